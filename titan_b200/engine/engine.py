"""The engine: a model on the GPU, its cache, the step function and the generation backend.

``Engine.step`` is the one step function.  It takes a batch of sequences, each
with the tokens it brings now (a whole prompt, or one token), runs exactly those
tokens as one packed batch from the cache that earlier steps left, and returns
float32 logits at the wanted places.  berniehans/titan's counterpart is
``ForwardDriver::prefill_chunked`` / ``decode`` for one sequence
(engine/engine-core/src/forward_driver.rs:939-1242, 3035-3070).

No length is committed if a step is refused: validation and page reservation
happen before the first kernel (the reference's InvalidSize guards,
forward_driver.rs:947-953, 3037-3043).  Pages reserved for a step that then
failed inside a kernel stay with their slot (they are room, not content) and
go back when the slot is freed.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels as K
from ..cache import PAGE_SIZE, CacheFull, SequenceCache
from ..config import load_config
from ..sampling import DeviceSampler, SamplerParams
from ..weights import DictWeights, FolderWeights, RandomWeights
from .batch import StepContext, StepEntry, StepLayout
from .decode_graph import DecodeGraph
from .generate import GenerationRequest, GenerationResult, generate, round_up
from .model import DecoderModel

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class StepError(ValueError):
    """A step that the engine refuses; the cache is as it was."""


@dataclass
class EngineOptions:
    dtype: object = "bfloat16"
    max_tokens: int = 8192            # tokens the cache holds over all live sequences (pages of 64)
    max_context: Optional[int] = None  # longest sequence; default: what the cache and the model's position limit allow (more than that limit is refused)
    max_slots: Optional[int] = None
    max_batch: int = 64               # sequences per generation batch
    gemm: str = "fast"                # "plain": CUDA-core matrix products even in bfloat16
    attention: str = "fast"           # "plain": the any-size attention kernels even where a tensor-core one fits
    attn_chunk: int = 256             # keys per split of decode attention
    mark_freed_pages: bool = False    # debugging: pages of a freed slot are overwritten with a large finite value, so a stale read shows
    fold_head_norm: bool = True       # decode steps: head norm, rotation and cache append inside the attention kernel where it can take them
    fold_norms: bool = True           # decode steps: a norm goes into the product that consumes it where the kernels can take it
    fold_norms_rows: int = 16         # ... in steps of up to this many rows (the kernels take up to 32; beyond 16 it was measured slower)
    early_pages: bool = True          # decode attention requests pages of older positions before it waits for the kernels before it
    decode_graphs: bool = True        # replay single-token steps as CUDA graphs once a batch size has run eagerly
    reproducible: bool = False        # bfloat16: partial sums along K add up in a fixed order, so the same requests in the same batches give the same bits on every run (slower)
    device: str = "cuda:0"


class Engine:
    def __init__(self, config, source_factory, options: EngineOptions):
        if not torch.cuda.is_available():
            raise RuntimeError("titan_b200 runs on a CUDA device (sm_100a); none is visible and there is no CPU path")
        self.options = options
        self.device = torch.device(options.device)
        torch.cuda.set_device(self.device)
        K.lib()                                   # build / load the kernels now, loudly
        self.dtype = _DTYPES[options.dtype]
        self.config = config
        self.spec = config.to_model_spec()
        self.model = DecoderModel(self.spec)
        self.model.load(source_factory(self.model.declared_weights(), self.dtype, self.device))
        num_pages = -(-options.max_tokens // PAGE_SIZE)
        limit = int(self.spec.max_positions)           # the model's own limit (max_position_embeddings)
        if options.max_context is not None and options.max_context > limit:
            raise StepError(f"max_context {options.max_context} is beyond the model's {limit} positions")
        max_context = min(options.max_context or limit, limit, num_pages * PAGE_SIZE)
        max_slots = options.max_slots or max(1, min(num_pages, (16 << 20) // max(1, -(-max_context // PAGE_SIZE))))
        self.cache = SequenceCache(self.model.cache_needs(), options.max_tokens, max_slots, max_context,
                                   self.dtype, self.device, mark_freed=options.mark_freed_pages)
        self.sampler = DeviceSampler(self.cache.state, max_slots, self.spec.vocab_size, self.device)
        self.scratch: Dict[str, torch.Tensor] = {}
        self.step_options = {"gemm": options.gemm, "attention": options.attention, "attn_chunk": options.attn_chunk,
                             "early_pages": options.early_pages, "fold_norms": options.fold_norms, "fold_head_norm": options.fold_head_norm,
                             "fold_norms_rows": options.fold_norms_rows,
                             "reproducible": options.reproducible,
                             "max_context": self.cache.max_context,
                             "sm_count": torch.cuda.get_device_properties(self.device).multi_processor_count}
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.steps_run = 0
        self.graph_launches = 0                   # launcher calls replayed through graphs
        self.last_logits: Optional[torch.Tensor] = None    # logits of the latest generation step, on the device; valid until the next step
        self._graphs: Dict[int, DecodeGraph] = {}
        self._ran_eagerly = set()
        # captured decode steps only if every part of the model allows it (Part.capturable)
        self._capturable = all(getattr(part, "capturable", True) for b in self.model.blocks for part in b.parts())

    # -- construction ------------------------------------------------------- #
    @classmethod
    def from_pretrained(cls, model_dir: str, dtype="bfloat16", **kw) -> "Engine":
        config = load_config(model_dir)
        ignorable = ["lm_head.weight"] if config.to_model_spec().lm_head is None else []
        return cls(config, lambda declared, dt, dev: FolderWeights(model_dir, declared, dt, dev, ignorable),
                   EngineOptions(dtype=dtype, **kw))

    @classmethod
    def from_random(cls, config, seed: int, dtype="bfloat16", **kw) -> "Engine":
        """Random weights made on the device (N(0, 0.02) matrices, 1 + N(0, 0.1) norm weights)."""
        return cls(config, lambda declared, dt, dev: RandomWeights(seed, dt, dev, store_dtype=torch.bfloat16),
                   EngineOptions(dtype=dtype, **kw))

    @classmethod
    def from_tensors(cls, config, tensors: Dict[str, torch.Tensor], dtype="bfloat16", **kw) -> "Engine":
        return cls(config, lambda declared, dt, dev: DictWeights(tensors, declared, dt, dev), EngineOptions(dtype=dtype, **kw))

    # -- properties the generation loop reads -------------------------------- #
    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    @property
    def max_context(self) -> int:
        return self.cache.max_context

    @property
    def max_batch(self) -> int:
        return min(self.options.max_batch, self.cache.max_slots)

    # -- slots --------------------------------------------------------------- #
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    # -- the step function ---------------------------------------------------- #
    def _context(self, layout: StepLayout) -> StepContext:
        return StepContext(layout, K.current_stream(), self.dtype, self.device, self.step_options, self.scratch)

    def _check_entries(self, entries: Sequence[StepEntry]) -> List[int]:
        if not entries:
            raise StepError("a step needs at least one sequence")
        seen = set()
        starts = []
        V = self.spec.vocab_size
        for e in entries:
            if not self.cache.is_live(e.slot):
                raise StepError(f"slot {e.slot} is not live")
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"slot {e.slot} brings no token")
            for t in e.tokens:
                if not 0 <= int(t) < V:
                    raise StepError(f"token id {t} lies outside the vocabulary of {V}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"logits wanted at place {w} of {n} tokens")
            starts.append(self.cache.length[e.slot])
        return starts

    def forward(self, entries: Sequence[StepEntry]) -> Tuple[torch.Tensor, StepLayout, StepContext]:
        """Run the tokens through the blocks; returns the residual stream [T, H]."""
        starts = self._check_entries(entries)
        try:
            self.cache.reserve({e.slot: s + len(e.tokens) for e, s in zip(entries, starts)})
        except CacheFull as err:
            raise StepError(str(err)) from None
        layout = StepLayout(entries, starts, self.device)
        self.h2d_bytes += layout.h2d_bytes
        self.steps_run += 1
        ctx = self._context(layout)
        try:
            self.sampler.observe(layout, ctx.stream)
            x = self.model.forward_hidden(ctx, self.cache)
            K.commit_lengths(layout.slot_of_seq, layout.kv_len, self.cache.state.seq_len, ctx.stream)
        except Exception:
            self.reset_accumulators()             # a kernel between a product and its consumer was refused
            raise
        for e, s in zip(entries, starts):
            self.cache.commit(e.slot, s + len(e.tokens))
        return x, layout, ctx

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Logits float32 [wanted, vocab] on the device, in the order of the entries and of
        their ``want`` lists; None if nothing is wanted."""
        x, layout, ctx = self.forward(entries)
        if layout.W == 0:
            return None
        return self.model.logits(x, ctx, layout.want)

    # -- backend of the generation loop ---------------------------------------- #
    def room_for(self, token_counts: Sequence[int]) -> bool:
        held = self.cache.tokens_held()
        want = sum(round_up(n, self.cache.page_size) for n in token_counts)
        return (held + want <= self.cache.num_pages * self.cache.page_size
                and self.cache.slots.free_count >= len(token_counts))

    def start(self, prompts, params, sequence_ids):
        slots = [self.cache.alloc_slot() for _ in prompts]
        try:
            self.sampler.configure(slots, params, sequence_ids)
            entries = [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]
            return slots, self._step_and_sample(entries)
        except Exception:
            for s in slots:
                self.cache.free_slot(s)
            raise

    def advance(self, slots, tokens):
        """One token for each sequence: host token ids in, sampled host token ids out."""
        B = len(slots)
        if not self.options.decode_graphs or not self._capturable or B not in self._ran_eagerly:
            self._ran_eagerly.add(B)              # the first step of a batch size runs eagerly (lazy set-up happens there)
            return self._step_and_sample([StepEntry(s, [t], [0]) for s, t in zip(slots, tokens)])
        g = self._prepare_graph_step(slots, 1)
        V = self.spec.vocab_size
        ids = np.asarray(tokens, dtype=np.int64)
        if ids.shape != (B,) or int(ids.min()) < 0 or int(ids.max()) >= V:
            bad = [int(t) for t in np.ravel(ids) if not 0 <= int(t) < V]
            raise StepError(f"token id {bad[0]} lies outside the vocabulary of {V}" if bad else f"{ids.size} tokens for {B} sequences")
        g.host_tokens_view[:] = ids                      # the pinned buffer, as numpy sees it
        g.tokens.copy_(g.host_tokens, non_blocking=True)
        self.h2d_bytes += 4 * B
        self.steps_run += 1
        self._replay(g, False)
        for s in slots:
            self.cache.commit(s, self.cache.length[s] + 1)
        g.host_out.copy_(g.out_tokens, non_blocking=True)       # into pinned memory, then one wait for the stream
        torch.cuda.current_stream(self.device).synchronize()
        self.d2h_bytes += 4 * B
        return g.host_out.tolist()

    def decode_on_device(self, slots, steps: int, keep_all: bool = False) -> torch.Tensor:
        """``steps`` decode steps without the host in the loop: every step feeds each sequence the
        token it sampled in the step before (``last_token`` of its slot).  Returns the last step's
        tokens as a device tensor [B], or with ``keep_all`` every step's [steps, B] (a device-to-device
        copy of B numbers per step); nothing is copied back to the host."""
        if not self._capturable:
            raise StepError("a part of this model cannot run in a captured step; decode with advance()")
        g = self._prepare_graph_step(slots, steps)
        history = torch.empty((steps, len(slots)), dtype=torch.int32, device=self.device) if keep_all else None
        for i in range(steps):
            self._replay(g, True)
            if keep_all:
                history[i].copy_(g.out_tokens, non_blocking=True)
        for s in slots:
            self.cache.commit(s, self.cache.length[s] + steps)
        self.steps_run += steps
        return history if keep_all else g.out_tokens

    def _prepare_graph_step(self, slots, steps: int) -> "DecodeGraph":
        g = self._graphs.get(len(slots))
        if steps == 1 and g is not None and g.slots == list(slots):
            # The sequences of the step before, which were checked then: a sequence whose length is inside a page needs
            # no new page for one more token (the host's share of a step at batch 64 is mostly these loops).
            length, page, limit = self.cache.length, self.cache.page_size, self.cache.max_context
            try:
                if all(length[s] % page and length[s] < limit for s in slots):
                    return g
            except KeyError:
                pass                                      # a slot was given back since: the checks below say so
        seen = set()
        for s in slots:
            if not self.cache.is_live(s) or s in seen:
                raise StepError(f"slot {s} is not live or appears twice")
            seen.add(s)
        try:
            self.cache.reserve({s: self.cache.length[s] + steps for s in slots})
        except CacheFull as err:
            raise StepError(str(err)) from None
        B = len(slots)
        if B not in self._graphs:
            self._graphs[B] = DecodeGraph(self, B)
        g = self._graphs[B]
        g.set_slots(slots)
        return g

    def reset_accumulators(self) -> None:
        """Zero the float32 buffers that decode products add into (``acc_*`` entries of the scratch).  Their
        consumers leave them zeroed after every use; a step that ended between a product and its consumer (a
        refused launch, a bounded wait that gave up) does not, and every later step of that shape would add
        onto stale sums.  Called after any failed step; in place, because captured graphs hold the addresses."""
        for scratch in [self.scratch] + [g.scratch for g in self._graphs.values()]:
            for key, t in scratch.items():
                if key.startswith("acc_"):
                    t.zero_()

    def _replay(self, g: "DecodeGraph", feed_last: bool) -> None:
        before = K.launch_count
        try:
            self.last_logits = g.replay(feed_last)
        except Exception:
            self.reset_accumulators()
            raise
        captured = K.launch_count - before
        if captured:                              # this call captured the graph: remember its size
            g.launches = captured
        self.graph_launches += g.launches

    def finish(self, slot) -> None:
        self.cache.free_slot(slot)

    def check_kernels(self) -> None:
        """Raise if a bounded wait inside a kernel gave up since the last check (the results of that step
        are invalid).  Synchronises the device; the generation loop calls it once per batch."""
        bad = K.wait_errors()
        if bad:
            self.reset_accumulators()
            raise StepError("a kernel's bounded wait gave up, results are invalid: " + ", ".join(f"{k} (code {v})" for k, v in bad.items()))

    def _step_and_sample(self, entries) -> List[int]:
        x, layout, ctx = self.forward(entries)
        logits = self.last_logits = self.model.logits(x, ctx, layout.want)
        tokens = self.sampler.sample(logits, layout.slot_of_seq, ctx.stream)
        host = tokens.cpu()
        self.d2h_bytes += host.numel() * 4
        return host.tolist()

    # -- the call a user makes --------------------------------------------------- #
    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 512,
                 params: Optional[SamplerParams] = None, stop_tokens: Optional[Sequence[int]] = None,
                 include_stop: bool = False) -> List[GenerationResult]:
        """Token ids in, token ids out.  ``stop_tokens`` defaults to the configuration's
        end-of-sequence ids (the reference uses literal Qwen ids, engine-server/src/server.rs:259)."""
        params = params or SamplerParams()
        stops = tuple(self.spec.stop_token_ids) if stop_tokens is None else tuple(int(t) for t in stop_tokens)
        reqs = [GenerationRequest(list(p), max_tokens, params, stops, include_stop) for p in prompts]
        return generate(self, reqs)
