"""A decode step captured as a CUDA graph: one launch per generated token instead of hundreds.

The captured step must not depend on host values that change between steps, so its layout arrays
are device buffers that a small kernel refreshes from the per-slot state at the start of every
replay (position = the slot's length, token = what the host put there or the slot's last sampled
token), and the number of attention splits is fixed at what the longest context needs.  What the
host still does per step is bookkeeping: pages for the next token, the host copy of the lengths.

berniehans/titan captures its decode pass the same way and feeds it through ``pos_dev`` and
``token_id_dev`` (engine/engine-core/src/forward_driver.rs:2413-2542, 2948-3032); there the split
count is frozen at capture time from the then-current position (:2240), which is not repeated here.
"""
from __future__ import annotations

import gc
import weakref
from typing import Dict, List, Optional, Sequence

import torch

from .. import kernels as K
from .batch import StepContext, StepLayout


class DecodeGraph:
    """Captured decode steps for exactly ``B`` sequences (which ones is data, not part of the graph)."""

    def __init__(self, engine, B: int):
        self._engine, self.B = weakref.ref(engine), B      # no cycle: an engine that is dropped frees its graphs at once
        dev = engine.device
        i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)
        ar = lambda n: torch.arange(n, dtype=torch.int32, device=dev)
        self.slot_of_seq, self.tokens, self.pos_of = i32(B), i32(B), i32(B)
        self.start_pos, self.kv_len, self.out_tokens = i32(B), i32(B), i32(B)
        self.layout = StepLayout.from_device_arrays(
            self.tokens, ar(B), self.pos_of, self.slot_of_seq, ar(B + 1), self.start_pos, self.kv_len, ar(B),
            max_new=1, max_kv_len=engine.max_context, all_single=True, all_fresh=False)
        self.layout.committed_len = engine.cache.state.seq_len     # kv_len = committed length + 1, known before the step
        self.options = dict(engine.step_options, fixed_splits=True)
        self.scratch: Dict[str, torch.Tensor] = {}
        self.graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self.slots: Optional[List[int]] = None
        self.launches = 0                      # launcher calls inside one replay
        self.logits: Dict[tuple, torch.Tensor] = {}    # per captured graph: the step's logits [B, vocab], valid until its next replay
        self.host_tokens = torch.zeros(B, dtype=torch.int32).pin_memory()
        self.host_tokens_view = self.host_tokens.numpy()
        self.host_slots = torch.zeros(B, dtype=torch.int32).pin_memory()
        self.host_out = torch.zeros(B, dtype=torch.int32).pin_memory()      # the step's sampled tokens, read by the host

    @property
    def engine(self):
        return self._engine()

    def set_slots(self, slots: Sequence[int]) -> None:
        if self.slots != list(slots):
            self.host_slots.copy_(torch.tensor(list(slots), dtype=torch.int32))
            self.slot_of_seq.copy_(self.host_slots, non_blocking=True)
            self.slots = list(slots)

    def _body(self, feed_last: bool) -> torch.Tensor:
        e = self.engine
        stream = K.current_stream()
        st = e.cache.state
        K.decode_prepare(self.slot_of_seq, st.seq_len, st.last_token, feed_last, self.tokens, self.pos_of,
                         self.start_pos, self.kv_len, stream)
        ctx = StepContext(self.layout, stream, e.dtype, e.device, self.options, self.scratch)
        if e.sampler.seen is not None:
            K.mark_seen(self.tokens, self.layout.seq_of, self.slot_of_seq, e.sampler.seen, self.B, stream)
        x = e.model.forward_hidden(ctx, e.cache)
        logits = e.model.logits(x, ctx, self.layout.want)
        e.sampler.sample(logits, self.slot_of_seq, stream, out=self.out_tokens)
        K.commit_lengths(self.slot_of_seq, self.kv_len, st.seq_len, stream)
        return logits

    def replay(self, feed_last: bool) -> torch.Tensor:
        """Run the step; returns its logits (memory of the graph: read them before the next replay)."""
        key = (feed_last, self.engine.sampler.seen is not None)
        g = self.graphs.get(key)
        if g is None:
            # Nothing may free device memory or destroy another graph while the stream is capturing (that
            # invalidates the capture), and Python's cycle collector can do both at any allocation when dead
            # objects that hold tensors or graphs are around: collect them now, and keep it off meanwhile.
            g = torch.cuda.CUDAGraph()
            gc.collect()
            was_enabled = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(g):
                    self.logits[key] = self._body(feed_last)
            finally:
                if was_enabled:
                    gc.enable()
            self.graphs[key] = g
        g.replay()
        return self.logits[key]
