"""Device-side sampler: per-slot options and counters, one kernel launch per step.

The options of a sequence live in device arrays indexed by its slot, next to
its other fixed-size state; the kernel reads them, draws, writes the token to
``last_token[slot]`` and advances ``sample_step[slot]``.  The uniform number of
a draw is a hash of (seed, sequence id, step): a sequence samples the same
tokens whatever else is in its batch.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import kernels as K
from .params import SamplerParams


class DeviceSampler:
    def __init__(self, slot_state, max_slots: int, vocab_size: int, device, parts: Optional[int] = None):
        self.state, self.V, self.device = slot_state, vocab_size, device
        f = lambda dt, v=0: torch.full((max_slots,), v, dtype=dt, device=device)
        self.temperature, self.top_p = f(torch.float32), f(torch.float32, 1.0)
        self.top_k, self.penalty = f(torch.int32), f(torch.float32, 1.0)
        self.max_slots = max_slots
        # several blocks per row look for the maximum when a row is long enough to keep them busy
        self.parts = (32 if vocab_size >= 32 * 1024 else 0) if parts is None else int(parts)
        self.part_best = torch.empty((max_slots, max(self.parts, 1)), dtype=torch.float32, device=device)
        self.part_idx = torch.empty((max_slots, max(self.parts, 1)), dtype=torch.int32, device=device)
        self.seen: Optional[torch.Tensor] = None          # [max_slots, ceil(V/32)] bits of context tokens
        self._penalised = set()

    def configure(self, slots: Sequence[int], params: Sequence[SamplerParams], sequence_ids: Sequence[int]) -> None:
        """Set the options of freshly started sequences (one small copy per array)."""
        for p in params:
            p.validate()
        idx = torch.tensor(list(slots), dtype=torch.long, device=self.device)
        put = lambda arr, vals, dt: arr.index_copy_(0, idx, torch.tensor(vals, dtype=dt, device=self.device))
        put(self.temperature, [p.temperature for p in params], torch.float32)
        put(self.top_p, [p.top_p for p in params], torch.float32)
        put(self.top_k, [p.top_k for p in params], torch.int32)
        put(self.penalty, [p.repetition_penalty for p in params], torch.float32)
        put(self.state.seed, [p.seed_value() for p in params], torch.int64)
        put(self.state.sequence_id, [int(s) & ((1 << 63) - 1) for s in sequence_ids], torch.int64)
        self.state.sample_step.index_fill_(0, idx, 0)
        if any(p.repetition_penalty > 1.0 for p in params):
            if self.seen is None:
                self.seen = torch.zeros((self.max_slots, -(-self.V // 32)), dtype=torch.int32, device=self.device)
            self.seen.index_fill_(0, idx, 0)
        for s, p in zip(slots, params):
            (self._penalised.add if p.repetition_penalty > 1.0 else self._penalised.discard)(s)

    def observe(self, layout, stream: int) -> None:
        """Record a step's tokens as context of the repetition penalty."""
        if self.seen is not None and self._penalised:
            K.mark_seen(layout.tokens, layout.seq_of, layout.slot_of_seq, self.seen, layout.T, stream)

    def sample(self, logits: torch.Tensor, slot_of_row: torch.Tensor, stream: int,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits float32 [B, V] -> int32 tokens [B] on the device."""
        B = logits.shape[0]
        if out is None:
            out = torch.empty(B, dtype=torch.int32, device=self.device)
        a = K.SampleArgs()
        a.logits, a.ld, a.V, a.B = logits.data_ptr(), logits.stride(0), self.V, B
        a.slot_of_row = slot_of_row.data_ptr()
        a.temperature, a.top_k = self.temperature.data_ptr(), self.top_k.data_ptr()
        a.top_p, a.penalty = self.top_p.data_ptr(), self.penalty.data_ptr()
        a.seed, a.sequence_id = self.state.seed.data_ptr(), self.state.sequence_id.data_ptr()
        a.sample_step, a.last_token = self.state.sample_step.data_ptr(), self.state.last_token.data_ptr()
        a.seen = None if self.seen is None else self.seen.data_ptr()
        a.seen_words = 0 if self.seen is None else self.seen.shape[1]
        a.out = out.data_ptr()
        a.parts = self.parts if B <= self.max_slots else 0
        a.part_best, a.part_idx = self.part_best.data_ptr(), self.part_idx.data_ptr()
        K.sample(a, stream)
        return out
