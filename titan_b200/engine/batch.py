"""The ragged layout of one step: which tokens run, for which sequence, at which position.

A step runs only the tokens it is given, packed without padding: the tokens of
all sequences are concatenated (``T`` rows), and small int32 arrays tell every
kernel which sequence a row belongs to and where in that sequence it stands.
The layout is mixer-agnostic; parts read it and never change it.

berniehans/titan runs one sequence, so its kernels derive the position from the
row index (``cur_pos = pos + blockIdx / n_heads``,
engine/engine-cuda/kernels/norm_rope.cu:19-22) or read ``*pos_ptr``
(kernels/paged_attention.cu:21-24).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import kernels as K


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()          # indices among ``tokens`` whose logits are wanted


class StepLayout:
    """Device arrays of one step (all int32), cut from one buffer that one copy fills:

    tokens[T] seq_of[T] pos_of[T] slot_of_seq[B] q_start[B+1] start_pos[B] kv_len[B] want[W]
    """

    def __init__(self, entries: Sequence[StepEntry], start_lengths: Sequence[int], device):
        B = len(entries)
        lens = [len(e.tokens) for e in entries]
        T = sum(lens)
        want_rows: List[int] = []
        q_start = np.zeros(B + 1, dtype=np.int32)
        q_start[1:] = np.cumsum(lens)
        for b, e in enumerate(entries):
            want_rows.extend(int(q_start[b]) + int(w) for w in e.want)
        W = len(want_rows)
        sizes = [T, T, T, B, B + 1, B, B, W]
        offs = np.concatenate([[0], np.cumsum([-(-s // 4) * 4 for s in sizes])])      # 16-byte aligned parts
        host = np.zeros(int(offs[-1]), dtype=np.int32)
        starts = np.asarray(start_lengths, dtype=np.int32)
        for b, e in enumerate(entries):
            a, z = int(q_start[b]), int(q_start[b + 1])
            host[offs[0] + a: offs[0] + z] = np.asarray(e.tokens, dtype=np.int32)
            host[offs[1] + a: offs[1] + z] = b
            host[offs[2] + a: offs[2] + z] = starts[b] + np.arange(z - a, dtype=np.int32)
        host[offs[3]: offs[3] + B] = [e.slot for e in entries]
        host[offs[4]: offs[4] + B + 1] = q_start
        host[offs[5]: offs[5] + B] = starts
        host[offs[6]: offs[6] + B] = starts + np.asarray(lens, dtype=np.int32)
        host[offs[7]: offs[7] + W] = want_rows
        pinned = torch.from_numpy(host)
        if torch.device(device).type == "cuda":
            pinned = pinned.pin_memory()
        self.buffer = pinned.to(device, non_blocking=True)
        self._host_keepalive = pinned
        cut = lambda i, n: self.buffer[int(offs[i]): int(offs[i]) + n]
        self.tokens, self.seq_of, self.pos_of = cut(0, T), cut(1, T), cut(2, T)
        self.slot_of_seq, self.q_start = cut(3, B), cut(4, B + 1)
        self.start_pos, self.kv_len, self.want = cut(5, B), cut(6, B), cut(7, W)
        self.T, self.B, self.W = T, B, W
        self.max_new = max(lens) if lens else 0
        self.max_kv_len = int((starts + np.asarray(lens, dtype=np.int32)).max()) if B else 0
        self.all_single = all(n == 1 for n in lens)       # a decode step: one token per sequence
        self.all_fresh = bool((starts == 0).all())        # every sequence starts at its first token
        self.h2d_bytes = host.nbytes
        self.lengths_by_copy = True            # kv_len is final before the step's first kernel runs
        self.committed_len = None
        self._c: Optional[K.Batch] = None

    @classmethod
    def from_device_arrays(cls, tokens, seq_of, pos_of, slot_of_seq, q_start, start_pos, kv_len, want,
                           max_new: int, max_kv_len: int, all_single: bool, all_fresh: bool) -> "StepLayout":
        """A layout over arrays that already live on the device (a captured decode step,
        whose arrays a kernel refreshes from the slot state before every replay)."""
        self = cls.__new__(cls)
        self.buffer = None
        self.tokens, self.seq_of, self.pos_of = tokens, seq_of, pos_of
        self.slot_of_seq, self.q_start, self.start_pos, self.kv_len, self.want = slot_of_seq, q_start, start_pos, kv_len, want
        self.T, self.B, self.W = tokens.numel(), slot_of_seq.numel(), want.numel()
        self.max_new, self.max_kv_len = max_new, max_kv_len
        self.all_single, self.all_fresh = all_single, all_fresh
        self.h2d_bytes = 0
        self.lengths_by_copy = False           # a kernel of the step writes kv_len ...
        self.committed_len = None              # ... as committed_len[slot] + 1, if the owner names that array (by slot)
        self._c = None
        return self

    def c_struct(self) -> K.Batch:
        if self._c is None:
            p = lambda t: t.data_ptr() if t.numel() else None
            self._c = K.Batch(p(self.tokens), p(self.seq_of), p(self.pos_of), p(self.slot_of_seq), p(self.q_start),
                              p(self.start_pos), p(self.kv_len), self.T, self.B, self.max_new, self.max_kv_len)
        return self._c


@dataclass
class StepContext:
    """What a part sees of a step besides its input rows."""
    layout: StepLayout
    stream: int
    dtype: torch.dtype                 # compute dtype of activations and cache
    device: torch.device
    options: Dict[str, object] = field(default_factory=dict)
    scratch: Dict[str, torch.Tensor] = field(default_factory=dict)   # long-lived buffers by name

    sites_taken: int = 0               # places of "row_sums" handed out in this step

    def row_sums(self) -> Optional[torch.Tensor]:
        """A float32 [16, 32] place of this step's own, for a product that leaves its rows' partial sums of squares
        (one row per K slice) to its consumer; None when the step has none left (the model provides one per run of
        a layer).  Nothing has to be cleared: every part a consumer reads was stored by the producer in the same step."""
        places = self.scratch.get("row_sums")
        if places is None or self.sites_taken >= places.shape[0]:
            return None
        self.sites_taken += 1
        return places[self.sites_taken - 1]

    def empty(self, shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)
