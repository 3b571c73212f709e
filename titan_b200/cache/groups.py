"""Storage of the cache, one group per kind of need.

Layers whose mixers need the same thing share a group, and each group has
storage, pages and a block table of its own:

* ``KVGroup`` with ``window=None`` keeps every key and value of a sequence;
* ``KVGroup`` with ``window=n`` keeps a ring of the last ``ring_rows`` rows
  (``n`` rounded up to whole pages): position ``p`` lives in ring row
  ``p % ring_rows``;
* ``StateGroup`` keeps a tensor of fixed size per sequence and layer (no time
  axis), zeroed when a slot is handed out.

Storage layout of a KV group, per layer: ``[2 (K,V), num_pages, kv_heads,
page_size, head_dim]``; one head's page is ``page_size * head_dim`` contiguous
elements.  Block table: ``int32 [max_slots, table_width]``, page id of the
sequence's i-th page (ring page for a window group).

berniehans/titan keeps one flat pool ``[capacity, 2, kv_heads, head_dim]`` per
layer behind a one-entry block table
(engine/engine-cuda/src/paged_kv.rs:9-15, engine/engine-core/src/forward_driver.rs:613-618).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .slots import PagePool


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer asks of the cache (``Mixer.cache_need``)."""
    kind: str                              # "kv" | "state"
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: torch.dtype = torch.float32

    def group_key(self):
        return (self.kind, self.num_kv_heads, self.head_dim, self.window, self.state_shape, self.state_dtype)


STALE_MARK = 3.0e4        # what a freed page holds when the cache is asked to mark freed pages


class KVGroup:
    def __init__(self, need: CacheNeed, layers: List[int], num_pages: int, page_size: int,
                 max_slots: int, max_context: int, dtype: torch.dtype, device):
        self.need, self.layers = need, list(layers)
        self.page_size, self.num_pages = page_size, num_pages
        pages_full = -(-max_context // page_size)
        if need.window is None:
            self.ring_rows = 0
            self.table_width = pages_full
        else:
            self.ring_rows = -(-need.window // page_size) * page_size
            self.table_width = min(self.ring_rows // page_size, pages_full)
            if self.table_width * page_size < self.ring_rows:      # the context is shorter than the ring
                self.ring_rows = 0
        self.pool = PagePool(num_pages)
        self.pages_of: Dict[int, List[int]] = {}
        # zeroed once: rows past a sequence's end are multiplied by a zero weight in the tensor-core
        # kernels, so they must hold finite numbers (a freed page keeps its old, finite, rows)
        self.storage = torch.zeros((len(layers), 2, num_pages, need.num_kv_heads, page_size, need.head_dim),
                                   dtype=dtype, device=device)
        self.table_host = torch.zeros((max_slots, self.table_width), dtype=torch.int32)
        if torch.device(device).type == "cuda":
            self.table_host = self.table_host.pin_memory()     # so that a page's table entry is copied without a sync
        self.table = torch.zeros((max_slots, self.table_width), dtype=torch.int32, device=device)

    # -- pages ---------------------------------------------------------- #
    def pages_for(self, length: int) -> int:
        return min(-(-length // self.page_size), self.table_width)

    def shortfall(self, slot: int, new_length: int) -> int:
        return max(0, self.pages_for(new_length) - len(self.pages_of.get(slot, ())))

    def extend(self, slot: int, new_length: int) -> None:
        have = self.pages_of.setdefault(slot, [])
        n = self.pages_for(new_length) - len(have)
        if n <= 0:
            return
        first = len(have)
        have.extend(self.pool.take_many(n))
        self.table_host[slot, first:len(have)] = torch.tensor(have[first:], dtype=torch.int32)
        self.table[slot, first:len(have)].copy_(self.table_host[slot, first:len(have)], non_blocking=True)

    def release(self, slot: int, mark: bool = False) -> None:
        """Give the slot's pages back.  ``mark``: first overwrite them with a large finite value, so that a
        later read of a row that its new owner never wrote shows in the result (not NaN or infinity: the
        tensor-core kernels multiply rows past a sequence's end by a weight of zero)."""
        pages = self.pages_of.pop(slot, [])
        if mark and pages:
            idx = torch.tensor(pages, dtype=torch.long, device=self.storage.device)
            self.storage.index_fill_(2, idx, STALE_MARK)
        for p in pages:
            self.pool.give_back(p)

    def layer_storage(self, index_in_group: int) -> torch.Tensor:
        return self.storage[index_in_group]

    def bytes(self) -> int:
        return self.storage.numel() * self.storage.element_size()


class StateGroup:
    def __init__(self, need: CacheNeed, layers: List[int], max_slots: int, device):
        self.need, self.layers = need, list(layers)
        self.storage = torch.zeros((len(layers), max_slots) + tuple(need.state_shape),
                                   dtype=need.state_dtype, device=device)

    def reset(self, slot: int) -> None:
        self.storage[:, slot].zero_()

    def layer_storage(self, index_in_group: int) -> torch.Tensor:
        return self.storage[index_in_group]

    def bytes(self) -> int:
        return self.storage.numel() * self.storage.element_size()
