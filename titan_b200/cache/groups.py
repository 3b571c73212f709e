"""Storage of the cache, one group per kind of need, and the registry of kinds.

A kind of need is a class registered under ``CacheNeed.kind``
(``register_cache_group``); ``SequenceCache`` builds one group per distinct need
as ``Class(need, layers, geometry)`` and talks to it only through the methods of
``CacheGroup`` below, so another kind of storage (a latent vector per token, a
window of inputs) is a class and a registration, not an edit of the cache.

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
    kind: str                              # a registered kind: "kv" | "state" | ...
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    state_dtype: torch.dtype = torch.float32
    extra: Tuple[Tuple[str, object], ...] = ()     # what a kind defined outside the package needs to know

    def group_key(self):
        return (self.kind, self.num_kv_heads, self.head_dim, self.window, self.state_shape, self.state_dtype, self.extra)

    def option(self, key: str, default=None):
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class CacheGeometry:
    """What every group is sized from."""
    num_pages: int
    page_size: int
    max_slots: int
    max_context: int
    dtype: torch.dtype                     # compute dtype of the engine
    device: object


class CacheGroup:
    """Interface of a group of storage.  ``layers`` are the runs of the layer order that share it; a run's
    storage is ``layer_storage(index_in_group)``.  All bookkeeping is on the host; nothing here may
    synchronise the device."""

    def __init__(self, need: CacheNeed, layers: List[int], geometry: CacheGeometry):
        self.need, self.layers = need, list(layers)

    def on_alloc(self, slot: int) -> None:
        """A slot is handed to a new sequence (fixed-size state starts from zero here)."""

    def room_error(self, wanted: Dict[int, int]) -> Optional[str]:
        """Why ``wanted`` (slot -> tokens it shall hold in total) cannot be held, or None.  Changes nothing."""
        return None

    def extend(self, slot: int, new_length: int) -> None:
        """Make room so that ``slot`` can hold ``new_length`` tokens (called only after ``room_error`` said None)."""

    def release(self, slot: int, mark: bool = False) -> None:
        """The slot's sequence has ended: give back what it held.  ``mark``: overwrite it with a large
        finite value first, so that a stale read shows."""

    def check(self, is_live) -> None:
        """Invariants for tests; raise ``CacheError``."""

    def layer_storage(self, index_in_group: int) -> torch.Tensor:
        raise NotImplementedError

    def bytes(self) -> int:
        return 0


_GROUP_KINDS: Dict[str, type] = {}


def register_cache_group(kind: str, cls: type) -> type:
    _GROUP_KINDS[kind] = cls
    return cls


def build_cache_group(need: CacheNeed, layers: List[int], geometry: CacheGeometry) -> CacheGroup:
    if need.kind not in _GROUP_KINDS:
        from .slots import CacheError
        raise CacheError(f"unknown cache need '{need.kind}'; registered kinds: {', '.join(sorted(_GROUP_KINDS))}")
    return _GROUP_KINDS[need.kind](need, layers, geometry)


STALE_MARK = 3.0e4        # what a freed page holds when the cache is asked to mark freed pages


class KVGroup(CacheGroup):
    def __init__(self, need: CacheNeed, layers: List[int], geometry: CacheGeometry):
        self.need, self.layers = need, list(layers)
        page_size, num_pages, device = geometry.page_size, geometry.num_pages, geometry.device
        self.page_size, self.num_pages = page_size, num_pages
        pages_full = -(-geometry.max_context // page_size)
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
                                   dtype=geometry.dtype, device=device)
        self.table = torch.zeros((geometry.max_slots, self.table_width), dtype=torch.int32, device=device)
        self._pin = torch.device(device).type == "cuda"

    # -- pages ---------------------------------------------------------- #
    def pages_for(self, length: int) -> int:
        return min(-(-length // self.page_size), self.table_width)

    def shortfall(self, slot: int, new_length: int) -> int:
        return max(0, self.pages_for(new_length) - len(self.pages_of.get(slot, ())))

    def room_error(self, wanted: Dict[int, int]) -> Optional[str]:
        short = sum(self.shortfall(slot, n) for slot, n in wanted.items())
        if short > self.pool.free_count:
            return (f"{short} more pages of {self.page_size} tokens wanted, "
                    f"{self.pool.free_count} of {self.pool.count} free")
        return None

    def extend(self, slot: int, new_length: int) -> None:
        have = self.pages_of.setdefault(slot, [])
        n = self.pages_for(new_length) - len(have)
        if n <= 0:
            return
        first = len(have)
        have.extend(self.pool.take_many(n))
        # Every copy has a staging tensor of its own: the copy is asynchronous, and a shared staging row could
        # be rewritten for the slot's next owner while an earlier copy of it is still queued.  (Pinned memory
        # from torch's host allocator is not handed out again before the copies that read it have run.)
        stage = torch.tensor(have[first:], dtype=torch.int32)
        if self._pin:
            stage = stage.pin_memory()
        self.table[slot, first:len(have)].copy_(stage, non_blocking=True)

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

    def check(self, is_live) -> None:
        from .slots import CacheError
        self.pool.check()
        held = [p for pages in self.pages_of.values() for p in pages]
        if len(set(held)) != len(held):
            raise CacheError("a page belongs to two sequences")
        if len(held) != self.pool.held_count:
            raise CacheError("a page is held by no sequence")
        for slot in self.pages_of:
            if not is_live(slot):
                raise CacheError(f"pages are held by slot {slot}, which is not live")

    def layer_storage(self, index_in_group: int) -> torch.Tensor:
        return self.storage[index_in_group]

    def bytes(self) -> int:
        return self.storage.numel() * self.storage.element_size()


class StateGroup(CacheGroup):
    def __init__(self, need: CacheNeed, layers: List[int], geometry: CacheGeometry):
        self.need, self.layers = need, list(layers)
        self.storage = torch.zeros((len(layers), geometry.max_slots) + tuple(need.state_shape),
                                   dtype=need.state_dtype, device=geometry.device)

    def on_alloc(self, slot: int) -> None:
        self.storage[:, slot].zero_()

    reset = on_alloc

    def layer_storage(self, index_in_group: int) -> torch.Tensor:
        return self.storage[index_in_group]

    def bytes(self) -> int:
        return self.storage.numel() * self.storage.element_size()


register_cache_group("kv", KVGroup)
register_cache_group("state", StateGroup)
