"""The cache of live sequences: slots, lengths, groups of storage, fixed-size state.

``SequenceCache`` is built from the needs of a model's layers (one
``CacheNeed`` or ``None`` per layer).  It owns

* the slot allocator and each sequence's length (host and device copies);
* one group of storage per distinct need, built from the registry of kinds
  (``groups.register_cache_group``: ``kv``, ``state``, and what else is
  registered), and the map from a layer to (group, index within the group);
* ``SlotState``: per-sequence state of fixed size that no layer owns (length,
  last token, sampling counters), the same place where a mixer's fixed-size
  state lies (a ``StateGroup``).

``reserve`` is all-or-nothing: it first asks every group whether the pages are
there, and only then takes them (berniehans/titan:
engine/engine-kvcache/src/cache.rs:166-172).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .groups import CacheGeometry, CacheGroup, CacheNeed, build_cache_group
from .slots import CacheError, CacheFull, SlotAllocator

PAGE_SIZE = 64


class SlotState:
    """Device arrays indexed by slot.  ``seq_len`` is the number of tokens whose
    keys are in the cache; the sampling fields make a draw depend on (seed,
    sequence id, step) only (berniehans/titan keeps pos_dev, token_id_dev and
    step_counter_dev, engine/engine-core/src/forward_driver.rs:547-575)."""

    def __init__(self, max_slots: int, device):
        z = lambda dt: torch.zeros(max_slots, dtype=dt, device=device)
        self.seq_len = z(torch.int32)
        self.last_token = z(torch.int32)
        self.sample_step = z(torch.int32)
        self.sequence_id = z(torch.int64)
        self.seed = z(torch.int64)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in vars(self).values())


class SequenceCache:
    def __init__(self, needs: Sequence[Optional[CacheNeed]], max_tokens: int, max_slots: int,
                 max_context: int, dtype: torch.dtype, device, page_size: int = PAGE_SIZE, mark_freed: bool = False):
        if max_tokens <= 0 or max_context <= 0:
            raise CacheError("max_tokens and max_context must be positive")
        self.page_size = page_size
        self.mark_freed = mark_freed           # a debugging aid: freed pages are overwritten with a large value
        self.num_pages = -(-max_tokens // page_size)
        self.max_context = min(max_context, self.num_pages * page_size)
        self.max_slots = max_slots
        self.device = device
        self.slots = SlotAllocator(max_slots)
        self.length: Dict[int, int] = {}
        self.state = SlotState(max_slots, device)
        self.groups: List[CacheGroup] = []
        geometry = CacheGeometry(self.num_pages, page_size, max_slots, self.max_context, dtype, device)
        self.layer_place: List[Optional[Tuple[int, int]]] = []
        by_key: Dict[tuple, List[int]] = {}
        for i, need in enumerate(needs):
            if need is not None:
                by_key.setdefault(need.group_key(), []).append(i)
        need_of = {need.group_key(): need for need in needs if need is not None}
        place: Dict[int, Tuple[int, int]] = {}
        for key, layers in by_key.items():
            need = need_of[key]
            g = build_cache_group(need, layers, geometry)
            for j, layer in enumerate(layers):
                place[layer] = (len(self.groups), j)
            self.groups.append(g)
        self.layer_place = [place.get(i) for i in range(len(needs))]

    # -- slots ---------------------------------------------------------- #
    def alloc_slot(self) -> int:
        slot = self.slots.take()
        self.length[slot] = 0
        self.state.seq_len[slot] = 0
        for g in self.groups:
            g.on_alloc(slot)
        return slot

    def free_slot(self, slot: int) -> None:
        self.slots.give_back(slot)          # raises on unknown / double free
        del self.length[slot]
        for g in self.groups:
            g.release(slot, self.mark_freed)

    def is_live(self, slot: int) -> bool:
        return self.slots.is_held(slot)

    # -- room ------------------------------------------------------------ #
    def reserve(self, wanted: Dict[int, int]) -> None:
        """Make room so that each slot can hold ``wanted[slot]`` tokens in total.
        Either every slot gets its pages or none does."""
        for slot, n in wanted.items():
            if not self.is_live(slot):
                raise CacheError(f"slot {slot} is not live")
            if n > self.max_context:
                raise CacheFull(f"slot {slot} would hold {n} tokens; the context holds {self.max_context}")
        for g in self.groups:
            why = g.room_error(wanted)
            if why:
                raise CacheFull(why)
        for g in self.groups:
            for slot, n in wanted.items():
                g.extend(slot, n)

    def commit(self, slot: int, new_length: int) -> None:
        """Host copy of the length after a step; the device copy is advanced by the step itself."""
        self.length[slot] = new_length

    # -- views ----------------------------------------------------------- #
    def view_for_layer(self, layer: int):
        place = self.layer_place[layer]
        if place is None:
            return None
        g = self.groups[place[0]]
        return g, place[1]

    def tokens_held(self) -> int:
        return sum(-(-n // self.page_size) * self.page_size for n in self.length.values())

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups) + self.state.bytes()

    def check(self) -> None:
        """Invariants for tests: no slot or page lost, held twice or freed twice."""
        self.slots.check()
        if sorted(self.length) != [i for i in range(self.max_slots) if self.slots.is_held(i)]:
            raise CacheError("lengths are kept for slots that are not held")
        for g in self.groups:
            g.check(self.is_live)
