"""Host-side bookkeeping of the cache: sequence slots and storage pages.

A *slot* is what one live sequence holds: a row in every block table, a row in
every fixed-size state tensor, and its length.  A *page* is ``page_size``
consecutive token rows of one cache group's storage.  Both are handed out
lowest-free-first and come back when the sequence ends; neither is cleared on
return, because a sequence's length gates every read.

berniehans/titan's CPU cache does the same with blocks per sequence
(engine/engine-kvcache/src/cache.rs:126-192; exhaustion leaves no partial
state, :166-172, 373-405) and its scheduler reuses slot ids lowest-first
(engine/engine-server/src/scheduler.rs:192-201).
"""
from __future__ import annotations

import heapq
from typing import List


class CacheError(RuntimeError):
    """Misuse of the cache: unknown slot, double free, and the like."""


class CacheFull(CacheError):
    """No free slot or not enough free pages; nothing was changed."""


class _LowestFree:
    def __init__(self, count: int, what: str):
        if count <= 0:
            raise CacheError(f"a cache needs at least one {what}")
        self.count, self.what = count, what
        self._free: List[int] = list(range(count))
        heapq.heapify(self._free)
        self._held = [False] * count

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.count - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.count and self._held[i]

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.count} are held)")
        i = heapq.heappop(self._free)
        self._held[i] = True
        return i

    def give_back(self, i: int) -> None:
        if not 0 <= i < self.count:
            raise CacheError(f"{self.what} {i} does not exist (there are {self.count})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is not held (freed twice?)")
        self._held[i] = False
        heapq.heappush(self._free, i)

    def check(self) -> None:
        """Invariant: every id is either free exactly once or held, never both."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise CacheError(f"a {self.what} is on the free list twice")
        for i in range(self.count):
            if self._held[i] == (i in set(free)):
                raise CacheError(f"{self.what} {i} is {'both held and free' if self._held[i] else 'lost'}")


class SlotAllocator(_LowestFree):
    def __init__(self, max_slots: int):
        super().__init__(max_slots, "slot")


class PagePool(_LowestFree):
    def __init__(self, num_pages: int):
        super().__init__(num_pages, "page")

    def take_many(self, n: int) -> List[int]:
        if n > self.free_count:
            raise CacheFull(f"{n} pages wanted, {self.free_count} of {self.count} free")
        return [self.take() for _ in range(n)]
