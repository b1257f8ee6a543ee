"""Host-side bookkeeping of the cache: which sequence holds which slot and which pages.

A *slot* stands for one live sequence: its length so far and, for each group of
layers, the pages that hold its keys and values.  A *page* holds ``page_size``
consecutive positions of one sequence for every layer of a group.  Slots and
pages come from free lists and go back to them when the sequence ends; handing
out something twice, freeing it twice or freeing what was never handed out is an
error, never silent.

The reference has one sequence and one contiguous cache that ``reset`` rewinds
(src/kv_cache.zig:11-57, src/engine.zig:287-289); its capacity errors are
``PromptExceedsContext`` and ``ContextFull`` (src/engine.zig:323,346), which
correspond to :class:`CacheFull` and :class:`SequenceTooLong` here.
"""
from __future__ import annotations

import heapq
import numpy as np
from typing import Dict, List, Optional


class CacheError(RuntimeError):
    """Misuse of the cache bookkeeping (double free, unknown slot, ...)."""


class NoFreeSlot(CacheError):
    """Every slot is held by a live sequence."""


class CacheFull(CacheError):
    """The pages that are free do not cover what the step needs."""


class SequenceTooLong(CacheError):
    """A sequence would grow beyond the positions the model or the cache allows."""


class FreeList:
    """Hands out the integers 0..n-1, lowest first, and takes them back."""

    def __init__(self, n: int, what: str):
        if n < 0:
            raise ValueError(f"cannot hold {n} {what}s")
        self.what = what
        self.capacity = n
        self._free: List[int] = list(range(n))               # a heap: the lowest comes first
        self._held = [False] * n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.capacity - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise (NoFreeSlot if self.what == "slot" else CacheFull)(f"no free {self.what} (all {self.capacity} are held)")
        i = heapq.heappop(self._free)
        self._held[i] = True
        return i

    def give_back(self, i: int) -> None:
        if not (0 <= i < self.capacity):
            raise CacheError(f"{self.what} {i} does not exist (there are {self.capacity})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is freed twice or was never handed out")
        self._held[i] = False
        heapq.heappush(self._free, i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.capacity and self._held[i]

    def check(self) -> None:
        """Every number is either free or held, exactly once."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise CacheError(f"a {self.what} is on the free list twice")
        for i in range(self.capacity):
            if self._held[i] == (i in set(free)):
                raise CacheError(f"{self.what} {i} is lost or held twice")


class GroupPages:
    """Pages of one group of layers: the pool and, per slot, the pages by position."""

    def __init__(self, n_pages: int, page_size: int, window: Optional[int]):
        self.pool = FreeList(n_pages, "page")
        self.page_size = page_size
        self.window = window
        self.pages_of: Dict[int, List[int]] = {}     # slot -> page per block index (-1: released)
        self.table: Optional[np.ndarray] = None      # the same as rows of an int32 array, once its size is known

    def mirror(self, n_slots: int, max_pages: int) -> None:
        """Keep the pages of every slot also as row ``slot`` of an int32 array [n_slots, max_pages] (-1: none),
        so that a step's block table is one indexing operation."""
        self.table = np.full((n_slots, max_pages), -1, dtype=np.int32)
        for slot, pages in self.pages_of.items():
            self.table[slot, :len(pages)] = pages

    def pages_needed(self, slot: int, new_len: int) -> int:
        have = len(self.pages_of.get(slot, ()))
        return max(0, -(-new_len // self.page_size) - have)

    def grow(self, slot: int, new_len: int) -> None:
        pages = self.pages_of.setdefault(slot, [])
        want = -(-new_len // self.page_size)
        while len(pages) < want:
            pages.append(self.pool.take())
            if self.table is not None and len(pages) <= self.table.shape[1]:
                self.table[slot, len(pages) - 1] = pages[-1]

    def release_behind_window(self, slot: int, length: int) -> None:
        """Give back pages whose every position lies before the window of the next token."""
        if self.window is None:
            return
        first_visible = max(0, length - self.window + 1)    # the next token sits at position `length`
        pages = self.pages_of.get(slot, [])
        for i in range(min(len(pages), first_visible // self.page_size)):
            if pages[i] >= 0:
                self.pool.give_back(pages[i])
                pages[i] = -1
                if self.table is not None and i < self.table.shape[1]:
                    self.table[slot, i] = -1

    def free(self, slot: int) -> None:
        for p in self.pages_of.pop(slot, []):
            if p >= 0:
                self.pool.give_back(p)
        if self.table is not None:
            self.table[slot, :] = -1


class SlotTable:
    """Slots of live sequences, their lengths, and their pages in every group."""

    def __init__(self, n_slots: int, groups: List[GroupPages], max_len: int):
        self.slots = FreeList(n_slots, "slot")
        self.groups = groups
        self.max_len = max_len
        self.length: Dict[int, int] = {}

    def alloc(self) -> int:
        s = self.slots.take()
        self.length[s] = 0
        return s

    def free(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"slot {slot} is freed twice or was never handed out")
        for g in self.groups:
            g.free(slot)
        del self.length[slot]
        self.slots.give_back(slot)

    def length_of(self, slot: int) -> int:
        try:
            return self.length[slot]
        except KeyError:
            raise CacheError(f"slot {slot} is not held by a live sequence") from None

    def reserve(self, growth: Dict[int, int]) -> None:
        """Make room for ``growth[slot]`` more positions in every slot named, or change nothing."""
        for slot, n in growth.items():
            cur = self.length_of(slot)
            if n < 0:
                raise CacheError("a sequence cannot shrink")
            if cur + n > self.max_len:
                raise SequenceTooLong(
                    f"slot {slot} would hold {cur + n} positions; the limit is {self.max_len}")
        for g in self.groups:
            need = sum(g.pages_needed(slot, self.length[slot] + n) for slot, n in growth.items())
            if need > g.pool.n_free:
                raise CacheFull(f"the step needs {need} more pages of {g.page_size} positions, "
                                f"{g.pool.n_free} of {g.pool.capacity} are free")
        for g in self.groups:
            for slot, n in growth.items():
                g.grow(slot, self.length[slot] + n)

    def advance(self, growth: Dict[int, int]) -> None:
        """The step has run: the sequences are longer now; windows let go of what fell behind."""
        for slot, n in growth.items():
            self.length[slot] += n
            for g in self.groups:
                g.release_behind_window(slot, self.length[slot])

    def check(self) -> None:
        self.slots.check()
        for g in self.groups:
            g.pool.check()
            seen = set()
            for slot, pages in g.pages_of.items():
                if not self.slots.is_held(slot):
                    raise CacheError(f"pages are kept for slot {slot}, which is free")
                for p in pages:
                    if p < 0:
                        continue
                    if p in seen or not g.pool.is_held(p):
                        raise CacheError(f"page {p} is held twice or not at all")
                    seen.add(p)
            if len(seen) != g.pool.n_held:
                raise CacheError("a page is held by no sequence (lost)")
