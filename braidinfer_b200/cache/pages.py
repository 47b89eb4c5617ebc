"""Host-side bookkeeping of the cache: a pool of pages and a table of sequence slots.

The reference keeps one sequence per model with a LIFO free list of 64-token chunks
(crates/braidinfer-runtime/src/paged_kv.rs:83-181 PageAllocator, :741-921 SequenceState);
here many sequences hold slots at once and every layer group has a pool of its own.
No CUDA in this file: it is tested on the CPU.
"""
from __future__ import annotations

from typing import Dict, List, Optional


class CacheError(RuntimeError):
    """Misuse or exhaustion of the cache (never undefined behaviour)."""


class PagePool:
    """Fixed number of pages, handed out and taken back; a page is held at most once."""

    def __init__(self, num_pages: int) -> None:
        if num_pages < 0:
            raise CacheError(f"a pool cannot have {num_pages} pages")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))    # LIFO: page 0 first
        self._held = [False] * num_pages

    @property
    def available(self) -> int:
        return len(self._free)

    @property
    def in_use(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise CacheError(f"the cache is full: all {self.num_pages} pages are in use")
        p = self._free.pop()
        self._held[p] = True
        return p

    def free(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise CacheError(f"page {page} is not in the pool of {self.num_pages}")
        if not self._held[page]:
            raise CacheError(f"page {page} is freed twice")
        self._held[page] = False
        self._free.append(page)


class SlotTable:
    """Sequence slots: taken when a batch starts, given back when its sequences end."""

    def __init__(self, max_slots: int) -> None:
        self.max_slots = max_slots
        self._free: List[int] = list(range(max_slots - 1, -1, -1))
        self._live = [False] * max_slots

    @property
    def available(self) -> int:
        return len(self._free)

    def is_live(self, slot: int) -> bool:
        return 0 <= slot < self.max_slots and self._live[slot]

    def alloc(self) -> int:
        if not self._free:
            raise CacheError(f"no free sequence slot: all {self.max_slots} are in use")
        s = self._free.pop()
        self._live[s] = True
        return s

    def free(self, slot: int) -> None:
        if not (0 <= slot < self.max_slots):
            raise CacheError(f"slot {slot} does not exist (there are {self.max_slots})")
        if not self._live[slot]:
            raise CacheError(f"slot {slot} is freed twice or was never taken")
        self._live[slot] = False
        self._free.append(slot)

    def live_slots(self) -> List[int]:
        return [i for i, l in enumerate(self._live) if l]


class GroupPages:
    """Pages of one layer group: for every live slot, the page of each logical block.

    kind "full" keeps every block; kind "window" gives back blocks that no later query
    can see: with window w, the next query (at position `length`) sees keys
    j > length - w, so a block whose last position is <= length - w is dead.
    """

    def __init__(self, num_pages: int, page_size: int, kind: str = "full", window: Optional[int] = None) -> None:
        if kind not in ("full", "window"):
            raise CacheError(f"unknown cache kind {kind!r}")
        if kind == "window" and not window:
            raise CacheError("a window group needs its window")
        self.pool = PagePool(num_pages)
        self.page_size = page_size
        self.kind = kind
        self.window = window
        self.blocks: Dict[int, List[int]] = {}      # slot -> page per logical block (-1: released)

    def open(self, slot: int) -> None:
        if slot in self.blocks:
            raise CacheError(f"slot {slot} is already open in this group")
        self.blocks[slot] = []

    def close(self, slot: int) -> None:
        for p in self.blocks.pop(slot):
            if p >= 0:
                self.pool.free(p)

    def pages_needed(self, slot: int, new_length: int) -> int:
        have = len(self.blocks[slot])
        need = (new_length + self.page_size - 1) // self.page_size
        return max(0, need - have)

    def grow(self, slot: int, new_length: int) -> None:
        """Make sure blocks exist for positions [0, new_length)."""
        b = self.blocks[slot]
        need = (new_length + self.page_size - 1) // self.page_size
        while len(b) < need:
            b.append(self.pool.alloc())

    def shrink(self, slot: int, length: int) -> None:
        """Give back what the window has passed, after a step left the slot at `length`."""
        if self.kind != "window":
            return
        b = self.blocks[slot]
        dead_upto = length - self.window            # positions <= this are never read again
        n_dead_blocks = max(0, (dead_upto + 1) // self.page_size)
        for i in range(min(n_dead_blocks, len(b))):
            if b[i] >= 0:
                self.pool.free(b[i])
                b[i] = -1
