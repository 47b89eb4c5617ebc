"""The cache on the device: keys and values per layer group, a fixed-size state area
per sequence, and the per-step page tables that kernels read.

Storage of a group: [layer_in_group][page][2 (K, V)][kv_head][page_size][head_dim] in
the run's element type.  A group collects the schedule entries whose mixers asked for
the same thing (`CacheRequest.group_key`): all keys, or a window of them.  The
reference's layout is one 64-token chunk holding all layers
(crates/braidinfer-runtime/src/paged_kv.rs:17-21); per-layer pools make a layer's pages
contiguous for the attention kernels instead.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.spec import CacheRequest
from ..csrc.build import page_size as _page_size
from .pages import CacheError, GroupPages, SlotTable

PAGE_SIZE = _page_size()      # csrc/page.h holds the number


@dataclass
class LayerCache:
    """What a mixer sees of the cache during one step."""
    storage: torch.Tensor            # [pages, 2, kv_heads, page_size, head_dim]
    page_size: int
    read_only: bool
    group: int
    page_table: Optional[torch.Tensor] = None    # [sequences of the step, blocks] int32, set per step


class CacheGroup:
    def __init__(self, request: CacheRequest, entries: List[int], num_pages: int, dtype, device) -> None:
        self.request = request
        self.entries = entries                   # schedule entries that own a layer here
        self.pages = GroupPages(num_pages, PAGE_SIZE, request.kind, request.window)
        self.storage = torch.zeros((len(entries), num_pages, 2, request.num_kv_heads, PAGE_SIZE, request.head_dim),
                                   dtype=dtype, device=device)

    def nbytes(self) -> int:
        return self.storage.numel() * self.storage.element_size()


class CacheManager:
    """Owns slots, groups and state.  `plan` comes from the model: for every schedule
    entry its (CacheRequest | None, cache_of | None, state_bytes)."""

    def __init__(self, plan: Sequence[Tuple[Optional[CacheRequest], Optional[int], int]], max_tokens: int,
                 max_slots: int, dtype: torch.dtype, device, max_blocks_per_seq: Optional[int] = None) -> None:
        self.device = device
        self.max_tokens = max_tokens
        self.num_pages = (max_tokens + PAGE_SIZE - 1) // PAGE_SIZE
        self.slots = SlotTable(max_slots)
        self.lengths: Dict[int, int] = {}
        self.groups: List[CacheGroup] = []
        self.entry_group: List[Optional[Tuple[int, int]]] = []   # entry -> (group, layer in group)
        self.entry_read_only: List[bool] = []
        by_key: Dict[tuple, int] = {}
        owners: List[Optional[Tuple[int, int]]] = []
        pending: List[Tuple[CacheRequest, List[int]]] = []
        for e, (req, cache_of, _sb) in enumerate(plan):
            if cache_of is not None:
                owners.append(None)
                continue
            if req is None:
                owners.append(None)
                continue
            key = req.group_key()
            if key not in by_key:
                by_key[key] = len(pending)
                pending.append((req, []))
            g = by_key[key]
            owners.append((g, len(pending[g][1])))
            pending[g][1].append(e)
        for req, entries in pending:
            self.groups.append(CacheGroup(req, entries, self.num_pages, dtype, device))
        for e, (req, cache_of, _sb) in enumerate(plan):
            if cache_of is not None:
                if owners[cache_of] is None:
                    raise CacheError(f"schedule entry {e} reads the cache of entry {cache_of}, which keeps none")
                self._check_reader(e, req, cache_of, plan[cache_of][0])
                self.entry_group.append(owners[cache_of])
                self.entry_read_only.append(True)
            else:
                self.entry_group.append(owners[e])
                self.entry_read_only.append(False)
        # fixed-size state per sequence and schedule entry
        self.state: List[Optional[torch.Tensor]] = []
        for (_req, _co, sb) in plan:
            self.state.append(torch.zeros((max_slots, sb), dtype=torch.uint8, device=device) if sb > 0 else None)
        self.max_blocks_per_seq = max_blocks_per_seq or self.num_pages

    @staticmethod
    def _check_reader(e: int, reader: Optional[CacheRequest], owner_entry: int, owner: CacheRequest) -> None:
        """A run that reads another run's cache must find there what its mixer expects: the
        same heads and head size (the layout's strides), and every key its own window still
        sees (a windowed owner gives pages back once its own window has passed them)."""
        if reader is None:
            return                            # a mixer that keeps nothing ignores the view it is handed
        if (reader.num_kv_heads, reader.head_dim) != (owner.num_kv_heads, owner.head_dim):
            raise CacheError(
                f"schedule entry {e} reads the cache of entry {owner_entry}, but its mixer expects "
                f"{reader.num_kv_heads} kv heads of {reader.head_dim} and that cache holds "
                f"{owner.num_kv_heads} of {owner.head_dim}")
        if owner.kind == "window":
            if reader.kind != "window" or reader.window is None or reader.window > owner.window:
                raise CacheError(
                    f"schedule entry {e} reads the cache of entry {owner_entry}, which keeps a window of "
                    f"{owner.window} positions only; the reader "
                    + ("sees every earlier position" if reader.kind != "window" else f"has a window of {reader.window}"))

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        s = self.slots.alloc()
        self.lengths[s] = 0
        for g in self.groups:
            g.pages.open(s)
        for st in self.state:
            if st is not None:
                st[s].zero_()
        return s

    def free_slot(self, slot: int) -> None:
        self.slots.free(slot)
        for g in self.groups:
            g.pages.close(slot)
        del self.lengths[slot]

    def length(self, slot: int) -> int:
        if not self.slots.is_live(slot):
            raise CacheError(f"slot {slot} is not live")
        return self.lengths[slot]

    def pages_in_use(self) -> List[int]:
        return [g.pages.pool.in_use for g in self.groups]

    # ------------------------------------------------------------------ steps
    def begin_step(self, slot_ids: Sequence[int], new_tokens: Sequence[int]) -> List[np.ndarray]:
        """Reserve pages for the tokens each sequence brings; return, per group, the page
        table [sequences, blocks] (int32, -1 where a block is absent or released)."""
        if len(set(slot_ids)) != len(slot_ids):
            raise CacheError("a slot appears twice in one step")
        for g in self.groups:
            need = sum(g.pages.pages_needed(s, self.length(s) + n) for s, n in zip(slot_ids, new_tokens))
            if need > g.pages.pool.available:
                raise CacheError(
                    f"the cache is full: this step needs {need} more pages of {PAGE_SIZE} tokens, "
                    f"{g.pages.pool.available} of {g.pages.pool.num_pages} are free "
                    f"(the cache was sized for {self.max_tokens} tokens)")
        tables = []
        for g in self.groups:
            for s, n in zip(slot_ids, new_tokens):
                g.pages.grow(s, self.lengths[s] + n)
            cols = max(1, max(len(g.pages.blocks[s]) for s in slot_ids))
            t = np.full((len(slot_ids), cols), -1, dtype=np.int32)
            for i, s in enumerate(slot_ids):
                b = g.pages.blocks[s]
                t[i, :len(b)] = b
            tables.append(t)
        return tables

    def end_step(self, slot_ids: Sequence[int], new_tokens: Sequence[int]) -> None:
        for s, n in zip(slot_ids, new_tokens):
            self.lengths[s] += n
            for g in self.groups:
                g.pages.shrink(s, self.lengths[s])

    def layer_view(self, entry: int) -> Optional[LayerCache]:
        where = self.entry_group[entry]
        if where is None:
            return None
        g, layer = where
        return LayerCache(self.groups[g].storage[layer], PAGE_SIZE, self.entry_read_only[entry], g)

    def state_view(self, entry: int) -> Optional[torch.Tensor]:
        return self.state[entry]

    def nbytes(self) -> int:
        return sum(g.nbytes() for g in self.groups) + sum(s.numel() for s in self.state if s is not None)
