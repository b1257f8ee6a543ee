"""Device storage of the cache: key/value pages per group of layers, and per-sequence state.

Places in the schedule that keep keys and values are grouped by what they need
(number of key/value heads, head size, all positions or a window); each group has
its own page pool and one allocation
    K, V: [places_in_group, n_pages, n_kv_heads, page_size, head_dim]
in the storage type of the run.  A page of one place is contiguous, so a head's
``page_size`` keys are one block of page_size*head_dim elements.  The reference
sizes one flat cache by the largest layer (src/cuda_model.zig:178-188,213-217)
and narrows only the read range for windowed layers (src/model.zig:661).

Beside the pages lies fixed-size state per sequence: for a place in the schedule
that asks for it, a tensor [n_slots, *shape] that is zeroed when a slot is handed
out.  This architecture asks for none; a mixer with a recurrent state would.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import KVNeed, LayerIO, StateNeed
from .slots import GroupPages, SlotTable

PAGE_SIZE = 64


class KVGroup:
    def __init__(self, need: KVNeed, places: List[int], n_pages: int, page_size: int, dtype: torch.dtype,
                 device: torch.device):
        self.need = need
        self.places = places
        self.page_size = page_size
        self.pages = GroupPages(n_pages, page_size, need.window)
        shape = (len(places), n_pages, need.n_kv_heads, page_size, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)

    def bytes_per_position(self) -> int:
        return 2 * len(self.places) * self.need.n_kv_heads * self.need.head_dim * self.k.element_size()


class CacheStorage:
    """All groups, the slot table above them, and the per-sequence state."""

    def __init__(self, kv_needs: Sequence[Optional[KVNeed]], reads_from: Sequence[Optional[int]],
                 state_needs: Sequence[Optional[StateNeed]], max_tokens: int, n_slots: int, max_len: int,
                 dtype: torch.dtype, device: torch.device, page_size: int = PAGE_SIZE,
                 window_pool_tokens: Optional[int] = None):
        """kv_needs[s], state_needs[s]: what place s of the schedule keeps.  reads_from[s]: the place
        whose keys and values place s reads instead of keeping its own (None: its own)."""
        if page_size <= 0 or page_size % 64:
            raise ValueError("the page size must be a positive multiple of 64 positions")
        self.page_size = page_size
        self.n_pages = -(-max_tokens // page_size)
        self.max_pages_per_seq = -(-max_len // page_size)
        self.groups: List[KVGroup] = []
        self.group_of: Dict[int, Tuple[int, int]] = {}    # place -> (group, index in group)
        by_need: Dict[KVNeed, List[int]] = {}
        for s, need in enumerate(kv_needs):
            if need is not None:
                by_need.setdefault(need, []).append(s)
        for need, places in by_need.items():
            n_pages = self.n_pages
            if need.window is not None and window_pool_tokens is not None:
                n_pages = min(n_pages, -(-window_pool_tokens // page_size))
            g = KVGroup(need, places, n_pages, page_size, dtype, device)
            for i, s in enumerate(places):
                self.group_of[s] = (len(self.groups), i)
            self.groups.append(g)
        self.reads_from = list(reads_from)
        for s, src in enumerate(self.reads_from):
            if src is not None and src not in self.group_of:
                raise ValueError(f"place {s} of the schedule reads the cache of place {src}, which keeps none")
        self.slots = SlotTable(n_slots, [g.pages for g in self.groups], max_len)
        for g in self.groups:
            g.pages.mirror(n_slots, self.max_pages_per_seq)
        self.states: Dict[int, torch.Tensor] = {}
        for s, need in enumerate(state_needs):
            if need is not None:
                self.states[s] = torch.zeros((n_slots,) + tuple(need.shape), dtype=need.dtype, device=device)

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        slot = self.slots.alloc()
        for st in self.states.values():
            st[slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        self.slots.free(slot)

    # ------------------------------------------------------------- block tables
    def block_table_rows(self, group: int, slots: Sequence[int], width: int):
        """Pages of the given slots as an int32 array [len(slots), width] (-1 where there is none)."""
        table = self.groups[group].pages.table
        if table is not None and width <= table.shape[1]:
            return table[list(slots), :width]
        pages = self.groups[group].pages.pages_of
        rows = []
        for s in slots:
            p = pages.get(s, [])
            rows.append(list(p[:width]) + [-1] * (width - len(p)))
        return rows

    def io_for(self, place: int, block_tables: Sequence[torch.Tensor]) -> LayerIO:
        """Storage of one place of the schedule, given the step's block tables by group."""
        src = self.reads_from[place]
        owner = place if src is None else src
        io = LayerIO(writes_cache=src is None, state=self.states.get(place))
        if owner in self.group_of:
            g, i = self.group_of[owner]
            grp = self.groups[g]
            io.k_pages, io.v_pages = grp.k[i], grp.v[i]
            io.block_table = block_tables[g]
            io.page_size = grp.page_size
        return io

    def bytes_per_position(self) -> int:
        return sum(g.bytes_per_position() for g in self.groups)
