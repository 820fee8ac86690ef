"""The cache on the device: per group the pooled keys and values of its lines and the page
table, and per state line the fixed-size state of every slot.

Layout of a line's keys (values alike): ``[pages, kv_heads, 64, head_dim]`` — the 64
positions of a page for one KV head are contiguous, so attention streams whole tiles.
The element type is the activation type of the engine (bfloat16, or float32 on the 32-bit
path); the reference keeps half floats or floats (``model.qwen3.cuda.pas:907-937``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .guards import Guards, alloc
from .pages import PAGE, CacheBook, GroupPlan


@dataclass
class CacheLine:
    """What a mixer gets of its line: pools, the page table of its group and the ring size."""
    k: torch.Tensor            # [pages, kv_heads, PAGE, head_dim]
    v: torch.Tensor
    page_table: torch.Tensor   # int32 [slots, max_pages] on the device
    max_pages: int
    ring_pages: int
    window: int
    kv_heads: int
    head_dim: int


class CacheStorage:
    def __init__(self, plans: List[GroupPlan], max_slots: int, dtype: torch.dtype,
                 device: torch.device, state_needs: Dict[int, "StateNeed"],
                 guards: Optional[Guards] = None):
        self.plans = plans
        self.pools: List[torch.Tensor] = []
        self.tables: List[torch.Tensor] = []
        self.tables_host: List[torch.Tensor] = []
        self.lines: Dict[int, CacheLine] = {}
        for g, plan in enumerate(plans):
            pool = alloc(guards, f"keys and values of group {g}",
                         (len(plan.lines), 2, plan.n_pages, plan.kv_heads, PAGE, plan.head_dim),
                         dtype, device)
            table = alloc(guards, f"page table of group {g}", (max_slots, plan.max_pages),
                          torch.int32, device)
            # pageable on purpose: the copy to the device then reads it before returning, so the
            # host may change it again at once
            host = torch.zeros((max_slots, plan.max_pages), dtype=torch.int32)
            self.pools.append(pool)
            self.tables.append(table)
            self.tables_host.append(host)
            for i, line in enumerate(plan.lines):
                self.lines[line] = CacheLine(pool[i, 0], pool[i, 1], table, plan.max_pages,
                                             plan.ring_pages, plan.window, plan.kv_heads,
                                             plan.head_dim)
        # fixed-size state per slot, at its initial value when a sequence starts; beside it a
        # copy of the same size that a step saves the slots it touches into, so that a step
        # that fails half way leaves the state it found
        self.state_init: Dict[int, float] = {l: float(n.init) for l, n in state_needs.items()}
        self.states: Dict[int, torch.Tensor] = {
            line: alloc(guards, f"state of line {line}", (max_slots,) + tuple(n.shape),
                        getattr(torch, n.dtype), device, float(n.init))
            for line, n in state_needs.items()}
        self.saved: Dict[int, torch.Tensor] = {l: torch.empty_like(s)
                                               for l, s in self.states.items()}

    def bytes(self) -> int:
        return (sum(p.numel() * p.element_size() for p in self.pools)
                + sum(2 * s.numel() * s.element_size() for s in self.states.values()))

    def map_pages(self, new_entries: List[List[Tuple[int, int, int]]]) -> None:
        """Writes the new table entries of ``CacheBook.reserve`` to the device tables."""
        for g, entries in enumerate(new_entries):
            if not entries:
                continue
            host = self.tables_host[g]
            where = np.asarray(entries, dtype=np.int64)     # [n, 3]: slot, entry, page
            host.numpy()[where[:, 0], where[:, 1]] = where[:, 2]
            lo, hi = int(where[:, 0].min()), int(where[:, 0].max())
            self.tables[g][lo:hi + 1].copy_(host[lo:hi + 1])

    def table_faults(self, book: CacheBook) -> List[str]:
        """Compares the page tables on the device with the bookkeeping: every entry that a
        sequence holds must name the page the book gave it, and no page may be held twice.
        Returns what is wrong (nothing, when all is well)."""
        out = []
        for g, table in enumerate(self.tables):
            dev = table.cpu()
            seen: Dict[int, int] = {}
            for slot in range(dev.shape[0]):
                for entry, page in enumerate(book.pages[g][slot]):
                    if int(dev[slot, entry]) != page:
                        out.append(f"group {g}, slot {slot}, entry {entry}: the device table "
                                   f"names page {int(dev[slot, entry])}, the book page {page}")
                    if page in seen:
                        out.append(f"group {g}: page {page} is held by slots {seen[page]} "
                                   f"and {slot}")
                    seen[page] = slot
        return out

    def reset_state(self, slot: int) -> None:
        for line, s in self.states.items():
            s[slot].fill_(self.state_init[line])

    def save_states(self, slots: torch.Tensor) -> None:
        """Keeps a copy of the state of ``slots`` (int64 indices on the device)."""
        for line, s in self.states.items():
            self.saved[line].index_copy_(0, slots, s.index_select(0, slots))

    def restore_states(self, slots: torch.Tensor) -> None:
        """Puts the copy of ``save_states`` back."""
        for line, s in self.states.items():
            s.index_copy_(0, slots, self.saved[line].index_select(0, slots))
