"""The cache on the device: per group the pooled keys and values of its lines and the page
table, and per state line the fixed-size state of every slot.

Layout of a line's keys (values alike): ``[pages, kv_heads, 64, head_dim]`` — the 64
positions of a page for one KV head are contiguous, so attention streams whole tiles.
The element type is the activation type of the engine (bfloat16, or float32 on the 32-bit
path); the reference keeps half floats or floats (``model.qwen3.cuda.pas:907-937``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch

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
                 device: torch.device, state_shapes: Dict[int, Tuple[int, ...]]):
        self.plans = plans
        self.pools: List[torch.Tensor] = []
        self.tables: List[torch.Tensor] = []
        self.tables_host: List[torch.Tensor] = []
        self.lines: Dict[int, CacheLine] = {}
        for plan in plans:
            pool = torch.zeros((len(plan.lines), 2, plan.n_pages, plan.kv_heads, PAGE,
                                plan.head_dim), dtype=dtype, device=device)
            table = torch.zeros((max_slots, plan.max_pages), dtype=torch.int32, device=device)
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
        # fixed-size state per slot, zero when a sequence starts
        self.states: Dict[int, torch.Tensor] = {
            line: torch.zeros((max_slots,) + tuple(shape), dtype=torch.float32, device=device)
            for line, shape in state_shapes.items()}

    def bytes(self) -> int:
        return (sum(p.numel() * p.element_size() for p in self.pools)
                + sum(s.numel() * 4 for s in self.states.values()))

    def map_pages(self, new_entries: List[List[Tuple[int, int, int]]]) -> None:
        """Writes the new table entries of ``CacheBook.reserve`` to the device tables."""
        for g, entries in enumerate(new_entries):
            if not entries:
                continue
            host = self.tables_host[g]
            lo, hi = host.shape[0], -1
            for slot, entry, page in entries:
                host[slot, entry] = page
                lo, hi = min(lo, slot), max(hi, slot)
            self.tables[g][lo:hi + 1].copy_(host[lo:hi + 1])

    def reset_state(self, slot: int) -> None:
        for s in self.states.values():
            s[slot].zero_()
