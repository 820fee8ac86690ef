"""The bookkeeping of the cache on the host: slots for sequences, pages of 64 positions for
their keys and values, and which sequence holds what. Pure Python, no device: the device
side (``cache/storage.py``) only mirrors the page tables that this file fills.

A *group* is a set of cache lines with the same needs (KV heads, head size, window); each
group has a page pool of its own. A line with a window keeps a ring of pages per sequence
(enough for the window and one step's new positions), a line without one keeps every page.
Slots and pages are given back when a sequence ends and are used again by later ones.
The reference has one context per sequence that grows (``decoder.pas:2306-2449``); slots,
pages and groups are this library's own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

from ..errors import CacheError

PAGE = 64


def pages_for(tokens: int) -> int:
    return (tokens + PAGE - 1) // PAGE


class FreeList:
    """Numbered things (slots, pages) that are taken and given back; refuses a thing that is
    given back twice or was never taken."""

    def __init__(self, count: int, what: str):
        self.what = what
        self.count = count
        self._free = list(range(count - 1, -1, -1))  # take() hands out 0 first
        self._held = [False] * count

    @property
    def free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what} (all {self.count} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def give(self, i: int) -> None:
        if not 0 <= i < self.count:
            raise CacheError(f"{self.what} {i} does not exist (there are {self.count})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is given back but not held")
        self._held[i] = False
        self._free.append(i)

    def held(self, i: int) -> bool:
        return 0 <= i < self.count and self._held[i]


@dataclass
class GroupPlan:
    """Sizes of one group. ``ring_pages`` 0: every page of a sequence is kept."""
    kv_heads: int
    head_dim: int
    window: int
    lines: List[int]
    n_pages: int
    max_pages: int      # entries of a sequence's page-table row
    ring_pages: int


def plan_groups(needs: Dict[int, Tuple[int, int, int]], max_tokens: int, max_context: int,
                max_slots: int, chunk: int) -> List[GroupPlan]:
    """Groups the lines by (kv_heads, head_dim, window) and sizes each group's pool.

    ``needs[line] = (kv_heads, head_dim, window)``; ``max_tokens`` is the most tokens that live
    sequences hold together (each rounded up to whole pages); ``chunk`` is the most new
    positions of one sequence in one pass of the model.
    """
    total_pages = pages_for(max_tokens)
    groups: Dict[Tuple[int, int, int], GroupPlan] = {}
    for line in sorted(needs):
        key = needs[line]
        if key not in groups:
            kvh, hd, window = key
            full = pages_for(max_context)
            ring = 0
            if window > 0:
                # positions pos-window+1 .. pos+chunk-1 are live at once; one more page for
                # where that span starts within a page
                span = pages_for(window + chunk - 1) + 1
                if span < full:
                    ring = span
            per_seq = ring if ring else full
            groups[key] = GroupPlan(kvh, hd, window, [], min(total_pages, max_slots * per_seq),
                                    per_seq, ring)
        groups[key].lines.append(line)
    return list(groups.values())


class CacheBook:
    """Who holds which slot and which pages, and how long each sequence is."""

    def __init__(self, plans: List[GroupPlan], max_slots: int, max_context: int):
        self.plans = plans
        self.max_context = max_context
        self.slots = FreeList(max_slots, "slot")
        self.pools = [FreeList(p.n_pages, "page") for p in plans]
        self.length = [0] * max_slots
        # the most positions that pages were ever reserved for since the slot was opened or
        # cut to nothing: keys may have been written up to there, also by a step that failed
        self.high = [0] * max_slots
        # pages[g][slot][i]: the page at entry i of the slot's table row, -1: none yet
        self.pages: List[List[List[int]]] = [
            [[] for _ in range(max_slots)] for _ in plans]

    # -- sequences
    def open(self) -> int:
        slot = self.slots.take()
        self.length[slot] = 0
        self.high[slot] = 0
        return slot

    def close(self, slot: int) -> None:
        if not self.slots.held(slot):
            raise CacheError(f"slot {slot} is closed but not open")
        for g, pool in enumerate(self.pools):
            for page in self.pages[g][slot]:
                if page >= 0:
                    pool.give(page)
            self.pages[g][slot] = []
        self.length[slot] = 0
        self.slots.give(slot)

    def check_open(self, slot: int) -> None:
        if not self.slots.held(slot):
            raise CacheError(f"slot {slot} is not open")

    # -- pages
    def entries_needed(self, g: int, length: int) -> int:
        plan = self.plans[g]
        n = pages_for(length)
        return min(n, plan.ring_pages) if plan.ring_pages else n

    def missing(self, slot: int, new_length: int) -> List[int]:
        """How many pages each group still has to map for the slot to hold new_length."""
        return [max(0, self.entries_needed(g, new_length) - len(self.pages[g][slot]))
                for g in range(len(self.plans))]

    def reserve(self, requests: List[Tuple[int, int]]) -> List[List[Tuple[int, int, int]]]:
        """Maps the pages that the slots need to reach their new lengths:
        ``requests = [(slot, new_length)]``. All or nothing: if a pool runs out, nothing is
        mapped and ``CacheError`` is raised. Returns, per group, the new table entries
        ``(slot, entry, page)``."""
        for slot, new_length in requests:
            self.check_open(slot)
            if new_length > self.max_context:
                raise CacheError(
                    f"slot {slot}: {new_length} positions exceed the context of {self.max_context}")
        want = [0] * len(self.plans)
        for slot, new_length in requests:
            for g, n in enumerate(self.missing(slot, new_length)):
                want[g] += n
        for g, pool in enumerate(self.pools):
            if want[g] > pool.free:
                raise CacheError(
                    f"the cache is full: {want[g]} more pages needed, {pool.free} of "
                    f"{pool.count} free")
        out: List[List[Tuple[int, int, int]]] = [[] for _ in self.plans]
        for slot, new_length in requests:
            for g, n in enumerate(self.missing(slot, new_length)):
                for _ in range(n):
                    page = self.pools[g].take()
                    self.pages[g][slot].append(page)
                    out[g].append((slot, len(self.pages[g][slot]) - 1, page))
        for slot, new_length in requests:
            self.high[slot] = max(self.high[slot], new_length)
        return out

    def commit(self, slot: int, new_length: int) -> None:
        self.length[slot] = new_length

    # -- going back
    def first_kept(self, g: int, slot: int) -> int:
        """The first position whose keys group g still holds for the slot: 0, or where the
        ring of pages of a windowed group began to overwrite itself."""
        ring = self.plans[g].ring_pages
        if not ring:
            return 0
        return max(0, pages_for(self.high[slot]) - ring) * PAGE

    def truncate(self, slot: int, new_length: int) -> List[List[Tuple[int, int]]]:
        """Shortens the slot's sequence to ``new_length`` positions. Whole pages beyond it go
        back to their pools (the partly filled one stays); a group whose ring already wrapped
        keeps its ring. Refused, with nothing changed, when a windowed group no longer holds
        the keys that the position after ``new_length`` would read. Returns, per group, the
        table entries ``(slot, entry)`` that were unmapped. The reference's
        ``TDecoderContext.Truncate`` (``decoder.pas:996-1018``) shortens its one growing
        buffer; pages and rings are this library's own."""
        self.check_open(slot)
        length = self.length[slot]
        if not 0 <= new_length <= length:
            raise CacheError(f"slot {slot}: truncate({new_length}) of {length} positions")
        if new_length > 0:
            for g, plan in enumerate(self.plans):
                if plan.ring_pages and max(0, new_length - plan.window + 1) < self.first_kept(g, slot):
                    raise CacheError(
                        f"slot {slot}: truncate({new_length}): a sliding window of "
                        f"{plan.window} no longer holds the keys of that position "
                        f"(kept from {self.first_kept(g, slot)} on)")
        out: List[List[Tuple[int, int]]] = [[] for _ in self.plans]
        for g, plan in enumerate(self.plans):
            held = self.pages[g][slot]
            wrapped = (plan.ring_pages and pages_for(self.high[slot]) > plan.ring_pages
                       and new_length > 0)
            keep = len(held) if wrapped else min(len(held), self.entries_needed(g, new_length))
            while len(held) > keep:
                page = held.pop()
                self.pools[g].give(page)
                out[g].append((slot, len(held)))
        self.length[slot] = new_length
        if new_length == 0:
            self.high[slot] = 0
        return out

    # -- checks for tests
    def held_pages(self, g: int) -> int:
        return self.pools[g].count - self.pools[g].free
