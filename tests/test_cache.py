"""The cache's bookkeeping (no GPU): no slot or page lost, held twice or freed twice; groups of
lines with different needs have pools of their own; a failed reservation changes nothing."""
import random

import pytest

from mormot2_ai_b200 import CacheError
from mormot2_ai_b200.cache import PAGE, CacheBook, FreeList, pages_for, plan_groups


def test_free_list():
    f = FreeList(3, "slot")
    got = [f.take(), f.take(), f.take()]
    assert sorted(got) == [0, 1, 2] and f.free == 0
    with pytest.raises(CacheError, match="no free slot"):
        f.take()
    f.give(1)
    with pytest.raises(CacheError, match="not held"):
        f.give(1)                       # freed twice
    with pytest.raises(CacheError, match="does not exist"):
        f.give(7)
    assert f.take() == 1                # used again


def book(max_tokens=1024, max_context=512, slots=8, chunk=64):
    needs = {0: (2, 16, 0), 1: (2, 16, 100), 2: (2, 16, 0), 3: (1, 32, 0)}
    plans = plan_groups(needs, max_tokens, max_context, slots, chunk)
    return CacheBook(plans, slots, max_context), plans


def test_groups_have_storage_of_their_own():
    b, plans = book()
    assert len(plans) == 3
    by_key = {(p.kv_heads, p.head_dim, p.window): p for p in plans}
    full, win, other = by_key[(2, 16, 0)], by_key[(2, 16, 100)], by_key[(1, 32, 0)]
    assert full.lines == [0, 2] and win.lines == [1] and other.lines == [3]
    assert full.ring_pages == 0 and full.max_pages == pages_for(512)
    # the window keeps a ring: window + chunk - 1 positions, and one page of slack
    assert win.ring_pages == pages_for(100 + 64 - 1) + 1 == 4 and win.max_pages == 4
    assert win.n_pages <= 8 * 4 and full.n_pages == 1024 // PAGE
    # a window that is no smaller than the context is stored like a full line
    wide = plan_groups({0: (1, 16, 600)}, 1024, 512, 4, 64)[0]
    assert wide.ring_pages == 0


def test_pages_follow_lengths_and_come_back():
    b, plans = book()
    s0, s1 = b.open(), b.open()
    new = b.reserve([(s0, 130), (s1, 5)])
    b.commit(s0, 130), b.commit(s1, 5)
    assert [len(g) for g in new] == [3 + 1, 3 + 1, 3 + 1]
    assert b.held_pages(0) == 4
    new = b.reserve([(s0, 131), (s1, 64)])           # nothing new: pages cover it
    assert all(not g for g in new)
    new = b.reserve([(s0, 400)])
    b.commit(s0, 400)
    win = [i for i, p in enumerate(plans) if p.window][0]
    assert len(b.pages[win][s0]) == 4                # the ring does not grow beyond its size
    assert len(b.pages[0][s0]) == pages_for(400)
    held = [b.held_pages(g) for g in range(3)]
    b.close(s0)
    assert [b.held_pages(g) for g in range(3)] == [held[0] - pages_for(400), held[1] - 4,
                                                    held[2] - pages_for(400)]
    with pytest.raises(CacheError, match="not open"):
        b.close(s0)                                  # closed twice
    with pytest.raises(CacheError, match="not open"):
        b.reserve([(s0, 10)])
    b.close(s1)
    assert all(b.held_pages(g) == 0 for g in range(3)) and b.slots.free == 8


def test_failed_reservation_changes_nothing():
    b, plans = book(max_tokens=256, max_context=256, slots=4)
    s0, s1 = b.open(), b.open()
    b.reserve([(s0, 128)])
    before = [b.held_pages(g) for g in range(len(plans))]
    with pytest.raises(CacheError, match="full"):
        b.reserve([(s0, 192), (s1, 192)])            # 1 + 3 pages wanted, 2 free
    assert [b.held_pages(g) for g in range(len(plans))] == before
    with pytest.raises(CacheError, match="exceed the context"):
        b.reserve([(s1, 300)])
    b.reserve([(s1, 128)])
    assert b.held_pages(0) == 4


def test_truncate_gives_whole_pages_back():
    b, plans = book()
    win = [i for i, p in enumerate(plans) if p.window][0]
    full = [i for i, p in enumerate(plans) if not p.window][0]
    s0 = b.open()
    b.reserve([(s0, 200)])
    b.commit(s0, 200)
    held = b.held_pages(full)
    gone = b.truncate(s0, 70)                       # pages 2 and 3 of 4 go, page 1 stays partly
    assert b.length[s0] == 70 and b.held_pages(full) == held - 2
    assert sorted(gone[full]) == [(s0, 2), (s0, 3)] and len(b.pages[full][s0]) == 2
    assert len(b.pages[win][s0]) == 2               # the ring had not wrapped: it shrinks too
    b.reserve([(s0, 130)])                          # and grows again
    b.commit(s0, 130)
    assert len(b.pages[full][s0]) == 3
    with pytest.raises(CacheError, match="truncate"):
        b.truncate(s0, 131)
    with pytest.raises(CacheError, match="truncate"):
        b.truncate(s0, -1)
    b.truncate(s0, 130)                             # to the present length: nothing changes
    assert len(b.pages[full][s0]) == 3
    b.truncate(s0, 0)
    assert all(b.held_pages(g) == 0 for g in range(len(plans))) and b.length[s0] == 0
    b.close(s0)
    with pytest.raises(CacheError, match="not open"):
        b.truncate(s0, 0)


def test_truncate_behind_a_windows_ring_is_refused():
    """The windowed group (window 100, ring of 4 pages) of a sequence of 400 positions holds
    keys from position 192 on: a cut whose next position would read older keys is refused and
    changes nothing; a cut that the ring still covers keeps the whole ring."""
    b, plans = book()
    win = [i for i, p in enumerate(plans) if p.window][0]
    s0 = b.open()
    b.reserve([(s0, 400)])
    b.commit(s0, 400)
    assert b.first_kept(win, s0) == (7 - 4) * PAGE == 192
    held = [b.held_pages(g) for g in range(len(plans))]
    with pytest.raises(CacheError, match="sliding window of 100 no longer holds"):
        b.truncate(s0, 290)                         # the next position reads keys from 191 on
    assert b.length[s0] == 400 and [b.held_pages(g) for g in range(len(plans))] == held
    b.truncate(s0, 291)                             # reads from 192 on: still there
    assert b.length[s0] == 291 and len(b.pages[win][s0]) == 4
    assert len(b.pages[0][s0]) == pages_for(291)
    # what the ring lost stays lost after the cut: positions before 192 cannot come back
    with pytest.raises(CacheError, match="no longer holds"):
        b.truncate(s0, 250)
    b.reserve([(s0, 500)])
    b.commit(s0, 500)
    assert len(b.pages[win][s0]) == 4 and len(b.pages[0][s0]) == pages_for(500)
    b.truncate(s0, 0)                               # to nothing is always allowed
    assert all(b.held_pages(g) == 0 for g in range(len(plans)))


def test_random_walk_loses_nothing():
    rng = random.Random(7)
    b, plans = book(max_tokens=2048, max_context=512, slots=6)
    live = {}
    for _ in range(2000):
        r = rng.random()
        if r < 0.3 and b.slots.free:
            live[b.open()] = 0
        elif r < 0.5 and live:
            s = rng.choice(list(live))
            b.close(s)
            del live[s]
        elif r < 0.6 and live:
            s = rng.choice(list(live))
            n = rng.randint(0, live[s])
            try:
                b.truncate(s, n)
                live[s] = n
            except CacheError:
                pass
        elif live:
            s = rng.choice(list(live))
            n = min(512, live[s] + rng.randint(1, 90))
            try:
                b.reserve([(s, n)])
                b.commit(s, n)
                live[s] = n
            except CacheError:
                pass
        for g, plan in enumerate(plans):
            held = [p for s in range(6) for p in b.pages[g][s]]
            assert len(held) == len(set(held)) == b.held_pages(g)     # none held twice
            for s, n in live.items():
                # a ring that wrapped before a cut may hold more than the length needs
                assert len(b.pages[g][s]) >= b.entries_needed(g, n)
                if not plan.ring_pages:
                    assert len(b.pages[g][s]) == b.entries_needed(g, n)
        assert b.slots.free == 6 - len(live)
    for s in list(live):
        b.close(s)
    assert all(b.held_pages(g) == 0 for g in range(len(plans)))       # none lost


def test_guard_bands_tell_a_write_outside_a_buffer():
    import torch
    from mormot2_ai_b200.cache.guards import BAND_BYTES, Guards, alloc
    g = Guards()
    a = g.alloc("a", (3, 5), torch.float32, "cpu")
    b = g.alloc("b", (7,), torch.int32, "cpu", fill=None)
    assert a.shape == (3, 5) and float(a.abs().max()) == 0.0 and b.dtype == torch.int32
    a.fill_(1.5)
    b.fill_(-1)
    assert g.damaged() == []                       # writes inside leave the bands alone
    raw = torch.tensor([], dtype=torch.uint8).set_(a.untyped_storage())
    assert raw.numel() == 2 * BAND_BYTES + 3 * 5 * 4
    raw[BAND_BYTES + 3 * 5 * 4] = 0                # the first byte behind a
    assert g.damaged() == ["a (behind)"]
    raw_b = torch.tensor([], dtype=torch.uint8).set_(b.untyped_storage())
    raw_b[BAND_BYTES - 1] = 7                      # the last byte before b
    assert g.damaged() == ["a (behind)", "b (before)"]
    assert alloc(None, "c", (2, 2), torch.float32, "cpu", 3.0).tolist() == [[3.0, 3.0]] * 2
