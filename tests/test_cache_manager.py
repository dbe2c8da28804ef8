"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed
twice, under random orders of requests; windows give pages back."""
import random

import pytest

from firefly_b200.cache import (BlockAllocator, CacheManager, OutOfPages, PageError, PagedKVSpec,
                                StateSpec)


def test_allocator_lifo_and_errors():
    a = BlockAllocator(4, first_id=1)
    got = a.allocate(3)
    assert got == [1, 2, 3] and a.num_free == 1
    assert a.allocate(2) is None and a.num_free == 1       # all or nothing
    a.free([2])
    assert a.allocate(1) == [2]                            # the page just freed comes back first
    with pytest.raises(PageError, match="twice"):
        a.free([4])                                        # never allocated
    a.free([1])
    with pytest.raises(PageError, match="twice"):
        a.free([1])
    with pytest.raises(PageError, match="does not belong"):
        a.free([0])
    got = a.allocate(2)
    before = a.num_free
    with pytest.raises(PageError, match="twice"):
        a.free([got[0], got[1], got[0]])                    # named twice in one call: nothing is freed
    assert a.num_free == before
    with pytest.raises(PageError, match="does not belong"):
        a.free([got[0], got[1], 77])                        # a foreign id behind valid ones: nothing is freed
    assert a.num_free == before
    a.free(got)                                             # ... and the valid ones can still be freed
    a.check()
    big = BlockAllocator(100000)
    ids = big.allocate(100000)
    assert ids[0] == 0 and ids[-1] == 99999 and big.allocate(1) is None
    big.free(reversed(ids))
    assert big.allocate(1) == [0]
    big.check()


def _manager(window=None, num_blocks=12, block=4, two_groups=False, state=False):
    specs = {0: PagedKVSpec(2, 16, None), 1: PagedKVSpec(2, 16, None)}
    if two_groups:
        specs[2] = PagedKVSpec(2, 16, window)
        specs[3] = PagedKVSpec(2, 16, window)
    if state:
        specs[4] = StateSpec((3, 5))
    return CacheManager(specs, block_size=block, num_blocks=num_blocks, max_requests=5)


def test_groups_by_need():
    m = _manager(window=6, two_groups=True, state=True)
    assert len(m.groups) == 2
    assert m.groups[0].slots == [0, 1] and m.groups[1].slots == [2, 3]
    assert m.slot_group == {0: 0, 1: 0, 2: 1, 3: 1}
    assert list(m.state_specs) == [4]
    assert m.bytes_per_block(__import__("torch").float32) == 2 * (2 * 2 * 2 * 4 * 16 * 4)


def test_grow_advance_free():
    m = _manager()
    a = m.admit("a")
    assert a.state_slot >= 1 and a.fresh
    assert m.grow(a, 9) and len(a.tables[0]) == 3
    m.advance(a, 9)
    assert a.num_tokens == 9 and not a.fresh
    assert m.grow(a, 12) and len(a.tables[0]) == 3          # room already there
    b = m.admit("b")
    assert not m.grow(b, 4 * 10) and b.tables[0] == []      # all or nothing
    assert m.grow(b, 4 * 9)
    m.check()
    with pytest.raises(PageError):
        m.advance(a, 100)                                    # more tokens than pages
    m.free(a)
    with pytest.raises(PageError, match="not live"):
        m.free(a)
    m.free(b)
    m.check()
    assert m.num_free_blocks == 12
    with pytest.raises(PageError, match="already live"):
        m.admit("c")
        m.admit("c")


def test_request_slots_run_out():
    m = _manager()
    for i in range(5):
        m.admit(i)
    assert not m.can_admit()
    with pytest.raises(OutOfPages):
        m.admit("x")


def test_window_gives_pages_back():
    m = _manager(window=6, two_groups=True, block=4, num_blocks=8)
    r = m.admit("r")
    n = 0
    for step in (5, 2, 7, 1, 1, 1, 9, 3):
        assert m.grow(r, n + step)
        m.advance(r, step)
        n += step
        first_needed = max(0, n - 6 + 1) // 4
        win = r.tables[1]
        assert all(b == -1 for b in win[:first_needed]) and all(b > 0 for b in win[first_needed:])
        assert all(b > 0 for b in r.tables[0])                # the full group keeps everything
        assert m.groups[1].allocator.num_held == len(win) - first_needed
        m.check()
    m.free(r)
    m.check()
    assert all(g.allocator.num_free == 8 for g in m.groups)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_invariants(seed):
    rng = random.Random(seed)
    m = _manager(window=rng.choice([None, 5, 17]), two_groups=True, block=rng.choice([2, 4, 8]),
                 num_blocks=rng.choice([6, 20, 50]), state=True)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.can_admit():
            live[next_id] = m.admit(next_id)
            next_id += 1
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            rc = live[rid]
            n = rng.choice([1, 1, 1, 2, 5, 13])
            before = [list(t) for t in rc.tables]
            if m.grow(rc, rc.num_tokens + n):
                m.advance(rc, n)
            else:
                assert [list(t) for t in rc.tables] == before     # nothing taken on failure
        elif live:
            rid = rng.choice(list(live))
            m.free(live.pop(rid))
        m.check()
    for rc in live.values():
        m.free(rc)
    m.check()
    assert all(g.allocator.num_free == m.num_blocks for g in m.groups)
