"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed
twice, under random orders of requests; windows give pages back."""
import random

import pytest
import torch

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


def test_groups_have_their_own_page_size_and_count():
    """A windowed group with small pages and few of them beside a group that keeps every key."""
    from firefly_b200.cache import plan_groups
    specs = {0: PagedKVSpec(2, 16, None), 1: PagedKVSpec(2, 16, 8, block_size=2), 2: PagedKVSpec(2, 16, None),
             3: PagedKVSpec(1, 32, None, block_size=8)}
    planned = plan_groups(specs, 4)
    assert [(sl, bs) for _, sl, bs in planned] == [([0, 2], 4), ([1], 2), ([3], 8)]
    m = CacheManager(specs, block_size=4, num_blocks=[20, 12, 10], max_requests=3)
    assert [(g.block_size, g.num_blocks) for g in m.groups] == [(4, 20), (2, 12), (8, 10)]
    assert m.num_blocks == 10 and m.bytes_per_block(torch.float32) == (2 * 2 * 2 * 16 * 4 + 2 * 2 * 16 * 2 + 2 * 32 * 8) * 4
    r = m.admit("r")
    n = 0
    for step in (5, 3, 9, 1, 1, 7, 13, 2):
        assert m.grow(r, n + step), (n, step)
        m.advance(r, step)
        n += step
        assert len(r.tables[0]) == -(-n // 4) and len(r.tables[2]) == -(-n // 8)
        live = [b for b in r.tables[1] if b >= 0]
        # the windowed group holds the pages of its window only: at most ceil(8 / 2) + 1
        assert len(live) <= 5 and len(r.tables[1]) == -(-n // 2)
        m.check()
    assert n == 41 and m.groups[1].allocator.num_free >= 7
    # what runs out first decides: group 0 has 20 pages of 4 = 80 tokens, group 2 10 of 8 = 80
    assert not m.grow(r, 80)                       # 39 tokens at once are more than the windowed group's 12 pages of 2
    while n < 80:
        step = min(8, 80 - n)
        assert m.grow(r, n + step)
        m.advance(r, step)
        n += step
    assert not m.grow(r, 81)
    assert m.why_it_cannot_fit(80, 8) is None
    assert "cache group 0" in m.why_it_cannot_fit(81, 8)
    # the windowed group refuses a portion that does not fit its pages: 8 + 16 tokens need 13 pages of 2
    assert m.why_it_cannot_fit(60, 12) is None and "cache group 1" in m.why_it_cannot_fit(60, 16)
    m.free(r)
    m.check()
    assert [g.allocator.num_free for g in m.groups] == [20, 12, 10]
    with pytest.raises(ValueError, match="page counts"):
        CacheManager(specs, block_size=4, num_blocks=[20, 9], max_requests=3)


@pytest.mark.parametrize("seed", range(4))
def test_random_orders_with_unequal_groups(seed):
    rng = random.Random(100 + seed)
    specs = {0: PagedKVSpec(2, 16, None), 1: PagedKVSpec(2, 16, rng.choice([3, 9]), block_size=rng.choice([1, 2, 4])),
             2: StateSpec((2, 2))}
    m = CacheManager(specs, block_size=rng.choice([4, 8]), num_blocks=[rng.choice([10, 30]), rng.choice([12, 25])],
                     max_requests=4)
    live = {}
    nid = 0
    for _ in range(500):
        op = rng.random()
        if op < 0.25 and m.can_admit():
            live[nid] = m.admit(nid)
            nid += 1
        elif op < 0.8 and live:
            rc = live[rng.choice(list(live))]
            n = rng.choice([1, 1, 2, 3])
            before = [list(t) for t in rc.tables]
            if m.grow(rc, rc.num_tokens + n):
                m.advance(rc, n)
            else:
                assert [list(t) for t in rc.tables] == before
        elif live:
            m.free(live.pop(rng.choice(list(live))))
        m.check()
    for rc in list(live.values()):
        m.free(rc)
    m.check()
    assert all(g.allocator.num_free == g.num_blocks for g in m.groups)


def test_engine_gives_a_windowed_group_far_fewer_pages():
    """The engine sizes each group from what it needs: every-key groups share the token capacity, a
    windowed group gets its window plus a portion per request and no more."""
    from types import SimpleNamespace
    from firefly_b200.engine.engine import Engine, EngineOptions
    model = SimpleNamespace(rt=SimpleNamespace(device=torch.device("cpu"), dtype=torch.bfloat16),
                            spec=SimpleNamespace(max_positions=4096, vocab_size=8),
                            cache_slot_specs=lambda: {0: PagedKVSpec(2, 16, None), 1: PagedKVSpec(2, 16, 64),
                                                      2: PagedKVSpec(2, 16, None)})
    opts = EngineOptions(num_kv_blocks=4096, kv_block_size=16, max_batch_size_limit=4, max_prefill_chunk_size=32,
                         use_cuda_graphs=False)
    eng = Engine(model, options=opts, runner=object(), sampler=object())
    full, win = eng.cache.groups
    assert full.num_blocks == 4096 and win.spec.window == 64
    assert win.num_blocks == 4 * ((64 + 32) // 16 + 2) == 32          # 128 times fewer than the full group
    assert eng.max_model_len == 4096
