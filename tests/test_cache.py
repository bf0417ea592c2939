"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; state slots."""
import random

import pytest
import torch

from lgml_b200.cache import CacheManager, FixedState, NoSlot, PagedKV, PagePool, PoolFull


def test_pool_takes_lowest_first_and_refuses_double_free():
    p = PagePool(5)
    got = [p.take() for _ in range(5)]
    assert got == [0, 1, 2, 3, 4]                      # lowest free first (lua/lgml/kvpool.lua:102-116)
    with pytest.raises(PoolFull, match="kv pool full"):
        p.take()
    p.release(3)
    p.release(1)
    assert p.take() == 1 and p.take() == 3
    p.release(2)
    with pytest.raises(ValueError, match="twice"):
        p.release(2)
    with pytest.raises(ValueError, match="outside"):
        p.release(9)
    p.ref(0)
    p.release(0)
    assert p.refcount(0) == 1 and p.n_free == 1
    p.check()


def manager(n_pages=8, slots=4, layout=None, **kw):
    layout = layout or {0: PagedKV(2, 8), 1: PagedKV(2, 8)}
    return CacheManager(layout, n_pages=n_pages, max_slots=slots, dtype=torch.float32, device="cpu", **kw)


def test_layers_with_equal_needs_share_a_group():
    cm = manager(layout={0: PagedKV(2, 8), 1: PagedKV(2, 8), 2: PagedKV(2, 8, window=100), 3: FixedState((4,)), 4: None})
    assert len(cm.groups) == 2 and cm.groups[0].layers == [0, 1] and cm.groups[1].layers == [2]
    assert cm.groups[0].k[1].shape == (8, 2, 64, 8)
    assert len(cm.state_groups) == 1 and cm.state_groups[0].state[3].shape == (4, 4)


def test_reserve_commit_close():
    cm = manager(n_pages=4)
    a = cm.open("a")
    assert cm.reserve(a, 65) and a.tables[0] == [0, 1]
    assert cm.reserve(a, 65) and a.tables[0] == [0, 1]          # asking again takes nothing
    cm.commit(a, 65)
    assert cm.reserve(a, 1) and len(a.tables[0]) == 2            # position 65 is in page 1
    b = cm.open("b")
    assert cm.reserve(b, 128) and b.tables[0] == [2, 3]
    assert not cm.reserve(a, 64)                                 # needs a third page, none free
    assert a.tables[0] == [0, 1]                                 # a failed reserve takes nothing
    cm.check()
    cm.close(b)
    assert cm.reserve(a, 64) and a.tables[0] == [0, 1, 2]        # b's page is used again
    with pytest.raises(ValueError, match="twice"):
        cm.close(b)
    cm.close(a)
    assert cm.n_free_pages == 4 and not cm.live
    cm.check()


def test_failed_reserve_rolls_back_every_group():
    cm = manager(n_pages=3, layout={0: PagedKV(2, 8), 1: PagedKV(1, 16)})
    a = cm.open("a")
    hog = cm.open("hog")
    cm.groups[1].pool.take(), cm.groups[1].pool.take()           # only the second group is short
    assert not cm.reserve(a, 128)
    assert a.tables == [[], []] and cm.groups[0].pool.n_free == 3
    cm.close(hog)


def test_slots_run_out_and_come_back():
    cm = manager(slots=2)
    a, b = cm.open("a"), cm.open("b")
    with pytest.raises(NoSlot):
        cm.open("c")
    with pytest.raises(ValueError, match="already live"):
        cm.open("a")
    slot = a.slot
    cm.close(a)
    assert cm.open("c").slot == slot


def test_window_gives_pages_back():
    cm = manager(n_pages=16, layout={0: PagedKV(2, 8), 1: PagedKV(2, 8, window=70)}, max_step_tokens=64)
    r = cm.open("r")
    held = []
    for _ in range(10):
        assert cm.reserve(r, 64)
        cm.commit(r, 64)
        held.append(cm.groups[1].pool.n_held)
        cm.check()
    assert cm.groups[0].pool.n_held == 10                        # the full group keeps everything
    assert max(held) <= 3                                        # the window group keeps ceil(70/64)+1
    # the pages still held cover every position a later query can reach
    lowest = r.n_tokens - 70 + 1
    assert all(p >= 0 for p in r.tables[1][lowest // 64:]) and all(p == -1 for p in r.tables[1][: lowest // 64])
    cm.close(r)
    cm.check()
    assert cm.groups[1].pool.n_held == 0


def test_state_slots_are_zeroed_at_open():
    cm = manager(layout={0: FixedState((3,))}, slots=2)
    a = cm.open("a")
    cm.state_groups[0].state[0][a.slot] += 5.0
    cm.close(a)
    b = cm.open("b")
    assert b.slot == a.slot and float(cm.state_groups[0].state[0][b.slot].abs().sum()) == 0.0


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    """Random opens, reserves, commits and closes: the invariants hold at every point and
    everything comes back at the end."""
    rng = random.Random(seed)
    cm = manager(n_pages=12, slots=4, layout={0: PagedKV(2, 8), 1: PagedKV(2, 8, window=90)}, max_step_tokens=80)
    live, n = {}, 0
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            live[n] = cm.open(n)
            n += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            k = rng.choice([1, 1, 2, 17, 64, 80])
            if cm.reserve(live[rid], k):
                cm.commit(live[rid], k)
            else:
                before = [list(t) for t in live[rid].tables]
                assert before == live[rid].tables
        elif live:
            rid = rng.choice(list(live))
            cm.close(live.pop(rid))
        cm.check()
    for r in live.values():
        cm.close(r)
    cm.check()
    assert all(g.pool.n_held == 0 for g in cm.groups)


# ---------------------------------------------------------------------------------------------
# prefix cache
# ---------------------------------------------------------------------------------------------

def _prefix_manager(n_pages=12, slots=4):
    from lgml_b200.cache import CacheManager, PagedKV
    return CacheManager({0: PagedKV(2, 16), 1: PagedKV(2, 16)}, n_pages=n_pages, max_slots=slots, dtype=torch.float32, device="cpu",
                        prefix_cache=True)


def test_prefix_cache_shares_full_pages_and_never_the_last_token():
    m = _prefix_manager()
    toks = list(range(200))
    a = m.open("a", toks)
    assert a.n_tokens == 0 and m.reserve(a, 200)
    m.commit(a, 200)
    assert m.publish(a, toks) == 3                       # three full pages of 64
    b = m.open("b", toks[:150] + [999] * 20)             # same first 150 tokens: two full pages in common
    assert b.n_tokens == 128 and b.tables[0] == a.tables[0][:2]
    assert m.groups[0].pool.refcount(a.tables[0][0]) == 2
    c = m.open("c", toks[:128])                          # all of it is cached, but its last token must run
    assert c.n_tokens == 64
    m.check()
    m.close(a)
    m.check()
    assert m.groups[0].pool.n_cached == 1                # the third page: keyed, nobody holds it
    d = m.open("d", toks)                                # takes up all three again
    assert d.n_tokens == 192 and m.groups[0].pool.n_cached == 0
    for r in (b, c, d):
        m.close(r)
    m.check()
    assert m.groups[0].pool.n_held == 0 and m.groups[0].pool.n_free == 12 and m.groups[0].pool.n_cached == 3


def test_prefix_cache_gives_cached_pages_up_when_the_pool_needs_them():
    m = _prefix_manager(n_pages=4, slots=2)
    toks = list(range(1000, 1130))
    a = m.open("a", toks)
    assert m.reserve(a, 130)
    m.commit(a, 130)
    m.publish(a, toks)
    m.close(a)
    pool = m.groups[0].pool
    assert pool.n_cached == 2 and pool.n_free == 4
    b = m.open("b", list(range(5, 250)))                 # other tokens: needs all four pages
    assert b.n_tokens == 0 and m.reserve(b, 245)
    assert pool.n_cached == 0 and pool.evicted_total == 2
    m.close(b)
    c = m.open("c", toks)                                # the keys went with the pages
    assert c.n_tokens == 0
    m.close(c)
    m.check()


def test_prefix_cache_refuses_windows_and_fixed_state():
    from lgml_b200.cache import CacheManager, FixedState, PagedKV
    with pytest.raises(ValueError, match="prefix_cache"):
        CacheManager({0: PagedKV(2, 16, window=100)}, n_pages=8, max_slots=2, dtype=torch.float32, device="cpu", prefix_cache=True)
    with pytest.raises(ValueError, match="prefix_cache"):
        CacheManager({0: PagedKV(2, 16), 1: FixedState((4,))}, n_pages=8, max_slots=2, dtype=torch.float32, device="cpu", prefix_cache=True)


def test_prefix_cache_random_orders_keep_the_books():
    import random
    rng = random.Random(5)
    m = _prefix_manager(n_pages=10, slots=3)
    families = [[rng.randrange(50) for _ in range(400)] for _ in range(3)]
    live = {}
    for step in range(400):
        if live and (len(live) == 3 or rng.random() < 0.4):
            rid = rng.choice(list(live))
            req, toks = live.pop(rid)
            if rng.random() < 0.8:
                m.publish(req, toks)
            m.close(req)
        else:
            fam = rng.choice(families)
            toks = fam[:rng.randrange(1, 300)] + [rng.randrange(50) for _ in range(rng.randrange(0, 80))]
            req = m.open(step, toks)
            assert req.n_tokens % 64 == 0 and req.n_tokens < len(toks)
            n = len(toks) - req.n_tokens
            if m.reserve(req, n):
                m.commit(req, n)
                live[step] = (req, toks)
            else:
                m.close(req)
        m.check()
    for req, _ in live.values():
        m.close(req)
    m.check()
    assert m.groups[0].pool.n_held == 0 and m.groups[0].pool.shared_total > 0


def test_a_step_that_finds_no_page_leaves_the_books_as_they_were():
    """Three entries, the third cannot fit: the first two give back what the call took for them."""
    from lgml_b200.engine.runner import ModelRunner

    cm = manager(n_pages=6, layout={0: PagedKV(2, 8), 1: PagedKV(2, 8, window=70)})
    a, b, c = cm.open("a"), cm.open("b"), cm.open("c")
    assert cm.reserve(a, 70)
    cm.commit(a, 70)
    assert cm.reserve(b, 10)
    cm.commit(b, 10)
    free = [g.pool.n_free for g in cm.groups]
    lens = [[len(t) for t in r.tables] for r in (a, b, c)]
    tables = [[list(t) for t in r.tables] for r in (a, b, c)]
    wanted = [(a, 60), (b, 64), (c, 129)]          # a and b need a page more each, c three: one too many
    assert cm.reserve_all(wanted) == 2
    assert [g.pool.n_free for g in cm.groups] == free
    assert [[len(t) for t in r.tables] for r in (a, b, c)] == lens
    assert [[list(t) for t in r.tables] for r in (a, b, c)] == tables
    cm.check()
    # the step function raises and changes nothing either (no device is touched before the pages are had)
    runner = ModelRunner.__new__(ModelRunner)
    runner.cache = cm
    with pytest.raises(PoolFull, match="kv pool full: request 'c'"):
        runner._reserve_all(wanted)
    assert [g.pool.n_free for g in cm.groups] == free and [[len(t) for t in r.tables] for r in (a, b, c)] == lens
    assert cm.reserve_all(wanted[:2]) is None and cm.n_free_pages == free[0] - 2
    with pytest.raises(ValueError, match="cannot cut"):
        cm.unreserve(a, [0, 0])                     # never below what holds keys
    cm.check()
