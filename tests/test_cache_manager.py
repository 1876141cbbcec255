"""The cache manager's bookkeeping: no page lost, held twice or freed twice, under random request orders."""
import numpy as np
import pytest

from xyntetik_runner_b200.cache.pages import CacheError, CacheManager, GroupSpec, OutOfPages, PagePool


def test_pool_rules():
    p = PagePool(3)
    a, b, c = p.take(), p.take(), p.take()
    assert sorted([a, b, c]) == [0, 1, 2] and p.n_free == 0
    with pytest.raises(OutOfPages):
        p.take()
    p.give(b)
    with pytest.raises(CacheError):
        p.give(b)                      # freed twice
    with pytest.raises(CacheError):
        p.give(7)
    assert p.take() == b               # used again


def test_reserve_commit_cancel_close():
    m = CacheManager([GroupSpec("full")], n_pages=6, page_size=4, max_requests=2, max_request_tokens=24)
    s = m.open("a")
    assert s in (0, 1) and m.length("a") == 0
    m.reserve("a", 5)                  # 2 pages
    assert m.free_pages() == [4] and (m.block_table(0, "a")[:2] >= 0).all() and m.block_table(0, "a")[2] == -1
    m.audit()
    m.cancel("a")                      # a planned step that never ran gives its pages back
    assert m.free_pages() == [6] and m.length("a") == 0
    m.reserve("a", 5); m.commit("a")
    assert m.length("a") == 5
    m.reserve("a", 3); m.commit("a")   # 8 tokens: still 2 pages
    assert m.free_pages() == [4]
    m.reserve("a", 1)                  # 9th token: a third page
    assert m.free_pages() == [3]
    m.cancel("a")
    assert m.free_pages() == [4] and m.length("a") == 8
    m.open("b")
    with pytest.raises(OutOfPages):
        m.open("c")                    # no slot
    with pytest.raises(OutOfPages):
        m.reserve("b", 17)             # 5 pages, 4 free: nothing is taken
    assert m.free_pages() == [4]
    m.audit()
    with pytest.raises(OutOfPages):
        m.reserve("a", 17)             # beyond the longest request
    m.close("a"); m.close("b")
    assert m.free_pages() == [6]
    with pytest.raises(CacheError):
        m.close("a")
    m.audit()


def test_window_group_releases_pages_behind_the_window():
    m = CacheManager([GroupSpec("full"), GroupSpec("w", window=6)], n_pages=8, page_size=4, max_requests=2,
                     max_request_tokens=32)
    m.open("a")
    m.reserve("a", 10); m.commit("a")          # positions 0..9: 3 pages in both groups
    assert m.free_pages() == [5, 5]
    m.reserve("a", 1); m.commit("a")           # query at 10 sees keys 5..10: page 0 (0..3) is behind the window
    assert m.free_pages() == [5, 6]
    assert m.block_table(1, "a")[0] == -1 and m.block_table(0, "a")[0] >= 0
    m.audit()
    for _ in range(13):
        m.reserve("a", 1); m.commit("a")       # up to 24 tokens
    assert m.length("a") == 24
    # window group holds pages for keys 18.. only (pages 4, 5); the full group all six
    assert m.free_pages() == [2, 6]
    m.audit()
    m.close("a")
    assert m.free_pages() == [8, 8]
    m.audit()


def test_window_lets_a_long_request_live_in_a_small_pool():
    m = CacheManager([GroupSpec("w", window=5)], n_pages=4, page_size=4, max_requests=1, max_request_tokens=400)
    m.open("a")
    for i in range(300):
        assert m.can_reserve("a", 1)
        m.reserve("a", 1); m.commit("a")
        m.audit()
    assert m.high_water[0] <= 3


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariants(seed):
    rng = np.random.RandomState(seed)
    groups = [GroupSpec("full"), GroupSpec("w", window=int(rng.randint(3, 20)))] if seed % 2 else [GroupSpec("full")]
    ps = int(rng.choice([1, 4, 8, 16]))
    m = CacheManager(groups, n_pages=int(rng.randint(8, 30)), page_size=ps, max_requests=4, max_request_tokens=ps * 12)
    live, next_id, held_pages = {}, 0, None
    for it in range(600):
        op = rng.rand()
        if op < 0.2 and m.has_free_slot():
            m.open(next_id); live[next_id] = 0; next_id += 1
        elif op < 0.75 and live:
            rid = list(live)[rng.randint(len(live))]
            n = int(rng.randint(1, 3 * ps))
            before = m.free_pages()
            if m.can_reserve(rid, n):
                m.reserve(rid, n)
                if rng.rand() < 0.15:
                    m.cancel(rid)
                    # cancel restores the pool except for pages the window let go
                    assert all(a >= b for a, b in zip(m.free_pages(), before))
                else:
                    m.commit(rid); live[rid] += n
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, n)
                assert m.free_pages() == before        # a failed reservation takes nothing
        elif live:
            rid = list(live)[rng.randint(len(live))]
            m.close(rid); del live[rid]
        m.audit()
        for rid, n in live.items():
            assert m.length(rid) == n
            tab = m.block_table(0, rid)
            assert (tab[:-(-n // ps)] >= 0).all() and (tab[-(-n // ps):] == -1).all()     # full group: ceil(len/ps) pages
    for rid in list(live):
        m.close(rid)
    m.audit()
    assert m.free_pages() == [p.n_pages for p in m.pools]


def test_describe_step_flattens_a_batch():
    """The step description: ids, positions (from the requests' lengths), segments, wanted rows, block-table rows,
    and filler segments at position 0 that point at the spare page."""
    m = CacheManager([GroupSpec("full"), GroupSpec("w", window=6)], n_pages=16, page_size=4, max_requests=4, max_request_tokens=32)
    for rid, held in (("a", 9), ("b", 0), ("c", 3)):
        m.open(rid)
        if held:
            m.reserve(rid, held); m.commit(rid)
    batch = [("c", [7], [0]), ("a", [11, 12, 13], [0, 2]), ("b", [5, 6], [])]
    for rid, toks, _ in batch:
        m.reserve(rid, len(toks))
    i32 = np.int32
    slots = np.array([m.slot_of(r) for r, _, _ in batch], dtype=i32)
    counts = np.array([len(t) for _, t, _ in batch], dtype=i32)
    tokens = np.array([x for _, t, _ in batch for x in t], dtype=i32)
    want_counts = np.array([len(w) for _, _, w in batch], dtype=i32)
    wants = np.array([x for _, _, w in batch for x in w], dtype=i32)
    fill, n, S, R, mp = 2, 6 + 2, 3 + 2, 3 + 2, m.max_pages_per_request
    arrs = [np.full(k, -9, dtype=i32) for k in (n, n, n, R, S, S, S, S)]
    bts = [np.full((S, mp), -9, dtype=i32) for _ in m.groups]
    max_kv = m.describe_step(slots, counts, tokens, want_counts, wants, fill, 16, [a.ctypes.data for a in arrs],
                             [b.ctypes.data for b in bts])
    tok, pos, seg, rows, s_start, s_len, s_pos0, s_slot = arrs
    assert max_kv == 12
    assert tok.tolist() == [7, 11, 12, 13, 5, 6, 0, 0] and pos.tolist() == [3, 9, 10, 11, 0, 1, 0, 0]
    assert seg.tolist() == [0, 1, 1, 1, 2, 2, 3, 4] and rows.tolist() == [0, 1, 3, 6, 7]
    assert s_start.tolist() == [0, 1, 4, 6, 7] and s_len.tolist() == [1, 3, 2, 1, 1] and s_pos0.tolist() == [3, 9, 0, 0, 0]
    assert s_slot.tolist()[:3] == slots.tolist()
    for g in range(2):
        for si, (rid, _, _) in enumerate(batch):
            assert (bts[g][si] == m.block_table(g, rid)).all()
        assert (bts[g][3:, 0] == 16).all() and (bts[g][3:, 1:] == -1).all()
    for rid, _, _ in batch:
        m.commit(rid)
    m.audit()
    m.close("b")
    with pytest.raises(CacheError):
        m.describe_step(slots, counts, tokens, want_counts, wants, 0, 16, [a.ctypes.data for a in arrs], [b.ctypes.data for b in bts])


@pytest.mark.parametrize("seed", range(4))
def test_pages_held_follow_the_formula(seed):
    """After every commit a request holds, in a group that keeps all keys, ceil(length / page) pages, and in a window
    group the pages from the one that holds the first key its next query can still read up to the last: counted here
    from lengths alone and compared with the pools."""
    rng = np.random.RandomState(50 + seed)
    ps, window, n_pages = int(rng.choice([2, 4, 8])), int(rng.randint(2, 30)), 200
    m = CacheManager([GroupSpec("full"), GroupSpec("w", window=window)], n_pages, ps, 5, ps * 30)
    lengths = {}

    released = {}                                   # request -> first page index still held in the window group
    for it in range(500):
        op = rng.rand()
        if op < 0.15 and m.has_free_slot():
            rid = f"r{it}"
            m.open(rid); lengths[rid] = 0; released[rid] = 0
        elif op < 0.85 and lengths:
            rid = list(lengths)[rng.randint(len(lengths))]
            n = int(rng.randint(1, 2 * ps + 2))
            if lengths[rid] + n <= ps * 30:
                # reserving releases what a query at the current length can no longer read
                first_key = max(0, lengths[rid] - window + 1)
                released[rid] = max(released[rid], min(first_key // ps, -(-lengths[rid] // ps)))
                m.reserve(rid, n); m.commit(rid)
                lengths[rid] += n
        elif lengths:
            rid = list(lengths)[rng.randint(len(lengths))]
            m.close(rid); del lengths[rid]; del released[rid]
        full = sum(-(-n // ps) for n in lengths.values())
        win = sum(-(-n // ps) - released[rid] for rid, n in lengths.items())
        assert m.free_pages() == [n_pages - full, n_pages - win], (it, lengths, released)
        for rid, n in lengths.items():
            tab = m.block_table(1, rid)
            assert (tab[:released[rid]] == -1).all() and (tab[released[rid]:-(-n // ps)] >= 0).all()
    m.audit()
