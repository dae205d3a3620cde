"""The host page pool against the reference's own pool tests (engine/ir/kv/src/pool_test.rs:5-103),
replayed call for call, plus the self-check after every random call."""
import pytest

from tessera_b200.kv import Pool, PoolError

T = 0


def err(fn, *a):
    with pytest.raises(PoolError) as e:
        fn(*a)
    return e.value.kind, e.value.detail


def test_admission_counts_worst():
    # pool_test.rs:5-18
    pool = Pool(4, 2)
    a = pool.reserve(T, 1, 6)
    assert err(pool.reserve, T, 1, 4) == ("NoRoom", 2)
    s = pool.stats()
    assert (s.size, s.active, s.worst) == (8, 2, 6)
    pool.retain(a)
    s = pool.stats()
    assert (s.live_runs, s.kept_runs, s.active) == (0, 1, 0)
    pool.release(a)
    pool.reserve(T, 1, 8)


def test_shared_writes_copy():
    # pool_test.rs:20-39
    pool = Pool(8, 2)
    a = pool.reserve(T, 3, 6)
    b = pool.fork(a, 3, 6)
    first, last = pool.pages(a)
    copies = pool.grow(b, 4)
    to = copies[0][1]
    assert copies == [(last, to, 1)]
    assert pool.pages(b) == [first, to]
    assert pool.grow(a, 4) == []


def test_retained_rows_fork():
    # pool_test.rs:41-53
    pool = Pool(4, 2)
    a = pool.reserve(T, 3, 8)
    pool.grow(a, 8)
    pool.truncate(a, 3)
    pool.retain(a)
    b = pool.fork(a, 3, 4)
    assert pool.pages(b) == pool.pages(a)
    pool.release(b)
    pool.reserve(T, 8, 8)
    assert err(pool.pages, a)[0] == "Unknown"


def test_full_pool_adopts():
    # pool_test.rs:55-69
    pool = Pool(2, 4)
    a = pool.reserve(T, 3, 4)
    pool.reserve(T, 3, 4)
    pool.retain(a)
    assert err(pool.fork, a, 2, 4) == ("NoRoom", 1)
    page = pool.pages(a)
    b = pool.adopt(a, 2, 4)
    assert err(pool.adopt, b, 2, 4)[0] == "Live"
    assert (pool.pages(b), pool.rows(b)) == (page, 2)
    assert err(pool.rows, a)[0] == "Unknown"
    pool.grow(b, 4)


def test_random_calls():
    # pool_test.rs:71-103: random calls on small pools; a failing call leaves the digest unchanged and
    # the pool stays consistent (holder counts match the runs, every promise fits) throughout
    mask = (1 << 64) - 1
    for pages in (4, 6, 8, 12):
        for seed in (1, 2, 3, 4):
            pool = Pool(pages, 4)
            runs = []
            for _ in range(1000):
                seed = (seed * 6364136223846793005 + 1) & mask
                pick = seed >> 33
                run = runs[pick // 8 % max(len(runs), 1)] if runs else None
                before = pool.digest()
                op = pick % 7
                try:
                    if op == 1 and run is not None:
                        runs.append(pool.fork(run, pick % 9, 16))
                    elif op == 2 and run is not None:
                        pool.grow(run, pick % 17)
                    elif op == 3 and run is not None:
                        pool.truncate(run, pick % 9)
                    elif op == 4 and run is not None:
                        pool.retain(run)
                    elif op == 5 and run is not None:
                        pool.release(run)
                        runs = [o for o in runs if o != run]
                    elif op == 6 and run is not None:
                        new = pool.adopt(run, pick % 9, 16)
                        runs = [o for o in runs if o != run] + [new]
                    else:
                        runs.append(pool.reserve(T, pick % 9, 8 + pick % 9))
                except PoolError:
                    assert pool.digest() == before
                assert pool.consistent()


def test_lowest_free_page_first_and_table_fill():
    import numpy as np
    pool = Pool(8, 16)
    a = pool.reserve(T, 20, 64)   # pages 0, 1
    b = pool.reserve(T, 1, 32)    # page 2
    assert pool.pages(a) == [0, 1] and pool.pages(b) == [2]
    pool.release(a)
    c = pool.reserve(T, 40, 48)   # lowest free first: 0, 1, 3
    assert pool.pages(c) == [0, 1, 3]
    table = np.full(2 * 4, 99, np.uint32)
    pool.fill_table(c, table, 1, 4)
    assert table.tolist() == [99, 99, 99, 99, 0, 1, 3, 99]


def test_skips_follow_rule():
    # engine/ir/kv/src/reuse_test.rs:3-14, case for case
    from tessera_b200.kv import begin
    cases = [
        (1031, 1030, 191, 2191, 64, 128, "Hit"),
        (1031, 1030, 63, 1999, 64, 0, "Grid"),
        (100, 0, 100, 99, 0, 0, "NoLcp"),
    ]
    for h, valid, lcp, limit, grid, skip, why in cases:
        assert begin([1] * h, valid, [1] * lcp, limit, grid) == (skip, lcp, why)
    assert begin([], 5, [1, 2, 3], 10, 1) == (0, 0, "First")          # no history
    assert begin([1, 2, 9], 3, [1, 2, 3, 4], 10, 1) == (2, 2, "Hit")   # the common rows stop at the first difference
    assert begin([1, 2, 3], 3, [1, 2, 3], 2, 1) == (2, 3, "Hit")       # the limit caps the skip, not the lcp


def test_prefixes_find_newest_longest():
    # engine/ir/kv/src/prefix.rs:34-55: runs of another tag and runs the pool no longer knows never match; the
    # longest skip wins and a later entry wins a tie
    from tessera_b200.kv import Prefixes
    pool = Pool(16, 4)
    kept = Prefixes(grid=4)
    prompt = list(range(100, 120))
    assert kept.find(pool, T, prompt, 64) is None
    runs = []
    for tag, history in ((T, prompt[:6] + [7, 7]), (T, prompt[:9]), (1, prompt[:16]), (T, prompt[:10])):
        r = pool.reserve(tag, len(history), len(history))
        pool.retain(r)
        kept.keep(r, history, len(history))
        runs.append(r)
    assert len(kept) == 4
    run, skip = kept.find(pool, T, prompt, 64)
    assert (run, skip) == (runs[3], 8)           # 9 and 10 common rows both skip 8: the newer run
    assert kept.find(pool, 1, prompt, 64) == (runs[2], 16)
    assert kept.find(pool, T, prompt, 7) == (runs[3], 4)   # the limit applies before the grid
    assert kept.find(pool, T, [5, 5, 5], 64) is None
    pool.release(runs[3])
    run, skip = kept.find(pool, T, prompt, 64)
    assert (run, skip) == (runs[1], 8) and len(kept) == 3  # the released run's entry left
    # a run adopted by a new request is no longer the retained run either
    pool.adopt(runs[1], 8, 12)
    assert kept.find(pool, T, prompt, 64) == (runs[0], 4) and len(kept) == 2
    assert pool.consistent()
