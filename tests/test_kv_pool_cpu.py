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


def test_kept_rows_resume():
    # engine/engine/tests/engine_test.rs:331-360 at the level of the slots: two dense slots of 16 rows, three tokens
    # made per request, one row fed per step.  A request feeds its prompt past the skip and all but the last token it
    # makes; those fed tokens are its history.
    from tessera_b200.kv import KeptSlots
    kept = KeptSlots(slots=2, context=16)

    def ask(prompt, made):
        slot, skip = kept.admit(prompt, len(prompt) - 1)
        history = list(prompt) + made[:-1]
        assert kept.grow(slot, len(history)) is None          # dense: no lanes
        kept.finish(slot, history)
        return skip, len(history) - skip                       # rows spared, rows fed (= steps at one row a step)

    first = [20, 21, 22]
    longer = [3, 9, 4] + first
    assert ask([3, 9, 4], first) == (0, 5)
    assert ask(longer, [23, 24, 25]) == (5, 3)                 # everything but the last prompt row is kept
    assert ask([3, 9, 7, 1], [26, 27, 28]) == (2, 4)           # the common rows of the one retained run
    slot, skip = kept.admit(longer, len(longer) - 1)           # still in flight below
    assert skip == 2                                           # Event::Kept(2): the adopting run was cut to two rows
    t = kept.totals()
    assert (t.hits, t.misses) == (3, 1)
    assert (t.pool.size, t.pool.active) == (32, 16)


def test_paged_slots_share():
    # engine/engine/tests/engine_test.rs:362-385: 16-row pages, two slots of 64 rows; both later prompts start at the
    # kept answer's first page and take a page of their own for the rest
    from tessera_b200.kv import KeptSlots
    kept = KeptSlots(slots=2, context=64, pages=8, page=16)
    base = [(i * 7 + 3) % 32 for i in range(20)]
    slot, skip = kept.admit(base, len(base) - 1)
    assert (slot, skip) == (0, 0)
    lanes = []
    for rows in range(1, 23):                                  # 20 prompt rows and two fed answers: 22 steps
        got = kept.grow(slot, rows)
        if got is not None:
            lanes.append((rows, got))
    assert [r for r, _ in lanes] == [1, 17] and lanes[1][1][0] == lanes[0][1][0]   # a page at row 1, another at row 17
    first_page = lanes[0][1][0]
    kept.finish(slot, base + [40, 41])
    a, b = base[:18] + [1, 2], base[:17] + [5]
    (sa, ka), (sb, kb) = kept.admit(a, len(a) - 1), kept.admit(b, len(b) - 1)
    assert (ka, kb) == (16, 16) and {sa, sb} == {0, 1}
    assert kept.admit([1, 2, 3], 2) is None                    # no slot left
    pa, pb = kept.grow(sa, 17), kept.grow(sb, 17)
    assert pa[0] == pb[0] == first_page and pa[1] != pb[1]     # the shared page, then one each
    fed = (len(a) + 2 - ka) + (len(b) + 2 - kb)
    assert fed == 10                                           # the reference's step count for the second round
    kept.finish(sa, a + [50, 51])
    kept.finish(sb, b + [60, 61])
    t = kept.totals()
    assert (t.hits, t.misses) == (2, 1) and t.pool.live_runs == 0 and t.pool.kept_runs == 3
    with pytest.raises(PoolError) as e:
        kept.grow(0, 5)                                        # a finished slot has no run
    assert e.value.kind == "RowPlace"
