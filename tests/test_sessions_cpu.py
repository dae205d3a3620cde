"""The host loop around the decode step (ts_sessions_*, through tessera_b200/sessions.py) against a stand-in decoder that keeps one token
per kept row, reads a row's whole past through the page table and answers with a hash of it: an answer is right only
if every earlier row of the sequence is where the table says, whoever wrote it.  No GPU."""
import numpy as np
import pytest

from tessera_b200 import TesseraError
from tessera_b200.sessions import Sessions


class KeptTokens:
    def __init__(self, slots, context, max_rows, page):
        self.slots, self.context, self.max_rows, self.page = slots, context, max_rows, page
        self.pages = -(-context // page) if page else 0
        self.rows = np.full(slots * (self.pages * page if page else context), -1, np.int64)
        self.table = np.arange(slots * self.pages, dtype=np.uint32)
        self.launches = []
        self.fed_slots = []

    def set_table(self, table):
        self.table = np.array(table, np.uint32)

    def _row(self, slot, position):
        if not self.page:
            return slot * self.context + position
        return int(self.table[slot * self.pages + position // self.page]) * self.page + position % self.page

    def step(self, tokens, slots, positions, out_rows=None):
        assert 1 <= len(tokens) <= self.max_rows
        self.launches.append(len(tokens))
        self.fed_slots.append(list(slots))
        for t, s, p in zip(tokens, slots, positions):   # append before anything attends (scatter.rs: K, V first)
            self.rows[self._row(s, p)] = t
        out = []
        for r in (out_rows if out_rows is not None else range(len(tokens))):
            s, p = slots[r], positions[r]
            past = [int(self.rows[self._row(s, q)]) for q in range(p + 1)]
            assert -1 not in past, f"slot {s} reads an unwritten row below {p}"
            h = 17
            for t in past:
                h = (h * 31 + t) % 1000003
            out.append(h % 997)
        return np.array(out, np.uint32)


def alone(prompt, new):
    """The answer of a sequence that has the decoder to itself."""
    dec = KeptTokens(1, 64, 64, 0)
    return Sessions(dec, reuse=False).generate([prompt], new)[0]


@pytest.mark.parametrize("page", [0, 16])
def test_answers_do_not_depend_on_what_was_kept(page):
    rng = np.random.default_rng(page)
    base = rng.integers(0, 900, size=40).tolist()
    prompts = [base, base[:37] + [5, 6, 7], base[:20], rng.integers(0, 900, size=9).tolist(), base + [1, 2, 3],
               base[:37] + [5, 6, 8, 9]]
    want = [alone(p, 4) for p in prompts]
    dec = KeptTokens(slots=2, context=64, max_rows=24, page=page)
    s = Sessions(dec)
    got = []
    for p in prompts:                       # one after another: each may continue what the earlier ones left
        got += s.generate([p], 4)
    assert got == want
    t = s.totals()
    assert t.hits >= 3 and t.hits + t.misses == len(prompts)
    assert max(dec.launches) <= 24          # prompts longer than a launch are fed in pieces
    # all at once: two slots, six prompts; they wait, share pages where they can, and answer the same
    both = Sessions(KeptTokens(slots=2, context=64, max_rows=24, page=page))
    assert both.generate(prompts, 4) == want


def test_reuse_spares_rows():
    base = list(range(100, 148))
    dec = KeptTokens(slots=2, context=64, max_rows=64, page=16)
    s = Sessions(dec)
    s.generate([base], 2)
    before = sum(dec.launches)
    s.generate([base[:40] + [7]], 2)
    assert sum(dec.launches) - before == (41 - 32) + 1     # 32 rows (two whole pages) were kept
    off = Sessions(KeptTokens(slots=2, context=64, max_rows=64, page=16), reuse=False)
    off.generate([base], 2)
    n = sum(off.dec.launches)
    off.generate([base[:40] + [7]], 2)
    assert sum(off.dec.launches) - n == 41 + 1


def test_prompts_that_cannot_fit_are_refused():
    s = Sessions(KeptTokens(slots=1, context=16, max_rows=16, page=0))
    with pytest.raises(TesseraError):
        s.generate([list(range(15))], 4)
    with pytest.raises(TesseraError):
        s.generate([[]], 1)


def test_step_counts_of_the_reference_cases():
    # engine/engine/tests/engine_test.rs:331-385 with its budget of one prompt row a step: the steps each request
    # takes are the rows it feeds (prompt past the skip, then all but the last token it makes)
    dec = KeptTokens(slots=2, context=16, max_rows=16, page=0)
    s = Sessions(dec, budget=1)

    def asked(prompts):
        before = s.steps
        return s.generate(prompts, 3), s.steps - before

    first, steps = asked([[3, 9, 4]])
    assert steps == 5
    longer = [3, 9, 4] + first[0]
    assert asked([longer])[1] == 3 and asked([[3, 9, 7, 1]])[1] == 4
    t = s.totals()
    assert (t.hits, t.misses) == (2, 1)

    paged = Sessions(KeptTokens(slots=2, context=64, max_rows=64, page=16), budget=1)
    base = [(i * 7 + 3) % 32 for i in range(20)]
    before = paged.steps
    paged.generate([base], 3)
    assert paged.steps - before == 22
    before = paged.steps
    got = paged.generate([base[:18] + [1, 2], base[:17] + [5]], 3)
    assert paged.steps - before == 10          # both start at the kept answer's first page; their rows share steps
    assert got == [alone(base[:18] + [1, 2], 3), alone(base[:17] + [5], 3)]


def test_first_step_feeds_decodes_first_then_prompts_in_turn():
    # through the library's loop: a one-token prompt is already decoding (its only row makes a token), prompts of
    # ten and three rows share what is left of a six-row budget a token each in turn: b c b c b
    dec = KeptTokens(slots=3, context=64, max_rows=64, page=0)
    Sessions(dec, reuse=False, budget=6).generate([list(range(10)), [7], [1, 2, 3]], 2)
    first = dec.fed_slots[0]
    assert len(first) == 6 and sorted(first.count(s) for s in set(first)) == [1, 2, 3]
    # rows of a sequence sit side by side in the launch
    assert all(first[i] == first[i + 1] or first[i] not in first[i + 1:] for i in range(len(first) - 1))
    tight = KeptTokens(slots=3, context=64, max_rows=4, page=0)      # the launch itself holds four rows
    Sessions(tight, reuse=False, budget=64).generate([list(range(10)), [7], [1, 2, 3]], 2)
    assert max(tight.launches) <= 4 and len(tight.fed_slots[0]) == 4


def test_fair_of_the_model_feeds_decodes_first_then_prompts_in_turn():
    from collections import deque
    from tests.sessions_model import _Seq, fair
    a = _Seq(0, 0, deque([7]), 9, [], 3)                 # decoding
    b = _Seq(1, 1, deque(range(10)), 0, [], 3)           # ten prompt rows
    c = _Seq(2, 2, deque(range(3)), 0, [], 3)            # three
    take = fair([b, a, c], budget=6, most=64)
    assert (take[id(a)], take[id(b)], take[id(c)]) == (1, 3, 2)     # 1 decode, then b c b c b: six rows
    take = fair([b, a, c], budget=64, most=64)
    assert (take[id(a)], take[id(b)], take[id(c)]) == (1, 10, 3)
    take = fair([b, a, c], budget=64, most=4)                        # the launch itself holds four rows
    assert sum(take.values()) == 4 and take[id(a)] == 1


@pytest.mark.parametrize("seed", range(6))
def test_random_rounds_of_related_prompts(seed):
    # prompts cut from a few stems at random lengths, in random-sized rounds, random page and budget: whatever
    # was kept, borrowed, adopted or reclaimed on the way, every answer equals the one of a decoder used once
    rng = np.random.default_rng(100 + seed)
    page = int(rng.choice([0, 16, 64]))
    slots, context = int(rng.integers(1, 4)), 128
    dec = KeptTokens(slots, context, max_rows=int(rng.choice([8, 32, 128])), page=page)
    s = Sessions(dec, budget=int(rng.choice([1, 5, 128])))
    stems = [rng.integers(0, 900, size=100).tolist() for _ in range(3)]
    asked = 0
    for _ in range(8):
        prompts = []
        for _ in range(int(rng.integers(1, 5))):
            stem = stems[int(rng.integers(0, 3))]
            cut = int(rng.integers(1, 100))
            tail = rng.integers(0, 900, size=int(rng.integers(0, 6))).tolist()
            prompts.append(stem[:cut] + tail)
        new = int(rng.integers(1, 5))
        assert s.generate(prompts, new) == [alone_in(context, p, new) for p in prompts]
        assert s.consistent()
        asked += len(prompts)
    t = s.totals()
    assert t.hits + t.misses == asked and t.pool.live_runs == 0


def alone_in(context, prompt, new):
    return Sessions(KeptTokens(1, context, context, 0), reuse=False).generate([prompt], new)[0]


@pytest.mark.parametrize("seed", range(4))
def test_the_library_loop_equals_the_python_model(seed):
    # ts_sessions_* (csrc/sessions.cu) driven through callbacks by the stand-in decoder: the same answers, the same
    # launches row for row, the same steps and totals as the plain Python statement of the loop in tests/sessions_model.py
    from tests.sessions_model import Sessions as Model
    rng = np.random.default_rng(200 + seed)
    page = int(rng.choice([0, 16, 64]))
    slots, context, rows = int(rng.integers(1, 4)), 128, int(rng.choice([8, 32, 128]))
    budget = int(rng.choice([1, 5, 128]))
    a, b = KeptTokens(slots, context, rows, page), KeptTokens(slots, context, rows, page)
    py, lib = Model(a, budget=budget), Sessions(b, budget=budget)
    stems = [rng.integers(0, 900, size=100).tolist() for _ in range(3)]
    for _ in range(6):
        prompts = [stems[int(rng.integers(0, 3))][: int(rng.integers(1, 100))] + rng.integers(0, 900, size=int(rng.integers(0, 6))).tolist()
                   for _ in range(int(rng.integers(1, 5)))]
        new = int(rng.integers(1, 5))
        assert lib.generate(prompts, new) == py.generate(prompts, new)
        assert lib.consistent()
    assert a.launches == b.launches and a.fed_slots == b.fed_slots and lib.steps == py.steps
    tp, tl = py.totals(), lib.totals()
    assert (tp.hits, tp.misses, tp.pool.kept_runs) == (tl.hits, tl.misses, tl.pool.kept_runs)


def test_the_library_loop_refuses_and_reports():
    s = Sessions(KeptTokens(1, 16, 16, 0))
    with pytest.raises(TesseraError):
        s.generate([list(range(15))], 4)           # does not fit the context with its answer
    with pytest.raises(TesseraError):
        s.generate([[]], 1)

    class Broken(KeptTokens):
        def step(self, *a, **k):
            raise RuntimeError("the device fell over")

    with pytest.raises(RuntimeError, match="fell over"):
        Sessions(Broken(1, 16, 16, 0)).generate([[1, 2, 3]], 2)


@pytest.mark.parametrize("page", [0, 16])
def test_a_failed_step_gives_its_slots_back(page):
    # A step that fails once must not strand the active sequences' slots and pages: the same sessions then answer
    # the next request, with the answers of a decoder that never failed (the reference retires a sequence on every
    # exit path: engine/engine/src/schedule.rs finish / retire).
    class FailsOnce(KeptTokens):
        armed = True

        def step(self, *a, **k):
            if self.armed and len(self.launches) == 2:
                self.armed = False
                raise RuntimeError("one bad launch")
            return super().step(*a, **k)

    prompts = [[5, 6, 7, 8], [9, 10], [11, 12, 13]]
    s = Sessions(FailsOnce(2, 64, 16, page), reuse=False)
    with pytest.raises(RuntimeError, match="one bad launch"):
        s.generate(prompts, 3)
    assert s.consistent()
    got = s.generate(prompts, 3)          # both slots are free again: three prompts over two slots
    assert s.consistent()
    assert got == [alone(p, 3) for p in prompts]
