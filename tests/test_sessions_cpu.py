"""The host loop around the decode step (tessera_b200/sessions.py) against a stand-in decoder that keeps one token
per kept row, reads a row's whole past through the page table and answers with a hash of it: an answer is right only
if every earlier row of the sequence is where the table says, whoever wrote it.  No GPU."""
import numpy as np
import pytest

from tessera_b200.sessions import Sessions


class KeptTokens:
    def __init__(self, slots, context, max_rows, page):
        self.slots, self.context, self.max_rows, self.page = slots, context, max_rows, page
        self.pages = -(-context // page) if page else 0
        self.rows = np.full(slots * (self.pages * page if page else context), -1, np.int64)
        self.table = np.arange(slots * self.pages, dtype=np.uint32)
        self.launches = []

    def set_table(self, table):
        self.table = np.array(table, np.uint32)

    def _row(self, slot, position):
        if not self.page:
            return slot * self.context + position
        return int(self.table[slot * self.pages + position // self.page]) * self.page + position % self.page

    def step(self, tokens, slots, positions, out_rows=None):
        assert 1 <= len(tokens) <= self.max_rows
        self.launches.append(len(tokens))
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
    with pytest.raises(ValueError):
        s.generate([list(range(15))], 4)
    with pytest.raises(ValueError):
        s.generate([[]], 1)
