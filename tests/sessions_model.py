"""A second statement of the session loop, in Python, for the tests to hold the library's loop against.

Test infrastructure, like the checker under oracle/: the product's loop is csrc/sessions.cu (ts_sessions_*).  This
one follows the reference's scheduler (engine/engine/src/schedule.rs:17-153, 227-345) over the page pool's ctypes face
and is deliberately plain: a waiting prompt is admitted (`KeptSlots.admit`), `fair` picks the rows of a step (decodes
first, then the prompts a token each in turn within the budget), fed slots get their pages (`KeptSlots.grow`), a
finished sequence's rows stay under the tokens that were fed (`KeptSlots.finish`).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np

from tessera_b200.kv import KeptSlots


@dataclass
class _Seq:
    """An answer in flight, in its slot (schedule.rs:17-31)."""
    index: int               # place in the caller's list
    slot: int
    pending: deque           # tokens to feed: the prompt past the skip, then each token made
    fed: int                 # rows of this sequence in the kept rows
    history: list            # the tokens behind those rows
    want: int
    made: list = field(default_factory=list)

    def prefilling(self) -> bool:
        return len(self.pending) > 1


def fair(seqs: list, budget: int, most: int) -> dict:
    """Rows per sequence for the next step: decodes first, then a prompt token each in turn while the step has
    fewer than `budget` rows (`Fair`, schedule.rs:127-153).  `most` is the launch's own limit, which decodes count
    against too."""
    take = {id(s): 1 for s in seqs if s.pending and not s.prefilling()}
    take = dict(list(take.items())[:most])
    rows = len(take)
    prompts = [s for s in seqs if s.prefilling()]
    for s in prompts:
        take[id(s)] = 0
    while True:
        more = False
        for s in prompts:
            if take[id(s)] < len(s.pending) and rows < min(budget, most):
                take[id(s)] += 1
                rows += 1
                more = True
        if not more:
            return take


class Sessions:
    def __init__(self, decoder, reuse: bool = True, budget: int | None = None):
        """`budget`: the most rows one step feeds to prompts (the scheduler's budget, schedule.rs:166-167); the
        decoder's `max_rows` by default."""
        self.dec, self.reuse = decoder, reuse
        self.budget = decoder.max_rows if budget is None else budget
        if self.budget < 1:
            raise ValueError("a step feeds at least one row")
        d = decoder
        if d.page:
            self.kept = KeptSlots(d.slots, d.context, pages=d.slots * d.pages, page=d.page)
            self.table = np.arange(d.slots * d.pages, dtype=np.uint32)   # each slot its own pages (lanes.rs:16-24)
            self.stale = True
        else:
            self.kept = KeptSlots(d.slots, d.context)
            self.table, self.stale = None, False
        self.steps = 0

    def totals(self):
        return self.kept.totals()

    def _admit(self, waiting: deque, active: list, new: int):
        while waiting:
            index, prompt = waiting[0]
            if len(prompt) == 0 or len(prompt) + new > self.dec.context:
                raise ValueError(f"prompt {index}: {len(prompt)} tokens and {new} new ones do not fit {self.dec.context} rows")
            # the last prompt row is always fed: its logits make the first token (schedule.rs:231)
            placed = self.kept.admit(prompt, (len(prompt) - 1) if self.reuse else 0)
            if placed is None:
                return
            waiting.popleft()
            slot, skip = placed
            active.append(_Seq(index, slot, deque(prompt[skip:]), skip, list(prompt[:skip]), new))

    def generate(self, prompts: list, new: int) -> list:
        """`new` greedy tokens for each prompt; prompts wait while every slot is taken."""
        if new < 1:
            raise ValueError("an answer has at least one token")
        waiting = deque((i, [int(t) for t in p]) for i, p in enumerate(prompts))
        active: list = []
        out = [None] * len(prompts)
        while waiting or active:
            self._admit(waiting, active, new)
            if not active:
                raise RuntimeError("nothing can be admitted: the pool has no room for one more sequence")
            take = fair(active, self.budget, self.dec.max_rows)
            tokens, slots, positions, ends, owners = [], [], [], [], []
            for seq in active:                     # a sequence's rows side by side, in position order
                n = take.get(id(seq), 0)
                if n == 0:
                    continue
                tokens += [seq.pending[i] for i in range(n)]
                slots += [seq.slot] * n
                positions += list(range(seq.fed, seq.fed + n))
                pages = self.kept.grow(seq.slot, seq.fed + n)          # Sched::page, schedule.rs:311-322
                if pages is not None:
                    first = seq.slot * self.dec.pages
                    self.table[first:first + len(pages)] = pages
                    self.stale = True
                ends.append(len(tokens) - 1)
                owners.append((seq, n))
            if self.stale:
                self.dec.set_table(self.table)
                self.stale = False
            ids = self.dec.step(tokens, slots, positions, out_rows=ends)
            self.steps += 1
            for (seq, n), token in zip(owners, ids):                   # Seq::advance, schedule.rs:52-76
                seq.history += [seq.pending.popleft() for _ in range(n)]
                seq.fed += n
                if seq.pending:
                    continue                                           # more of the prompt to feed: the id is not used
                seq.made.append(int(token))
                if len(seq.made) >= seq.want:
                    out[seq.index] = seq.made
                    self.kept.finish(seq.slot, seq.history)            # Sched::retire
                    active.remove(seq)
                else:
                    seq.pending.append(int(token))
        return out
