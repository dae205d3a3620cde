"""Greedy answers over a decoder whose kept rows outlive the request that wrote them.

The host loop around the decode step, as the reference's scheduler runs it (engine/engine/src/schedule.rs:227-345):
a waiting prompt is admitted to a slot (`KeptSlots.admit`, engine/engine/src/kept.rs:69-106) and skips the rows an
earlier answer left in the kept rows; every step feeds each active sequence its pending prompt rows (as many as the
launch has room for) or the token it made last; before the launch each fed slot gets the pages its rows need
(`KeptSlots.grow`, the table as `Lanes.set`, engine/engine/src/lanes.rs:41-46); a finished sequence's rows stay under
the tokens that were fed (`KeptSlots.finish`).  The decoder is anything with `step(tokens, slots, positions,
out_rows)`, `set_table(table)` and `slots`, `context`, `max_rows`, `page`, `pages` (tessera_b200.runner.Decoder).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np

from .kv import KeptSlots


@dataclass
class _Seq:
    index: int               # place in the caller's list
    slot: int
    pending: deque           # prompt tokens not fed yet
    fed: int                 # rows of this sequence in the kept rows
    history: list            # the tokens behind those rows
    want: int
    made: list = field(default_factory=list)


class Sessions:
    def __init__(self, decoder, reuse: bool = True):
        self.dec, self.reuse = decoder, reuse
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
        waiting = deque((i, [int(t) for t in p]) for i, p in enumerate(prompts))
        active: list = []
        out = [None] * len(prompts)
        while waiting or active:
            self._admit(waiting, active, new)
            if not active:
                raise RuntimeError("nothing can be admitted: the pool has no room for one more sequence")
            tokens, slots, positions, out_rows, owners = [], [], [], [], []
            room = self.dec.max_rows
            for seq in active:
                if room == 0:
                    break
                if seq.pending:
                    n = min(len(seq.pending), room)
                    feed = [seq.pending.popleft() for _ in range(n)]
                else:
                    feed = [seq.made[-1]]
                    n = 1
                room -= n
                tokens += feed
                slots += [seq.slot] * n
                positions += list(range(seq.fed, seq.fed + n))
                seq.history += feed
                seq.fed += n
                pages = self.kept.grow(seq.slot, seq.fed)
                if pages is not None:
                    first = seq.slot * self.dec.pages
                    self.table[first:first + len(pages)] = pages
                    self.stale = True
                if not seq.pending:               # the sequence's newest row makes its next token
                    out_rows.append(len(tokens) - 1)
                    owners.append(seq)
            if self.stale:
                self.dec.set_table(self.table)
                self.stale = False
            ids = self.dec.step(tokens, slots, positions, out_rows=out_rows or [len(tokens) - 1])
            self.steps += 1
            for seq, token in zip(owners, ids):
                seq.made.append(int(token))
                if len(seq.made) == seq.want:
                    out[seq.index] = seq.made
                    self.kept.finish(seq.slot, seq.history)
                    active.remove(seq)
        return out
