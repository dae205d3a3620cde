"""Greedy answers over a decoder whose kept rows outlive the request that wrote them.

The host loop around the decode step, as the reference's scheduler runs it (engine/engine/src/schedule.rs:227-345):
a waiting prompt is admitted to a slot (`KeptSlots.admit`, engine/engine/src/kept.rs:69-106) and skips the rows an
earlier answer left in the kept rows; every step feeds the rows the `Fair` policy picks (every decoding sequence the
token it made last, then the prompts a token each in turn within the step's row budget, schedule.rs:127-153);
before the launch each fed slot gets the pages its rows need
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


# ---- the same loop in the library (csrc/sessions.cu): ts_sessions_* over a ts_decoder or a host's own stepper ----
import ctypes as _C

_u32, _u64, _vp, _i32 = _C.c_uint32, _C.c_uint64, _C.c_void_p, _C.c_int
_STEP = _C.CFUNCTYPE(_i32, _vp, _C.POINTER(_u32), _C.POINTER(_u32), _C.POINTER(_u32), _u32, _C.POINTER(_u32), _u32,
                     _C.POINTER(_u32))
_TABLE = _C.CFUNCTYPE(_i32, _vp, _C.POINTER(_u32), _u32)


class _Stepper(_C.Structure):
    _fields_ = [("self", _vp), ("slots", _u32), ("context", _u32), ("max_rows", _u32), ("page", _u32), ("step", _STEP),
                ("set_table", _TABLE)]


def _bind():
    from . import runner   # sets the argument types of ts_sessions_* (runner.RUN_SIGNATURES)
    from ._lib import lib
    from .kv import Totals
    assert "ts_sessions_new" in runner.RUN_SIGNATURES
    return lib, Totals


class NativeSessions:
    """ts_sessions_*: the loop of `Sessions` as host code inside the library.  Over a tessera_b200.runner.Decoder it
    calls ts_decoder_step / ts_decoder_set_table directly; over any other decoder it calls back into Python."""

    def __init__(self, decoder, reuse: bool = True, budget: int | None = None):
        self._lib, self._Totals = _bind()
        self.dec = decoder
        handle = getattr(decoder, "_h", None)
        if handle is not None and hasattr(decoder, "run_resident"):      # the library's own decoder
            self._h = self._lib.ts_sessions_on_decoder(handle, int(reuse), budget or 0)
        else:
            def step(_, tokens, slots, positions, rows, out_rows, n_out, out_ids):
                try:
                    ids = decoder.step([tokens[i] for i in range(rows)], [slots[i] for i in range(rows)],
                                       [positions[i] for i in range(rows)], out_rows=[out_rows[i] for i in range(n_out)])
                    for i in range(n_out):
                        out_ids[i] = int(ids[i])
                    return 0
                except Exception:        # a Python exception cannot cross the C frames: report a failed step
                    self.error = __import__("sys").exc_info()[1]
                    return 5

            def set_table(_, table, entries):
                decoder.set_table(np.array([table[i] for i in range(entries)], np.uint32))
                return 0

            self.error = None
            self._keep = (_STEP(step), _TABLE(set_table))                 # the callbacks live as long as the loop
            st = _Stepper(None, decoder.slots, decoder.context, decoder.max_rows, decoder.page, *self._keep)
            self._h = self._lib.ts_sessions_new(_C.byref(st), int(reuse), budget or 0)
        if not self._h:
            raise ValueError("the decoder's slots, context and max_rows must be positive")

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.ts_sessions_free(self._h)
            self._h = None

    def generate(self, prompts: list, new: int) -> list:
        from ._lib import check
        flat = np.ascontiguousarray([t for p in prompts for t in p], dtype=np.uint32)
        offsets = np.ascontiguousarray(np.concatenate([[0], np.cumsum([len(p) for p in prompts])]), dtype=np.uint64)
        out = np.zeros((len(prompts), max(new, 1)), np.uint32)
        code = self._lib.ts_sessions_generate(self._h, flat.ctypes.data_as(_vp), offsets.ctypes.data_as(_vp), len(prompts),
                                              new, out.ctypes.data_as(_vp))
        if code and getattr(self, "error", None) is not None:
            err, self.error = self.error, None
            raise err
        check(code)
        return out.tolist()

    @property
    def steps(self) -> int:
        return int(self._lib.ts_sessions_steps(self._h))

    def totals(self):
        t = self._Totals()
        self._lib.ts_sessions_totals(self._h, _C.byref(t))
        return t

    def consistent(self) -> bool:
        return bool(self._lib.ts_sessions_consistent(self._h))
