"""Greedy answers over a decoder whose kept rows outlive the request that wrote them: the face on `ts_sessions_*`.

The host loop around the decode step, as the reference's scheduler runs it (engine/engine/src/schedule.rs:227-345),
lives in the library (csrc/sessions.cu), one implementation for every host language: a waiting prompt is admitted to
a slot (engine/engine/src/kept.rs:69-106) and skips the rows an earlier answer left in the kept rows; every step feeds
the rows the `Fair` policy picks (every decoding sequence the token it made last, then the prompts a token each in
turn within the step's row budget, schedule.rs:127-153); before the launch each fed slot gets the pages its rows need
(the table as `Lanes.set`, engine/engine/src/lanes.rs:41-46); a finished sequence's rows stay under the tokens that
were fed.  The decoder is a tessera_b200.runner.Decoder (the loop then calls ts_decoder_step / ts_decoder_set_table
directly) or anything with `step(tokens, slots, positions, out_rows)`, `set_table(table)` and `slots`, `context`,
`max_rows`, `page` (called back through function pointers, the way a host in another language would).
"""
from __future__ import annotations

import ctypes as _C

import numpy as np

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


class Sessions:
    """`budget`: the most rows one step feeds to prompts (the scheduler's budget, schedule.rs:166-167); the decoder's
    `max_rows` by default.  Refusals (a prompt that cannot fit, an empty one) raise TesseraError before any launch; an
    exception inside a Python decoder's step comes back as itself."""

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


NativeSessions = Sessions   # the name this class had while a Python loop stood beside it
