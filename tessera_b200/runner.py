"""Python face of the C++ decode runner (include/tessera_b200_run.h)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib

u32, f32, vp, sz, i32 = C.c_uint32, C.c_float, C.c_void_p, C.c_size_t, C.c_int


class DecoderConfig(C.Structure):
    _fields_ = [(n, u32) for n in ("layers", "hidden", "heads", "kv_heads", "head_dim", "ffn", "vocab", "slots",
                                   "context", "page", "max_rows")]
    _fields_ += [("eps", f32), ("theta", f32), ("qk_norm", i32), ("graphs", i32), ("pdl", i32)]


RUN_SIGNATURES = {
    "ts_decoder_create": (i32, [C.POINTER(DecoderConfig), C.POINTER(vp)]),
    "ts_decoder_destroy": (None, [vp]),
    "ts_decoder_load": (i32, [vp, C.c_char_p, vp, sz]),
    "ts_decoder_set_table": (i32, [vp, vp, u32]),
    "ts_decoder_copy_pages": (i32, [vp, vp, u32, vp]),
    "ts_decoder_step": (i32, [vp, vp, vp, vp, u32, vp, u32, vp, vp]),
    "ts_decoder_run_resident": (i32, [vp, u32, vp]),
    "ts_decoder_read_ids": (i32, [vp, vp, u32, vp]),
    "ts_decoder_read_hidden": (i32, [vp, vp, u32, vp]),
    "ts_decoder_read_logits": (i32, [vp, vp, u32, vp]),
    "ts_decoder_launches_per_step": (u32, [vp, u32, u32]),
    "ts_decoder_graph_replays": (C.c_uint64, [vp]),
    "ts_decoder_graphs": (u32, [vp]),
    "ts_decoder_prepare": (i32, [vp, u32, vp]),
    "ts_decoder_profile": (i32, [vp, u32, vp]),
    "ts_decoder_take_profile": (i32, [vp, C.c_char_p, sz]),
    "ts_decoder_get_config": (i32, [vp, C.POINTER(DecoderConfig)]),
    "ts_decoder_use_step_kernel": (i32, [vp, i32]),
    # the request loop (tessera_b200/sessions.py binds the stepper's callback types)
    "ts_sessions_new": (vp, [vp, i32, u32]),
    "ts_sessions_on_decoder": (vp, [vp, i32, u32]),
    "ts_sessions_free": (None, [vp]),
    "ts_sessions_generate": (i32, [vp, vp, vp, u32, u32, vp]),
    "ts_sessions_steps": (C.c_uint64, [vp]),
    "ts_sessions_totals": (None, [vp, vp]),
    "ts_sessions_consistent": (i32, [vp]),
}
for _name, (_res, _args) in RUN_SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype, _fn.argtypes = _res, _args


def _u(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


class Decoder:
    """A Qwen3-shaped decoder on one GPU: load weights, feed rows, read greedy ids."""

    def __init__(self, cfg: dict, slots: int, context: int, max_rows: int, page: int = 64, graphs: bool = True,
                 pdl: bool = False, qk_norm: bool = True):
        self.cfg = dict(cfg)
        c = DecoderConfig(cfg["layers"], cfg["hidden"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["ffn"],
                          cfg["vocab"], slots, context, page, max_rows, cfg.get("eps", 1e-6), cfg.get("theta", 1e6),
                          int(qk_norm), int(graphs), int(pdl))
        self._h = vp()
        check(lib.ts_decoder_create(C.byref(c), C.byref(self._h)))
        self.slots, self.context, self.max_rows, self.page = slots, context, max_rows, page
        self.pages = -(-context // page) if page else 0

    def close(self):
        if self._h:
            lib.ts_decoder_destroy(self._h)
            self._h = vp()

    def __del__(self):
        self.close()

    def load(self, name: str, array: np.ndarray):
        a = np.ascontiguousarray(array)
        check(lib.ts_decoder_load(self._h, name.encode(), a.ctypes.data_as(vp), a.nbytes))

    def load_all(self, named_arrays):
        for name, a in named_arrays:
            self.load(name, a)

    def set_table(self, table):
        t = _u(table)
        check(lib.ts_decoder_set_table(self._h, t.ctypes.data_as(vp), t.size))

    def copy_pages(self, copies, stream=None):
        """Applies a pool's planned page copies [(from, to, rows), ...] (kv.Pool.grow) to every layer's kept rows."""
        if not copies:
            return
        flat = np.ascontiguousarray(copies, dtype=np.uint32).reshape(-1, 3)
        check(lib.ts_decoder_copy_pages(self._h, flat.ctypes.data_as(vp), flat.shape[0], vp(stream or 0)))

    def step(self, tokens, slots, positions, out_rows=None, stream=None) -> np.ndarray:
        tokens, slots, positions = _u(tokens), _u(slots), _u(positions)
        rows = tokens.size
        orows = _u(out_rows) if out_rows is not None else None
        n_out = orows.size if orows is not None else rows
        ids = np.empty(n_out, np.uint32)
        check(lib.ts_decoder_step(self._h, tokens.ctypes.data_as(vp), slots.ctypes.data_as(vp),
                                  positions.ctypes.data_as(vp), rows,
                                  orows.ctypes.data_as(vp) if orows is not None else None, n_out,
                                  ids.ctypes.data_as(vp), vp(stream or 0)))
        return ids

    def run_resident(self, steps: int, stream=None):
        check(lib.ts_decoder_run_resident(self._h, steps, vp(stream or 0)))

    def read_ids(self, rows: int, stream=None) -> np.ndarray:
        ids = np.empty(rows, np.uint32)
        check(lib.ts_decoder_read_ids(self._h, ids.ctypes.data_as(vp), rows, vp(stream or 0)))
        return ids

    def read_hidden(self, rows: int, stream=None) -> np.ndarray:
        out = np.empty((rows, self.cfg["hidden"]), np.uint16)
        check(lib.ts_decoder_read_hidden(self._h, out.ctypes.data_as(vp), rows, vp(stream or 0)))
        return out

    def read_logits(self, n_out: int, stream=None) -> np.ndarray:
        out = np.empty((n_out, self.cfg["vocab"]), np.float32)
        check(lib.ts_decoder_read_logits(self._h, out.ctypes.data_as(vp), n_out, vp(stream or 0)))
        return out

    def launches_per_step(self, rows: int, keys: int) -> int:
        return int(lib.ts_decoder_launches_per_step(self._h, rows, keys))

    def prepare(self, rows: int, stream=None):
        """Captures the decode-step graphs of `rows` rows for every context bucket ahead of time."""
        check(lib.ts_decoder_prepare(self._h, rows, vp(stream or 0)))

    def use_step_kernel(self, on: bool) -> bool:
        """Chooses between the one persistent kernel per decode step and one launch per product; returns whether
        the persistent kernel exists for this decoder's shapes."""
        return bool(lib.ts_decoder_use_step_kernel(self._h, int(on)))

    def graphs(self) -> int:
        """Graphs captured so far (one per bucket of row counts, context bucket and kind of launch)."""
        return int(lib.ts_decoder_graphs(self._h))

    def graph_replays(self) -> int:
        return int(lib.ts_decoder_graph_replays(self._h))

    def profile(self, steps: int, stream=None) -> dict:
        """Per-kernel device milliseconds over `steps` resident decode launches: {name: (ms, intervals)}."""
        import json
        check(lib.ts_decoder_profile(self._h, steps, vp(stream or 0)))
        buf = C.create_string_buffer(1 << 14)
        check(lib.ts_decoder_take_profile(self._h, buf, len(buf)))
        return {k: (v[0], int(v[1])) for k, v in json.loads(buf.value.decode()).items()}

    # -- the decode loop a user drives (engine/engine/src/lib.rs:498-507 `generate`, greedy) --
    def prefill(self, prompts: list, chunk: int | None = None) -> np.ndarray:
        """Feeds every prompt (slot i = prompt i) and returns each slot's first generated id."""
        chunk = chunk or self.max_rows
        toks, slts, poss, last = [], [], [], {}
        for s, p in enumerate(prompts):
            for i, t in enumerate(p):
                toks.append(int(t)); slts.append(s); poss.append(i)
        first = np.zeros(len(prompts), np.uint32)
        n = len(toks)
        for a in range(0, n, chunk):
            b = min(n, a + chunk)
            # rows that end a prompt inside this chunk
            ends = [i - a for i in range(a, b) if (i + 1 == n or slts[i + 1] != slts[i])]
            if ends:
                ids = self.step(toks[a:b], slts[a:b], poss[a:b], out_rows=ends)
                for e, t in zip(ends, ids):
                    first[slts[a + e]] = t
            else:
                self.step(toks[a:b], slts[a:b], poss[a:b], out_rows=[b - a - 1])
        return first

    def generate(self, prompts: list, new: int) -> np.ndarray:
        """Greedy decode: returns [len(prompts), new] ids, fed and read through host memory each step."""
        out = np.zeros((len(prompts), new), np.uint32)
        cur = self.prefill(prompts)
        out[:, 0] = cur
        slots = np.arange(len(prompts), dtype=np.uint32)
        pos = np.array([len(p) for p in prompts], np.uint32)
        for t in range(1, new):
            cur = self.step(cur, slots, pos)
            out[:, t] = cur
            pos += 1
        return out
