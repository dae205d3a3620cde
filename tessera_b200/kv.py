"""Python face of the host page pool (include/tessera_b200_kv.h; tessera-kv's Pool restated)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import lib

u32, u64, vp, i32 = C.c_uint32, C.c_uint64, C.c_void_p, C.c_int


class Run(C.Structure):
    _fields_ = [("at", u32), ("generation", u32)]

    def __eq__(self, other):
        return isinstance(other, Run) and (self.at, self.generation) == (other.at, other.generation)

    def __hash__(self):
        return hash((self.at, self.generation))

    def __repr__(self):
        return f"Run(at={self.at}, generation={self.generation})"


class PageCopy(C.Structure):
    _fields_ = [("src", u32), ("dst", u32), ("rows", u32)]


class Stats(C.Structure):
    _fields_ = [(n, u64) for n in ("size", "active", "worst", "live_runs", "kept_runs")]


class Totals(C.Structure):
    """engine/engine/src/kept.rs:14-25."""
    _fields_ = [("pool", Stats), ("hits", u64), ("misses", u64)]


class _Begin(C.Structure):
    _fields_ = [("skip", u64), ("lcp", u64), ("why", i32)]


KV_SIGNATURES = {
    "ts_kv_pool_new": (vp, [u32, u32]),
    "ts_kv_pool_free": (None, [vp]),
    "ts_kv_last_detail": (u64, [vp]),
    "ts_kv_reserve": (i32, [vp, u64, u64, u64, C.POINTER(Run)]),
    "ts_kv_fork": (i32, [vp, Run, u64, u64, C.POINTER(Run)]),
    "ts_kv_grow": (i32, [vp, Run, u64, C.POINTER(PageCopy), u32, C.POINTER(u32)]),
    "ts_kv_truncate": (i32, [vp, Run, u64]),
    "ts_kv_retain": (i32, [vp, Run]),
    "ts_kv_adopt": (i32, [vp, Run, u64, u64, C.POINTER(Run)]),
    "ts_kv_release": (i32, [vp, Run]),
    "ts_kv_pages": (i32, [vp, Run, vp, u32, C.POINTER(u32)]),
    "ts_kv_rows": (i32, [vp, Run, C.POINTER(u64)]),
    "ts_kv_tag": (i32, [vp, Run, C.POINTER(u64)]),
    "ts_kv_spare": (u64, [vp]),
    "ts_kv_promised": (u64, [vp]),
    "ts_kv_get_stats": (None, [vp, C.POINTER(Stats)]),
    "ts_kv_digest": (u64, [vp]),
    "ts_kv_consistent": (i32, [vp]),
    "ts_kv_fill_table": (i32, [vp, Run, vp, u32, u32]),
    "ts_kv_copy_pages": (i32, [vp, C.POINTER(PageCopy), u32, u32, C.c_size_t, vp]),
    "ts_kv_begin_rows": (None, [vp, u64, u64, vp, u64, u64, u64, C.POINTER(_Begin)]),
    "ts_kv_prefixes_new": (vp, [u64]),
    "ts_kv_prefixes_free": (None, [vp]),
    "ts_kv_prefixes_keep": (i32, [vp, Run, vp, u64, u64]),
    "ts_kv_prefixes_find": (i32, [vp, vp, u64, vp, u64, u64, C.POINTER(Run), C.POINTER(u64), C.POINTER(i32)]),
    "ts_kv_prefixes_len": (u64, [vp]),
    "ts_kept_slots_dense": (vp, [u32, u32]),
    "ts_kept_slots_paged": (vp, [u32, u32, u32, u32]),
    "ts_kept_slots_free": (None, [vp]),
    "ts_kept_slots_admit": (i32, [vp, vp, u64, u64, C.POINTER(u32), C.POINTER(u64), C.POINTER(i32)]),
    "ts_kept_slots_grow": (i32, [vp, u32, u64, vp, u32, C.POINTER(u32)]),
    "ts_kept_slots_finish": (i32, [vp, u32, vp, u64]),
    "ts_kept_slots_totals": (None, [vp, vp]),
    "ts_kept_slots_pool": (vp, [vp]),
}
for _name, (_res, _args) in KV_SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype, _fn.argtypes = _res, _args

ERRORS = {1: "NoRoom", 2: "PastWorst", 3: "PastSource", 4: "Live", 5: "Retained", 6: "Unknown", 7: "BadArgument",
          8: "RowPlace", 9: "SharedPage"}


class PoolError(Exception):
    """engine/ir/kv/src/pool.rs:25-40: every error leaves the pool as it was."""

    def __init__(self, code: int, detail: int):
        super().__init__(f"{ERRORS.get(code, code)}({detail})")
        self.kind, self.detail = ERRORS.get(code, str(code)), detail


class Pool:
    def __init__(self, pages: int, page: int):
        self._h = lib.ts_kv_pool_new(pages, page)
        self.page = page

    def __del__(self):
        if getattr(self, "_h", None):
            lib.ts_kv_pool_free(self._h)
            self._h = None

    def _check(self, code):
        if code:
            raise PoolError(code, int(lib.ts_kv_last_detail(self._h)))

    def reserve(self, tag: int, rows: int, worst: int) -> Run:
        out = Run()
        self._check(lib.ts_kv_reserve(self._h, tag, rows, worst, C.byref(out)))
        return out

    def fork(self, source: Run, rows: int, worst: int) -> Run:
        out = Run()
        self._check(lib.ts_kv_fork(self._h, source, rows, worst, C.byref(out)))
        return out

    def grow(self, run: Run, rows: int) -> list:
        copies, n = (PageCopy * 2)(), u32(0)
        self._check(lib.ts_kv_grow(self._h, run, rows, copies, 2, C.byref(n)))
        return [(c.src, c.dst, c.rows) for c in copies[: n.value]]

    def truncate(self, run: Run, rows: int):
        self._check(lib.ts_kv_truncate(self._h, run, rows))

    def retain(self, run: Run):
        self._check(lib.ts_kv_retain(self._h, run))

    def adopt(self, run: Run, rows: int, worst: int) -> Run:
        out = Run()
        self._check(lib.ts_kv_adopt(self._h, run, rows, worst, C.byref(out)))
        return out

    def release(self, run: Run):
        self._check(lib.ts_kv_release(self._h, run))

    def pages(self, run: Run) -> list:
        n = u32(0)
        self._check(lib.ts_kv_pages(self._h, run, None, 0, C.byref(n)))
        buf = (u32 * max(n.value, 1))()
        self._check(lib.ts_kv_pages(self._h, run, buf, n.value, C.byref(n)))
        return list(buf[: n.value])

    def rows(self, run: Run) -> int:
        out = u64(0)
        self._check(lib.ts_kv_rows(self._h, run, C.byref(out)))
        return out.value

    def stats(self) -> Stats:
        s = Stats()
        lib.ts_kv_get_stats(self._h, C.byref(s))
        return s

    def spare(self) -> int:
        return int(lib.ts_kv_spare(self._h))

    def promised(self) -> int:
        return int(lib.ts_kv_promised(self._h))

    def digest(self) -> int:
        return int(lib.ts_kv_digest(self._h))

    def consistent(self) -> bool:
        return bool(lib.ts_kv_consistent(self._h))

    def fill_table(self, run: Run, table: np.ndarray, slot: int, kept_pages: int):
        assert table.dtype == np.uint32 and table.flags.c_contiguous
        self._check(lib.ts_kv_fill_table(self._h, run, table.ctypes.data_as(vp), slot, kept_pages))


WHY = ("First", "NoLcp", "Grid", "Hit")   # engine/ir/kv/src/reuse.rs:3-14


def _ids(tokens) -> np.ndarray:
    return np.ascontiguousarray(tokens, dtype=np.uint32)


def begin(history, valid: int, prompt, limit: int, grid: int) -> tuple:
    """(skip, lcp, why): the rows of `prompt` that `valid` kept rows spare (engine/ir/kv/src/reuse.rs:24-37)."""
    h, p = _ids(history), _ids(prompt)
    out = _Begin()
    lib.ts_kv_begin_rows(h.ctypes.data_as(vp), h.size, valid, p.ctypes.data_as(vp), p.size, limit, grid, C.byref(out))
    return int(out.skip), int(out.lcp), WHY[out.why]


class Prefixes:
    """The tokens of retained runs, oldest first (engine/ir/kv/src/prefix.rs:11-55)."""

    def __init__(self, grid: int):
        self._h = lib.ts_kv_prefixes_new(grid)

    def __del__(self):
        if getattr(self, "_h", None):
            lib.ts_kv_prefixes_free(self._h)
            self._h = None

    def __len__(self):
        return int(lib.ts_kv_prefixes_len(self._h))

    def keep(self, run: Run, history, valid: int):
        h = _ids(history)
        code = lib.ts_kv_prefixes_keep(self._h, run, h.ctypes.data_as(vp), h.size, valid)
        if code:
            raise PoolError(code, 0)

    def find(self, pool: "Pool", tag: int, prompt, limit: int):
        """(run, skip) of the newest run with the longest skip, or None."""
        p = _ids(prompt)
        run, skip, found = Run(), u64(0), i32(0)
        code = lib.ts_kv_prefixes_find(self._h, pool._h, tag, p.ctypes.data_as(vp), p.size, limit, C.byref(run),
                                       C.byref(skip), C.byref(found))
        if code:
            raise PoolError(code, 0)
        return (run, int(skip.value)) if found.value else None


class KeptSlots:
    """Which slot a prompt gets and how many of its rows the kept rows spare: the engine's `Kept`
    (engine/engine/src/kept.rs:27-159) over the pool and the prefix index."""

    def __init__(self, slots: int, context: int, pages: int | None = None, page: int | None = None):
        """Dense (each slot one page of `context` rows) unless `pages` and `page` are given (slots share whole pages)."""
        self.paged = pages is not None
        self._h = lib.ts_kept_slots_paged(slots, context, pages, page) if self.paged else lib.ts_kept_slots_dense(slots, context)
        if not self._h:
            raise ValueError("slots, context, pages and page must be positive")
        self.capacity = -(-context // page) if self.paged else 1

    def __del__(self):
        if getattr(self, "_h", None):
            lib.ts_kept_slots_free(self._h)
            self._h = None

    def admit(self, prompt, limit: int):
        """(slot, skip), or None while no slot or room is free (kept.rs:69-106)."""
        p = _ids(prompt)
        slot, skip, ok = u32(0), u64(0), i32(0)
        code = lib.ts_kept_slots_admit(self._h, p.ctypes.data_as(vp), p.size, limit, C.byref(slot), C.byref(skip), C.byref(ok))
        if code:
            raise PoolError(code, 0)
        return (int(slot.value), int(skip.value)) if ok.value else None

    def grow(self, slot: int, rows: int):
        """Paged: the slot's pages if its lane lacks some, else None (kept.rs:133-148)."""
        pages, n = (u32 * self.capacity)(), u32(0)
        code = lib.ts_kept_slots_grow(self._h, slot, rows, pages, self.capacity, C.byref(n))
        if code:
            raise PoolError(code, int(lib.ts_kv_last_detail(lib.ts_kept_slots_pool(self._h))))
        return list(pages[: n.value]) if n.value else None

    def finish(self, slot: int, history):
        h = _ids(history)
        code = lib.ts_kept_slots_finish(self._h, slot, h.ctypes.data_as(vp), h.size)
        if code:
            raise PoolError(code, 0)

    def totals(self) -> Totals:
        t = Totals()
        lib.ts_kept_slots_totals(self._h, C.byref(t))
        return t

    def consistent(self) -> bool:
        """The pool's self-check (page counts, owners and promises add up)."""
        return bool(lib.ts_kv_consistent(lib.ts_kept_slots_pool(self._h)))
