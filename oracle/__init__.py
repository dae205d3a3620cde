"""TEST INFRASTRUCTURE ONLY: ctypes + numpy face of the CPU checker.

The C file beside this module restates tessera-interp (the reference's CPU
interpreter) op by op; this module loads it, adds the kept-row store
(engine/ir/interp/src/run.rs:90-177) and the model-level compositions
(engine/models/src/decoder.rs:58-84, 281-389) on top, in numpy.  Only tests, the
smoke check and the CPU-baseline leg of the benchmark may import it; the shipped
package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtessera_oracle.so")

ACC = {"f32": 0, "f16": 1, "bf16": 2}
ACT = {"gelu_tanh": 0, "silu": 1, "sigmoid": 2, "relu": 3, "softplus": 4, "exp": 5, "tanh": 6}
MASK = {"causal": 0, "bidirectional": 1, "within": 2, "back": 3}
PAIRS = {"adjacent": 0, "halves": 1}
KEPT = {"dense": 0, "interleaved": 1, "paged": 2, "paged16": 2}
PAGE = {"paged": 64, "paged16": 16}


def build(force: bool = False) -> str:
    """Compiles the checker with gcc when the shared object is missing or stale."""
    src = os.path.join(_HERE, "tessera_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libtessera_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.to_bf16_narrow.restype = C.c_uint16
        _lib.to_bf16_narrow.argtypes = [C.c_float]
        _lib.to_bf16_widen.restype = C.c_float
        _lib.to_bf16_widen.argtypes = [C.c_uint16]
        _lib.to_acc_sum.restype = C.c_float
        _lib.to_kept_row.restype = C.c_uint32
    return _lib


def _f(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _z(n) -> C.c_size_t:
    return C.c_size_t(int(n))


# ---- narrow floats -------------------------------------------------------

def bf16_bits(x) -> np.ndarray:
    x = _f(x)
    out = np.empty(x.shape, np.uint16)
    lib().to_bf16_narrow_array(_p(x), _p(out), _z(x.size))
    return out


def bf16_widen(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, np.float32)
    lib().to_bf16_widen_array(_p(bits), _p(out), _z(bits.size))
    return out


def bf16_round(x) -> np.ndarray:
    x = _f(x)
    out = np.empty_like(x)
    lib().to_bf16_round_array(_p(x), _p(out), _z(x.size))
    return out


def acc_sum(values, acc="f32") -> float:
    v = _f(values)
    return float(lib().to_acc_sum(C.c_int(ACC[acc]), _p(v), _z(v.size)))


class Noise:
    """engine/ir/testkit/src/noise.rs:1-10."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed)

    def draw(self, *shape) -> np.ndarray:
        out = np.empty(shape, np.float32)
        lib().to_noise(C.byref(self.state), _p(out), _z(out.size))
        return out


# ---- ops -----------------------------------------------------------------

def matmul(x, w, acc="f32") -> np.ndarray:
    """x [..., k] times w [n, k] transposed; w float32 or bf16 bits (uint16)."""
    w = np.ascontiguousarray(w)
    x = _f(x)
    k = x.shape[-1]
    m = x.size // k
    n = w.shape[0]
    out = np.empty(x.shape[:-1] + (n,), np.float32)
    if w.dtype == np.uint16:
        assert acc == "f32"
        lib().to_matmul_bf16w(_p(x), _p(w), _p(out), _z(m), _z(n), _z(k))
    else:
        w = _f(w)
        lib().to_matmul(C.c_int(ACC[acc]), _p(x), _p(w), _p(out), _z(m), _z(n), _z(k))
    return out


def q8_0_pack(data) -> np.ndarray:
    """engine/ir/mem/src/block.rs Block::pack for Q8_0: bytes of an f16 scale and 32 signed codes a block."""
    data = _f(data).reshape(-1)
    lib().to_q8_0_bytes.restype = C.c_size_t
    out = np.zeros(lib().to_q8_0_bytes(_z(data.size)), np.uint8)
    lib().to_q8_0_pack(_p(data), _z(data.size), _p(out))
    return out


def q8_0_unpack(packed, elements) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty(elements, np.float32)
    lib().to_q8_0_unpack(_p(packed), _z(elements), _p(out))
    return out


def matmul_q8_0(x, packed, n) -> np.ndarray:
    """x [m, k] times a Q8_0 matrix [n, k] transposed, every output by Form::dot (block.rs:204-221)."""
    x = _f(x)
    k = x.shape[-1]
    m = x.size // k
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    assert k % 32 == 0 and packed.size == n * (k // 32) * 34
    out = np.empty(x.shape[:-1] + (n,), np.float32)
    lib().to_matmul_q8_0(_p(x), _p(packed), _p(out), _z(m), _z(n), _z(k))
    return out


def matmul_picked(x, table, ids, first=0) -> np.ndarray:
    """engine/ir/interp/src/cpu.rs:89-105: x [m, k], table [experts, n, k], ids [rows]."""
    x, table, ids = _f(x), _f(table), _u(ids)
    experts, n, k = table.shape
    m = x.size // k
    rows = ids.size
    out = np.empty(ids.shape + (n,), np.float32)
    lib().to_matmul_picked(_p(x), _p(table), _p(ids), _p(out), _z(m), _z(rows), _z(experts),
                           _z(n), _z(k), _z(first))
    return out


def act(x, name) -> np.ndarray:
    out = _f(x).copy()
    lib().to_act(C.c_int(ACT[name]), _p(out), _z(out.size))
    return out


def softmax(x, acc="f32") -> np.ndarray:
    out = _f(x).copy()
    width = out.shape[-1]
    lib().to_softmax(C.c_int(ACC[acc]), _p(out), _z(out.size // max(width, 1)), _z(width))
    return out


def rms_norm(x, w=None, eps=1e-6, acc="f32") -> np.ndarray:
    out = _f(x).copy()
    width = out.shape[-1]
    wp = _p(_f(w)) if w is not None else None
    lib().to_rms_norm(C.c_int(ACC[acc]), _p(out), wp, _z(out.size // width), _z(width), C.c_float(eps))
    return out


def rope(x, positions, theta, pairs="halves", turned=None) -> np.ndarray:
    """x [positions..., heads, width]; one position per leading row."""
    out = _f(x).copy()
    positions = _u(positions)
    width = out.shape[-1]
    span = out.size // max(positions.size, 1)
    lib().to_rope(_p(out), _p(positions), _z(positions.size), _z(span), _z(width), C.c_float(theta),
                  C.c_int(PAIRS[pairs]), _z(width if turned is None else turned))
    return out


def hadamard(x, block) -> np.ndarray:
    out = _f(x).copy()
    lib().to_hadamard(_p(out), _z(out.size), _z(block))
    return out


def mean(x, axis, weights=None, acc="f32") -> np.ndarray:
    x = _f(x)
    outer = int(np.prod(x.shape[:axis], dtype=np.int64))
    count = x.shape[axis]
    inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    out = np.empty(x.shape[:axis] + x.shape[axis + 1:], np.float32)
    wp = _p(_f(weights)) if weights is not None else None
    lib().to_mean(C.c_int(ACC[acc]), _p(x), wp, _p(out), _z(outer), _z(count), _z(inner))
    return out


def take(x, ids) -> np.ndarray:
    x, ids = _f(x), _u(ids)
    width = x.shape[-1]
    rows = x.size // width
    picks = ids.size // max(rows, 1)
    out = np.empty(ids.shape, np.float32)
    lib().to_take(_p(x), _p(ids), _p(out), _z(rows), _z(width), _z(picks))
    return out


def gather(table, ids, first=0) -> np.ndarray:
    table = np.ascontiguousarray(table)
    ids = _u(ids)
    rows = table.shape[0]
    row_bytes = table.nbytes // max(rows, 1)
    out = np.empty(ids.shape + table.shape[1:], table.dtype)
    lib().to_gather(_p(table), _p(ids), _p(out), _z(rows), _z(row_bytes), _z(ids.size), _z(first))
    return out


def top_k(x, k) -> np.ndarray:
    x = _f(x)
    width = x.shape[-1]
    rows = x.size // max(width, 1)
    out = np.empty(x.shape[:-1] + (k,), np.uint32)
    lib().to_top_k(_p(x), _p(out), _z(rows), _z(width), _z(k))
    return out


def top_k_numpy(x, k) -> np.ndarray:
    """Numpy twin of top_k (engine/ir/interp/src/run.rs:577-591), for cross-checking."""
    x = np.asarray(x, np.float32)
    width = x.shape[-1]
    flat = x.reshape(-1, width)
    out = np.full((flat.shape[0], k), width, np.uint32)
    for r, row in enumerate(flat):
        keep = np.nonzero(row > -np.inf)[0]
        # stable descending: sort on the negated value, ties keep the lower index
        vals = -row[keep]
        vals = np.where(vals == 0.0, 0.0, vals)
        order = keep[np.argsort(vals, kind="stable")]
        out[r, : min(k, order.size)] = order[:k]
    return out.reshape(x.shape[:-1] + (k,))


def _mask(mask):
    if isinstance(mask, tuple):
        return MASK[mask[0]], int(mask[1])
    return MASK[mask], 0


def attend(q, k, v, mask="causal", scale=1.0, acc="f32") -> np.ndarray:
    """engine/ir/interp/src/cpu.rs:171-225.  mask: 'causal' | 'bidirectional' | ('within', n) | ('back', n)."""
    q, k, v = _f(q), _f(k), _f(v)
    seqs, queries, heads, d = q.shape
    keys, kv_heads, dv = k.shape[1], k.shape[2], v.shape[3]
    out = np.empty((seqs, queries, heads, dv), np.float32)
    kind, n = _mask(mask)
    rc = lib().to_attend(C.c_int(ACC[acc]), C.c_int(kind), _z(n), C.c_float(scale), _p(q), _p(k), _p(v),
                         _p(out), _z(seqs), _z(queries), _z(keys), _z(heads), _z(kv_heads), _z(d), _z(dv))
    if rc:
        raise ValueError(f"{queries} queries, {keys} keys")
    return out


def attend_rows(q, k, v, slots, positions, mask="causal", scale=1.0, acc="f32") -> np.ndarray:
    """engine/ir/interp/src/cpu.rs:292-351 over a dense store [seqs, keys, kv_heads, d]."""
    q, k, v = _f(q), _f(k), _f(v)
    slots, positions = _u(slots), _u(positions)
    rows, heads, d = q.shape
    keys, kv_heads, dv = k.shape[1], k.shape[2], v.shape[3]
    if slots.size and int(slots.max()) >= k.shape[0]:
        raise ValueError("slot outside the store")
    out = np.empty((rows, heads, dv), np.float32)
    kind, n = _mask(mask)
    rc = lib().to_attend_rows(C.c_int(ACC[acc]), C.c_int(kind), _z(n), C.c_float(scale), _p(q), _p(k),
                              _p(v), _p(slots), _p(positions), _p(out), _z(rows), _z(keys), _z(heads),
                              _z(kv_heads), _z(d), _z(dv))
    if rc:
        raise ValueError(f"row {rc - 1} is past {keys} keys")
    return out


def kept_row(layout, slot, position, scalar, table=None) -> int:
    """engine/plan/codegen/src/kept.rs:135-194.  scalar = kept_stride | kept_slots | kept_pages."""
    t = _u(table if table is not None else [0])
    return int(lib().to_kept_row(C.c_int(KEPT[layout]), C.c_uint32(slot), C.c_uint32(position),
                                 C.c_uint32(scalar), C.c_uint32(PAGE.get(layout, 1)), _p(t)))


def kept_rows(layout, slots, positions, scalar, table=None) -> np.ndarray:
    return np.array([kept_row(layout, int(s), int(p), scalar, table) for s, p in zip(slots, positions)],
                    np.uint32)


class Store:
    """One kept tensor, held between launches: engine/ir/interp/src/run.rs:104-177.

    Rows stay where they were and the store only grows; a launch is refused when a
    row sits outside `seqs` x max(held, ctx) or reads a position never written.
    """

    def __init__(self):
        self.kept = None  # [seqs, len, ...]
        self.written = None  # [seqs, len]

    def __len__(self):
        return 0 if self.kept is None else self.kept.shape[1]

    def append(self, rows, slots, positions, seqs, ctx) -> np.ndarray:
        rows = _f(rows)
        slots, positions = _u(slots), _u(positions)
        tail = rows.shape[1:]
        had = len(self)
        length = max(had, ctx)
        all_ = np.zeros((seqs, length) + tail, np.float32)
        written = np.zeros((seqs, length), bool)
        if self.kept is not None:
            all_[:, :had] = self.kept[:seqs]
            written[:, :had] = self.written[:seqs]
        for r in range(rows.shape[0]):
            s, p = int(slots[r]), int(positions[r])
            if s >= seqs or p >= length:
                raise ValueError(f"row {r} at slot {s}, position {p} is outside the kept rows")
            all_[s, p] = rows[r]
            written[s, p] = True
        for r in range(rows.shape[0]):
            s, p = int(slots[r]), int(positions[r])
            gaps = np.nonzero(~written[s, :p])[0]
            if gaps.size:
                raise ValueError(f"row {r} at slot {s} reads unwritten position {int(gaps[0])}")
        self.kept, self.written = all_, written
        return all_[:, :ctx].copy()


# ---- model-level compositions -------------------------------------------

def swiglu(h, gate, up, down, round_inner=False) -> np.ndarray:
    inner = act(matmul(h, gate), "silu") * matmul(h, up)
    if round_inner:
        inner = bf16_round(inner)
    return matmul(inner, down)


def moe_block(h, router, w_in, w_out, top, first=0, count=None, round_inner=False):
    """engine/models/src/decoder.rs:70-84.  h [rows, H]; router [E, H]; w_in [E, 2F, H]
    (gate rows then up rows); w_out [E, H, F].  Weights as float32 (bf16-valued).
    Returns (y, ids, gates)."""
    h = _f(h)
    rows = h.shape[0]
    experts, two_f, _ = w_in.shape
    ffn = two_f // 2
    count = experts if count is None else count
    scores = matmul(h, router)
    ids = top_k(scores, top)
    gates = softmax(take(scores, ids))
    flat = ids.reshape(-1)
    gate = act(matmul_picked(h, w_in[first:first + count, :ffn], flat, first), "silu")
    inner = gate * matmul_picked(h, w_in[first:first + count, ffn:], flat, first)
    if round_inner:
        inner = bf16_round(inner)
    # one output row per pick, each on its own expert
    out = matmul_picked(inner, w_out[first:first + count], flat, first)
    y = mean(out.reshape(rows, top, -1), 1, weights=gates)
    return y, ids, gates


class DecoderConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in
                ("layers", "hidden", "heads", "kv_heads", "head_dim", "ffn", "vocab", "context", "slots")]
    _fields_ += [("eps", C.c_float), ("theta", C.c_float)]


class _DecoderWeights(C.Structure):
    _fields_ = [("embed", C.c_void_p)] + [(n, C.POINTER(C.c_void_p)) for n in
                ("q", "k", "v", "o", "gate", "up", "down", "ln1", "ln2", "q_norm", "k_norm")]
    _fields_ += [("norm", C.c_void_p)]


class Decoder:
    """The Qwen3-shaped decoder of engine/models/src/decoder.rs:281-389 over a dense kept store.

    weights: dict with 'embed' (uint16 [vocab, hidden]), 'norm' (float32 [hidden]) and
    per-layer lists 'q','k','v','o','gate','up','down' (uint16 bf16 bits, [out, in]) and
    'ln1','ln2','q_norm','k_norm' (float32).
    """

    def __init__(self, cfg: dict, weights: dict):
        self.cfg = DecoderConfig(**cfg)
        self.w = weights
        L = self.cfg.layers
        self._keep = []
        sw = _DecoderWeights()
        sw.embed = weights["embed"].ctypes.data
        sw.norm = weights["norm"].ctypes.data
        for name in ("q", "k", "v", "o", "gate", "up", "down", "ln1", "ln2", "q_norm", "k_norm"):
            arr = (C.c_void_p * L)(*[weights[name][l].ctypes.data for l in range(L)])
            self._keep.append(arr)
            setattr(sw, name, C.cast(arr, C.POINTER(C.c_void_p)))
        self._sw = sw
        kw = self.cfg.kv_heads * self.cfg.head_dim
        shape = (self.cfg.slots, self.cfg.context, kw)
        self.keys = [np.zeros(shape, np.float32) for _ in range(L)]
        self.values = [np.zeros(shape, np.float32) for _ in range(L)]
        self._kp = (C.c_void_p * L)(*[a.ctypes.data for a in self.keys])
        self._vp = (C.c_void_p * L)(*[a.ctypes.data for a in self.values])

    def step(self, tokens, slots, positions, want_logits=False, want_hidden=False):
        tokens, slots, positions = _u(tokens), _u(slots), _u(positions)
        rows = tokens.size
        ids = np.empty(rows, np.uint32)
        logits = np.empty((rows, self.cfg.vocab), np.float32) if want_logits else None
        hidden = np.empty((rows, self.cfg.hidden), np.float32) if want_hidden else None
        rc = lib().to_decoder_step(C.byref(self.cfg), C.byref(self._sw), self._kp, self._vp, _p(tokens),
                                   _p(slots), _p(positions), _z(rows),
                                   _p(hidden) if hidden is not None else None,
                                   _p(logits) if logits is not None else None, _p(ids))
        if rc:
            raise ValueError("a row sits outside the kept store")
        return ids, logits, hidden


# ---- the timed CPU baseline (cpu_rules.c) ----------------------------------

_RULES_PATH = os.path.join(_HERE, "libtessera_cpu_rules.so")
_rules = None


def build_rules(force: bool = False) -> str:
    src = os.path.join(_HERE, "cpu_rules.c")
    if force or not os.path.exists(_RULES_PATH) or os.path.getmtime(_RULES_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libtessera_cpu_rules.so"], stdout=subprocess.DEVNULL)
    return _RULES_PATH


def rules() -> C.CDLL:
    global _rules
    if _rules is None:
        _rules = C.CDLL(build_rules())
        _rules.cr_threads.restype = C.c_int
    return _rules


class CpuRulesDecoder:
    """The reference's native CPU rules restated (threads + SIMD), for the timed baseline:
    f32 activations, bf16 weights widened per block, dense f32 kept rows."""

    def __init__(self, cfg: dict, weights: dict):
        self.cfg = DecoderConfig(**cfg)
        L = self.cfg.layers
        self._keep = []
        sw = _DecoderWeights()
        sw.embed = weights["embed"].ctypes.data
        sw.norm = weights["norm"].ctypes.data
        for name in ("q", "k", "v", "o", "gate", "up", "down", "ln1", "ln2", "q_norm", "k_norm"):
            arr = (C.c_void_p * L)(*[weights[name][l].ctypes.data for l in range(L)])
            self._keep.append(arr)
            setattr(sw, name, C.cast(arr, C.POINTER(C.c_void_p)))
        self._sw = sw
        self.w = weights
        kw = self.cfg.kv_heads * self.cfg.head_dim
        shape = (self.cfg.slots, self.cfg.context, kw)
        self.keys = [np.zeros(shape, np.float32) for _ in range(L)]
        self.values = [np.zeros(shape, np.float32) for _ in range(L)]
        self._kp = (C.c_void_p * L)(*[a.ctypes.data for a in self.keys])
        self._vp = (C.c_void_p * L)(*[a.ctypes.data for a in self.values])
        try:
            cores = len(os.sched_getaffinity(0))
        except AttributeError:
            cores = os.cpu_count() or 1
        rules().cr_set_threads(C.c_int(cores))  # torchrun exports OMP_NUM_THREADS=1; use every host core
        self.threads = int(rules().cr_threads())

    def step(self, tokens, slots, positions) -> np.ndarray:
        tokens, slots, positions = _u(tokens), _u(slots), _u(positions)
        ids = np.empty(tokens.size, np.uint32)
        rules().cr_decoder_step(C.byref(self.cfg), C.byref(self._sw), self._kp, self._vp, _p(tokens), _p(slots),
                                _p(positions), _z(tokens.size), _p(ids))
        return ids
