"""Each C-ABI entry point over torch CUDA tensors.

torch is plumbing here: device memory and the current stream.  Every function passes raw
device pointers to libtessera_b200.so and raises TesseraError on a non-zero status.  A call
with tensors that are not on a CUDA device is refused; there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import EPILOGUE, KEPT_KIND, KEPT_PAGE, LINEAR_PATH, TS_BF16, TS_F32, TsKept, check, lib

_workspaces: dict = {}


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise _lib.TesseraError(_lib.TS_ERR_BAD_INPUT, "tensors must live on a CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise _lib.TesseraError(_lib.TS_ERR_BAD_INPUT, "tensors must be contiguous")
    return C.c_void_p(t.data_ptr())


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return TS_BF16
    if dtype == torch.float32:
        return TS_F32
    raise _lib.TesseraError(_lib.TS_ERR_BAD_INPUT, f"dtype {dtype} is not bf16 or f32")


def workspace(nbytes: int, device) -> torch.Tensor | None:
    """A caller-owned scratch buffer, grown on demand and reused: one per device and stream, so that launches on
    two streams that may run side by side never share scratch."""
    if nbytes == 0:
        return None
    dev = torch.device(device)
    key = (dev.index or 0, torch.cuda.current_stream(dev).cuda_stream if dev.type == "cuda" else 0)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def set_pdl(enabled: bool) -> None:
    check(lib.ts_set_pdl(1 if enabled else 0))


def device_status() -> int:
    return lib.ts_device_status()


def linear(x, w, a0=None, *, epilogue="none", scale=1.0, out_dtype=torch.bfloat16, path="auto", out=None):
    """out[m, n] = sum_k x[m, k] w[n, k] (+ epilogue): ts_linear_bf16."""
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    gated = epilogue in ("swiglu", "geglu")
    if out is None:
        out = torch.empty((m, n // 2 if gated else n), dtype=out_dtype, device=x.device)
    nbytes = lib.ts_linear_workspace_bytes(m, n, k, EPILOGUE[epilogue], LINEAR_PATH[path])
    ws = workspace(nbytes, x.device)
    check(lib.ts_linear_bf16(_ptr(x), _ptr(w), _ptr(a0), _ptr(out), m, n, k, EPILOGUE[epilogue], scale,
                             _dtype_code(out.dtype), LINEAR_PATH[path], _ptr(ws), nbytes, _stream()))
    return out


def router_scores(x, router):
    """A router's scores, f32 [rows, experts], every sum in the interpreter's order (path "ordered"): top-k over
    them picks the interpreter's experts, near ties included."""
    return linear(x, router, out_dtype=torch.float32, path="ordered")


def q8_0_pack(w: torch.Tensor) -> torch.Tensor:
    """A float matrix [n, k] (k a multiple of 32) in the reference's Q8_0 block form: uint8 [n, k / 32 * 34], on the
    device of `w` (packed on the host by ts_q8_0_pack)."""
    import numpy as np
    n, k = w.shape
    assert k % 32 == 0
    data = np.ascontiguousarray(w.detach().float().cpu().numpy())
    out = np.zeros(lib.ts_q8_0_bytes(data.size), np.uint8)
    check(lib.ts_q8_0_pack(data.ctypes.data_as(C.c_void_p), data.size, out.ctypes.data_as(C.c_void_p)))
    return torch.from_numpy(out.reshape(n, k // 32 * 34)).to(w.device)


def linear_q8_0(x, w_q8, a0=None, *, epilogue="none", scale=1.0, out_dtype=torch.bfloat16, out=None):
    """out[m, n] = sum_k x[m, k] w[n, k] over Q8_0 weights (uint8 [n, k / 32 * 34]): ts_linear_q8_0."""
    m, k = x.shape
    n = w_q8.shape[0]
    assert w_q8.shape[1] == k // 32 * 34
    out_n = n // 2 if epilogue in ("swiglu", "geglu") else n
    if out is None:
        out = torch.empty((m, out_n), dtype=out_dtype, device=x.device)
    nbytes = lib.ts_linear_q8_0_workspace_bytes(m, n, k)
    ws = workspace(nbytes, x.device)
    check(lib.ts_linear_q8_0(_ptr(x), _ptr(w_q8), _ptr(a0), _ptr(out), m, n, k, EPILOGUE[epilogue], scale, _dtype_code(out_dtype),
                             _ptr(ws), nbytes, _stream()))
    return out


def linear_fused(x, w, a0=None, *, epilogue="none", scale=1.0, out_dtype=torch.bfloat16, out=None, rows=None,
                 next_gain=None):
    """ts_linear_fused_bf16.  rows = (partial sums of squares f32 [m, parts], eps): x is bf16(row * gain) and the
    output rows get the 1/rms factor.  next_gain (f32 [n]): also returns xs = bf16(out * next_gain) and the
    per-tile sums of squares of the output rows, f32 [m, ts_linear_sumsq_parts]: (out, xs, ss)."""
    from ._lib import TsLinearFused
    m, k = x.shape
    n = w.shape[0]
    gated = epilogue in ("swiglu", "geglu")
    if out is None:
        out = torch.empty((m, n // 2 if gated else n), dtype=out_dtype, device=w.device)
    f = TsLinearFused()
    if rows is not None:
        ss_in, eps = rows
        assert ss_in.dtype == torch.float32 and ss_in.is_contiguous() and ss_in.shape[0] == m
        f.row_ss, f.row_parts, f.row_eps = ss_in.data_ptr(), ss_in.shape[1], eps
    xs = ss = None
    if next_gain is not None:
        parts = lib.ts_linear_sumsq_parts(m, n, k, EPILOGUE[epilogue])
        if parts == 0:
            raise ValueError(f"no sums of squares from a linear of m={m} n={n} k={k}")
        ss = torch.empty((m, parts), dtype=torch.float32, device=w.device)
        xs = torch.empty((m, n), dtype=torch.bfloat16, device=w.device)
        assert next_gain.dtype == torch.float32 and next_gain.numel() == n
        f.ss_out, f.xs_out, f.xs_gain = ss.data_ptr(), xs.data_ptr(), next_gain.data_ptr()
    check(lib.ts_linear_fused_bf16(_ptr(x), _ptr(w), _ptr(a0), _ptr(out), m, n, k, EPILOGUE[epilogue], scale,
                                   _dtype_code(out.dtype), C.byref(f), _stream()))
    return (out, xs, ss) if next_gain is not None else out


@dataclass
class Kept:
    """Where a slot's row at a position lives (engine/plan/codegen/src/kept.rs:8-24)."""
    layout: str            # dense | interleaved | paged | paged16
    scalar: int            # kept_stride | kept_slots | kept_pages
    table: torch.Tensor | None = None  # u32 (stored as int32) [slots * kept_pages]
    rows: int = 0
    page: int | None = None  # rows per page when it is neither 64 ("paged") nor 16 ("paged16")

    def c(self) -> TsKept:
        t = self.table
        return TsKept(KEPT_KIND[self.layout], self.page or KEPT_PAGE[self.layout], self.scalar,
                      t.data_ptr() if t is not None else None, t.numel() if t is not None else 0, self.rows)


def attend_rows(q, k_rows, v_rows, slots, positions, kept: Kept, keys: int, *, scale: float, back=0xFFFFFFFF,
                out=None):
    """Ragged causal attention over kept rows: ts_attend_rows_bf16."""
    rows, heads, width = q.shape
    kv_heads = k_rows.shape[-2]
    if out is None:
        out = torch.empty_like(q)
    nbytes = lib.ts_attend_rows_workspace_bytes(rows, keys, heads, kv_heads, width)
    ws = workspace(nbytes, q.device)
    kc = kept.c()
    if kc.rows == 0:
        kc.rows = k_rows.numel() // (kv_heads * width)
    check(lib.ts_attend_rows_bf16(_ptr(q), _ptr(k_rows), _ptr(v_rows), _ptr(out), _ptr(slots), _ptr(positions),
                                  C.byref(kc), rows, keys, heads, kv_heads, width, back, scale, _ptr(ws), nbytes,
                                  _stream()))
    return out


def attend_rows_append(qkv, q_norm, k_norm, inv_freq, k_rows, v_rows, slots, positions, kept: Kept, keys: int, heads: int,
                       *, eps: float, scale: float, out=None):
    """ts_attend_rows_append_bf16: per-head norm + rotation + append + causal attention in one launch.
    Every row must sit in a slot of its own."""
    rows = qkv.shape[0]
    kv_heads, width = k_rows.shape[-2], k_rows.shape[-1]
    if out is None:
        out = torch.empty((rows, heads, width), dtype=torch.bfloat16, device=qkv.device)
    nbytes = lib.ts_attend_rows_workspace_bytes(rows, keys, heads, kv_heads, width)
    ws = workspace(nbytes, qkv.device)
    kc = kept.c()
    if kc.rows == 0:
        kc.rows = k_rows.numel() // (kv_heads * width)
    check(lib.ts_attend_rows_append_bf16(_ptr(qkv), _ptr(q_norm), _ptr(k_norm), _ptr(inv_freq), _ptr(k_rows), _ptr(v_rows),
                                         _ptr(out), _ptr(slots), _ptr(positions), C.byref(kc), rows, keys, heads, kv_heads,
                                         width, eps, scale, _ptr(ws), nbytes, _stream()))
    return out


FAR = 0xFFFFFFFF
MASKS = {"causal": (FAR, 0), "bidirectional": (FAR, FAR)}


def attend(q, k, v, *, mask="causal", scale: float, cu_seqlens=None, max_len=None, out=None):
    """Whole-sequence attention: ts_attend_bf16.  mask: 'causal' | 'bidirectional' | ('within', n) | ('back', n).
    Fixed layout: q [seqs, queries, heads, width], k/v [seqs, keys, kv_heads, width].
    Packed: q/k/v [total, heads, width] with cu_seqlens (int32 [seqs + 1]) and max_len."""
    if isinstance(mask, tuple):
        back, ahead = (mask[1], mask[1]) if mask[0] == "within" else (mask[1], 0)
    else:
        back, ahead = MASKS[mask]
    if cu_seqlens is None:
        seqs, queries, heads, width = q.shape
        keys, kv_heads = k.shape[1], k.shape[2]
    else:
        total, heads, width = q.shape
        kv_heads = k.shape[1]
        seqs, queries, keys = cu_seqlens.numel() - 1, int(max_len), total
    if out is None:
        out = torch.empty_like(q)
    nbytes = lib.ts_attend_workspace_bytes(seqs, queries, keys, heads, kv_heads, width)
    ws = workspace(nbytes, q.device)
    check(lib.ts_attend_bf16(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(cu_seqlens), seqs, queries, keys, heads,
                             kv_heads, width, back, ahead, scale, _ptr(ws), nbytes, _stream()))
    return out


def scatter(x, slots, positions, out, kept: Kept):
    rows = x.shape[0]
    width = x.numel() // max(rows, 1)
    kc = kept.c()
    check(lib.ts_scatter_bf16(_ptr(x), _ptr(slots), _ptr(positions), _ptr(out), C.byref(kc), rows, width, _stream()))
    return out


def rope_inv_freq(theta: float, width: int, device) -> torch.Tensor:
    buf = (C.c_float * (width // 2))()
    lib.ts_rope_inv_freq(theta, width, buf)
    return torch.tensor(list(buf), dtype=torch.float32, device=device)


def rope_angles(positions, width: int, theta: float, turned: int | None = None) -> torch.Tensor:
    """[count, width] f32: (cos, sin) per pair, the reference's `angles` launch (engine/rules/kernels/src/rope.rs:36-60)."""
    out = torch.empty((positions.numel(), width), dtype=torch.float32, device=positions.device)
    check(lib.ts_rope_angles(_ptr(positions), _ptr(out), positions.numel(), width, theta,
                             width // 2 if turned is None else turned, _stream()))
    return out


def rope(x, freqs, heads: int, width: int, adjacent: bool = False):
    """Rotates x [positions, heads, width] (f32 or bf16) in place by `freqs` (rope.rs:10-34)."""
    positions = x.numel() // (heads * width)
    check(lib.ts_rope(_ptr(x), _dtype_code(x.dtype), _ptr(freqs), positions, heads, width, int(adjacent), _stream()))
    return x


def qk_norm_rope_append(qkv, q_norm, k_norm, inv_freq, slots, positions, q_out, k_rows, v_rows, kept: Kept, heads,
                        kv_heads, width, eps):
    rows = qkv.shape[0]
    kc = kept.c()
    check(lib.ts_qk_norm_rope_append_bf16(_ptr(qkv), _ptr(q_norm), _ptr(k_norm), _ptr(inv_freq), _ptr(slots),
                                          _ptr(positions), _ptr(q_out), _ptr(k_rows), _ptr(v_rows), C.byref(kc), rows,
                                          heads, kv_heads, width, eps, _stream()))
    return q_out


def rms_norm(x, w=None, eps=1e-6, out_dtype=torch.bfloat16, out=None):
    width = x.shape[-1]
    rows = x.numel() // width
    if out is None:
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    check(lib.ts_rms_norm(_ptr(x), _dtype_code(x.dtype), _ptr(w), _ptr(out), _dtype_code(out.dtype), rows, width, eps,
                          _stream()))
    return out


def gather_scaled(table, ids, gain, parts: int):
    """ts_gather_scaled_bf16: (rows f32, bf16(rows * gain), sums of squares f32 [rows, parts])."""
    rows = ids.numel()
    table_rows, width = table.shape
    out = torch.empty((rows, width), dtype=torch.float32, device=table.device)
    xs = torch.empty((rows, width), dtype=torch.bfloat16, device=table.device)
    ss = torch.empty((rows, parts), dtype=torch.float32, device=table.device)
    check(lib.ts_gather_scaled_bf16(_ptr(table), _ptr(ids), _ptr(out), _ptr(xs), _ptr(gain), _ptr(ss), parts, rows, table_rows,
                                    width, _stream()))
    return out, xs, ss


def gather(table, ids, out_dtype=torch.float32, first=0):
    rows = ids.numel()
    table_rows, width = table.shape
    out = torch.empty(tuple(ids.shape) + (width,), dtype=out_dtype, device=table.device)
    check(lib.ts_gather_bf16(_ptr(table), _ptr(ids), _ptr(out), _dtype_code(out_dtype), rows, table_rows, width, first,
                             _stream()))
    return out


def top_k(x, k: int):
    width = x.shape[-1]
    rows = x.numel() // width
    ids = torch.empty(x.shape[:-1] + (k,), dtype=torch.int32, device=x.device)
    nbytes = lib.ts_top_k_workspace_bytes(rows, width, k)
    ws = workspace(nbytes, x.device)
    check(lib.ts_top_k(_ptr(x), _dtype_code(x.dtype), _ptr(ids), rows, width, k, _ptr(ws), nbytes, _stream()))
    return ids


def take_softmax(x, ids):
    rows, width = x.shape
    k = ids.shape[-1]
    gates = torch.empty((rows, k), dtype=torch.float32, device=x.device)
    check(lib.ts_take_softmax(_ptr(x), _ptr(ids), _ptr(gates), rows, width, k, _stream()))
    return gates


def moe_permutation(ids, experts: int, first: int = 0):
    """ts_moe_permutation: (order, place, offsets, batch_tiles) of the picks in `ids` (int32, any shape)."""
    picks = ids.numel()
    dev = ids.device
    order = torch.empty(picks, dtype=torch.int32, device=dev)
    place = torch.empty(picks, dtype=torch.int32, device=dev)
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=dev)
    tiles = torch.empty(experts + 1, dtype=torch.int32, device=dev)
    check(lib.ts_moe_permutation(_ptr(ids), _ptr(order), _ptr(place), _ptr(offsets), _ptr(tiles), picks, experts, first,
                                 _stream()))
    return order, place, offsets, tiles


def moe_experts(x, ids, w_in, w_out, *, repeat: int = 1, first: int = 0):
    """out[i] = expert_{ids[i]}(x[i // repeat]): ts_moe_experts_bf16.  w_in [E, 2F, H], w_out [E, H, F]."""
    experts, two_f, hidden = w_in.shape
    picks = ids.numel()
    out = torch.empty((picks, hidden), dtype=torch.float32, device=x.device)
    nbytes = lib.ts_moe_workspace_bytes(picks, experts, hidden, two_f // 2)
    ws = workspace(nbytes, x.device)
    check(lib.ts_moe_experts_bf16(_ptr(x), _ptr(ids), _ptr(w_in), _ptr(w_out), _ptr(out), picks, repeat, experts, first,
                                  hidden, two_f // 2, _ptr(ws), nbytes, _stream()))
    return out


def moe(h, ids, gates, w_in, w_out, *, add=None, first: int = 0):
    """y[r] = sum_p gates[r, p] expert_{ids[r, p]}(h[r]) (+ add[r]): ts_moe_bf16."""
    experts, two_f, hidden = w_in.shape
    rows, top = ids.shape
    y = torch.empty((rows, hidden), dtype=torch.float32, device=h.device)
    nbytes = lib.ts_moe_workspace_bytes(rows * top, experts, hidden, two_f // 2)
    ws = workspace(nbytes, h.device)
    check(lib.ts_moe_bf16(_ptr(h), _ptr(ids), _ptr(gates), _ptr(add), _ptr(w_in), _ptr(w_out), _ptr(y), rows, top,
                          experts, first, hidden, two_f // 2, _ptr(ws), nbytes, _stream()))
    return y


def picked(x, w, ids, n: int, *, count: int | None = None, stride: int | None = None, offset: int = 0, repeat: int = 1,
           first: int = 0):
    """out[i] = x[i // repeat] . w[(ids[i] - first) * stride + offset + (0..n)]^T, zeros for ids outside
    [first, first + count): ts_picked_bf16 (engine/rules/linear/src/picked.rs:28-60).  w bf16 [matrices, stride, k]
    or any row-major table of `count * stride` rows."""
    k = x.shape[-1]
    rows = ids.numel()
    stride = stride if stride is not None else (w.shape[-2] if w.dim() == 3 else n)
    count = count if count is not None else w.numel() // (stride * k)
    out = torch.empty((rows, n), dtype=torch.float32, device=x.device)
    nbytes = lib.ts_picked_workspace_bytes(rows, n, k, count)
    ws = workspace(nbytes, x.device)
    check(lib.ts_picked_bf16(_ptr(x), _ptr(w), _ptr(ids), _ptr(out), rows, n, k, count, stride, offset, repeat, first,
                             _ptr(ws), nbytes, _stream()))
    return out


def moe_mix(y_picks, gates, add=None):
    """out[r] = sum_p gates[r, p] y_picks[r * top + p] (+ add[r]) in pick order: ts_moe_mix."""
    rows, top = gates.shape
    hidden = y_picks.shape[-1]
    out = torch.empty((rows, hidden), dtype=torch.float32, device=y_picks.device)
    check(lib.ts_moe_mix(_ptr(y_picks), _ptr(gates), _ptr(add), _ptr(out), rows, top, hidden, _stream()))
    return out


def mean_pool(x, cu_seqlens, normalize=True):
    """Per-sequence mean of packed rows, then unit length: ts_mean_pool."""
    seqs = cu_seqlens.numel() - 1
    width = x.shape[-1]
    out = torch.empty((seqs, width), dtype=torch.float32, device=x.device)
    check(lib.ts_mean_pool(_ptr(x), _ptr(cu_seqlens), _ptr(out), seqs, width, int(normalize), _stream()))
    return out
