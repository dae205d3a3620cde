"""Loads libtessera_b200.so and declares the C ABI of include/tessera_b200.h for ctypes.

There is no fallback: if the shared library is missing the import of this module raises,
and every compute call on a machine without a CUDA device returns TS_ERR_CUDA.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libtessera_b200.so")

TS_OK, TS_ERR_ABI, TS_ERR_PEER, TS_ERR_BAD_INPUT, TS_ERR_TIMEOUT, TS_ERR_PROTOCOL, TS_ERR_CUDA = range(7)
TS_BF16, TS_F32 = 0, 1
EPILOGUE = {"none": 0, "add": 1, "swiglu": 2, "scale": 3, "geglu": 4}
LINEAR_PATH = {"auto": 0, "skinny": 1, "umma": 2, "stream": 3, "pair": 4, "plain": 5, "ordered": 6}
KEPT_KIND = {"dense": 0, "interleaved": 1, "paged": 2, "paged16": 2}
KEPT_PAGE = {"dense": 1, "interleaved": 1, "paged": 64, "paged16": 16}

u32, f32, vp, sz, i32 = C.c_uint32, C.c_float, C.c_void_p, C.c_size_t, C.c_int


class TsKept(C.Structure):
    """ts_kept: engine/plan/codegen/src/kept.rs:135-194 as one record."""
    _fields_ = [("kind", i32), ("page", u32), ("kept_scalar", u32), ("table", vp), ("table_len", u32), ("rows", u32)]


class TsLinearFused(C.Structure):
    """ts_linear_fused: the RMS norm folded into a decode-sized linear's input and output."""
    _fields_ = [("row_ss", vp), ("row_parts", u32), ("row_eps", f32), ("ss_out", vp), ("xs_out", vp), ("xs_gain", vp)]


class TsArg(C.Structure):
    class _V(C.Union):
        _fields_ = [("ptr", vp), ("u32", u32), ("f32", f32)]
    _fields_ = [("kind", i32), ("v", _V)]


class TsShape(C.Structure):
    _fields_ = [("across", u32), ("down", u32), ("threads", u32)]


class TsKernelInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("signature", C.c_char_p), ("order", i32)]


# name -> (restype, argtypes); every symbol include/tessera_b200.h declares.
SIGNATURES = {
    "ts_last_error": (C.c_char_p, []),
    "ts_kernel_count": (i32, []),
    "ts_kernel_info_at": (i32, [i32, C.POINTER(TsKernelInfo)]),
    "ts_launch_workspace_bytes": (sz, [C.c_char_p, C.POINTER(TsArg), i32, C.POINTER(TsShape)]),
    "ts_launch": (i32, [C.c_char_p, C.POINTER(TsArg), i32, C.POINTER(TsShape), vp, sz, vp]),
    "ts_abi_version": (i32, []),
    "ts_set_pdl": (i32, [i32]),
    "ts_device_status": (i32, []),
    "ts_wait_runs_out": (i32, [C.c_uint64, vp]),
    "ts_platform_info": (i32, [C.c_char_p, sz]),
    "ts_q8_0_bytes": (sz, [sz]),
    "ts_q8_0_pack": (i32, [vp, sz, vp]),
    "ts_q8_0_unpack": (i32, [vp, sz, vp]),
    "ts_linear_q8_0_workspace_bytes": (sz, [u32, u32, u32]),
    "ts_linear_q8_0": (i32, [vp, vp, vp, vp, u32, u32, u32, i32, f32, i32, vp, sz, vp]),
    "ts_linear_workspace_bytes": (sz, [u32, u32, u32, i32, i32]),
    "ts_linear_bf16": (i32, [vp, vp, vp, vp, u32, u32, u32, i32, f32, i32, i32, vp, sz, vp]),
    "ts_gather_scaled_bf16": (i32, [vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, vp]),
    "ts_linear_sumsq_parts": (u32, [u32, u32, u32, i32]),
    "ts_linear_fused_bf16": (i32, [vp, vp, vp, vp, u32, u32, u32, i32, f32, i32, C.POINTER(TsLinearFused), vp]),
    "ts_attend_rows_workspace_bytes": (sz, [u32, u32, u32, u32, u32]),
    "ts_attend_rows_bf16": (i32, [vp, vp, vp, vp, vp, vp, C.POINTER(TsKept), u32, u32, u32, u32, u32, u32, f32, vp, sz, vp]),
    "ts_attend_rows_append_bf16": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, C.POINTER(TsKept), u32, u32, u32, u32, u32, f32,
                                         f32, vp, sz, vp]),
    "ts_attend_workspace_bytes": (sz, [u32, u32, u32, u32, u32, u32]),
    "ts_attend_bf16": (i32, [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, u32, f32, vp, sz, vp]),
    "ts_scatter_bf16": (i32, [vp, vp, vp, vp, C.POINTER(TsKept), u32, u32, vp]),
    "ts_qk_norm_rope_append_bf16": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, C.POINTER(TsKept), u32, u32, u32, u32, f32, vp]),
    "ts_rope_inv_freq": (None, [f32, u32, vp]),
    "ts_rope_angles": (i32, [vp, vp, u32, u32, f32, u32, vp]),
    "ts_rope": (i32, [vp, i32, vp, u32, u32, u32, i32, vp]),
    "ts_rms_norm": (i32, [vp, i32, vp, vp, i32, u32, u32, f32, vp]),
    "ts_gather_bf16": (i32, [vp, vp, vp, i32, u32, u32, u32, u32, vp]),
    "ts_top_k_workspace_bytes": (sz, [u32, u32, u32]),
    "ts_top_k": (i32, [vp, i32, vp, u32, u32, u32, vp, sz, vp]),
    "ts_top_1_static": (i32, [vp, i32, vp, u32, u32, vp]),
    "ts_moe_workspace_bytes": (sz, [u32, u32, u32, u32]),
    "ts_moe_experts_bf16": (i32, [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, vp, sz, vp]),
    "ts_moe_bf16": (i32, [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, vp, sz, vp]),
    "ts_picked_workspace_bytes": (sz, [u32, u32, u32, u32]),
    "ts_picked_bf16": (i32, [vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, u32, vp, sz, vp]),
    "ts_moe_mix": (i32, [vp, vp, vp, vp, u32, u32, u32, vp]),
    "ts_moe_permutation": (i32, [vp, vp, vp, vp, vp, u32, u32, u32, vp]),
    "ts_mean_pool": (i32, [vp, vp, vp, u32, u32, i32, vp]),
    "ts_take_softmax": (i32, [vp, vp, vp, u32, u32, u32, vp]),
}


class TesseraError(RuntimeError):
    """A non-zero ts_status, with the library's message (tessera_run::Error in the reference)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"tessera_b200 status {code}: {message}")
        self.code = code


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m tessera_b200.build` (there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.ts_abi_version() != 1:
        raise ImportError("libtessera_b200.so has a different ABI version")
    return lib


lib = _load()


def check(code: int) -> None:
    if code != TS_OK:
        raise TesseraError(code, lib.ts_last_error().decode())
