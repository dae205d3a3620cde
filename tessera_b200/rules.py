"""The reference's kernels by name, with arguments in the reference's order.

tessera's lowering rules end in `Launch { args, shape }` records whose `args` follow the kernel's
parameter list (engine/plan/lower/src/rule.rs:241-261; the lists below cite each kernel).  A host that
walks such records can hand them to `launch(name, args, ...)` here unchanged: buffers as device tensors,
scalars as Python numbers, in the reference's order.  What the reference keeps outside the argument
list (element types, the kept layout's trailing scalars, epilogue stages fused by the lowering) comes in
as keywords.  Unknown names and wrong argument counts raise `KeyError` / `TypeError` before anything is
launched, as `Error::Launch` does in the reference.

    launch("lanes", [x, w, out, n, k])                      # engine/rules/linear/src/lanes.rs:21-32
    launch("attend_rows", [q, k, v, out, slots, positions, rows, keys, heads, kv_heads, width, back],
           kept=ops.Kept("paged", pages, table), scale=d ** -0.5)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable


@dataclass(frozen=True)
class Rule:
    name: str
    params: tuple[str, ...]   # the reference kernel's parameters, in order
    cites: str                # where the reference declares them
    run: Callable             # (args by name, keywords) -> output tensor


def _linear(a, kw):
    from . import ops
    x, w, out = a["x"], a["w"], a["out"]
    n, k = int(a["n"]), int(a["k"])
    if w.shape != (n, k) or x.shape[-1] != k:
        raise TypeError(f"linear: w is {tuple(w.shape)}, x is {tuple(x.shape)}, the launch says n={n} k={k}")
    return ops.linear(x.reshape(-1, k), w, kw.get("a0"), epilogue=kw.get("epilogue", "none"), scale=kw.get("scale", 1.0),
                      out_dtype=out.dtype, path=kw.get("path", "auto"), out=out)


def _attend_rows(a, kw):
    from . import ops
    q = a["q"]
    rows, heads, kv_heads, width = int(a["rows"]), int(a["heads"]), int(a["kv_heads"]), int(a["width"])
    if q.numel() != rows * heads * width:
        raise TypeError(f"attend_rows: q holds {q.numel()} elements, the launch says {rows} x {heads} x {width}")
    if "kept" not in kw or "scale" not in kw:
        raise TypeError("attend_rows: the kept layout and the score scale come as keywords")
    k_rows = a["k"].reshape(-1, kv_heads, width)
    v_rows = a["v"].reshape(-1, kv_heads, width)
    return ops.attend_rows(q.reshape(rows, heads, width), k_rows, v_rows, a["slots"], a["positions"], kw["kept"],
                           int(a["keys"]), scale=float(kw["scale"]), back=int(a["back"]),
                           out=a["out"].reshape(rows, heads, width))


def _scatter(a, kw):
    from . import ops
    if "kept" not in kw:
        raise TypeError("scatter: the kept layout comes as a keyword")
    rows, width = int(a["rows"]), int(a["width"])
    return ops.scatter(a["x"].reshape(rows, width), a["slots"], a["positions"], a["out"].reshape(-1, width), kw["kept"])


def _top_k(a, kw):
    from . import ops
    rows, width, k = int(a["rows"]), int(a["width"]), int(a["k"])
    ids = ops.top_k(a["x"].reshape(rows, width), k)
    a["out"].reshape(rows, k).copy_(ids.reshape(rows, k))
    return a["out"]


def _lane_norm(a, kw):
    from . import ops
    rows, width = int(a["rows"]), int(a["width"])
    return ops.rms_norm(a["x"].reshape(rows, width), a["w"], float(a["eps"]), out_dtype=a["out"].dtype,
                        out=a["out"].reshape(rows, width))


def _picked(a, kw):
    from . import ops
    rows, n, k = int(a["rows"]), int(a["n"]), int(a["k"])
    if a["ids"].numel() != rows or a["out"].numel() != rows * n:
        raise TypeError(f"picked: {a['ids'].numel()} ids and {a['out'].numel()} outputs, the launch says {rows} rows of {n}")
    got = ops.picked(a["x"].reshape(-1, k), a["w"], a["ids"], n, count=int(a["count"]), stride=int(a["stride"]),
                     offset=int(a["offset"]), repeat=int(a["repeat"]), first=int(a["first"]))
    a["out"].reshape(rows, n).copy_(got)
    return a["out"]


def _angles(a, kw):
    from . import ops
    count, width = int(a["count"]), int(a["width"])
    a["out"].reshape(count, width).copy_(ops.rope_angles(a["positions"], width, float(a["theta"]), int(a["turned"])))
    return a["out"]


def _rope(adjacent):
    def run(a, kw):
        from . import ops
        return ops.rope(a["x"], a["freqs"], int(a["heads"]), int(a["width"]), adjacent)
    return run


_LINEAR_PARAMS = ("x", "w", "out", "n", "k")
RULES = {r.name: r for r in (
    # The linear family shares one parameter list; m rides in the launch shape (lanes.rs:21-32, thin.rs, tiled.rs:295-304).
    Rule("lanes", _LINEAR_PARAMS, "engine/rules/linear/src/lanes.rs:21-32", _linear),
    Rule("thin", _LINEAR_PARAMS, "engine/rules/linear/src/thin.rs", _linear),
    Rule("tiled", _LINEAR_PARAMS, "engine/rules/linear/src/tiled.rs:295-304", _linear),
    Rule("picked", ("x", "w", "ids", "out", "rows", "n", "k", "count", "stride", "offset", "repeat", "first"),
         "engine/rules/linear/src/picked.rs:28-41", _picked),
    Rule("angles", ("positions", "out", "count", "width", "theta", "turned"), "engine/rules/kernels/src/rope.rs:36-44", _angles),
    Rule("rope", ("x", "freqs", "positions", "heads", "width"), "engine/rules/kernels/src/rope.rs:10-16", _rope(False)),
    Rule("rope_adjacent", ("x", "freqs", "positions", "heads", "width"), "engine/rules/kernels/src/rope.rs:10-16", _rope(True)),
    Rule("attend_rows", ("q", "k", "v", "out", "slots", "positions", "rows", "keys", "heads", "kv_heads", "width", "back"),
         "engine/rules/attention/src/attend.rs:126-139", _attend_rows),
    Rule("scatter", ("x", "slots", "positions", "out", "rows", "width"), "engine/plan/lower/src/kernels/scatter.rs:12-19", _scatter),
    Rule("top_k", ("x", "out", "rows", "width", "k"), "engine/rules/kernels/src/argmax.rs:39", _top_k),
    Rule("lane_norm", ("x", "w", "out", "rows", "width", "eps"), "engine/rules/kernels/src/lane_norm.rs:10-17", _lane_norm),
)}


def kernels() -> dict:
    """The C entry point's table: {name: (signature, order)}; signature letters p = pointer, u = u32, f = f32."""
    import ctypes as C
    from ._lib import TsKernelInfo, check, lib
    out = {}
    for i in range(lib.ts_kernel_count()):
        info = TsKernelInfo()
        check(lib.ts_kernel_info_at(i, C.byref(info)))
        out[info.name.decode()] = (info.signature.decode(), info.order)
    return out


def launch_c(name: str, args, down: int = 0):
    """ts_launch: `args` in the reference's order, tensors for buffers, int / float for scalars.  The workspace
    comes from this library's pool; `down` fills shape->down (the rows of a five-argument linear)."""
    import ctypes as C
    import torch
    from . import ops
    from ._lib import TsArg, TsShape, check, lib
    arr = (TsArg * len(args))()
    for i, a in enumerate(args):
        if isinstance(a, torch.Tensor):
            arr[i].kind, arr[i].v.ptr = 0, ops._ptr(a)
        elif isinstance(a, float):
            arr[i].kind, arr[i].v.f32 = 2, a
        else:
            arr[i].kind, arr[i].v.u32 = 1, int(a)
    shape = TsShape(0, down, 0)
    device = next(a.device for a in args if isinstance(a, torch.Tensor))
    nbytes = lib.ts_launch_workspace_bytes(name.encode(), arr, len(args), C.byref(shape))
    ws = ops.workspace(nbytes, device)
    check(lib.ts_launch(name.encode(), arr, len(args), C.byref(shape), ops._ptr(ws), nbytes, ops._stream()))


def launch(name: str, args, **keywords):
    """Runs the kernel `name` on `args` (the reference's order).  Returns the tensor written."""
    rule = RULES[name]
    args = list(args)
    if len(args) != len(rule.params):
        raise TypeError(f"{name} takes {len(rule.params)} arguments ({', '.join(rule.params)}), got {len(args)}")
    return rule.run(dict(zip(rule.params, args)), keywords)
