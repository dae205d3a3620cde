"""The reference's kernels by name, with arguments in the reference's order: a face on `ts_launch`.

tessera's lowering rules end in `Launch { args, shape }` records whose `args` follow the kernel's
parameter list (engine/plan/lower/src/rule.rs:241-261; the lists below cite each kernel).  A host that
walks such records can hand them to `launch(name, args, ...)` here unchanged: buffers as device tensors,
scalars as Python numbers, in the reference's order.  The launch itself happens in the library's by-name
table (`ts_launch`, one implementation for every host language); this module only names the parameters,
picks the table entry that the element types and the kept layout select (`attend_rows` + a 16-row paged
layout -> `attend_rows_paged16`, as `plan_attend_rows_{layout}` does in
engine/rules/attention/src/attend.rs:182-186), puts the layout's page table and scalar where the
reference's argument list has them, and turns the library's refusals into exceptions.  Unknown names and
wrong argument counts raise `KeyError` / `TypeError` before anything is launched, as `Error::Launch` does
in the reference.  As in the reference, queries arrive already scaled and epilogue stages are not part of
a by-name launch (a host that fuses them calls the typed entry points in `ops`).

    launch("lanes", [x, w, out, n, k])                      # engine/rules/linear/src/lanes.rs:21-32
    launch("attend_rows", [q, k, v, out, slots, positions, rows, keys, heads, kv_heads, width, back],
           kept=ops.Kept("paged", pages, table))
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable


@dataclass(frozen=True)
class Rule:
    name: str
    params: tuple[str, ...]   # the reference kernel's parameters, in order
    cites: str                # where the reference declares them
    entry: Callable           # (args by name, keywords) -> (table entry name, its argument list, rows for shape->down)
    written: str = "out"      # the parameter the kernel writes


def _linear(name):
    def entry(a, kw):
        x, w, n, k = a["x"], a["w"], int(a["n"]), int(a["k"])
        if tuple(w.shape) != (n, k) or x.shape[-1] != k:
            raise TypeError(f"{name}: w is {tuple(w.shape)}, x is {tuple(x.shape)}, the launch says n={n} k={k}")
        # m is a build parameter in the reference and shows only in the launch shape
        return f"{name}_bf16", [x, w, a["out"], n, k], x.numel() // k
    return entry


def _layout(name, a, kw, buffers, scalars):
    if "kept" not in kw:
        raise TypeError(f"{name}: the kept layout comes as a keyword")
    kept = kw["kept"]
    if kept.page not in (None, 64 if kept.layout == "paged" else 16):
        raise TypeError(f"{name}: the by-name table holds 64- and 16-row pages, not {kept.page}")
    table = [kept.table] if kept.layout in ("paged", "paged16") else []
    return f"{name}_{kept.layout}", [a[b] for b in buffers] + table + [int(a[s]) for s in scalars] + [int(kept.scalar)], 0


def _attend_rows(a, kw):
    rows, heads, width = int(a["rows"]), int(a["heads"]), int(a["width"])
    if a["q"].numel() != rows * heads * width:
        raise TypeError(f"attend_rows: q holds {a['q'].numel()} elements, the launch says {rows} x {heads} x {width}")
    return _layout("attend_rows", a, kw, ("q", "k", "v", "out", "slots", "positions"),
                   ("rows", "keys", "heads", "kv_heads", "width", "back"))


def _scatter(a, kw):
    return _layout("scatter", a, kw, ("x", "slots", "positions", "out"), ("rows", "width"))


def _plain(name, floats=(), by_dtype=None):
    def entry(a, kw):
        import torch
        entry_name = name
        if by_dtype and a[by_dtype].dtype == torch.bfloat16:
            entry_name += "_bf16"
        return entry_name, [float(v) if p in floats else v for p, v in a.items()], 0
    return entry


def _picked(a, kw):
    rows, n = int(a["rows"]), int(a["n"])
    if a["ids"].numel() != rows or a["out"].numel() != rows * n:
        raise TypeError(f"picked: {a['ids'].numel()} ids and {a['out'].numel()} outputs, the launch says {rows} rows of {n}")
    return "picked_bf16", list(a.values()), 0


_LINEAR_PARAMS = ("x", "w", "out", "n", "k")
_ROPE_PARAMS = ("x", "freqs", "positions", "heads", "width")
RULES = {r.name: r for r in (
    # The linear family shares one parameter list; m rides in the launch shape (lanes.rs:21-32, thin.rs, tiled.rs:295-304).
    Rule("lanes", _LINEAR_PARAMS, "engine/rules/linear/src/lanes.rs:21-32", _linear("lanes")),
    Rule("thin", _LINEAR_PARAMS, "engine/rules/linear/src/thin.rs", _linear("thin")),
    Rule("tiled", _LINEAR_PARAMS, "engine/rules/linear/src/tiled.rs:295-304", _linear("tiled")),
    Rule("picked", ("x", "w", "ids", "out", "rows", "n", "k", "count", "stride", "offset", "repeat", "first"),
         "engine/rules/linear/src/picked.rs:28-41", _picked),
    Rule("angles", ("positions", "out", "count", "width", "theta", "turned"), "engine/rules/kernels/src/rope.rs:36-44",
         _plain("angles", floats=("theta",))),
    Rule("rope", _ROPE_PARAMS, "engine/rules/kernels/src/rope.rs:10-16", _plain("rope", by_dtype="x"), written="x"),
    Rule("rope_adjacent", _ROPE_PARAMS, "engine/rules/kernels/src/rope.rs:10-16", _plain("rope_adjacent", by_dtype="x"),
         written="x"),
    Rule("attend_rows", ("q", "k", "v", "out", "slots", "positions", "rows", "keys", "heads", "kv_heads", "width", "back"),
         "engine/rules/attention/src/attend.rs:126-139", _attend_rows),
    Rule("scatter", ("x", "slots", "positions", "out", "rows", "width"), "engine/plan/lower/src/kernels/scatter.rs:12-19", _scatter),
    Rule("top_k", ("x", "out", "rows", "width", "k"), "engine/rules/kernels/src/argmax.rs:39", _plain("top_k")),
    Rule("lane_norm", ("x", "w", "out", "rows", "width", "eps"), "engine/rules/kernels/src/lane_norm.rs:10-17",
         _plain("lane_norm", floats=("eps",), by_dtype="out")),
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
    """Runs the kernel `name` on `args` (the reference's order) through `ts_launch`.  Returns the tensor written."""
    rule = RULES[name]
    args = list(args)
    if len(args) != len(rule.params):
        raise TypeError(f"{name} takes {len(rule.params)} arguments ({', '.join(rule.params)}), got {len(args)}")
    by_name = dict(zip(rule.params, args))
    entry, c_args, down = rule.entry(by_name, keywords)
    launch_c(entry, c_args, down=down)
    return by_name[rule.written]
