"""The by-name launch table: names, parameter lists in the reference's order, and refusals before any launch."""
import pytest


def test_table_lists_the_reference_parameters():
    from tessera_b200 import rules
    assert rules.RULES["attend_rows"].params == ("q", "k", "v", "out", "slots", "positions", "rows", "keys", "heads",
                                                 "kv_heads", "width", "back")   # attend.rs:126-139
    assert rules.RULES["scatter"].params == ("x", "slots", "positions", "out", "rows", "width")   # scatter.rs:12-19
    assert rules.RULES["top_k"].params == ("x", "out", "rows", "width", "k")   # argmax.rs:39
    assert rules.RULES["lane_norm"].params == ("x", "w", "out", "rows", "width", "eps")   # lane_norm.rs:10-17
    assert rules.RULES["picked"].params == ("x", "w", "ids", "out", "rows", "n", "k", "count", "stride", "offset", "repeat",
                                            "first")   # picked.rs:28-41
    assert rules.RULES["angles"].params == ("positions", "out", "count", "width", "theta", "turned")   # rope.rs:36-44
    assert rules.RULES["rope"].params == rules.RULES["rope_adjacent"].params == ("x", "freqs", "positions", "heads", "width")
    for name in ("lanes", "thin", "tiled"):
        assert rules.RULES[name].params == ("x", "w", "out", "n", "k")
    assert all(r.cites.startswith("engine/") for r in rules.RULES.values())


def test_unknown_names_and_wrong_counts_are_refused():
    from tessera_b200 import rules
    with pytest.raises(KeyError):
        rules.launch("no_such_kernel", [])
    with pytest.raises(TypeError):
        rules.launch("top_k", [1, 2, 3])


def test_c_table_lists_the_reference_kernel_names():
    # ts_kernel_info_at: loads the library (no GPU needed) and reads the by-name table
    from tessera_b200 import rules
    table = rules.kernels()
    for name in ("lanes_bf16", "thin_bf16", "tiled_bf16", "parts_bf16", "attend_rows_dense", "attend_rows_paged",
                 "attend_rows_paged16", "flash_rows_paged", "scatter_dense", "scatter_paged16", "top_k", "lane_norm",
                 "flash_128", "flash_256", "picked_bf16", "angles", "rope", "rope_adjacent", "rope_bf16"):
        assert name in table
    # read buffers, output, [page table], then scalars; the layout's scalar last (rule.rs:62-109)
    assert table["attend_rows_dense"][0] == "pppppp" + "u" * 7
    assert table["attend_rows_paged"][0] == "ppppppp" + "u" * 7
    assert table["scatter_paged"][0] == "ppppp" + "uuu"
    assert table["lane_norm"][0] == "pppuuf"
    assert table["picked_bf16"] == ("pppp" + "u" * 8, 1) and table["angles"][0] == "ppuufu" and table["rope"] == ("ppuuu", 0)
    assert table["top_k"] == ("ppuuu", 0) and table["scatter_dense"][1] == 0   # Order::Fixed
    assert table["tiled_bf16"][1] == 1 and table["flash_128"][1] == 1          # Order::PerConfig


def test_c_launch_refuses_bad_lists_without_a_gpu():
    import ctypes as C
    from tessera_b200._lib import TsArg, TsShape, lib
    arr = (TsArg * 2)()
    shape = TsShape(0, 0, 0)
    assert lib.ts_launch(b"no_such_kernel", arr, 2, C.byref(shape), None, 0, None) == 3
    assert b"no kernel is called" in lib.ts_last_error()
    assert lib.ts_launch(b"top_k", arr, 2, C.byref(shape), None, 0, None) == 3     # wrong count and NULL pointers
    assert b"ppuuu" in lib.ts_last_error()


def test_face_builds_the_table_entry_and_its_argument_list():
    # no launch: only what `launch` would hand ts_launch (entry name by element type and kept layout, the page table
    # after the buffers, the layout's scalar last, a linear's rows in shape->down)
    import torch
    from tessera_b200 import ops, rules
    q = torch.zeros(2, 4 * 128, dtype=torch.bfloat16)
    kv = torch.zeros(3 * 64, 2 * 128, dtype=torch.bfloat16)
    out, sl, ps = torch.zeros_like(q), torch.zeros(2, dtype=torch.int32), torch.zeros(2, dtype=torch.int32)
    table = torch.arange(12, dtype=torch.int32)
    a = dict(zip(rules.RULES["attend_rows"].params, [q, kv, kv, out, sl, ps, 2, 64, 4, 2, 128, 0xFFFFFFFF]))
    name, args, down = rules.RULES["attend_rows"].entry(a, {"kept": ops.Kept("paged16", 4, table)})
    assert name == "attend_rows_paged16" and down == 0
    assert args[6] is table and args[7:] == [2, 64, 4, 2, 128, 0xFFFFFFFF, 4]
    name, args, _ = rules.RULES["attend_rows"].entry(a, {"kept": ops.Kept("dense", 64)})
    assert name == "attend_rows_dense" and len(args) == 13 and args[-1] == 64
    with pytest.raises(TypeError):
        rules.RULES["attend_rows"].entry(a, {})                       # the layout is not optional
    with pytest.raises(TypeError):
        rules.RULES["attend_rows"].entry(a, {"kept": ops.Kept("paged", 4, table, page=32)})   # not in the by-name table
    s = dict(zip(rules.RULES["scatter"].params, [q, sl, ps, kv, 2, 256]))
    name, args, _ = rules.RULES["scatter"].entry(s, {"kept": ops.Kept("paged", 4, table)})
    assert name == "scatter_paged" and args[4] is table and args[5:] == [2, 256, 4]
    x, w = torch.zeros(24, 256, dtype=torch.bfloat16), torch.zeros(512, 256, dtype=torch.bfloat16)
    lin = dict(zip(rules.RULES["tiled"].params, [x, w, torch.zeros(24, 512, dtype=torch.bfloat16), 512, 256]))
    assert rules.RULES["tiled"].entry(lin, {})[0::2] == ("tiled_bf16", 24)
    norm = dict(zip(rules.RULES["lane_norm"].params, [torch.zeros(5, 300), torch.zeros(300), torch.zeros(5, 300, dtype=torch.bfloat16), 5, 300, 1]))
    name, args, _ = rules.RULES["lane_norm"].entry(norm, {})
    assert name == "lane_norm_bf16" and isinstance(args[-1], float)    # eps travels as f32 whatever the host passed
    rope = dict(zip(rules.RULES["rope"].params, [torch.zeros(4, 2, 128, dtype=torch.bfloat16), torch.zeros(4, 128), 4, 2, 128]))
    assert rules.RULES["rope"].entry(rope, {})[0] == "rope_bf16" and rules.RULES["rope"].written == "x"
