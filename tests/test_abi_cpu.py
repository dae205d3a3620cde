"""CPU-side checks of the boundary: the shared library loads, exports every symbol the headers
declare, refuses bad arguments on the host, and has no CPU compute path."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ts_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from tessera_b200 import _lib
    names = _declared("tessera_b200.h") + _declared("tessera_b200_run.h") + _declared("tessera_b200_kv.h")
    assert len(names) > 20
    for name in names:
        assert hasattr(_lib.lib, name), f"{name} is declared but not exported"
    assert _lib.lib.ts_abi_version() == 1


def test_python_signatures_cover_the_header():
    from tessera_b200 import _lib, runner
    declared = set(_declared("tessera_b200.h"))
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert set(_declared("tessera_b200_run.h")) == set(runner.RUN_SIGNATURES)
    from tessera_b200 import kv
    assert set(_declared("tessera_b200_kv.h")) == set(kv.KV_SIGNATURES)


def test_bad_arguments_are_refused_on_the_host():
    from tessera_b200 import _lib
    lib = _lib.lib
    rc = lib.ts_linear_bf16(None, None, None, None, 1, 1, 64, 0, 1.0, 0, 0, None, 0, None)
    assert rc == _lib.TS_ERR_BAD_INPUT and b"NULL" in lib.ts_last_error()
    buf = (C.c_char * 256)()
    p = C.cast(buf, C.c_void_p).value
    p = (p + 15) // 16 * 16
    rc = lib.ts_linear_bf16(p, p, None, p, 1, 1, 100, 0, 1.0, 0, 2, None, 0, None)   # path 2: the tiled tensor-core kernel
    assert rc == _lib.TS_ERR_BAD_INPUT and b"multiples of 64" in lib.ts_last_error()
    rc = lib.ts_linear_bf16(p, p, None, p, 1, 1, 100, 0, 1.0, 0, 9, None, 0, None)
    assert rc == _lib.TS_ERR_BAD_INPUT and b"path 9" in lib.ts_last_error()
    rc = lib.ts_linear_bf16(p, p, None, p, 1, 1, 0, 0, 1.0, 0, 0, None, 0, None)
    assert rc == _lib.TS_ERR_BAD_INPUT and b"k is zero" in lib.ts_last_error()
    rc = lib.ts_linear_bf16(p + 2, p, None, p, 1, 1, 64, 0, 1.0, 0, 0, None, 0, None)
    assert rc == _lib.TS_ERR_BAD_INPUT and b"aligned" in lib.ts_last_error()
    kept = _lib.TsKept(2, 48, 4, None, 0, 0)  # page 48 is not a power of two
    rc = lib.ts_scatter_bf16(p, p, p, p, C.byref(kept), 1, 8, None)
    assert rc == _lib.TS_ERR_BAD_INPUT and b"power of two" in lib.ts_last_error()


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_there_is_no_cpu_path():
    from tessera_b200 import TesseraError, ops, runner
    x = torch.zeros((4, 64), dtype=torch.bfloat16)
    with pytest.raises(TesseraError):
        ops.linear(x, x)
    with pytest.raises(TesseraError) as e:
        runner.Decoder(dict(layers=1, hidden=256, heads=4, kv_heads=2, head_dim=64, ffn=256, vocab=100), 1, 16, 4)
    assert e.value.code == 6  # TS_ERR_CUDA


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "tessera_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text, f
                assert "tessera_oracle" not in text, f


def test_rope_table_matches_the_checker():
    import oracle as O
    from tessera_b200 import _lib
    out = (C.c_float * 64)()
    _lib.lib.ts_rope_inv_freq(1e6, 128, out)
    # the checker's angle at position 1 is the same f32 power (engine/ir/interp/src/cpu.rs:31-34)
    x = np.zeros((1, 1, 128), np.float32)
    x[0, 0, :64] = 1.0
    turned = O.rope(x, [1], 1e6, "halves")
    assert np.allclose(turned[0, 0, :64], np.cos(np.array(out[:], np.float32)), atol=1e-7)


def test_synthetic_weights_are_reproducible():
    from tessera_b200 import synth
    cfg = dict(layers=2, hidden=64, heads=2, kv_heads=1, head_dim=32, ffn=128, vocab=50)
    a = dict(synth.decoder_weights(cfg, 3))
    b = dict(synth.decoder_weights(cfg, 3))
    assert list(a) == synth.decoder_weight_names(2)
    assert all(np.array_equal(a[k], b[k]) for k in a)
    import oracle as O
    rng = np.random.default_rng(0)
    x = rng.standard_normal(5000).astype(np.float32)
    assert np.array_equal(synth.bf16_bits(x), O.bf16_bits(x))
    total = sum(int(np.prod(synth.decoder_weight_shape(n, synth.QWEN3_0_6B))) for n in synth.decoder_weight_names(28))
    assert total == 596_049_920  # tools/parity/tests/qwen3/mod.rs:16


def test_platform_row_reads_through_the_abi():
    """ts_platform_info needs no device: its row is the committed platforms/cuda-b200.json (the record a maintainer
    adds to engine/gpu/platform/platforms/), shaped like the reference's Row (platform.rs:11-29), and it refines the
    sm_10x row's mma.sync tiles to the tcgen05 one."""
    import json
    from tessera_b200 import _lib
    buf = C.create_string_buffer(4096)
    assert _lib.lib.ts_platform_info(buf, len(buf)) == 0
    info = json.loads(buf.value.decode())
    row = info["row"]
    committed = json.load(open(os.path.join(ROOT, "tessera_b200", "platforms", "cuda-b200.json")))
    assert row == committed
    assert set(row) >= {"matches", "tile", "bf16_tile", "pdl", "check", "note"}        # the reference's Row fields
    assert row["matches"] == ["cuda sm_100"] and row["tile"] == [128, 256, 16] and row["pdl"] is True
    assert row["b200"]["abi"] == _lib.lib.ts_abi_version() and row["b200"]["cluster"] == 8
    if not torch.cuda.is_available():
        assert info["asked"] is None
    small = C.create_string_buffer(16)
    assert _lib.lib.ts_platform_info(small, len(small)) == _lib.TS_ERR_BAD_INPUT
