"""Linear kernels against the CPU checker on the same seeded inputs.

Tolerance: bf16 outputs with f32 sums must sit within 1e-2 of the checker relative to the
output's largest magnitude (the bar the build states for floating-point outputs); f32 outputs
(the residual-add epilogue) within 1e-4, which is summation-order noise.  One-hot inputs must
read weights back bit-exactly, as engine/rules/linear/tests/lanes_test.rs:96-106 demands.
"""
import numpy as np
import pytest
import torch

import oracle as O
from tests.util import from_bits, normal_bf16, rel_error, widen

pytestmark = pytest.mark.gpu

BF16_TOL = 1e-2
F32_TOL = 1e-4


def _case(m, n, k, seed):
    rng = np.random.default_rng(seed)
    x = normal_bf16(rng, (m, k), 1.0)
    w = normal_bf16(rng, (n, k), 0.02)
    return x, w


def _run(x_bits, w_bits, path, **kw):
    from tessera_b200 import ops
    out = ops.linear(from_bits(x_bits), from_bits(w_bits), path=path, **kw)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return out


SKINNY = [(1, 2048, 1024), (5, 1024, 1024), (16, 1024, 2048), (33, 6144, 1024), (64, 1024, 3072),
          (64, 2048, 1024), (7, 1000, 512), (64, 72, 256)]
UMMA = [(1, 2048, 1024), (16, 1024, 2048), (64, 1024, 3072), (64, 6144, 1024), (100, 2048, 1024),
        (128, 1024, 1024), (200, 512, 1024), (384, 1024, 512), (1024, 640, 256), (129, 200, 64),
        (256, 128, 4096), (300, 100, 2048)]   # a router's shape: two tiles, k split sixteen ways over blocks


STREAM = [(1, 2048, 1024), (16, 1024, 2048), (64, 1024, 3072), (64, 6144, 1024), (100, 2048, 1024),
          (128, 1024, 1024), (64, 4096, 1024), (33, 1000, 512), (64, 72, 256), (17, 128, 64), (64, 20000, 1024)]


@pytest.mark.parametrize("m,n,k", STREAM)
def test_stream_matches_oracle(m, n, k):
    x, w = _case(m, n, k, seed=m * 13 + n + k)
    want = O.matmul(O.bf16_widen(x), w)
    got = widen(_run(x, w, "stream"))
    assert rel_error(got, want) <= BF16_TOL
    got32 = widen(_run(x, w, "stream", out_dtype=torch.float32))
    assert rel_error(got32, want) <= F32_TOL


@pytest.mark.parametrize("m,n,k", SKINNY)
def test_skinny_matches_oracle(m, n, k):
    x, w = _case(m, n, k, seed=m * 7 + n + k)
    want = O.matmul(O.bf16_widen(x), w)
    got = widen(_run(x, w, "skinny"))
    assert rel_error(got, want) <= BF16_TOL
    got32 = widen(_run(x, w, "skinny", out_dtype=torch.float32))
    assert rel_error(got32, want) <= F32_TOL


@pytest.mark.parametrize("m,n,k", UMMA)
def test_umma_matches_oracle(m, n, k):
    x, w = _case(m, n, k, seed=m * 11 + n + k)
    want = O.matmul(O.bf16_widen(x), w)
    got = widen(_run(x, w, "umma"))
    assert rel_error(got, want) <= BF16_TOL
    got32 = widen(_run(x, w, "umma", out_dtype=torch.float32))
    assert rel_error(got32, want) <= F32_TOL


@pytest.mark.parametrize("path,m", [("skinny", 8), ("umma", 8), ("umma", 160), ("stream", 8), ("stream", 77)])
def test_one_hot_rows_read_weights_back(path, m):
    # engine/rules/linear/tests/lanes_test.rs:96-106
    n, k = 256, 512
    rng = np.random.default_rng(5)
    w = normal_bf16(rng, (n, k), 0.02)
    hot = rng.integers(0, k, size=m)
    x = np.zeros((m, k), np.float32)
    x[np.arange(m), hot] = 1.0
    got = _run(O.bf16_bits(x), w, path)
    from tests.util import to_bits
    assert np.array_equal(to_bits(got), w[:, hot].T)


@pytest.mark.parametrize("path", ["skinny", "umma", "stream"])
@pytest.mark.parametrize("m", [3, 64])
def test_residual_add_epilogue(path, m):
    n, k = 1024, 2048
    x, w = _case(m, n, k, seed=90 + m)
    rng = np.random.default_rng(91)
    res = rng.standard_normal((m, n), dtype=np.float32)
    want = O.matmul(O.bf16_widen(x), w) + res
    got = widen(_run(x, w, path, a0=torch.from_numpy(res).cuda(), epilogue="add", out_dtype=torch.float32))
    assert rel_error(got, want) <= F32_TOL


def test_few_tiles_split_k_with_residual():
    # m > 128 with a handful of output tiles: k slices meet in the reduce kernel, which adds the residual
    m, n, k = 256, 128, 2048
    x, w = _case(m, n, k, seed=77)
    res = np.random.default_rng(78).standard_normal((m, n), dtype=np.float32)
    want = O.matmul(O.bf16_widen(x), w) + res
    got = widen(_run(x, w, "umma", a0=torch.from_numpy(res).cuda(), epilogue="add", out_dtype=torch.float32))
    assert rel_error(got, want) <= F32_TOL
    again = widen(_run(x, w, "umma", a0=torch.from_numpy(res).cuda(), epilogue="add", out_dtype=torch.float32))
    assert np.array_equal(got, again)     # slices add in a fixed order


@pytest.mark.parametrize("path,m", [("skinny", 4), ("skinny", 64), ("umma", 64), ("umma", 256), ("stream", 4),
                                    ("stream", 64), ("stream", 128)])
@pytest.mark.parametrize("act", ["swiglu", "geglu"])
def test_gated_epilogue(path, m, act):
    ffn, k = 768, 512
    x, w = _case(m, 2 * ffn, k, seed=33 + m)
    xs = O.bf16_widen(x)
    gate, up = O.matmul(xs, w[:ffn]), O.matmul(xs, w[ffn:])
    want = O.act(gate, "silu" if act == "swiglu" else "gelu_tanh") * up
    got = widen(_run(x, w, path, epilogue=act))
    assert got.shape == (m, ffn)
    assert rel_error(got, want) <= BF16_TOL


def test_stream_gated_wide_enough_for_one_block_per_tile():
    # (n/2) / 64 tiles >= SM count: no cluster, the pairing goes through the block's own buffer
    m, ffn, k = 20, 64 * 160, 128
    x, w = _case(m, 2 * ffn, k, seed=77)
    xs = O.bf16_widen(x)
    want = O.act(O.matmul(xs, w[:ffn]), "silu") * O.matmul(xs, w[ffn:])
    got = widen(_run(x, w, "stream", epilogue="swiglu"))
    assert rel_error(got, want) <= BF16_TOL


@pytest.mark.parametrize("path", ["skinny", "umma", "stream"])
def test_scale_epilogue(path):
    x, w = _case(9, 512, 256, seed=3)
    want = O.matmul(O.bf16_widen(x), w) * np.float32(0.125)
    got = widen(_run(x, w, path, epilogue="scale", scale=0.125, out_dtype=torch.float32))
    assert rel_error(got, want) <= F32_TOL


def test_lm_head_shape_small_batch():
    # (151936, 1024): the tied unembedding, at the decode parity batch
    m, n, k = 2, 151936, 1024
    x, w = _case(m, n, k, seed=1)
    want = O.matmul(O.bf16_widen(x), w)
    for path in ("skinny", "umma", "stream"):
        got = widen(_run(x, w, path, out_dtype=torch.float32))
        assert rel_error(got, want) <= F32_TOL


def test_rerun_is_bit_identical():
    # Order::PerConfig (engine/ir/graph/src/numerics.rs:26-35): one configuration, one sum order
    x, w = _case(64, 1024, 3072, seed=8)
    for path in ("skinny", "umma", "stream"):
        a = _run(x, w, path, out_dtype=torch.float32)
        b = _run(x, w, path, out_dtype=torch.float32)
        assert torch.equal(a, b)


def test_bad_arguments_are_refused():
    from tessera_b200 import TesseraError, ops
    x = torch.zeros((4, 100), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((8, 100), dtype=torch.bfloat16, device="cuda")
    for path in ("skinny", "umma", "stream", "pair"):
        with pytest.raises(TesseraError) as e:
            ops.linear(x, w, path=path)
        assert e.value.code == 3  # TS_ERR_BAD_INPUT: the tensor-core kernels take k in multiples of 64
    assert ops.linear(x, w).shape == (4, 8)   # left to itself the library takes the plain kernel
    with pytest.raises(TesseraError):
        ops.linear(x.cpu(), w.cpu())
    with pytest.raises(TesseraError):
        ops.linear(x[:, :99].contiguous(), w[:7, :99].contiguous(), epilogue="swiglu")   # a gated epilogue with odd n


def test_every_size_of_the_reference_tiled_cases():
    # engine/rules/linear/tests/tiled_test.rs:57-67: Noise(29); sizes off the block, on it, beyond it, over bands;
    # x drawn first, then w; the reference sees the weights in the stored (bf16) form.  Activations are bf16 here.
    from tessera_b200 import ops
    draws = O.Noise(29)
    for m, n, k in [(1, 3, 4), (37, 50, 72), (64, 64, 64), (600, 40, 512), (256, 512, 1024)]:
        x = O.bf16_bits(draws.draw(m, k))
        w = O.bf16_bits(draws.draw(n, k))
        want = O.matmul(O.bf16_widen(x), w)
        got = ops.linear(from_bits(x), from_bits(w), out_dtype=torch.float32)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        assert rel_error(widen(got), want) <= F32_TOL, (m, n, k)
        plain = ops.linear(from_bits(x), from_bits(w), out_dtype=torch.float32, path="plain")
        assert rel_error(widen(plain), want) <= F32_TOL, (m, n, k)
        assert rel_error(widen(ops.linear(from_bits(x), from_bits(w))), want) <= BF16_TOL, (m, n, k)


@pytest.mark.parametrize("act", ["swiglu", "geglu"])
def test_plain_kernel_epilogues(act):
    from tessera_b200 import ops
    m, ffn, k = 5, 9, 40                     # nothing here sits on a tile or a 16-byte row
    x, w = _case(m, 2 * ffn, k, seed=61)
    xs = O.bf16_widen(x)
    want = O.act(O.matmul(xs, w[:ffn]), "silu" if act == "swiglu" else "gelu_tanh") * O.matmul(xs, w[ffn:])
    got = ops.linear(from_bits(x), from_bits(w), epilogue=act, out_dtype=torch.float32)
    assert got.shape == (m, ffn) and rel_error(widen(got), want) <= 1e-3   # tanh / exp of the device's libm
    res = np.random.default_rng(62).standard_normal((m, 2 * ffn), dtype=np.float32)
    added = ops.linear(from_bits(x), from_bits(w), torch.from_numpy(res).cuda(), epilogue="add", out_dtype=torch.float32)
    assert rel_error(widen(added), O.matmul(xs, w) + res) <= F32_TOL
    scaled = ops.linear(from_bits(x), from_bits(w), epilogue="scale", scale=0.25, out_dtype=torch.float32)
    assert rel_error(widen(scaled), O.matmul(xs, w) * np.float32(0.25)) <= F32_TOL


@pytest.mark.parametrize("m", [64, 37, 128, 9])
def test_norms_folded_into_the_projections(m):
    # The decode step's pair: a residual-adding projection that also leaves bf16(out * gain) and per-tile
    # sums of squares, and a projection that takes those and multiplies its rows by 1/rms.  Checked
    # against the checker's rms_norm -> bf16 -> matmul chain (the folded product rounds the normed row
    # before instead of after the 1/rms factor: same tolerance) and against the unfolded launches.
    from tessera_b200 import ops
    rng = np.random.default_rng(m)
    hidden, inner, wide, eps = 1024, 2048, 4096, 1e-6
    a = normal_bf16(rng, (m, inner), 1.0)
    w1 = normal_bf16(rng, (hidden, inner), 0.02)
    x0 = rng.standard_normal((m, hidden)).astype(np.float32)
    gain = (1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
    w2 = normal_bf16(rng, (wide, hidden), 0.02)
    wgu = normal_bf16(rng, (2 * 3072, hidden), 0.02)

    x0_d, gain_d = torch.from_numpy(x0).cuda(), torch.from_numpy(gain).cuda()
    y, xs, ss = ops.linear_fused(from_bits(a), from_bits(w1), x0_d, epilogue="add", out_dtype=torch.float32,
                                 next_gain=gain_d)
    torch.cuda.synchronize()
    want_y = O.matmul(O.bf16_widen(a), w1) + x0
    assert rel_error(y.cpu().numpy(), want_y) <= F32_TOL
    assert ss.shape == (m, hidden // 128)
    tiles = (y.double() ** 2).reshape(m, hidden // 128, 128).sum(-1)
    assert torch.allclose(ss.double(), tiles, rtol=1e-5, atol=1e-6)
    assert torch.equal(xs, (y * gain_d).to(torch.bfloat16))   # one rounding of an f32 product: bit-exact

    h = O.bf16_round(O.rms_norm(y.cpu().numpy(), gain, eps))
    for w, epi in ((w2, "none"), (wgu, "swiglu")):
        got = ops.linear_fused(xs, from_bits(w), epilogue=epi, rows=(ss, eps))
        unfused = ops.linear(ops.rms_norm(y, gain_d, eps), from_bits(w), epilogue=epi, path="stream")
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        z = O.matmul(h, w)
        want = z if epi == "none" else (z[:, :3072] / (1.0 + np.exp(-z[:, :3072])) * z[:, 3072:]).astype(np.float32)
        assert rel_error(widen(got), want) <= BF16_TOL
        assert rel_error(widen(got), widen(unfused)) <= BF16_TOL


def test_sums_of_squares_are_refused_where_k_is_not_split():
    from tessera_b200 import TesseraError, ops
    x, w = _case(64, 20000, 1024, 5)   # one block per tile: no cluster reduce to hang the sums on
    with pytest.raises((TesseraError, ValueError)):
        ops.linear_fused(from_bits(x), from_bits(w), torch.zeros((64, 20000), device="cuda"), epilogue="add",
                         out_dtype=torch.float32, next_gain=torch.ones(20000, device="cuda"))


PAIR = [(512, 512, 256), (1024, 640, 256), (700, 1024, 512), (1300, 2304, 768), (512, 256, 64)]


@pytest.mark.parametrize("m,n,k", PAIR)
def test_pair_matches_oracle(m, n, k):
    # 256 x 256 tiles on pairs of SMs: ragged last row tile (m % 256), ragged last column tile (n % 256)
    x, w = _case(m, n, k, seed=m * 3 + n + k)
    want = O.matmul(O.bf16_widen(x), w)
    got = widen(_run(x, w, "pair"))
    assert rel_error(got, want) <= BF16_TOL
    got32 = widen(_run(x, w, "pair", out_dtype=torch.float32))
    assert rel_error(got32, want) <= F32_TOL


def test_pair_epilogues():
    m, n, k = 640, 768, 256
    x, w = _case(m, n, k, seed=12)
    base = O.matmul(O.bf16_widen(x), w)
    rng = np.random.default_rng(13)
    res = rng.standard_normal((m, n), dtype=np.float32)
    got = widen(_run(x, w, "pair", a0=torch.from_numpy(res).cuda(), epilogue="add", out_dtype=torch.float32))
    assert rel_error(got, base + res) <= F32_TOL
    got = widen(_run(x, w, "pair", epilogue="scale", scale=0.25, out_dtype=torch.float32))
    assert rel_error(got, base * np.float32(0.25)) <= F32_TOL
    ffn = n // 2   # 384 = 3 gated tiles of 128
    for act in ("swiglu", "geglu"):
        want = O.act(base[:, :ffn], "silu" if act == "swiglu" else "gelu_tanh") * base[:, ffn:]
        got = widen(_run(x, w, "pair", epilogue=act))
        assert got.shape == (m, ffn) and rel_error(got, want) <= BF16_TOL


def test_pair_equals_one_sm_tiles_bit_for_bit():
    # same k order inside the tensor core: the two tilings give the same f32 sums (64 one-SM tiles: enough
    # of them that the one-SM kernel keeps its k loop whole)
    x, w = _case(1024, 2048, 512, seed=4)
    a = _run(x, w, "pair", out_dtype=torch.float32)
    b = _run(x, w, "umma", out_dtype=torch.float32)
    assert torch.equal(a, b)


def test_norms_folded_into_the_paired_projections():
    # the prefill-sized pair: same contract as the decode-sized one, on the two-SM kernel
    from tessera_b200 import ops
    rng = np.random.default_rng(77)
    m, hidden, inner, eps = 640, 768, 512, 1e-6
    a = normal_bf16(rng, (m, inner), 1.0)
    w1 = normal_bf16(rng, (hidden, inner), 0.02)
    x0 = rng.standard_normal((m, hidden)).astype(np.float32)
    gain = (1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
    w2 = normal_bf16(rng, (1280, hidden), 0.02)
    wgu = normal_bf16(rng, (2 * 1152, hidden), 0.02)
    x0_d, gain_d = torch.from_numpy(x0).cuda(), torch.from_numpy(gain).cuda()
    y, xs, ss = ops.linear_fused(from_bits(a), from_bits(w1), x0_d, epilogue="add", out_dtype=torch.float32, next_gain=gain_d)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    want_y = O.matmul(O.bf16_widen(a), w1) + x0
    assert rel_error(y.cpu().numpy(), want_y) <= F32_TOL
    assert ss.shape == (m, hidden // 256)
    tiles = (y.double() ** 2).reshape(m, hidden // 256, 256).sum(-1)
    assert torch.allclose(ss.double(), tiles, rtol=1e-5, atol=1e-6)
    assert torch.equal(xs, (y * gain_d).to(torch.bfloat16))
    h = O.bf16_round(O.rms_norm(y.cpu().numpy(), gain, eps))
    for w, epi in ((w2, "none"), (wgu, "geglu")):
        got = ops.linear_fused(xs, from_bits(w), epilogue=epi, rows=(ss, eps))
        torch.cuda.synchronize()
        z = O.matmul(h, w)
        want = z if epi == "none" else O.act(z[:, :1152], "gelu_tanh") * z[:, 1152:]
        assert rel_error(widen(got), want) <= BF16_TOL
