"""Row kernels against the CPU checker: RMS norm, gather, top-k (bit-exact), take + softmax."""
import math

import numpy as np
import pytest
import torch

import oracle as O
from tests.util import dev_u32, from_bits, normal_bf16, rel_error, to_bits, u32, widen

pytestmark = pytest.mark.gpu


def test_rms_norm_f32_to_bf16():
    from tessera_b200 import ops
    rng = np.random.default_rng(0)
    x = rng.standard_normal((37, 1024), dtype=np.float32) * 3
    w = rng.standard_normal(1024, dtype=np.float32)
    want = O.rms_norm(x, w, 1e-6)
    got = ops.rms_norm(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), 1e-6)
    assert rel_error(widen(got), want) <= 1e-2
    got32 = ops.rms_norm(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), 1e-6, out_dtype=torch.float32)
    assert rel_error(widen(got32), want) <= 1e-5
    plain = ops.rms_norm(torch.from_numpy(x).cuda(), None, 1e-6, out_dtype=torch.float32)
    assert rel_error(widen(plain), O.rms_norm(x, None, 1e-6)) <= 1e-5


@pytest.mark.parametrize("width", [768, 1024, 2048])
def test_rms_norm_many_rows(width):
    # from 1024 rows on a warp takes a row (registers, one read); the last block is ragged
    from tessera_b200 import ops
    rng = np.random.default_rng(width)
    rows = 1024 + 13
    x = rng.standard_normal((rows, width), dtype=np.float32) * 2
    w = rng.standard_normal(width, dtype=np.float32)
    want = O.rms_norm(x, w, 1e-6)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    assert rel_error(widen(ops.rms_norm(xd, wd, 1e-6)), want) <= 1e-2
    assert rel_error(widen(ops.rms_norm(xd, wd, 1e-6, out_dtype=torch.float32)), want) <= 1e-5
    assert rel_error(widen(ops.rms_norm(xd, None, 1e-6, out_dtype=torch.float32)), O.rms_norm(x, None, 1e-6)) <= 1e-5


def test_rms_known_answer():
    # engine/ir/interp/src/cpu_test.rs:131-149, through the device kernel
    from tessera_b200 import ops
    x = torch.tensor([[1., -3., 5., -1.], [2., 0., 0., -2.]], device="cuda")
    w = torch.tensor([1., 2., -1., 0.5], device="cuda")
    got = widen(ops.rms_norm(x, w, 7.0, out_dtype=torch.float32)).reshape(-1)
    want = np.array([0.25, -1.5, -1.25, -0.125, 2. / 3., 0., 0., -1. / 3.], np.float32)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-6)


def test_gather_rows():
    from tessera_b200 import ops
    rng = np.random.default_rng(1)
    table = normal_bf16(rng, (50, 64))
    ids = np.array([3, 0, 49, 50, 3, 7], np.uint32)  # 50 is past the table: zeros
    got = ops.gather(from_bits(table), dev_u32(ids), out_dtype=torch.bfloat16)
    assert np.array_equal(to_bits(got), O.gather(table, ids))
    got32 = ops.gather(from_bits(table), dev_u32(ids), out_dtype=torch.float32)
    assert np.array_equal(widen(got32), O.bf16_widen(O.gather(table, ids)))
    shifted = ops.gather(from_bits(table), dev_u32(ids + 10), out_dtype=torch.bfloat16, first=10)
    assert np.array_equal(to_bits(shifted), O.gather(table, ids + 10, first=10))


def test_top_k_ties_known_answer():
    # engine/ir/interp/src/run_test.rs:54-67, on the device
    from tessera_b200 import ops
    inf, nan = math.inf, math.nan
    x = torch.tensor([2., 7., 7., -1., -inf, 3., nan, -inf, -0.0, 0.0, -0.0, inf], device="cuda").reshape(3, 4)
    got = u32(ops.top_k(x, 3)).reshape(-1).tolist()
    assert got == [1, 2, 0, 1, 4, 4, 3, 0, 1]


@pytest.mark.parametrize("rows,width,k", [(256, 128, 8), (64, 128, 1), (5, 1000, 32), (3, 7, 4), (6, 600, 1), (6, 32, 1),
                                          (4, 3000, 5), (3, 20000, 3), (7, 200, 8), (2, 1024, 2)])
def test_top_k_is_bit_exact(rows, width, k):
    from tessera_b200 import ops
    x = O.Noise(rows + width).draw(rows, width)
    x[0, 1] = x[0, width - 1]  # ties keep the lower index
    x[rows - 1, :] = 0.25      # a whole row of ties
    want = O.top_k(x, k)
    got = u32(ops.top_k(torch.from_numpy(x).cuda(), k))
    assert np.array_equal(got, want)


@pytest.mark.parametrize("width", [16, 128, 700, 5000])
def test_top_k_spare_slots_hold_the_width(width):
    # engine/ir/interp/src/run.rs:577-591: -inf and NaN never rank; slots past the rankable entries hold the width
    from tessera_b200 import ops
    x = np.full((3, width), -np.inf, np.float32)
    x[0, [3, width - 1]] = [1.0, 2.0]          # two rankable entries, k = 4
    x[1, 5] = np.nan                           # nothing ranks
    x[2, :] = np.nan
    x[2, [0, 1, 2, 7, 9]] = [0.5, 0.5, -1.0, 0.5, 3.0]
    want = O.top_k(x, 4)
    assert want[0].tolist() == [width - 1, 3, width, width] and want[1].tolist() == [width] * 4
    assert want[2].tolist() == [9, 0, 1, 7]
    got = u32(ops.top_k(torch.from_numpy(x).cuda(), 4))
    assert np.array_equal(got, want)


def test_argmax_over_the_vocabulary():
    from tessera_b200 import ops
    rng = np.random.default_rng(9)
    x = rng.standard_normal((6, 151936), dtype=np.float32)
    x[2, 77] = x[2, 150000] = 9.0  # a tie across parts: the lower index wins
    x[3, :] = -np.inf              # nothing ranks: the spare value is the width
    want = O.top_k(x, 1)
    got = u32(ops.top_k(torch.from_numpy(x).cuda(), 1))
    assert np.array_equal(got, want)


def test_take_softmax():
    from tessera_b200 import ops
    x = O.Noise(3).draw(40, 128) * 4
    ids = O.top_k(x, 8)
    want = O.softmax(O.take(x, ids))
    got = ops.take_softmax(torch.from_numpy(x).cuda(), dev_u32(ids))
    assert rel_error(widen(got), want) <= 1e-5


def test_launch_by_name_with_the_reference_argument_order():
    from tessera_b200 import ops, rules
    rng = np.random.default_rng(8)
    m, n, k = 24, 512, 256
    x = from_bits(normal_bf16(rng, (m, k)))
    w = from_bits(normal_bf16(rng, (n, k), 0.02))
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    rules.launch("lanes", [x, w, out, n, k])
    assert torch.equal(out, ops.linear(x, w))
    with pytest.raises(TypeError):
        rules.launch("tiled", [x, w, out, n + 1, k])

    xs = torch.randn(5, 300, device="cuda")
    ids = torch.empty((5, 3), dtype=torch.int32, device="cuda")
    rules.launch("top_k", [xs, ids, 5, 300, 3])
    assert torch.equal(ids, ops.top_k(xs, 3))

    g = torch.randn(300, device="cuda")
    normed = torch.empty((5, 300), dtype=torch.float32, device="cuda")
    rules.launch("lane_norm", [xs, g, normed, 5, 300, 1e-6])
    assert torch.equal(normed, ops.rms_norm(xs, g, 1e-6, out_dtype=torch.float32))

    # attend_rows over a dense layout, then scatter a new row into it by name
    slots, context, heads, kv_heads, width = 3, 40, 4, 2, 128
    kept = ops.Kept("dense", context, None, slots * context)
    kr = from_bits(normal_bf16(rng, (slots * context, kv_heads * width)))
    vr = from_bits(normal_bf16(rng, (slots * context, kv_heads * width)))
    q = from_bits(normal_bf16(rng, (2, heads * width), 0.1))
    sl, ps = dev_u32([2, 0]), dev_u32([17, 39])
    o = torch.empty_like(q)
    # by name the queries arrive already scaled, as in the reference (its scale is a launch of its own)
    rules.launch("attend_rows", [q, kr, vr, o, sl, ps, 2, context, heads, kv_heads, width, 0xFFFFFFFF], kept=kept)
    want = ops.attend_rows(q.reshape(2, heads, width), kr.reshape(-1, kv_heads, width), vr.reshape(-1, kv_heads, width), sl, ps,
                           kept, context, scale=1.0)
    # the by-name entry does not know how many kept rows the buffers hold, so it may pick another kernel of the
    # family than the typed call: same values to rounding, not the same bits
    assert rel_error(widen(o.reshape(2, heads, width)), widen(want)) <= 1e-2
    new = from_bits(normal_bf16(rng, (2, kv_heads * width)))
    rules.launch("scatter", [new, sl, ps, kr, 2, kv_heads * width], kept=kept)
    assert torch.equal(kr[2 * context + 17], new[0]) and torch.equal(kr[39], new[1])


def test_ts_launch_by_name():
    # the C entry point: argument lists in the reference's order, checked against the kernel's signature
    from tessera_b200 import TesseraError, ops, rules
    rng = np.random.default_rng(18)
    m, n, k = 24, 512, 256
    x = from_bits(normal_bf16(rng, (m, k)))
    w = from_bits(normal_bf16(rng, (n, k), 0.02))
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    rules.launch_c("tiled_bf16", [x, w, out, m, n, k])
    assert torch.equal(out, ops.linear(x, w))
    out.zero_()
    rules.launch_c("lanes_bf16", [x, w, out, n, k], down=m)   # m from the launch shape, as in the reference
    assert torch.equal(out, ops.linear(x, w))
    with pytest.raises(TesseraError):
        rules.launch_c("lanes_bf16", [x, w, out, n, k])       # no rows anywhere
    with pytest.raises(TesseraError):
        rules.launch_c("tiled_bf16", [x, w, n, k, out])       # buffers after scalars

    xs = torch.randn(5, 300, device="cuda")
    ids = torch.empty((5, 3), dtype=torch.int32, device="cuda")
    rules.launch_c("top_k", [xs, ids, 5, 300, 3])
    assert torch.equal(ids, ops.top_k(xs, 3))
    g = torch.randn(300, device="cuda")
    normed = torch.empty((5, 300), dtype=torch.float32, device="cuda")
    rules.launch_c("lane_norm", [xs, g, normed, 5, 300, 1e-6])
    assert torch.equal(normed, ops.rms_norm(xs, g, 1e-6, out_dtype=torch.float32))

    # paged16 attention: the table after the last buffer, kept_pages as the last scalar
    slots, context, heads, kv_heads, width = 3, 48, 4, 2, 128
    pages = context // 16
    table = dev_u32(rng.permutation(slots * pages))
    kept = ops.Kept("paged16", pages, table, slots * pages * 16)
    kr = from_bits(normal_bf16(rng, (slots * pages * 16, kv_heads, width)))
    vr = from_bits(normal_bf16(rng, (slots * pages * 16, kv_heads, width)))
    q = from_bits(normal_bf16(rng, (2, heads, width)))
    sl, ps = dev_u32([2, 0]), dev_u32([17, 47])
    o = torch.empty_like(q)
    rules.launch_c("attend_rows_paged16", [q, kr, vr, o, sl, ps, table, 2, context, heads, kv_heads, width, 0xFFFFFFFF, pages])
    assert torch.equal(o, ops.attend_rows(q, kr, vr, sl, ps, kept, context, scale=1.0))
    new = from_bits(normal_bf16(rng, (2, kv_heads * width)))
    rules.launch_c("scatter_paged16", [new, sl, ps, kr, table, 2, kv_heads * width, pages])
    want = kr.clone()
    ops.scatter(new, sl, ps, want.reshape(-1, kv_heads * width), kept)
    assert torch.equal(kr, want)

    # one whole sequence, causal: q, k, v, out, queries, keys, past, heads, kv_heads, back, ahead
    seq = 200
    fq = from_bits(normal_bf16(rng, (1, seq, heads, width)))
    fk = from_bits(normal_bf16(rng, (1, seq, kv_heads, width)))
    fv = from_bits(normal_bf16(rng, (1, seq, kv_heads, width)))
    fo = torch.empty_like(fq)
    rules.launch_c("flash_128", [fq, fk, fv, fo, seq, seq, 0, heads, kv_heads, 0xFFFFFFFF, 0])
    assert torch.equal(fo, ops.attend(fq, fk, fv, mask="causal", scale=1.0))


@pytest.mark.parametrize("width,heads,adjacent,turned", [(128, 4, False, None), (64, 3, True, None), (256, 2, False, 40), (6, 1, True, 2)])
def test_rope_launches_match_oracle(width, heads, adjacent, turned):
    """The reference's `angles` and `rope` / `rope_adjacent` launches (rope.rs:10-60) against the CPU interpreter's
    rope (cpu.rs:31-47).  The rotation itself is exact in f32 given the angles; the device's sine and cosine may
    differ from the host's in the last bits, which the tolerance covers."""
    from tessera_b200 import ops, rules
    rng = np.random.default_rng(width + heads)
    count, theta = 9, 10000.0
    positions = rng.integers(0, 4096, size=count).astype(np.uint32)
    x = rng.standard_normal((count, heads, width)).astype(np.float32)
    want = O.rope(x, positions, theta, pairs="adjacent" if adjacent else "halves", turned=turned)
    freqs = ops.rope_angles(dev_u32(positions), width, theta, turned)
    pairs = width // 2
    upto = pairs if turned is None else min(turned, pairs)
    f = widen(freqs).reshape(count, pairs, 2)
    # The checker's cosines and sines: what its rope makes of the pair (1, 0).
    a = np.arange(pairs) * 2 if adjacent else np.arange(pairs)
    b = a + 1 if adjacent else a + pairs
    unit = np.zeros((count, 1, width), np.float32)
    unit[:, :, a] = 1.0
    turned_unit = O.rope(unit, positions, theta, pairs="adjacent" if adjacent else "halves", turned=turned)[:, 0]
    assert np.abs(f[:, :, 0] - turned_unit[:, a]).max() <= 1e-6 and np.abs(f[:, :, 1] - turned_unit[:, b]).max() <= 1e-6
    assert (f[:, upto:, 0] == 1.0).all() and (f[:, upto:, 1] == 0.0).all()    # pairs past `turned` keep angle zero
    got = ops.rope(torch.from_numpy(x).cuda(), freqs, heads, width, adjacent)
    assert np.abs(widen(got) - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    # by name, and in bf16
    xb = torch.from_numpy(x).cuda()
    fr = torch.empty_like(freqs)
    rules.launch_c("angles", [dev_u32(positions), fr, count, width, theta, pairs if turned is None else turned])
    assert torch.equal(fr, freqs)
    rules.launch_c("rope_adjacent" if adjacent else "rope", [xb, fr, count, heads, width])
    assert torch.equal(xb, got)
    xh = torch.from_numpy(x).cuda().to(torch.bfloat16)
    want_h = O.rope(widen(xh), positions, theta, pairs="adjacent" if adjacent else "halves", turned=turned)
    ops.rope(xh, freqs, heads, width, adjacent)
    assert rel_error(widen(xh), want_h) <= 1e-2
