"""Pins the CPU checker to every literal known-answer test the reference holds for
the hot path.  Each test names the reference test it replays; inputs and expected
values are the reference's own literals."""
import math

import numpy as np
import pytest

import oracle as O


def close(got, want):
    """engine/ir/interp/src/cpu_test.rs:55-64: 1e-5 relative to max(|want|, 1)."""
    got = np.asarray(got, np.float32).reshape(-1)
    want = np.asarray(want, np.float32).reshape(-1)
    assert got.shape == want.shape
    assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(np.abs(want), 1.0)), (got, want)


def test_top_k_ties():
    # engine/ir/interp/src/run_test.rs:54-67
    inf, nan = math.inf, math.nan
    x = np.array([2., 7., 7., -1., -inf, 3., nan, -inf, -0.0, 0.0, -0.0, inf], np.float32).reshape(3, 4)
    want = [1, 2, 0, 1, 4, 4, 3, 0, 1]
    assert O.top_k(x, 3).reshape(-1).tolist() == want
    assert O.top_k_numpy(x, 3).reshape(-1).tolist() == want


def test_top_k_twin_agrees_on_noise():
    x = O.Noise(11).draw(64, 128)
    x[3, 5] = x[3, 90]  # a tie
    assert np.array_equal(O.top_k(x, 8), O.top_k_numpy(x, 8))


def test_rms_divides_rows():
    # engine/ir/interp/src/cpu_test.rs:131-149
    x = np.array([1., -3., 5., -1., 2., 0., 0., -2.], np.float32).reshape(2, 4)
    w = np.array([1., 2., -1., 0.5], np.float32)
    close(O.rms_norm(x, None, 7.0), [0.25, -0.75, 1.25, -0.25, 2. / 3., 0., 0., -2. / 3.])
    close(O.rms_norm(x, w, 7.0), [0.25, -1.5, -1.25, -0.125, 2. / 3., 0., 0., -1. / 3.])


def test_softmax_rows():
    # engine/ir/interp/src/cpu_test.rs:163-173
    x = np.array([0., math.log(2), math.log(3), math.log(4), 500., 500., -math.inf, 500.], np.float32)
    close(O.softmax(x.reshape(2, 4)), [0.1, 0.2, 0.3, 0.4, 1. / 3., 1. / 3., 0., 1. / 3.])


def test_act_values():
    # engine/ir/interp/src/cpu_test.rs:175-199
    x = np.array([-2., 0., 1., 3.], np.float32)
    close(O.act(x, "relu"), [0., 0., 1., 3.])
    close(O.act(x, "sigmoid"), [0.119_202_92, 0.5, 0.731_058_6, 0.952_574_1])
    close(O.act(x, "silu"), [-0.238_405_84, 0., 0.731_058_6, 2.857_722_4])
    close(O.act(x, "gelu_tanh"), [-0.045_402_3, 0., 0.841_192, 2.996_362_6])
    close(O.act(x, "softplus"), [0.126_928, math.log(2), 1.313_261_7, 3.048_587_4])
    close(O.act(x, "exp"), [0.135_335_28, 1., math.e, 20.085_537])
    close(O.act(x, "tanh"), [-0.964_027_6, 0., 0.761_594_2, 0.995_055])


def test_gather_rows():
    # engine/ir/interp/src/cpu_test.rs:201-212
    table = np.arange(1, 9, dtype=np.float32).reshape(4, 2)
    close(O.gather(table, [3, 0, 3]), [7., 8., 1., 2., 7., 8.])
    close(O.gather(table, [4, 1]), [0., 0., 3., 4.])


def test_mean_each_axis():
    # engine/ir/interp/src/cpu_test.rs:214-220
    x = np.arange(12, dtype=np.float32).reshape(2, 3, 2)
    close(O.mean(x, 0), [3., 4., 5., 6., 7., 8.])
    close(O.mean(x, 1), [2., 3., 8., 9.])
    close(O.mean(x, 2), [0.5, 2.5, 4.5, 6.5, 8.5, 10.5])


def _turned(x, pairs):
    # engine/ir/interp/src/cpu_test.rs:66-91: rows at position 0, then at 3: angles 3, 1.5
    s0, c0 = np.float32(math.sin(3.0)), np.float32(math.cos(3.0))
    s1, c1 = np.float32(math.sin(1.5)), np.float32(math.cos(1.5))
    want = list(x[:8])
    for r in x[8:].reshape(-1, 4):
        a, b, c, d = r
        if pairs == "adjacent":
            want += [a * c0 - b * s0, a * s0 + b * c0, c * c1 - d * s1, c * s1 + d * c1]
        else:
            want += [a * c0 - c * s0, b * c1 - d * s1, a * s0 + c * c0, b * s1 + d * c1]
    return want


@pytest.mark.parametrize("pairs", ["adjacent", "halves"])
def test_rope_both_pairs(pairs):
    # engine/ir/interp/src/cpu_test.rs:116-129: [Rows=2, Heads=2, width=4], theta 4
    x = np.arange(16, dtype=np.float32) - 5.5
    out = O.rope(x.reshape(2, 2, 4), [0, 3], 4.0, pairs)
    close(out, _turned(x, pairs))


def test_hadamard_blocks():
    # engine/ir/interp/src/cpu_test.rs:151-161
    close(O.hadamard([1., 2., 3., 4., -1., 0., 2., 5.], 4), [5., -1., -2., 0., 3., -2., -4., 1.])
    x = np.array([((i * 37) % 11) - 5.0 for i in range(128)], np.float32)
    scale = 1.0 / math.sqrt(128)
    want = [sum(v if bin(i & j).count("1") % 2 == 0 else -v for j, v in enumerate(x)) * scale for i in range(128)]
    close(O.hadamard(x, 128), want)


def test_sums_round():
    # engine/ir/interp/src/round_test.rs:4-18
    xs = [2048.0, 1.0, 1.0, 1.0]
    assert O.acc_sum(xs, "f32") == 2051.0
    assert O.acc_sum(xs, "f16") == 2048.0
    assert O.acc_sum(xs, "bf16") == 2048.0


def test_accumulators_follow_numerics():
    # engine/ir/interp/src/interp_test.rs:203-217: x [1,3] times ones [2,3]
    x = np.array([[2048.0, 1.0, 1.0]], np.float32)
    ones = np.ones((2, 3), np.float32)
    assert O.matmul(x, ones, "f32").tolist() == [[2050.0, 2050.0]]
    assert O.matmul(x, ones, "f16").tolist() == [[2048.0, 2048.0]]
    assert O.matmul(x, ones, "bf16").tolist() == [[2048.0, 2048.0]]


def _qkv():
    # engine/ir/interp/src/interp_test.rs:68-74
    wave = lambda seed: np.sin(np.arange(48, dtype=np.float32) * np.float32(seed)).astype(np.float32).reshape(2, 4, 2, 3)
    return wave(0.3), wave(0.7), wave(1.1)


def test_causal_first_row():
    # engine/ir/interp/src/interp_test.rs:76-86
    q, k, v = _qkv()
    o = O.attend(q, k, v, "causal", 0.5).reshape(-1)
    vf = v.reshape(-1)
    assert np.array_equal(o[:6], vf[:6])
    assert np.array_equal(o[24:30], vf[24:30])
    both = O.attend(q, k, v, "bidirectional", 0.5).reshape(-1)
    assert not np.array_equal(both[:6], vf[:6])


def test_decode_sees_past_keys():
    # engine/ir/interp/src/interp_test.rs:167-176: one query row sees all four keys either way
    q, k, v = _qkv()
    q1 = q.reshape(-1)[:12].reshape(2, 1, 2, 3)
    assert np.array_equal(O.attend(q1, k, v, "causal", 0.5), O.attend(q1, k, v, "bidirectional", 0.5))
    with pytest.raises(ValueError):
        O.attend(q, k[:, :3], v[:, :3], "causal", 0.5)  # fewer keys than queries


def test_narrow_values():
    # engine/ir/interp/src/interp_test.rs:122-138: values one wide
    q, k, _ = _qkv()
    v = np.arange(16, dtype=np.float32).reshape(2, 4, 2, 1)
    o = O.attend(q, k, v, "causal", 0.5)
    assert o.shape == (2, 4, 2, 1)
    assert np.array_equal(o.reshape(-1)[:2], v.reshape(-1)[:2])
    assert np.array_equal(o.reshape(-1)[8:10], v.reshape(-1)[8:10])


def _window(rows, v):
    # engine/ir/interp/src/interp_test.rs:258-268: zero queries average the keys they see
    q = np.zeros((1, rows, 1, 2), np.float32)
    kv = np.asarray(v, np.float32).reshape(1, -1, 1, 2)
    return O.attend(q, kv, kv, ("within", 1), 1.0)


def test_window_edges():
    # engine/ir/interp/src/interp_test.rs:293-301
    v = [x for t in range(4) for x in (float(1 << t), -float(t))]
    want = [1.5, -0.5, 7. / 3., -1., 14. / 3., -2., 6., -2.5]
    close(_window(4, v), want)
    close(_window(1, v), want[6:])


def _rows_over(positions):
    # engine/ir/interp/src/interp_test.rs:270-291: two rows, 4 query heads over 2 key heads
    ln3 = math.log(3.0)
    k = [0., ln3, 0., 0., ln3, 0., 0., 0., 99., 99., 99., 99.] + [9.] * 12
    v = [4., -8., 0., 2., 8., 4., 4., 0., 99., 99., 99., 99.]
    v += [-1., 2., 3., -3., 50., 50., 50., 50., 60., 60., 60., 60.]
    q = np.array([1., 0., 0., 1.] * 4, np.float32).reshape(2, 4, 2)
    k = np.array(k, np.float32).reshape(2, 3, 2, 2)
    v = np.array(v, np.float32).reshape(2, 3, 2, 2)
    return O.attend_rows(q, k, v, [1, 0], positions, "causal", 1.0)


def test_rows_read_slots():
    # engine/ir/interp/src/interp_test.rs:303-312
    want = [-1., 2., -1., 2., 3., -3., 3., -3., 7., 1., 5., -5., 2., 1., 2., 1.]
    close(_rows_over([0, 1]), want)
    with pytest.raises(ValueError):
        _rows_over([0, 3])


def test_store_keeps_rows():
    # engine/ir/interp/src/run_test.rs:86-110.  The kept graph there (run_test.rs:10-39):
    # zero queries [n,2,2], one kv head of width 2 whose rows are [v, 0], Seqs 2, Context 3;
    # keys and values are the same appended rows, so each output is the mean of the
    # values its slot holds up to the row's position.
    ks, vs = O.Store(), O.Store()

    def step(rows, k_store=None, v_store=None):
        k_store = ks if k_store is None else k_store
        v_store = vs if v_store is None else v_store
        n = len(rows)
        x = np.array([[v, 0.0] for _, _, v in rows], np.float32).reshape(n, 1, 2)
        slots = [r[0] for r in rows]
        positions = [r[1] for r in rows]
        ctx = max(positions) + 1
        if ctx > 3:
            raise ValueError("past the context bound")
        k = k_store.append(x, slots, positions, 2, ctx)
        v = v_store.append(x, slots, positions, 2, ctx)
        q = np.zeros((n, 2, 2), np.float32)
        return O.attend_rows(q, k, v, slots, positions, "causal", 1.0).reshape(-1)[::4]

    close(step([(0, 0, 1.), (0, 1, 3.), (1, 0, 10.)]), [1., 2., 10.])
    with pytest.raises(ValueError, match="position 0"):
        step([(0, 2, 5.)], O.Store(), O.Store())
    close(step([(0, 2, 5.)]), [3.])
    close(step([(1, 1, 20.)]), [15.])
    with pytest.raises(ValueError):
        step([(0, 4, 1.)])
    assert len(ks) == 3
    with pytest.raises(ValueError):
        step([(2, 0, 1.)])
    with pytest.raises(ValueError):
        step([(1, 3, 1.)])


def test_store_grows_past_three():
    # engine/ir/interp/src/run_test.rs:109: the last step of store_keeps_rows in a
    # store whose context bound admits position 3
    ks = O.Store()
    x = lambda v: np.array([[[v, 0.0]]], np.float32)
    for p, v in enumerate([1., 3., 5.]):
        ks.append(x(v), [0], [p], 2, p + 1)
    out = ks.append(x(7.), [0], [3], 2, 4)
    assert out.shape == (2, 4, 1, 2)
    q = np.zeros((1, 2, 2), np.float32)
    close(O.attend_rows(q, out, out, [0], [3], "causal", 1.0).reshape(-1)[::4], [4.])


def test_noise_stream():
    # engine/ir/testkit/src/noise.rs:1-10: values lie in [-1, 1) and the stream is fixed
    a = O.Noise(7).draw(1000)
    assert a.min() >= -1.0 and a.max() < 1.0
    s = (7 * 6364136223846793005 + 1442695040888963407) % (1 << 64)
    assert a[0] == np.float32((s >> 40) / float(1 << 23) - 1.0)
    assert np.array_equal(a, O.Noise(7).draw(1000))


def test_bf16_rounds_to_even():
    # engine/ir/graph/src/scalar.rs:21-43
    cases = {1.0: 0x3F80, 1.00390625: 0x3F80, 1.01171875: 0x3F82, -2.5: 0xC020, 0.0: 0x0000}
    for x, bits in cases.items():
        assert int(O.bf16_bits([x])[0]) == bits, x
    assert int(O.bf16_bits([math.nan])[0]) & 0x7FC0 == 0x7FC0
    assert int(O.bf16_bits([math.inf])[0]) == 0x7F80
    import torch
    x = O.Noise(3).draw(4096) * 100
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.bf16_bits(x), want)


def test_kept_rows():
    # engine/plan/codegen/src/kept.rs:135-194
    assert O.kept_row("dense", 2, 5, 8) == 21
    assert O.kept_row("interleaved", 2, 5, 4) == 22
    table = np.array([3, 0, 2, 1], np.uint32)  # 2 slots x 2 pages
    assert O.kept_row("paged16", 1, 17, 2, table) == (1 << 4) | 1
    assert O.kept_row("paged", 0, 70, 2, table) == (0 << 6) | 6
    assert O.kept_row("paged", 1, 3, 2, table) == (2 << 6) | 3
