"""Parity at the benchmark configurations' own sizes.

The other test files check each kernel on small and awkward shapes; here every isolated configuration runs at full
size on the device and the CPU checker judges a sample of it (the checker is single-threaded C: full outputs at
these sizes would take hours, a few rows and columns take seconds).  Samples always hold the first and last row
and column of the output, the edges of the first and last tile, and seeded random picks in between.

Tolerances are the build's per-op bars: bf16 outputs with f32 sums within 1e-2 of the checker relative to the
largest magnitude of the sample; integer outputs (router ids, token permutation) bit-exact.
"""
import numpy as np
import pytest
import torch

import oracle as O
from tests.util import dev_u32, from_bits, normal_bf16, rel_error, to_bits, u32, widen

pytestmark = pytest.mark.gpu

TOL = 1e-2

# (N, K): q-proj, kv-proj, o-proj, fused gate/up, down, lm-head of the Qwen3-0.6B shape
LINEAR_SHAPES = [(2048, 1024), (1024, 1024), (1024, 2048), (6144, 1024), (1024, 3072), (151936, 1024)]
LINEAR_ROWS = [1, 16, 64, 128, 2048, 8192]


def _sample(n, count, rng, edges=(0, 1, 63, 64, 127, 128, 255, 256)):
    picks = {i for i in edges if i < n} | {n - 1 - i for i in edges if i < n}
    want = min(count, n)
    while len(picks) < want:
        picks.add(int(rng.integers(0, n)))
    return np.array(sorted(picks)[:max(want, 1)] if len(picks) > want else sorted(picks))


@pytest.fixture(scope="module")
def linear_weights():
    """One seeded weight matrix per shape, made on the device (N(0, 0.02), rounded to bf16) and kept for every m."""
    out = {}
    for n, k in LINEAR_SHAPES:
        g = torch.Generator(device="cuda").manual_seed(n * 7 + k)
        out[(n, k)] = (torch.randn((n, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    return out


@pytest.mark.parametrize("m", LINEAR_ROWS)
@pytest.mark.parametrize("n,k", LINEAR_SHAPES)
def test_linear_sweep_matches_oracle(linear_weights, m, n, k):
    """Every (M, N, K) of the isolated linear sweep through the kernel the sizes pick (path "auto"): skinny,
    streaming, tiled and paired-SM kernels all appear.  bf16 out; a second run must give the same bits."""
    from tessera_b200 import ops
    rng = np.random.default_rng(m * 31 + n + k)
    w = linear_weights[(n, k)]
    g = torch.Generator(device="cuda").manual_seed(m * 13 + n)
    x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    got = ops.linear(x, w)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    rows, cols = _sample(m, 12, rng), _sample(n, 96, rng)
    want = O.matmul(O.bf16_widen(to_bits(x[rows])), to_bits(w[cols]))
    sample = widen(got[rows][:, cols])
    assert rel_error(sample, want) <= TOL, (m, n, k)
    again = ops.linear(x, w)
    torch.cuda.synchronize()
    assert torch.equal(got, again)


def test_causal_prefill_4_by_4096():
    """Config 3a: 4 sequences x 4096 tokens, 16 query / 8 kv heads x 128, causal; 40 sampled query rows a sequence
    (the first and last rows, the rows either side of every 128-row tile edge near the ends, random ones between)."""
    from tessera_b200 import ops
    seqs, n, heads, kv_heads, width = 4, 4096, 16, 8, 128
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn((seqs, n, heads, width), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn((seqs, n, kv_heads, width), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((seqs, n, kv_heads, width), generator=g, device="cuda").to(torch.bfloat16)
    scale = float(1.0 / np.sqrt(width))
    got = ops.attend(q, k, v, mask="causal", scale=scale)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    rng = np.random.default_rng(3)
    for s in range(seqs):
        rows = _sample(n, 40, rng)
        kd, vd = O.bf16_widen(to_bits(k[s:s + 1])), O.bf16_widen(to_bits(v[s:s + 1]))
        want = O.attend_rows(O.bf16_widen(to_bits(q[s, rows])), kd, vd, [0] * len(rows), rows.tolist(), "causal", scale)
        assert rel_error(widen(got[s, rows]), want) <= TOL, s


@pytest.mark.parametrize("page", [64, 16])
def test_paged_decode_64_ragged_sequences(page):
    """Config 3b: batch 64, context lengths uniform in [512, 8192] (seed 4), the kept rows in pages behind a seeded
    random page table; every row is checked."""
    from tessera_b200 import ops, synth
    slots, heads, kv_heads, width = 64, 16, 8, 128
    rng = np.random.default_rng(4)
    lengths = rng.integers(512, 8193, size=slots)
    context = 8192
    pages = context // page
    table = synth.page_permutation(slots * pages, seed=4)
    total = slots * pages * page
    kb = torch.zeros((total, kv_heads, width), dtype=torch.bfloat16, device="cuda")
    vb = torch.zeros_like(kb)
    q = normal_bf16(rng, (slots, heads, width))
    scale = float(1.0 / np.sqrt(width))
    wants = []
    for s in range(slots):
        n = int(lengths[s])
        ks, vs = normal_bf16(rng, (n, kv_heads, width)), normal_bf16(rng, (n, kv_heads, width))
        pos = np.arange(n)
        rows = table[s * pages + pos // page].astype(np.int64) * page + pos % page
        at = torch.from_numpy(rows).cuda()
        kb[at], vb[at] = from_bits(ks), from_bits(vs)
        wants.append(O.attend_rows(O.bf16_widen(q[s:s + 1]), O.bf16_widen(ks)[None], O.bf16_widen(vs)[None], [0], [n - 1],
                                   "causal", scale)[0])
    kept = ops.Kept("paged" if page == 64 else "paged16", pages, dev_u32(table), total)
    got = ops.attend_rows(from_bits(q), kb, vb, dev_u32(np.arange(slots)), dev_u32(lengths - 1), kept, context, scale=scale)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert rel_error(widen(got), np.stack(wants)) <= TOL
    again = ops.attend_rows(from_bits(q), kb, vb, dev_u32(np.arange(slots)), dev_u32(lengths - 1), kept, context, scale=scale)
    torch.cuda.synchronize()
    assert torch.equal(got, again)


@pytest.mark.parametrize("seed", range(8))
def test_router_ids_bit_exact_at_the_moe_shape(seed):
    """Config 5's router: 256 rows x 128 experts over hidden 4096, top-8, scores from the device linear.  The
    ids must equal the checker's bit for bit: any flip counts, there is no tolerance on integer outputs."""
    from tessera_b200 import ops
    rows, experts, hidden, top = 256, 128, 4096, 8
    rng = np.random.default_rng(100 + seed)
    h = normal_bf16(rng, (rows, hidden))
    router = normal_bf16(rng, (experts, hidden), 0.02)
    scores = ops.router_scores(from_bits(h), from_bits(router))
    ids = ops.top_k(scores, top)
    gates = ops.take_softmax(scores, ids)
    torch.cuda.synchronize()
    want_scores = O.matmul(O.bf16_widen(h), router)
    want_ids = O.top_k(want_scores, top)
    assert np.array_equal(u32(ids), want_ids)
    assert rel_error(widen(gates), O.softmax(O.take(want_scores, want_ids))) <= 1e-4


def test_moe_layer_at_full_shape_on_sampled_rows():
    """One routed block at config 5's size (256 rows, hidden 4096, 128 experts of ffn 1536, top-8) through
    ts_moe_bf16; the checker recomputes three sampled rows from the experts those rows picked."""
    from tessera_b200 import ops
    rows, experts, hidden, ffn, top = 256, 128, 4096, 1536, 8
    g = torch.Generator(device="cuda").manual_seed(5)
    h = torch.randn((rows, hidden), generator=g, device="cuda").to(torch.bfloat16)
    router = (torch.randn((experts, hidden), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    w_in = (torch.randn((experts, 2 * ffn, hidden), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    w_out = (torch.randn((experts, hidden, ffn), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    scores = ops.router_scores(h, router)
    ids = ops.top_k(scores, top)
    gates = ops.take_softmax(scores, ids)
    y = ops.moe(h, ids, gates, w_in, w_out)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    want_scores = O.matmul(O.bf16_widen(to_bits(h)), to_bits(router))
    want_ids = O.top_k(want_scores, top)
    assert np.array_equal(u32(ids), want_ids)
    want_gates = O.softmax(O.take(want_scores, want_ids))
    for r in (0, 131, 255):
        x = O.bf16_widen(to_bits(h[r:r + 1]))
        out = np.zeros((top, hidden), np.float32)
        for j, e in enumerate(want_ids[r]):
            wi = O.bf16_widen(to_bits(w_in[int(e)]))
            out[j] = O.swiglu(x, wi[:ffn], wi[ffn:], O.bf16_widen(to_bits(w_out[int(e)])), round_inner=True)[0]
        want = O.mean(out[None], 1, weights=want_gates[r:r + 1])[0]
        assert rel_error(widen(y[r]), want) <= TOL, r
