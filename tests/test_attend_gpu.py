"""Whole-sequence attention (tcgen05 path at width 128, ragged-rows path at widths 64 / 256)
against the CPU checker, over the case grid of engine/rules/attention/tests/attention_test.rs:43-102
(sequence/row/key counts x masks x head shapes).  bf16 outputs with f32 sums: within 1e-2 of the
checker relative to the largest output."""
import numpy as np
import pytest
import torch

import oracle as O
from tests.util import dev_u32, from_bits, normal_bf16, rel_error, widen

pytestmark = pytest.mark.gpu
TOL = 1e-2

CASES = [(1, 128, 128), (2, 200, 200), (2, 70, 300), (1, 513, 513), (3, 1, 257), (1, 1000, 1000)]
MASKS = ["causal", "bidirectional", ("within", 17), ("back", 33), ("back", 300)]
HEADS = [(16, 8, 128), (4, 4, 128), (8, 2, 128)]


def _run(q, k, v, mask, scale, **kw):
    from tessera_b200 import ops
    out = ops.attend(from_bits(q), from_bits(k), from_bits(v), mask=mask, scale=scale, **kw)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return widen(out)


@pytest.mark.parametrize("seqs,queries,keys", CASES)
@pytest.mark.parametrize("mask", MASKS)
def test_flash_matches_oracle(seqs, queries, keys, mask):
    heads, kv_heads, width = 4, 2, 128
    rng = np.random.default_rng(seqs * 1000 + queries + keys)
    q = normal_bf16(rng, (seqs, queries, heads, width))
    k = normal_bf16(rng, (seqs, keys, kv_heads, width))
    v = normal_bf16(rng, (seqs, keys, kv_heads, width))
    scale = float(1.0 / np.sqrt(width))
    want = O.attend(O.bf16_widen(q), O.bf16_widen(k), O.bf16_widen(v), mask, scale)
    got = _run(q, k, v, mask, scale)
    assert rel_error(got, want) <= TOL


@pytest.mark.parametrize("heads,kv_heads,width", HEADS + [(4, 2, 64), (3, 1, 256)])
@pytest.mark.parametrize("mask", ["causal", "bidirectional"])
def test_head_shapes(heads, kv_heads, width, mask):
    rng = np.random.default_rng(heads * 7 + width)
    seqs, n = 2, 160
    q = normal_bf16(rng, (seqs, n, heads, width))
    k = normal_bf16(rng, (seqs, n, kv_heads, width))
    v = normal_bf16(rng, (seqs, n, kv_heads, width))
    scale = float(1.0 / np.sqrt(width))
    want = O.attend(O.bf16_widen(q), O.bf16_widen(k), O.bf16_widen(v), mask, scale)
    got = _run(q, k, v, mask, scale)
    assert rel_error(got, want) <= TOL


@pytest.mark.parametrize("mask", ["causal", "bidirectional"])
def test_packed_sequences_width_256(mask):
    # the embedding encoder's attention shape: 3 query heads over 1 kv head, 256 wide, ragged lengths
    rng = np.random.default_rng(6)
    lens = [32, 200, 65, 512, 64, 129]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
    total, heads, kv_heads, width = int(cu[-1]), 3, 1, 256
    q = normal_bf16(rng, (total, heads, width))
    k = normal_bf16(rng, (total, kv_heads, width))
    v = normal_bf16(rng, (total, kv_heads, width))
    scale = float(1.0 / np.sqrt(width))
    got = _run(q, k, v, mask, scale, cu_seqlens=dev_u32(cu), max_len=max(lens))
    for s, n in enumerate(lens):
        a, b = int(cu[s]), int(cu[s + 1])
        want = O.attend(O.bf16_widen(q[a:b])[None], O.bf16_widen(k[a:b])[None], O.bf16_widen(v[a:b])[None], mask, scale)[0]
        assert rel_error(got[a:b], want) <= TOL, (s, n)


def test_large_score_range_rescales():
    # scores that keep growing along the keys force the lagging maximum to be rescaled block after block
    rng = np.random.default_rng(8)
    n, heads, width = 700, 2, 128
    q = normal_bf16(rng, (1, n, heads, width))
    ramp = np.linspace(0.2, 6.0, n, dtype=np.float32)[None, :, None, None]
    k = O.bf16_bits(O.bf16_widen(q[:, :, :1]) * ramp)  # key j aligned with query j, growing norm
    v = normal_bf16(rng, (1, n, 1, width))
    for mask in ("causal", "bidirectional"):
        want = O.attend(O.bf16_widen(q), O.bf16_widen(k), O.bf16_widen(v), mask, 0.5)
        got = _run(q, k, v, mask, 0.5)
        assert rel_error(got, want) <= TOL


@pytest.mark.parametrize("mask", ["causal", "bidirectional"])
def test_packed_sequences(mask):
    # ragged lengths packed back to back, the embedding batch's shape (lengths 32..512)
    rng = np.random.default_rng(5)
    lens = [32, 300, 129, 512, 1, 77]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
    total, heads, kv_heads, width = int(cu[-1]), 4, 2, 128
    q = normal_bf16(rng, (total, heads, width))
    k = normal_bf16(rng, (total, kv_heads, width))
    v = normal_bf16(rng, (total, kv_heads, width))
    scale = 0.1
    got = _run(q, k, v, mask, scale, cu_seqlens=dev_u32(cu), max_len=max(lens))
    for s, n in enumerate(lens):
        a, b = int(cu[s]), int(cu[s + 1])
        want = O.attend(O.bf16_widen(q[a:b])[None], O.bf16_widen(k[a:b])[None], O.bf16_widen(v[a:b])[None], mask, scale)[0]
        assert rel_error(got[a:b], want) <= TOL, (s, n)


def test_causal_first_row_reads_first_value():
    # engine/ir/interp/src/interp_test.rs:76-86 on the device: causal row 0 equals V row 0
    rng = np.random.default_rng(1)
    q = normal_bf16(rng, (2, 130, 4, 128))
    k = normal_bf16(rng, (2, 130, 4, 128))
    v = normal_bf16(rng, (2, 130, 4, 128))
    got = _run(q, k, v, "causal", 0.5)
    assert np.array_equal(got[:, 0], O.bf16_widen(v)[:, 0])


def test_prefill_shape_spot_check():
    # batch 1 x 2048 tokens of the isolated attention configuration (16q / 8kv heads, 128 wide), causal;
    # the checker on a sample of query rows (full checker cost grows with tokens squared)
    rng = np.random.default_rng(3)
    n, heads, kv_heads, width = 2048, 16, 8, 128
    q = normal_bf16(rng, (1, n, heads, width))
    k = normal_bf16(rng, (1, n, kv_heads, width))
    v = normal_bf16(rng, (1, n, kv_heads, width))
    scale = float(1.0 / np.sqrt(width))
    got = _run(q, k, v, "causal", scale)
    rows = [0, 1, 127, 128, 129, 1000, 2047]
    kd, vd = O.bf16_widen(k), O.bf16_widen(v)
    want = O.attend_rows(O.bf16_widen(q)[0, rows], kd, vd, [0] * len(rows), rows, "causal", scale)
    assert rel_error(got[0, rows], want) <= TOL
    again = _run(q, k, v, "causal", scale)
    assert np.array_equal(got, again)  # same bits on a re-run


def test_reference_case_grid_with_its_noise():
    """engine/rules/attention/tests/attention_test.rs:43-102, `flash_matches_cpu`: Noise(41); rows off, on and past
    the block, with older keys; five masks; heads x width (2, 16), (4, 64), (2, 128); q, k, v drawn in that order.
    Inputs are rounded to bf16 here (the reference feeds f32) and the checker sees the rounded values."""
    draws = O.Noise(41)
    cases = [(1, 1, 1), (1, 1, 38), (2, 7, 7), (1, 33, 33), (2, 70, 93), (1, 128, 128)]
    masks = ["causal", "bidirectional", ("within", 5), ("within", 40), ("back", 5)]
    worst = 0.0
    for mask in masks:
        for heads, width in [(2, 16), (4, 64), (2, 128)]:
            for seqs, rows, keys in cases:
                q = O.bf16_bits(draws.draw(seqs, rows, heads, width))
                k = O.bf16_bits(draws.draw(seqs, keys, heads, width))
                v = O.bf16_bits(draws.draw(seqs, keys, heads, width))
                want = O.attend(O.bf16_widen(q), O.bf16_widen(k), O.bf16_widen(v), mask, 1.0)
                got = _run(q, k, v, mask, 1.0)
                off = rel_error(got, want)
                worst = max(worst, off)
                assert off <= TOL, (mask, heads, width, seqs, rows, keys, off)
    print(f"worst relative error over the grid: {worst:.2e}")


@pytest.mark.parametrize("width", [16, 32])
def test_narrow_heads_over_kept_rows(width):
    # ragged rows over paged kept rows at the narrow widths the reference's cases use
    from tessera_b200 import ops
    rng = np.random.default_rng(width)
    slots, context, heads, kv_heads, page = 3, 96, 4, 2, 16
    pages = context // page
    table = rng.permutation(slots * pages).astype(np.uint32)
    kd = normal_bf16(rng, (slots, context, kv_heads, width))
    vd = normal_bf16(rng, (slots, context, kv_heads, width))
    kr = np.zeros((slots * pages * page, kv_heads, width), np.uint16)
    vr = np.zeros_like(kr)
    for s in range(slots):
        for p in range(context):
            at = int(table[s * pages + p // page]) * page + p % page
            kr[at], vr[at] = kd[s, p], vd[s, p]
    row_slots, row_pos = [2, 0, 1, 2], [95, 0, 40, 17]
    q = normal_bf16(rng, (4, heads, width))
    want = O.attend_rows(O.bf16_widen(q), O.bf16_widen(kd), O.bf16_widen(vd), row_slots, row_pos, "causal", 0.25)
    kept = ops.Kept("paged16", pages, dev_u32(table), slots * pages * page)
    got = ops.attend_rows(from_bits(q), from_bits(kr), from_bits(vr), dev_u32(row_slots), dev_u32(row_pos), kept, context,
                          scale=0.25)
    torch.cuda.synchronize()
    assert ops.device_status() == 0 and rel_error(widen(got), want) <= TOL
