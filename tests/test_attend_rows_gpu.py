"""Paged / dense ragged attention and the append kernels against the CPU checker.

The checker keeps a dense [slots, keys, kv_heads, width] store; paging is a pure address
permutation, so checker(dense) must equal kernel(any layout, any table).  Page-table gathers
are integer work and are checked bit-exactly through the appended rows; attention outputs are
bf16 with f32 sums and must sit within 1e-2 of the checker relative to the largest output
(cases follow engine/rules/attention/tests/attention_test.rs:145-236: dense and paged16 with a
reversed page table, two successive launches into the same store).
"""
import numpy as np
import pytest
import torch

import oracle as O
from tests.util import dev_u32, from_bits, normal_bf16, rel_error, to_bits, widen

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _layout(name, slots, context, rng, order="random"):
    """Returns (ops.Kept, kept_rows(slot, pos) -> row as numpy fn, total rows)."""
    from tessera_b200 import ops
    if name == "dense":
        return ops.Kept("dense", context, None, slots * context), (lambda s, p: s * context + p), slots * context
    if name == "interleaved":
        return ops.Kept("interleaved", slots, None, slots * context), (lambda s, p: p * slots + s), slots * context
    page = O.PAGE[name]
    pages = -(-context // page)
    total = slots * pages
    if order == "reversed":
        table = np.arange(total, dtype=np.uint32)[::-1].copy()
    elif order == "identity":
        table = np.arange(total, dtype=np.uint32)
    else:
        table = rng.permutation(total).astype(np.uint32)
    kept = ops.Kept(name, pages, dev_u32(table), total * page)
    shift = page.bit_length() - 1

    def row(s, p):
        return (int(table[s * pages + (p >> shift)]) << shift) | (p & (page - 1))
    return kept, row, total * page


def _fill_store(rng, slots, lengths, kv_heads, width, row_fn, total_rows):
    """Dense checker store plus the same rows placed by row_fn into the device layout."""
    context = max(lengths)
    kd = np.zeros((slots, context, kv_heads, width), np.float32)
    vd = np.zeros_like(kd)
    kb = np.zeros((total_rows, kv_heads, width), np.uint16)
    vb = np.zeros_like(kb)
    for s in range(slots):
        n = lengths[s]
        kbits = normal_bf16(rng, (n, kv_heads, width))
        vbits = normal_bf16(rng, (n, kv_heads, width))
        kd[s, :n] = O.bf16_widen(kbits)
        vd[s, :n] = O.bf16_widen(vbits)
        rows = np.array([row_fn(s, p) for p in range(n)])
        kb[rows] = kbits
        vb[rows] = vbits
    return kd, vd, kb, vb


@pytest.mark.parametrize("layout,order", [("dense", ""), ("interleaved", ""), ("paged16", "reversed"),
                                          ("paged", "random"), ("paged16", "random")])
@pytest.mark.parametrize("heads,kv_heads,width", [(16, 8, 128), (4, 4, 128), (8, 2, 128), (4, 2, 64)])
def test_rows_match_oracle(layout, order, heads, kv_heads, width):
    from tessera_b200 import ops
    rng = np.random.default_rng(hash((layout, heads, width)) % 1000)
    slots = 6
    lengths = [int(v) for v in rng.integers(1, 300, size=slots)]
    lengths[0], lengths[1] = 1, 257
    context = max(lengths)
    kept, row_fn, total = _layout(layout, slots, context, rng, order or "random")
    kd, vd, kb, vb = _fill_store(rng, slots, lengths, kv_heads, width, row_fn, total)
    # one row per slot at its last position, plus two mid-sequence rows
    row_slots = list(range(slots)) + [1, 1]
    row_pos = [n - 1 for n in lengths] + [100, 31]
    q = normal_bf16(rng, (len(row_slots), heads, width))
    scale = 1.0 / np.sqrt(width)
    want = O.attend_rows(O.bf16_widen(q), kd, vd, row_slots, row_pos, "causal", scale)
    got = ops.attend_rows(from_bits(q), from_bits(kb), from_bits(vb), dev_u32(row_slots), dev_u32(row_pos), kept,
                          context, scale=float(scale))
    torch.cuda.synchronize()
    assert rel_error(widen(got), want) <= TOL


@pytest.mark.parametrize("page_layout,kv_heads", [("paged", 8), ("paged16", 8), ("paged", 4), ("dense", 4)])
def test_long_ragged_contexts_split_and_merge(page_layout, kv_heads):
    # the decode shape of the isolated attention config, scaled down: contexts 40..2100, GQA 16/8 (two heads
    # per key: the scalar kernels) and 16/4 (four: the warp-MMA kernel)
    from tessera_b200 import ops
    rng = np.random.default_rng(4)
    slots, heads, width = 5, 16, 128
    lengths = [40, 513, 1024, 2100, 777]
    context = max(lengths)
    kept, row_fn, total = _layout(page_layout, slots, context, rng)
    kd, vd, kb, vb = _fill_store(rng, slots, lengths, kv_heads, width, row_fn, total)
    row_slots = list(range(slots))
    row_pos = [n - 1 for n in lengths]
    q = normal_bf16(rng, (slots, heads, width))
    scale = 1.0 / np.sqrt(width)
    want = O.attend_rows(O.bf16_widen(q), kd, vd, row_slots, row_pos, "causal", scale)
    args = (from_bits(q), from_bits(kb), from_bits(vb), dev_u32(row_slots), dev_u32(row_pos), kept, context)
    got = ops.attend_rows(*args, scale=float(scale))
    again = ops.attend_rows(*args, scale=float(scale))
    torch.cuda.synchronize()
    assert rel_error(widen(got), want) <= TOL
    assert torch.equal(got, again)  # fixed merge order: same bits on a re-run


@pytest.mark.parametrize("kv_heads", [4, 2])
@pytest.mark.parametrize("layout", ["dense", "paged"])
def test_unwritten_rows_may_hold_anything(layout, kv_heads):
    # Rows past a slot's last position (a page's tail, a dense slot's unused part) are never written;
    # whatever bits they hold must not reach the output.
    from tessera_b200 import ops
    rng = np.random.default_rng(21)
    slots, heads, width = 4, 8, 128
    lengths = [1, 33, 70, 190]
    context = 256
    kept, row_fn, total = _layout(layout, slots, context, rng)
    kd, vd, kb, vb = _fill_store(rng, slots, lengths, kv_heads, width, row_fn, total)
    written = np.zeros(total, bool)
    for s in range(slots):
        written[[row_fn(s, p) for p in range(lengths[s])]] = True
    kb[~written] = 0x7FC0  # NaN
    vb[~written] = 0x7F80  # +inf
    row_slots, row_pos = list(range(slots)), [n - 1 for n in lengths]
    q = normal_bf16(rng, (slots, heads, width))
    want = O.attend_rows(O.bf16_widen(q), kd[:, :max(lengths)], vd[:, :max(lengths)], row_slots, row_pos, "causal", 0.09)
    got = ops.attend_rows(from_bits(q), from_bits(kb), from_bits(vb), dev_u32(row_slots), dev_u32(row_pos), kept,
                          context, scale=0.09)
    torch.cuda.synchronize()
    assert torch.isfinite(got.float()).all()
    assert rel_error(widen(got), want) <= TOL


def test_window_back():
    # Mask::Back(n): keys at most n back (engine/ir/graph/src/node.rs:162-187)
    from tessera_b200 import ops
    rng = np.random.default_rng(12)
    slots, heads, kv_heads, width, n = 3, 4, 2, 128, 200
    kept, row_fn, total = _layout("paged", slots, n, rng)
    kd, vd, kb, vb = _fill_store(rng, slots, [n] * slots, kv_heads, width, row_fn, total)
    row_slots, row_pos = [0, 1, 2, 2], [199, 150, 10, 70]
    q = normal_bf16(rng, (4, heads, width))
    want = O.attend_rows(O.bf16_widen(q), kd, vd, row_slots, row_pos, ("back", 37), 0.1)
    got = ops.attend_rows(from_bits(q), from_bits(kb), from_bits(vb), dev_u32(row_slots), dev_u32(row_pos), kept, n,
                          scale=0.1, back=37)
    torch.cuda.synchronize()
    assert rel_error(widen(got), want) <= TOL


@pytest.mark.parametrize("layout", ["dense", "paged", "paged16"])
def test_norm_rope_append_then_attend_two_launches(layout):
    # Two successive launches into the same kept rows (attention_test.rs:145-236), through the
    # fused per-head norm + rotation + append; appended rows must equal the checker's bits.
    from tessera_b200 import ops
    rng = np.random.default_rng(21)
    slots, heads, kv_heads, width, context = 3, 4, 2, 128, 40
    eps, theta = 1e-6, 1e6
    kept, row_fn, total = _layout(layout, slots, context, rng, "reversed")
    k_rows = torch.zeros((total, kv_heads, width), dtype=torch.bfloat16, device="cuda")
    v_rows = torch.zeros_like(k_rows)
    qn = rng.standard_normal(width).astype(np.float32)
    kn = rng.standard_normal(width).astype(np.float32)
    inv_freq = ops.rope_inv_freq(theta, width, "cuda")
    kd = np.zeros((slots, context, kv_heads, width), np.float32)
    vd = np.zeros_like(kd)
    launches = [([0, 0, 0, 1, 2, 2], [0, 1, 2, 0, 0, 1]), ([0, 1, 1, 2], [3, 1, 2, 2])]
    for row_slots, row_pos in launches:
        rows = len(row_slots)
        qkv = normal_bf16(rng, (rows, (heads + 2 * kv_heads) * width))
        wide = O.bf16_widen(qkv).reshape(rows, heads + 2 * kv_heads, width)
        q = O.bf16_round(O.rope(O.rms_norm(wide[:, :heads], qn, eps), row_pos, theta, "halves"))
        k = O.bf16_round(O.rope(O.rms_norm(wide[:, heads:heads + kv_heads], kn, eps), row_pos, theta, "halves"))
        v = wide[:, heads + kv_heads:]
        for r, (s, p) in enumerate(zip(row_slots, row_pos)):
            kd[s, p], vd[s, p] = k[r], v[r]
        q_out = torch.empty((rows, heads, width), dtype=torch.bfloat16, device="cuda")
        ds, dp = dev_u32(row_slots), dev_u32(row_pos)
        ops.qk_norm_rope_append(from_bits(qkv), torch.from_numpy(qn).cuda(), torch.from_numpy(kn).cuda(), inv_freq, ds,
                                dp, q_out, k_rows, v_rows, kept, heads, kv_heads, width, eps)
        torch.cuda.synchronize()
        # rotation goes through sin/cos of the device's libm: allow one bf16 step on q and k
        assert rel_error(widen(q_out), q) <= 1e-2
        placed = np.array([row_fn(s, p) for s, p in zip(row_slots, row_pos)])
        assert np.array_equal(to_bits(v_rows)[placed], O.bf16_bits(v))  # values are copied: bit-exact
        assert rel_error(widen(k_rows)[placed], k) <= 1e-2
        keys = max(row_pos) + 1
        want = O.attend_rows(q, kd, vd, row_slots, row_pos, "causal", 0.3)
        got = ops.attend_rows(q_out, k_rows, v_rows, ds, dp, kept, keys, scale=0.3)
        torch.cuda.synchronize()
        assert rel_error(widen(got), want) <= 2e-2  # q and k carry the rotation's rounding


@pytest.mark.parametrize("layout,heads,kv_heads,context", [("dense", 16, 8, 200), ("paged", 16, 8, 200), ("paged", 8, 2, 700),
                                                           ("paged", 4, 4, 1500)])
def test_append_inside_attention_equals_the_two_launches(layout, heads, kv_heads, context):
    # A decode step (every row in a slot of its own): one launch that norms, rotates, appends and attends
    # must leave the same kept rows and the same outputs, bit for bit, as append followed by attention.
    from tessera_b200 import ops
    rng = np.random.default_rng(heads * 7 + context)
    slots, width, eps, theta = 9, 128, 1e-6, 1e6
    kept, row_fn, total = _layout(layout, slots, context, rng)
    lengths = [int(v) for v in rng.integers(1, context, size=slots)]
    lengths[0], lengths[1], lengths[2] = 1, 33, context   # first position, just past a tile, the last position
    # the past of every slot (at least one row, so that the store's shape is fixed); the row at the last
    # position is what the launches append
    kd, vd, kb, vb = _fill_store(rng, slots, [max(n - 1, 1) for n in lengths], kv_heads, width, row_fn, total)
    row_slots = list(rng.permutation(slots))[:7]
    row_pos = [lengths[s] - 1 for s in row_slots]
    rows = len(row_slots)
    qkv = from_bits(normal_bf16(rng, (rows, (heads + 2 * kv_heads) * width)))
    qn = torch.from_numpy(rng.standard_normal(width).astype(np.float32)).cuda()
    kn = torch.from_numpy(rng.standard_normal(width).astype(np.float32)).cuda()
    inv_freq = ops.rope_inv_freq(theta, width, "cuda")
    ds, dp = dev_u32(row_slots), dev_u32(row_pos)

    k1, v1 = from_bits(kb), from_bits(vb)
    q_out = torch.empty((rows, heads, width), dtype=torch.bfloat16, device="cuda")
    ops.qk_norm_rope_append(qkv, qn, kn, inv_freq, ds, dp, q_out, k1, v1, kept, heads, kv_heads, width, eps)
    want = ops.attend_rows(q_out, k1, v1, ds, dp, kept, context, scale=0.11)

    k2, v2 = from_bits(kb), from_bits(vb)
    got = ops.attend_rows_append(qkv, qn, kn, inv_freq, k2, v2, ds, dp, kept, context, heads, eps=eps, scale=0.11)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    assert torch.equal(got, want)


def test_append_inside_attention_refuses_other_layouts():
    from tessera_b200 import TesseraError, ops
    rng = np.random.default_rng(1)
    kept, row_fn, total = _layout("paged16", 2, 64, rng)
    z = torch.zeros((total, 2, 128), dtype=torch.bfloat16, device="cuda")
    qkv = torch.zeros((2, 8 * 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(TesseraError):
        ops.attend_rows_append(qkv, None, None, ops.rope_inv_freq(1e6, 128, "cuda"), z, z.clone(), dev_u32([0, 1]),
                               dev_u32([3, 4]), kept, 64, 4, eps=1e-6, scale=0.1)


def test_scatter_places_rows_bit_exactly():
    from tessera_b200 import ops
    rng = np.random.default_rng(2)
    slots, context, width = 4, 100, 256
    for layout in ("dense", "interleaved", "paged", "paged16"):
        kept, row_fn, total = _layout(layout, slots, context, rng)
        out = torch.zeros((total, width), dtype=torch.bfloat16, device="cuda")
        row_slots = rng.integers(0, slots, size=50)
        row_pos = rng.permutation(context)[:50]
        x = normal_bf16(rng, (50, width))
        ops.scatter(from_bits(x), dev_u32(row_slots), dev_u32(row_pos), out, kept)
        torch.cuda.synchronize()
        placed = np.array([row_fn(int(s), int(p)) for s, p in zip(row_slots, row_pos)])
        want = np.zeros((total, width), np.uint16)
        want[placed] = x
        assert np.array_equal(to_bits(out), want)
        # and the device's address agrees with the checker's kept_row
        table = None if kept.table is None else kept.table.cpu().numpy().view(np.uint32)
        for s, p, r in zip(row_slots[:8], row_pos[:8], placed[:8]):
            assert O.kept_row(layout, int(s), int(p), kept.scalar, table) == r
