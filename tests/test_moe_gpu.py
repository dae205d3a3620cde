"""Routed experts against the CPU checker (engine/models/src/decoder.rs:70-84 composed from the
checker's matmul_picked, top_k, take, softmax and mix).

Router ids and the token permutation are integer work: bit-exact.  Expert outputs are f32 sums of
bf16 products with a bf16 inner row: within 1e-2 of the checker relative to the largest output
(engine/rules/linear/tests/lanes_test.rs:112-149 asks `picked` for 1e-3 relative and cos > 0.9999 in
f32; the bf16 inner row sets the looser bar here, the cosine bar is kept)."""
import numpy as np
import pytest
import torch

import oracle as O
from tests.util import dev_u32, from_bits, normal_bf16, rel_error, u32, widen

pytestmark = pytest.mark.gpu


def _weights(rng, experts, hidden, ffn):
    w_in = normal_bf16(rng, (experts, 2 * ffn, hidden), 0.05)
    w_out = normal_bf16(rng, (experts, hidden, ffn), 0.05)
    return w_in, w_out


def _cos(a, b):
    a, b = a.reshape(-1).astype(np.float64), b.reshape(-1).astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30))


@pytest.mark.parametrize("picks,experts,first", [(2048, 128, 0), (100, 16, 0), (333, 16, 8), (5, 4, 0), (64, 1, 0)])
def test_permutation_is_stable_and_exact(picks, experts, first):
    from tessera_b200 import ops
    rng = np.random.default_rng(picks + experts)
    total = experts + 2 * first
    ids = rng.integers(0, max(total, 1), size=picks).astype(np.uint32)
    order, place, offsets, tiles = [u32(t) for t in ops.moe_permutation(dev_u32(ids), experts, first)]
    local = (ids >= first) & (ids - first < experts)
    want_order = np.array(sorted(np.nonzero(local)[0], key=lambda i: (ids[i], i)), np.uint32)  # stable by pick index
    n = want_order.size
    assert np.array_equal(order[:n], want_order)
    counts = np.bincount(ids[local] - first, minlength=experts)
    assert np.array_equal(offsets, np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32))
    assert np.array_equal(tiles, np.concatenate([[0], np.cumsum((counts + 31) // 32)]).astype(np.uint32))
    want_place = np.full(picks, 0xFFFFFFFF, np.uint32)
    want_place[want_order] = np.arange(n, dtype=np.uint32)
    assert np.array_equal(place, want_place)


@pytest.mark.parametrize("rows,experts,top,hidden,ffn", [(24, 8, 2, 256, 128), (256, 16, 4, 512, 256), (7, 4, 4, 128, 64)])
def test_moe_block_matches_oracle(rows, experts, top, hidden, ffn):
    from tessera_b200 import ops
    rng = np.random.default_rng(rows * 3 + experts)
    h = normal_bf16(rng, (rows, hidden))
    router = normal_bf16(rng, (experts, hidden), 0.1)
    w_in, w_out = _weights(rng, experts, hidden, ffn)
    want, want_ids, want_gates = O.moe_block(O.bf16_widen(h), O.bf16_widen(router), O.bf16_widen(w_in),
                                             O.bf16_widen(w_out), top, round_inner=True)
    hd = from_bits(h)
    scores = ops.linear(hd, from_bits(router), out_dtype=torch.float32)
    ids = ops.top_k(scores, top)
    gates = ops.take_softmax(scores, ids)
    torch.cuda.synchronize()
    assert np.array_equal(u32(ids), want_ids)          # router indices: bit-exact
    assert rel_error(widen(gates), want_gates) <= 1e-4
    y = ops.moe(hd, ids, gates, from_bits(w_in), from_bits(w_out))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = widen(y)
    assert rel_error(got, want) <= 1e-2 and _cos(got, want) > 0.9999


def test_experts_held_elsewhere_give_zero_and_parts_add_up():
    # The reference splits experts over ranks: each computes its own picks, the others read zeros, and
    # the parts sum to the whole (engine/rules/linear/src/picked.rs:49-59, interp cpu.rs:100-104).
    from tessera_b200 import ops
    rng = np.random.default_rng(9)
    rows, experts, top, hidden, ffn = 40, 8, 2, 256, 128
    h = normal_bf16(rng, (rows, hidden))
    w_in, w_out = _weights(rng, experts, hidden, ffn)
    ids = rng.integers(0, experts, size=(rows, top)).astype(np.uint32)
    gates = rng.random((rows, top), dtype=np.float32)
    hd, idd, gd = from_bits(h), dev_u32(ids), torch.from_numpy(gates).cuda()
    whole = widen(ops.moe(hd, idd, gd, from_bits(w_in), from_bits(w_out)))
    parts = np.zeros_like(whole)
    for first in (0, 4):
        part = widen(ops.moe(hd, idd, gd, from_bits(w_in[first:first + 4]), from_bits(w_out[first:first + 4]), first=first))
        want, _, _ = None, None, None
        parts += part
    assert rel_error(parts, whole) <= 1e-5
    # per-pick outputs: a pick of an expert held elsewhere is a zero row
    out = widen(ops.moe_experts(hd, idd.reshape(-1), from_bits(w_in[:4]), from_bits(w_out[:4]), repeat=top, first=0))
    away = ids.reshape(-1) >= 4
    assert np.all(out[away] == 0.0) and np.all(np.abs(out[~away]).max(axis=1) > 0)


def test_shared_expert_adds_in():
    from tessera_b200 import ops
    rng = np.random.default_rng(10)
    rows, experts, top, hidden, ffn = 16, 4, 2, 128, 64
    h = normal_bf16(rng, (rows, hidden))
    w_in, w_out = _weights(rng, experts, hidden, ffn)
    ids = rng.integers(0, experts, size=(rows, top)).astype(np.uint32)
    gates = np.full((rows, top), 0.5, np.float32)
    add = rng.standard_normal((rows, hidden), dtype=np.float32)
    base = widen(ops.moe(from_bits(h), dev_u32(ids), torch.from_numpy(gates).cuda(), from_bits(w_in), from_bits(w_out)))
    with_add = widen(ops.moe(from_bits(h), dev_u32(ids), torch.from_numpy(gates).cuda(), from_bits(w_in), from_bits(w_out),
                             add=torch.from_numpy(add).cuda()))
    assert np.allclose(with_add, base + add, rtol=1e-6, atol=1e-6)


def test_uneven_routing_many_rows_on_one_expert():
    # more rows on one expert than a batch tile holds, and experts with none
    from tessera_b200 import ops
    rng = np.random.default_rng(11)
    rows, experts, hidden, ffn = 150, 6, 256, 128
    h = normal_bf16(rng, (rows, hidden))
    w_in, w_out = _weights(rng, experts, hidden, ffn)
    ids = np.where(np.arange(rows) % 10 == 0, 5, 2).astype(np.uint32).reshape(rows, 1)
    gates = np.ones((rows, 1), np.float32)
    want = np.zeros((rows, hidden), np.float32)
    hs = O.bf16_widen(h)
    for e in (2, 5):
        sel = ids[:, 0] == e
        want[sel] = O.swiglu(hs[sel], O.bf16_widen(w_in[e, :ffn]), O.bf16_widen(w_in[e, ffn:]), O.bf16_widen(w_out[e]),
                             round_inner=True)
    got = widen(ops.moe(from_bits(h), dev_u32(ids), torch.from_numpy(gates).cuda(), from_bits(w_in), from_bits(w_out)))
    assert rel_error(got, want) <= 1e-2


@pytest.mark.parametrize("rows,repeat,count,first,n,k", [(64, 4, 8, 0, 256, 128), (300, 1, 16, 4, 128, 192), (7, 7, 3, 0, 384, 64)])
def test_picked_alone_matches_oracle(rows, repeat, count, first, n, k):
    """The reference's `picked` launch (picked.rs:28-60): each row against the matrix its id names, the gate or
    the up half of a fused table through stride / offset, zeros for ids this rank does not hold."""
    from tessera_b200 import ops, rules
    rng = np.random.default_rng(rows + n)
    x = normal_bf16(rng, (rows // repeat, k))
    table = normal_bf16(rng, (count, 2 * n, k), 0.05)          # two halves per matrix, as gate | up
    ids = rng.integers(0, count + 2 * first, size=rows).astype(np.uint32)
    xd, td, idd = from_bits(x), from_bits(table), dev_u32(ids)
    for offset in (0, n):
        want = O.matmul_picked(O.bf16_widen(x), O.bf16_widen(table)[:, offset:offset + n], ids, first)
        got = ops.picked(xd, td, idd, n, count=count, stride=2 * n, offset=offset, repeat=repeat, first=first)
        torch.cuda.synchronize()
        assert ops.device_status() == 0
        held = (ids >= first) & (ids - first < count)
        assert not widen(got)[~held].any()                    # exactly zero, not small
        assert rel_error(widen(got), want) <= 1e-2 and _cos(widen(got), want) > 0.9999
        by_name = torch.full((rows, n), 7.0, dtype=torch.float32, device="cuda")
        rules.launch_c("picked_bf16", [xd, td, idd, by_name, rows, n, k, count, 2 * n, offset, repeat, first])
        assert torch.equal(by_name, got)                       # same kernels, same order: same bits


def test_picked_refuses_what_it_cannot_tile():
    from tessera_b200 import ops
    from tessera_b200._lib import TesseraError
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((2, 100, 64), dtype=torch.bfloat16, device="cuda")
    ids = dev_u32([0, 1, 0, 1])
    with pytest.raises(TesseraError):
        ops.picked(x, w, ids, 100)                             # n is not a multiple of 128
    w = torch.zeros((2, 128, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(TesseraError):
        ops.picked(x, w, ids, 128, stride=64)                  # matrices would overlap
