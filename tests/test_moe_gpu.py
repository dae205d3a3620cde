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


def test_block_lands_on_the_residual_rows():
    # moe_forward(..., residual=x) is x + block: the shared expert's down projection adds x in its epilogue and the
    # routed mix adds that, with no elementwise launch in between
    from tessera_b200 import moe
    rng = np.random.default_rng(12)
    rows, experts, top, hidden, ffn, shared = 40, 8, 2, 256, 128, 256
    h = from_bits(normal_bf16(rng, (rows, hidden)))
    w_in, w_out = _weights(rng, experts, hidden, ffn)
    w = moe.MoeWeights(from_bits(normal_bf16(rng, (experts, hidden), 0.1)), from_bits(w_in), from_bits(w_out),
                       from_bits(normal_bf16(rng, (2 * shared, hidden), 0.05)), from_bits(normal_bf16(rng, (hidden, shared), 0.05)),
                       first=0, experts_total=experts)
    x = torch.from_numpy(rng.standard_normal((rows, hidden), dtype=np.float32)).cuda()
    base, ids, _ = moe.moe_forward(h, w, top)
    onto, ids2, _ = moe.moe_forward(h, w, top, residual=x)
    torch.cuda.synchronize()
    assert torch.equal(ids, ids2)
    assert torch.allclose(onto, base + x, rtol=1e-5, atol=1e-5)
    w.shared_in = w.shared_out = None          # no shared expert: the residual rows are the add
    bare, _, _ = moe.moe_forward(h, w, top)
    onto, _, _ = moe.moe_forward(h, w, top, residual=x)
    torch.cuda.synchronize()
    assert torch.allclose(onto, bare + x, rtol=1e-5, atol=1e-5)


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


@pytest.mark.parametrize("count,n,k,rows,repeat", [(4, 32, 64, 10, 2), (4, 64, 32, 10, 2), (3, 7, 52, 5, 1), (2, 128, 40, 9, 3)])
def test_picked_takes_every_size(count, n, k, rows, repeat):
    # engine/rules/linear/tests/lanes_test.rs:112-149: two of four experts per row from one stacked set of 64 x 32;
    # sizes off the tiles run the plain kernel (1e-3 relative and cos > 0.9999 is the reference's bar)
    from tessera_b200 import ops
    draws = O.Noise(11)
    table = O.bf16_bits(draws.draw(count, n, k))
    x = O.bf16_bits(draws.draw(-(-rows // repeat), k))
    ids = (np.arange(rows) * 7 % (count + 1)).astype(np.uint32)     # one id past the table: zeros
    each = np.repeat(O.bf16_widen(x), repeat, axis=0)[:rows]       # row i reads x[i // repeat]
    want = O.matmul_picked(each, O.bf16_widen(table), ids, 0)
    got = ops.picked(from_bits(x), from_bits(table), dev_u32(ids), n, count=count, stride=n, repeat=repeat)
    torch.cuda.synchronize()
    assert not widen(got)[ids >= count].any()
    assert rel_error(widen(got), want) <= 1e-3 and _cos(widen(got), want) > 0.9999


def test_picked_refuses_overlapping_matrices():
    from tessera_b200 import ops
    from tessera_b200._lib import TesseraError
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    ids = dev_u32([0, 1, 0, 1])
    w = torch.zeros((2, 128, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(TesseraError):
        ops.picked(x, w, ids, 128, stride=64)                  # matrices would overlap


SMALL_MOE = dict(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=128, experts=8, top=2, ffn=128, shared_ffn=128,
                 eps=1e-6, theta=1e4)


def _moe_decoder_want(dec, x, slots, positions, keys):
    """One decode step of the MoE layer stack from the checker's ops, rounding to bf16 where the device stores bf16."""
    c = dec.cfg
    d, heads, kvh, eps = c["head_dim"], c["heads"], c["kv_heads"], c["eps"]
    rows = x.shape[0]
    table = u32(dec.table)
    x = x.copy()
    for i, L in enumerate(dec.layers):
        h = O.bf16_round(O.rms_norm(x, widen(L["ln1"]), eps))
        qkv = O.bf16_round(O.matmul(h, widen(L["wqkv"])))
        q = qkv[:, :heads * d].reshape(rows, heads, d)
        k = qkv[:, heads * d:(heads + kvh) * d].reshape(rows, kvh, d)
        v = qkv[:, (heads + kvh) * d:].reshape(rows, kvh, d)
        q = O.bf16_round(O.rope(O.rms_norm(q.reshape(-1, d), widen(L["q_norm"]), eps).reshape(rows, heads, d), positions, c["theta"]))
        k = O.bf16_round(O.rope(O.rms_norm(k.reshape(-1, d), widen(L["k_norm"]), eps).reshape(rows, kvh, d), positions, c["theta"]))
        # the slots' kept rows as a dense store, with this step's rows appended
        kr, vr = widen(dec.k_rows[i]), widen(dec.v_rows[i])      # read before the device step appends
        dense_k = np.zeros((dec.slots, keys, kvh, d), np.float32)
        dense_v = np.zeros_like(dense_k)
        for s in range(dec.slots):
            for p in range(keys):
                at = int(table[s * dec.pages + p // 64]) * 64 + p % 64
                dense_k[s, p], dense_v[s, p] = kr[at], vr[at]
        for r in range(rows):
            dense_k[slots[r], positions[r]], dense_v[slots[r], positions[r]] = k[r], v[r]
        a = O.bf16_round(O.attend_rows(q, dense_k, dense_v, slots, positions, scale=d ** -0.5))
        x = x + O.matmul(a.reshape(rows, heads * d), widen(L["wo"]))
        h = O.bf16_round(O.rms_norm(x, widen(L["ln2"]), eps))
        m = L["moe"]
        y, _, _ = O.moe_block(h, widen(m.router), widen(m.w_in), widen(m.w_out), c["top"], round_inner=True)
        w_sh = widen(m.shared_in)
        y = y + O.swiglu(h, w_sh[:c["shared_ffn"]], w_sh[c["shared_ffn"]:], widen(m.shared_out), round_inner=True)
        x = x + y
    return x


def test_moe_decoder_step_matches_oracle_and_its_graph_replay():
    """The GLM-style layer stack (decoder.rs:327-389 with the Moe feed-forward, decoder.rs:58-84) on one GPU: a decode
    step over paged kept rows against the checker's composition, and the same step replayed from a CUDA graph."""
    from tessera_b200.moe_decoder import MoeDecoder
    rng = np.random.default_rng(12)
    rows, context, keys = 6, 192, 128
    dec = MoeDecoder(SMALL_MOE, slots=rows, context=context, seed=3)
    dec.fill_kept(seed=4)
    dec.set_table(rng.permutation(rows * dec.pages))
    slots = np.arange(rows, dtype=np.uint32)
    positions = np.array([5, 63, 64, 100, 0, 127], np.uint32)
    x = rng.standard_normal((rows, SMALL_MOE["hidden"])).astype(np.float32)
    want = _moe_decoder_want(dec, x, slots, positions, keys)
    xd, sd, pd = torch.from_numpy(x).cuda(), dev_u32(slots), dev_u32(positions)
    got = dec.step(xd.clone(), sd, pd, keys)
    torch.cuda.synchronize()
    assert rel_error(widen(got), want) <= 1e-2 and _cos(widen(got), want) > 0.9999
    again = dec.step_graphed(xd, sd, pd, keys)          # appends the same rows again: same bits
    assert torch.equal(again, got)
    moved = dec.step_graphed(xd * 0.5, sd, pd, keys)     # replays the graph on new inputs
    assert torch.equal(moved, dec.step((xd * 0.5).clone(), sd, pd, keys))
