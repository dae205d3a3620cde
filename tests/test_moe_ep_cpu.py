"""Expert-parallel dispatch / combine on two CPU ranks over gloo, with the CPU checker injected as the
compute: the exchange logic (owner of each pick, stable grouping, counts all-to-all, rows out, outputs
back, pick-order mix) must reproduce the single-rank MoE block of engine/models/src/decoder.rs:70-84,
router ids bit-exact."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O

HIDDEN, FFN, EXPERTS, TOP, ROWS = 32, 16, 8, 2, 12


def _weights():
    rng = np.random.default_rng(3)
    bf = lambda *s, std=0.2: O.bf16_round(rng.standard_normal(s, dtype=np.float32) * std)
    return dict(router=bf(EXPERTS, HIDDEN), w_in=bf(EXPERTS, 2 * FFN, HIDDEN), w_out=bf(EXPERTS, HIDDEN, FFN),
                h=bf(2 * ROWS, HIDDEN, std=1.0))


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tessera_b200.moe import ExpertParallel, MoeWeights
    w = _weights()
    per = EXPERTS // world
    mw = MoeWeights(router=torch.from_numpy(w["router"]), w_in=torch.from_numpy(w["w_in"][rank * per:(rank + 1) * per]),
                    w_out=torch.from_numpy(w["w_out"][rank * per:(rank + 1) * per]), first=rank * per,
                    experts_total=EXPERTS)

    def route(h, mw, top):
        scores = O.matmul(h.numpy(), mw.router.numpy())
        ids = O.top_k(scores, top)
        return torch.from_numpy(ids.astype(np.int64)), torch.from_numpy(O.softmax(O.take(scores, ids)))

    def experts(x, ids, mw):
        # the checker's `picked` chain on this rank's table (ids outside it would read zeros)
        xs, flat = x.numpy(), ids.numpy().astype(np.uint32)
        w_in, w_out = mw.w_in.numpy(), mw.w_out.numpy()
        inner = O.act(O.matmul_picked(xs, w_in[:, :FFN], flat, mw.first), "silu") * O.matmul_picked(xs, w_in[:, FFN:], flat, mw.first)
        return torch.from_numpy(O.matmul_picked(inner, w_out, flat, mw.first))

    def mix(y_picks, gates, add):
        y = O.mean(y_picks.numpy().reshape(gates.shape[0], gates.shape[1], -1), 1, weights=gates.numpy())
        return torch.from_numpy(y)

    def local(h_all, ids, gates, mw):
        # the whole routed block against this rank's experts: foreign picks contribute zeros (picked.rs:49-59)
        per_pick = experts(torch.from_numpy(np.repeat(h_all.numpy(), TOP, axis=0)), ids.reshape(-1), mw)
        return mix(per_pick, gates, None)

    ep = ExpertParallel(experts_fn=experts, route_fn=route, shared_fn=lambda h, mw: None, mix_fn=mix, local_fn=local)
    h = torch.from_numpy(w["h"][rank * ROWS:(rank + 1) * ROWS])
    y, ids, gates = ep.forward(h, mw, TOP)
    y2, ids2, _ = ep.forward(h, mw, TOP, scheme="replicate")
    out[rank] = (y.numpy(), ids.numpy(), y2.numpy(), ids2.numpy())
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_rank_block():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    w = _weights()
    want, want_ids, _ = O.moe_block(w["h"], w["router"], w["w_in"], w["w_out"], TOP)
    got = np.concatenate([out[0][0], out[1][0]])
    ids = np.concatenate([out[0][1], out[1][1]])
    assert np.array_equal(ids.astype(np.uint32), want_ids)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-7)
    # the replicate scheme (all-gather rows, local experts with zeros for foreign picks, sum over ranks)
    got2 = np.concatenate([out[0][2], out[1][2]])
    ids2 = np.concatenate([out[0][3], out[1][3]])
    assert np.array_equal(ids2.astype(np.uint32), want_ids)
    assert np.allclose(got2, want, rtol=1e-5, atol=1e-6)
