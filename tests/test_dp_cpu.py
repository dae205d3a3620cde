"""The data-parallel plumbing on two CPU ranks over gloo: balanced dealing of ragged units, the
max-over-ranks time, and the final gather."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tessera_b200 import dp


def test_serpentine_deal_balances_lengths():
    rng = np.random.default_rng(0)
    lengths = rng.integers(32, 513, size=1024)
    for world in (1, 2, 4, 8):
        shards = [dp.shard_by_length(lengths, r, world) for r in range(world)]
        assert sorted(i for s in shards for i in s) == list(range(1024))
        totals = [int(lengths[s].sum()) for s in shards]
        assert max(totals) - min(totals) <= 512 and max(len(s) for s in shards) - min(len(s) for s in shards) <= 1


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lengths = [5, 9, 2, 7, 7, 1, 3]
    mine = dp.shard_by_length(lengths, rank, world)
    local = torch.tensor([[float(i), float(lengths[i])] for i in mine])
    got = dp.gather_rows(local, mine, len(lengths))
    # the loop form: the widest shard known beforehand, so that the gather asks the ranks nothing
    widest = max(len(dp.shard_by_length(lengths, r, world)) for r in range(world))
    again = dp.gather_rows(local, mine, len(lengths), width=widest)
    assert (got is None) == (again is None) and (got is None or torch.equal(got, again))
    slow = dp.max_over_ranks(1.0 + rank)
    out[rank] = (None if got is None else got.numpy(), slow)
    dist.destroy_process_group()


def test_two_ranks_gather_and_time():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    rows, slow0 = out[0]
    assert out[1][0] is None and slow0 == 2.0 and out[1][1] == 2.0
    assert np.array_equal(rows, np.array([[i, l] for i, l in enumerate([5, 9, 2, 7, 7, 1, 3])], np.float32))
