"""Data-parallel plumbing: independent units (sequences, texts) are dealt to ranks, weights are
replicated, and nothing crosses ranks on the data path; only timing and the final gather do.

The reference has no cross-device data parallelism (independent slots of one batch only,
engine/engine/src/schedule.rs:157-188); this is the natural sharding of its independent units.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_by_length(lengths, rank: int, world: int) -> list[int]:
    """Indices of the units rank `rank` owns: units sorted by length (longest first, index as the tie
    break) and dealt in serpentine order, so every rank gets the same count (within one) and nearly the
    same total length."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    mine = []
    for j, i in enumerate(order):
        lap, pos = divmod(j, world)
        owner = pos if lap % 2 == 0 else world - 1 - pos
        if owner == rank:
            mine.append(i)
    return mine


def max_over_ranks(seconds: float, device=None, group=None) -> float:
    """The slowest rank's time: what a multi-GPU number is reported on."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return seconds
    t = torch.tensor([seconds], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def gather_rows(local: torch.Tensor, indices: list[int], total: int, group=None, width: int | None = None) -> torch.Tensor | None:
    """Rank 0 receives every rank's rows (e.g. embeddings or token ids) placed at their unit indices.

    `width`: the largest number of rows any rank holds, when the caller already knows it (a loop that gathers
    every step asks the ranks once, outside the loop, and the gather then never touches the host)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        out = local.new_zeros((total,) + tuple(local.shape[1:]))
        out[torch.tensor(indices, dtype=torch.long, device=local.device)] = local
        return out
    idx = torch.tensor(indices, dtype=torch.long, device=local.device)
    if width is None:
        counts = [None] * world
        dist.all_gather_object(counts, int(idx.numel()), group=group)
        width = max(counts)
    pad_rows = local.new_zeros((width,) + tuple(local.shape[1:]))
    pad_rows[: idx.numel()] = local
    pad_idx = idx.new_full((width,), -1)
    pad_idx[: idx.numel()] = idx
    rows = [torch.empty_like(pad_rows) for _ in range(world)]
    ids = [torch.empty_like(pad_idx) for _ in range(world)]
    dist.all_gather(rows, pad_rows, group=group)
    dist.all_gather(ids, pad_idx, group=group)
    if dist.get_rank(group) != 0:
        return None
    out = local.new_zeros((total,) + tuple(local.shape[1:]))
    for r, i in zip(rows, ids):
        keep = i >= 0
        out[i[keep]] = r[keep]
    return out
