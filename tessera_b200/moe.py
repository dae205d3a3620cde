"""The routed block of a decoder layer, on one GPU or expert-parallel over several.

Mirrors engine/models/src/decoder.rs:70-84 (`Moe::apply`): scores = h router^T, ids = top_k(scores),
gates = softmax(take(scores, ids)), y = sum_p gates[p] expert_{ids[p]}(h) in pick order, plus a shared
expert (engine/models/src/mla.rs:466-467).

Expert parallel: rank r of g holds experts [r E/g, (r+1) E/g) - the reference's axis-0 split with its
`first` / `count` (engine/plan/lower/src/sites/matmul.rs:64, engine/rules/linear/src/picked.rs:49-53) -
and its own share of the token rows.  Where the reference lets every rank compute zeros for foreign
picks and all-reduces, this module has two schemes.  `dispatch` moves the picks: counts all-to-all, rows
to the owning rank (NCCL all_to_all over NVLink), grouped expert kernels there, per-pick outputs back,
gate-weighted sum at the source in pick order; its exchange sizes pass through the host, so it suits large
launches (prefill), where each rank's picks are far fewer than the rows of all ranks.  `replicate` is the
reference's scheme with the all-reduce split in two: all-gather the token rows, every rank routes all of
them (the same kernels on the same bits: the same ids everywhere) and runs the whole routed block against
its own experts with foreign picks contributing zeros, then a reduce-scatter sums the ranks' partial rows
and leaves each rank its own.  Nothing passes through the host, so a decode step with it can be captured in
a CUDA graph; with top-k >= ranks it moves no more bytes than dispatch.  The exchange logic is
device-agnostic (tested on CPU ranks over gloo with injected compute); the compute callbacks default to
the CUDA kernels of this library.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist


@dataclass
class MoeWeights:
    router: torch.Tensor   # bf16 [E, H] (all experts, replicated)
    w_in: torch.Tensor     # bf16 [E_local, 2F, H] gate rows then up rows
    w_out: torch.Tensor    # bf16 [E_local, H, F]
    shared_in: torch.Tensor | None = None   # bf16 [2Fs, H]
    shared_out: torch.Tensor | None = None  # bf16 [H, Fs]
    first: int = 0         # global id of the first local expert
    experts_total: int = 0


def _cuda_route(h, w: MoeWeights, top: int):
    from . import ops
    scores = ops.router_scores(h, w.router)   # the interpreter's summation order: ids are bit-exact, near ties included
    ids = ops.top_k(scores, top)
    return ids, ops.take_softmax(scores, ids)


def _cuda_experts(x, ids, w: MoeWeights):
    from . import ops
    return ops.moe_experts(x, ids, w.w_in, w.w_out, repeat=1, first=w.first)


def _cuda_shared(h, w: MoeWeights, residual=None):
    """The shared expert's rows, f32; with `residual` the down projection adds it in its epilogue, so the block's
    output lands on the residual stream without an elementwise launch of its own."""
    from . import ops
    if w.shared_in is None:
        return residual
    inner = ops.linear(h, w.shared_in, epilogue="swiglu")
    if residual is None:
        return ops.linear(inner, w.shared_out, out_dtype=torch.float32)
    return ops.linear(inner, w.shared_out, residual, epilogue="add", out_dtype=torch.float32)


def _cuda_local(h_all, ids, gates, w: MoeWeights):
    from . import ops
    return ops.moe(h_all, ids, gates, w.w_in, w.w_out, first=w.first)


def _cuda_mix(y_picks, gates, add):
    from . import ops
    return ops.moe_mix(y_picks, gates, add)


def moe_forward(h, w: MoeWeights, top: int, residual=None):
    """Single GPU: every expert is local.  With `residual` (f32 [rows, H]) the result is residual + block."""
    from . import ops
    ids, gates = _cuda_route(h, w, top)
    return ops.moe(h, ids, gates, w.w_in, w.w_out, add=_cuda_shared(h, w, residual), first=w.first), ids, gates


class ExpertParallel:
    """Dispatch / combine of picks between ranks.  `experts_fn(x [n, H], ids [n]) -> [n, H] f32` runs on
    the rank that holds the experts; `mix_fn(y_picks [rows * top, H], gates, add) -> [rows, H]` at the source."""

    def __init__(self, group=None, experts_fn: Callable | None = None, route_fn: Callable | None = None,
                 shared_fn: Callable | None = None, mix_fn: Callable | None = None, local_fn: Callable | None = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.experts_fn = experts_fn or _cuda_experts
        self.route_fn = route_fn or _cuda_route
        self.shared_fn = shared_fn or _cuda_shared
        self.mix_fn = mix_fn or _cuda_mix
        self.local_fn = local_fn or _cuda_local   # (h_all, ids, gates, w) -> [rows of all ranks, H] f32, this rank's experts only

    def plan(self, ids: torch.Tensor, experts_total: int):
        """Which rank owns each pick, the stable order that groups picks by owner, and per-owner counts."""
        per = experts_total // self.world
        owner = (ids.reshape(-1).to(torch.int64) // per).clamp_(max=self.world - 1)
        order = torch.argsort(owner, stable=True)
        counts = torch.bincount(owner, minlength=self.world)
        return order, counts

    def _add(self, h, w: MoeWeights, residual):
        """What is added to the routed rows: the shared expert's output and, when given, the residual rows."""
        if self.shared_fn is _cuda_shared:
            return _cuda_shared(h, w, residual)
        add = self.shared_fn(h, w)
        if residual is None:
            return add
        return residual if add is None else add + residual

    def forward_replicated(self, h, w: MoeWeights, top: int, residual=None):
        """all-gather rows -> route everywhere -> local experts on all rows -> reduce-scatter.  No host reads."""
        rows, hidden = h.shape
        h_all = torch.empty((self.world * rows, hidden), dtype=h.dtype, device=h.device)
        dist.all_gather_into_tensor(h_all, h.contiguous(), group=self.group)
        ids, gates = self.route_fn(h_all, w, top)
        part = self.local_fn(h_all, ids, gates, w)
        if dist.get_backend(self.group) == "gloo":      # no reduce-scatter there: all-reduce and keep this rank's rows
            dist.all_reduce(part, group=self.group)
            y = part[self.rank * rows:(self.rank + 1) * rows].clone()
        else:
            y = torch.empty((rows, hidden), dtype=part.dtype, device=part.device)
            dist.reduce_scatter_tensor(y, part, group=self.group)
        add = self._add(h, w, residual)
        if add is not None:
            y += add
        mine = slice(self.rank * rows, (self.rank + 1) * rows)
        return y, ids[mine], gates[mine]

    def forward(self, h, w: MoeWeights, top: int, scheme: str = "dispatch", residual=None):
        """With `residual` (f32 [rows, H]) the result is residual + block."""
        if scheme == "replicate":
            return self.forward_replicated(h, w, top, residual)
        rows, hidden = h.shape
        ids, gates = self.route_fn(h, w, top)
        order, send_counts = self.plan(ids, w.experts_total)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        send = [int(v) for v in send_counts.tolist()]   # the exchange sizes must be known on the host
        recv = [int(v) for v in recv_counts.tolist()]
        flat_ids = ids.reshape(-1)
        x_send = h[(order // top)].contiguous()          # pick i reads row i // top
        id_send = flat_ids[order].contiguous()
        x_recv = torch.empty((sum(recv), hidden), dtype=h.dtype, device=h.device)
        id_recv = torch.empty(sum(recv), dtype=flat_ids.dtype, device=h.device)
        dist.all_to_all_single(x_recv, x_send, recv, send, group=self.group)
        dist.all_to_all_single(id_recv, id_send, recv, send, group=self.group)
        y_recv = self.experts_fn(x_recv, id_recv, w) if sum(recv) else torch.empty((0, hidden), dtype=torch.float32,
                                                                                    device=h.device)
        y_back = torch.empty((sum(send), hidden), dtype=torch.float32, device=h.device)
        dist.all_to_all_single(y_back, y_recv.contiguous(), send, recv, group=self.group)
        y_picks = torch.empty_like(y_back)
        y_picks[order] = y_back                           # back to pick order
        return self.mix_fn(y_picks, gates, self._add(h, w, residual)), ids, gates


class OneRankOfMany(ExpertParallel):
    """One rank's share of an expert-parallel step with no peers: the all-gather is `world` copies of this rank's
    rows and the reduce-scatter keeps this rank's slice of its own partial sums.  The kernels, their shapes and
    their order are those of rank `rank` of `world` (the values are not): for timing and profiling one rank's
    launches on one GPU, where a profiler cannot wrap a multi-rank command."""

    def __init__(self, world: int, rank: int = 0):
        self.group, self.world, self.rank = None, world, rank
        self.experts_fn, self.route_fn, self.shared_fn = _cuda_experts, _cuda_route, _cuda_shared
        self.mix_fn, self.local_fn = _cuda_mix, _cuda_local

    def forward(self, h, w: MoeWeights, top: int, scheme: str = "replicate", residual=None):
        rows = h.shape[0]
        h_all = h.repeat(self.world, 1)
        ids, gates = self.route_fn(h_all, w, top)
        part = self.local_fn(h_all, ids, gates, w)
        mine = slice(self.rank * rows, (self.rank + 1) * rows)
        y = part[mine].clone()
        add = _cuda_shared(h, w, residual)
        if add is not None:
            y += add
        return y, ids[mine], gates[mine]
