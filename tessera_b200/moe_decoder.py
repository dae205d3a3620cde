"""A GLM-style mixture-of-experts decoder layer stack for decode steps over paged kept rows, on the
library's kernels; experts local or expert-parallel.

Per layer (engine/models/src/decoder.rs:327-389 with the `Moe` feed-forward of decoder.rs:58-84 and the
shared expert of engine/models/src/mla.rs:466-467): rms_norm, fused q|k|v linear, per-head norm +
rotation + append to the slot's pages, ragged attention over the kept rows, o linear + residual,
rms_norm, router -> top-k -> softmax gates, shared expert + routed experts (dispatched to their owning
rank when expert-parallel), residual.
"""
from __future__ import annotations

import torch

from . import ops
from .moe import ExpertParallel, MoeWeights, OneRankOfMany, moe_forward

GLM_MOE = dict(layers=8, hidden=4096, heads=32, kv_heads=8, head_dim=128, experts=128, top=8, ffn=1536,
               shared_ffn=1536, eps=1e-6, theta=1e6)


def _bf16_normal(shape, std, gen, device):
    return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


class MoeDecoder:
    def __init__(self, cfg: dict, slots: int, context: int, rank: int = 0, world: int = 1, seed: int = 0,
                 group=None, device="cuda", scheme: str = "replicate", alone: bool = False):
        self.cfg, self.device, self.world, self.rank = dict(cfg), device, world, rank
        self.scheme = scheme          # how picks meet their experts across ranks: see tessera_b200/moe.py
        self._graphs: dict = {}       # (rows, keys) -> (graph, output); static inputs in self._static
        c = cfg
        h, d = c["hidden"], c["head_dim"]
        qw, kw = c["heads"] * d, c["kv_heads"] * d
        per = c["experts"] // world
        shared = torch.Generator(device=device).manual_seed(seed)          # replicated weights: same on every rank
        local = torch.Generator(device=device).manual_seed(seed * 1000 + 17 + rank)
        self.layers = []
        for _ in range(c["layers"]):
            L = dict(ln1=torch.ones(h, device=device), ln2=torch.ones(h, device=device),
                     q_norm=torch.ones(d, device=device), k_norm=torch.ones(d, device=device),
                     wqkv=_bf16_normal((qw + 2 * kw, h), 0.02, shared, device), wo=_bf16_normal((h, qw), 0.02, shared, device))
            L["moe"] = MoeWeights(router=_bf16_normal((c["experts"], h), 0.02, shared, device),
                                  w_in=_bf16_normal((per, 2 * c["ffn"], h), 0.02, local, device),
                                  w_out=_bf16_normal((per, h, c["ffn"]), 0.02, local, device),
                                  shared_in=_bf16_normal((2 * c["shared_ffn"], h), 0.02, shared, device),
                                  shared_out=_bf16_normal((h, c["shared_ffn"]), 0.02, shared, device),
                                  first=rank * per, experts_total=c["experts"])
            self.layers.append(L)
        self.page = 64
        self.pages = -(-context // self.page)
        self.slots, self.context = slots, context
        rows = slots * self.pages * self.page
        self.k_rows = [torch.zeros((rows, c["kv_heads"], d), dtype=torch.bfloat16, device=device) for _ in self.layers]
        self.v_rows = [torch.zeros_like(k) for k in self.k_rows]
        self.table = torch.arange(slots * self.pages, dtype=torch.int32, device=device)
        self.inv_freq = ops.rope_inv_freq(c["theta"], d, device)
        # alone: this rank's kernels with stand-ins for the collectives (see moe.OneRankOfMany)
        self.ep = (OneRankOfMany(world, rank) if alone else ExpertParallel(group)) if world > 1 else None

    def close(self):
        """Drops the captured graphs.  Call before torch.distributed.destroy_process_group(): a live graph that holds
        captured collectives keeps the communicator busy and the teardown waits on it forever."""
        torch.cuda.synchronize()
        self._graphs.clear()
        self.__dict__.pop("_static", None)
        torch.cuda.synchronize()

    def set_table(self, table):
        self.table.copy_(torch.as_tensor(table, dtype=torch.int32, device=self.device))

    def fill_kept(self, seed: int = 1):
        """Synthetic kept rows ~ N(0, 1): decode cost does not depend on their values."""
        gen = torch.Generator(device=self.device).manual_seed(seed)
        for k, v in zip(self.k_rows, self.v_rows):
            k.copy_(torch.randn(k.shape, generator=gen, device=self.device).to(torch.bfloat16))
            v.copy_(torch.randn(v.shape, generator=gen, device=self.device).to(torch.bfloat16))

    def step(self, x: torch.Tensor, slots: torch.Tensor, positions: torch.Tensor, keys: int) -> torch.Tensor:
        """x f32 [rows, hidden] (the residual rows), one row per slot -> the rows after every layer."""
        c = self.cfg
        rows, d, heads, kvh, eps = x.shape[0], c["head_dim"], c["heads"], c["kv_heads"], c["eps"]
        kept = ops.Kept("paged", self.pages, self.table, self.k_rows[0].shape[0])
        q = torch.empty((rows, heads, d), dtype=torch.bfloat16, device=self.device)
        for i, L in enumerate(self.layers):
            h = ops.rms_norm(x, L["ln1"], eps)
            qkv = ops.linear(h, L["wqkv"])
            # one row per slot: per-head norm, rotation, append and attention in one launch (the same bits as
            # ops.qk_norm_rope_append followed by ops.attend_rows)
            a = ops.attend_rows_append(qkv, L["q_norm"], L["k_norm"], self.inv_freq, self.k_rows[i], self.v_rows[i], slots,
                                       positions, kept, keys, heads, eps=eps, scale=d ** -0.5, out=q)
            x = ops.linear(a.view(rows, heads * d), L["wo"], x, epilogue="add", out_dtype=torch.float32, out=x)
            h = ops.rms_norm(x, L["ln2"], eps)
            # the block's output lands on the residual rows inside its own kernels (the shared expert's down
            # projection adds them in its epilogue, the routed mix adds that)
            if self.ep is None:
                x, _, _ = moe_forward(h, L["moe"], c["top"], residual=x)
            else:
                x, _, _ = self.ep.forward(h, L["moe"], c["top"], scheme=self.scheme, residual=x)
        return x

    def step_graphed(self, x: torch.Tensor, slots: torch.Tensor, positions: torch.Tensor, keys: int) -> torch.Tensor:
        """`step` replayed from a CUDA graph per (rows, keys): a decode step is some hundred short launches and, across
        ranks, two collectives per layer; replaying them removes the host's share of a step that takes about a
        millisecond of device time per rank.  Needs a scheme with no host reads (`replicate`, or one rank).  The
        returned tensor is overwritten by the next call with the same (rows, keys)."""
        if self.ep is not None and self.scheme != "replicate":
            return self.step(x, slots, positions, keys)
        rows = x.shape[0]
        st = self.__dict__.setdefault("_static", {})
        if rows not in st:
            st[rows] = (torch.empty_like(x), torch.empty_like(slots), torch.empty_like(positions))
        gx, gs, gp = st[rows]
        gx.copy_(x)
        gs.copy_(slots)
        gp.copy_(positions)
        entry = self._graphs.get((rows, keys))
        if entry is None:
            cur = torch.cuda.current_stream()
            side = torch.cuda.Stream()
            side.wait_stream(cur)
            with torch.cuda.stream(side):      # the launches once outside a capture: scratch buffers, attributes, communicators
                for _ in range(2):
                    self.step(gx.clone(), gs, gp, keys)
            cur.wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self.step(gx.clone(), gs, gp, keys)
            entry = self._graphs[(rows, keys)] = (graph, out)
        entry[0].replay()
        return entry[1]
