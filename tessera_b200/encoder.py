"""A bidirectional text encoder of the EmbeddingGemma-300M shape on the library's kernels: packed ragged
sequences in, one unit-length embedding per sequence out.

Layer order follows the reference's decoder trunk (engine/models/src/decoder.rs:327-389) with the
embedding model's differences (engine/models/src/eg2.rs): a bidirectional mask, a GeGLU feed-forward
(tanh GELU), mean pooling over each text's rows and a unit scale (frontend/tasks/src/embed.rs:47-52,
148-154).  Where the reference groups texts of equal length because it has no kernel for ragged keys
(frontend/tasks/src/embed.rs:14-17), every text of a batch shares one launch here: rows are packed
back to back and the attention kernel takes the sequence bounds.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from . import ops
from ._lib import EPILOGUE, lib

EMBEDDING_300M = dict(layers=24, hidden=768, heads=3, kv_heads=1, head_dim=256, ffn=1152, vocab=262144,
                      eps=1e-6, theta=1e6)


def encoder_weight_names(layers: int) -> list[str]:
    names = ["embed"]
    for i in range(layers):
        names += [f"layers.{i}.{f}" for f in ("ln1", "q", "k", "v", "q_norm", "k_norm", "o", "ln2", "mlp.gate", "mlp.up",
                                              "mlp.down")]
    return names + ["norm"]


class Encoder:
    def __init__(self, cfg: dict, named_weights, device="cuda"):
        self.cfg = dict(cfg)
        L = cfg["layers"]
        raw = dict(named_weights)
        bf = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16).to(device)
        f32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device)
        self.embed = bf(raw["embed"])
        self.norm = f32(raw["norm"])
        self.layers = []
        for i in range(L):
            g = lambda f: raw[f"layers.{i}.{f}"]
            self.layers.append(dict(
                ln1=f32(g("ln1")), ln2=f32(g("ln2")), q_norm=f32(g("q_norm")), k_norm=f32(g("k_norm")),
                wqkv=bf(np.concatenate([g("q"), g("k"), g("v")], axis=0)), wo=bf(g("o")),
                wgu=bf(np.concatenate([g("mlp.gate"), g("mlp.up")], axis=0)), wdown=bf(g("mlp.down"))))
        self.inv_freq = ops.rope_inv_freq(cfg["theta"], cfg["head_dim"], device)
        self.device = device

    def forward(self, tokens: torch.Tensor, cu_seqlens: torch.Tensor, max_len: int) -> torch.Tensor:
        """tokens int32 [total] packed, cu_seqlens int32 [seqs + 1] -> float32 [seqs, hidden], unit rows."""
        c = self.cfg
        total, seqs = tokens.numel(), cu_seqlens.numel() - 1
        heads, kvh, d, eps = c["heads"], c["kv_heads"], c["head_dim"], c["eps"]
        lens = (cu_seqlens[1:] - cu_seqlens[:-1]).to(torch.int64)
        slots = torch.repeat_interleave(torch.arange(seqs, device=self.device), lens).to(torch.int32)
        positions = (torch.arange(total, device=self.device) - cu_seqlens[:-1].to(torch.int64)[slots.long()]).to(torch.int32)
        # Kept layout with one-row pages: table[s * max_len + t] = row of token t of text s in the packed buffer.
        table = torch.zeros(seqs * max_len, dtype=torch.int32, device=self.device)
        table[slots.long() * max_len + positions.long()] = torch.arange(total, dtype=torch.int32, device=self.device)
        kept = ops.Kept("paged", max_len, table, total, page=1)
        q = torch.empty((total, heads, d), dtype=torch.bfloat16, device=self.device)
        k = torch.empty((total, kvh, d), dtype=torch.bfloat16, device=self.device)
        v = torch.empty_like(k)
        scale = float(d) ** -0.5
        hidden_w, inner_w = c["hidden"], heads * d
        # The two norms of a layer can fold into the projections around them (TS_ENCODER_FOLD=1) when the
        # residual-adding ones can leave the rows' sums of squares (ts_linear_sumsq_parts > 0).  Off by default:
        # at 273 K rows the paired kernel's epilogue (a thread per row: 16-byte pieces of 32 different rows per
        # store instruction) is what bounds these short-k projections, and the extra scaled copy it then writes
        # costs more (157 ms per pass) than the norm launches it removes (140 ms).
        parts = lib.ts_linear_sumsq_parts(total, hidden_w, inner_w, EPILOGUE["add"])
        fold = (os.environ.get("TS_ENCODER_FOLD", "0") == "1" and parts > 0 and
                lib.ts_linear_sumsq_parts(total, hidden_w, c["ffn"], EPILOGUE["add"]) == parts)
        if fold:
            x, xs, ss = ops.gather_scaled(self.embed, tokens, self.layers[0]["ln1"], parts)
        else:
            x = ops.gather(self.embed, tokens, out_dtype=torch.float32)
        for i, L in enumerate(self.layers):
            if fold:
                qkv = ops.linear_fused(xs, L["wqkv"], rows=(ss, eps))
            else:
                qkv = ops.linear(ops.rms_norm(x, L["ln1"], eps), L["wqkv"])
            ops.qk_norm_rope_append(qkv, L["q_norm"], L["k_norm"], self.inv_freq, slots, positions, q, k, v, kept,
                                    heads, kvh, d, eps)
            a = ops.attend(q, k, v, mask="bidirectional", scale=scale, cu_seqlens=cu_seqlens, max_len=max_len)
            if fold:
                x, xs, ss = ops.linear_fused(a.view(total, inner_w), L["wo"], x, epilogue="add", out_dtype=torch.float32, out=x,
                                             next_gain=L["ln2"])
                act = ops.linear_fused(xs, L["wgu"], epilogue="geglu", rows=(ss, eps))
                nxt = self.layers[i + 1]["ln1"] if i + 1 < len(self.layers) else self.norm
                x, xs, ss = ops.linear_fused(act, L["wdown"], x, epilogue="add", out_dtype=torch.float32, out=x, next_gain=nxt)
            else:
                x = ops.linear(a.view(total, inner_w), L["wo"], x, epilogue="add", out_dtype=torch.float32, out=x)
                act = ops.linear(ops.rms_norm(x, L["ln2"], eps), L["wgu"], epilogue="geglu")
                x = ops.linear(act, L["wdown"], x, epilogue="add", out_dtype=torch.float32, out=x)
        hidden = ops.rms_norm(x, self.norm, eps, out_dtype=torch.float32)
        return ops.mean_pool(hidden, cu_seqlens, normalize=True)
