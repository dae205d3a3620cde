"""Seeded synthetic weights and inputs of the benchmark configurations.

Weights are N(0, 0.02) rounded to bf16 (round-to-nearest-even), norm gains are 1, the
unembedding is tied to the embedding: the random initialisation the configurations name.
numpy's PCG64 streams are reproducible across machines, so the CPU checker and the GPU path
can both be fed the same bytes from a seed.  Tensors are drawn in the declaration order of
engine/models/src/decoder.rs:225-255, one child seed per tensor.
"""
from __future__ import annotations

import numpy as np

QWEN3_0_6B = dict(layers=28, hidden=1024, heads=16, kv_heads=8, head_dim=128, ffn=3072, vocab=151936,
                  eps=1e-6, theta=1e6)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bits, round to nearest even (engine/ir/graph/src/scalar.rs:21-43)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))) >> np.uint32(16)
    return rounded.astype(np.uint16)


def decoder_weight_names(layers: int) -> list[str]:
    names = ["embed"]
    for i in range(layers):
        names += [f"layers.{i}.{f}" for f in
                  ("ln1", "q", "k", "v", "q_norm", "k_norm", "o", "ln2", "mlp.gate", "mlp.up", "mlp.down")]
    return names + ["norm"]


def decoder_weight_shape(name: str, cfg: dict) -> tuple:
    h, d = cfg["hidden"], cfg["head_dim"]
    qw, kw, f = cfg["heads"] * d, cfg["kv_heads"] * d, cfg["ffn"]
    leaf = name.split(".", 2)[-1] if name.startswith("layers.") else name
    return {"embed": (cfg["vocab"], h), "norm": (h,), "ln1": (h,), "ln2": (h,), "q_norm": (d,), "k_norm": (d,),
            "q": (qw, h), "k": (kw, h), "v": (kw, h), "o": (h, qw), "mlp.gate": (f, h), "mlp.up": (f, h),
            "mlp.down": (h, f)}[leaf]


def decoder_weights(cfg: dict, seed: int = 0, std: float = 0.02, gains: str = "ones"):
    """Yields (name, array): linears as uint16 bf16 bits [out, in], gains as float32."""
    names = decoder_weight_names(cfg["layers"])
    children = np.random.SeedSequence(seed).spawn(len(names))
    for name, child in zip(names, children):
        shape = decoder_weight_shape(name, cfg)
        rng = np.random.default_rng(child)
        if len(shape) == 1:
            if gains == "ones":
                yield name, np.ones(shape, np.float32)
            else:  # gains near one, for tests that must notice a dropped gain
                yield name, (1.0 + 0.1 * rng.standard_normal(shape, dtype=np.float32)).astype(np.float32)
        else:
            yield name, bf16_bits(rng.standard_normal(shape, dtype=np.float32) * np.float32(std))


def prompt_tokens(vocab: int, count: int, seed: int = 0) -> np.ndarray:
    """`count` token ids uniform in [0, vocab)."""
    return np.random.default_rng(np.random.SeedSequence([seed, 0xBEEF])).integers(0, vocab, size=count,
                                                                                   dtype=np.int64).astype(np.uint32)


def page_permutation(entries: int, seed: int = 0) -> np.ndarray:
    """A seeded random page-to-slot map: a permutation of all pages."""
    return np.random.default_rng(np.random.SeedSequence([seed, 0xFA6E])).permutation(entries).astype(np.uint32)
