"""Writes tests/golden/qwen3_0p6b_greedy.json: the CPU checker's greedy tokens for the
Qwen3-0.6B-shaped decoder (random init from seed 0, norms = 1, tied embeddings), batch 1, a
prompt of 128 uniform token ids, 64 greedy steps.  Run from the repository root:

    python tests/golden/make_qwen3_tokens.py

Takes a few minutes on one core.  The GPU parity test replays the same seed and must reproduce
the first 32 generated ids exactly.
"""
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle as O  # noqa: E402
from tessera_b200 import synth  # noqa: E402  (only the seeded weight generator: no device code)


def oracle_weights(cfg, seed, gains="ones"):
    w = {k: [] for k in ("q", "k", "v", "o", "gate", "up", "down", "ln1", "ln2", "q_norm", "k_norm")}
    for name, a in synth.decoder_weights(cfg, seed, gains=gains):
        if name in ("embed", "norm"):
            w[name] = a
        else:
            w[name.split(".", 2)[2].replace("mlp.", "")].append(a)
    return w


def greedy(cfg, seed, prompt, new, context):
    dec = O.Decoder(dict(cfg, context=context, slots=1), oracle_weights(cfg, seed))
    n = len(prompt)
    ids, _, _ = dec.step(prompt, [0] * n, list(range(n)))
    out = [int(ids[-1])]
    for t in range(1, new):
        ids, _, _ = dec.step([out[-1]], [0], [n + t - 1])
        out.append(int(ids[0]))
    return out


if __name__ == "__main__":
    cfg = synth.QWEN3_0_6B
    prompt = synth.prompt_tokens(cfg["vocab"], 128, seed=0)
    t0 = time.time()
    tokens = greedy(cfg, 0, prompt.tolist(), 64, 192)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "qwen3_0p6b_greedy.json")
    with open(path, "w") as f:
        json.dump({"config": cfg, "seed": 0, "prompt_seed": 0, "prompt_len": 128, "new": 64,
                   "prompt_head": prompt[:8].tolist(), "tokens": tokens, "numpy": np.__version__,
                   "seconds": round(time.time() - t0, 1)}, f, indent=1)
    print(path, tokens[:8], f"{time.time() - t0:.0f}s")
