"""Writes tests/golden/qwen3_0p6b_greedy.json: the CPU checker's greedy tokens for the
Qwen3-0.6B-shaped decoder (random init from seed 0, norms = 1, tied embeddings), batch 1, a
prompt of 128 uniform token ids, 64 greedy steps.  Run from the repository root:

    python tests/golden/make_qwen3_tokens.py

Takes a few minutes per seed on one core.  The GPU parity test replays the same seed and must
reproduce the first 32 generated ids exactly.

Greedy decoding is discontinuous: where the two largest logits nearly tie, summing in another order
(which every parallel kernel does) is enough to pick the other token, and from then on the sequences
differ.  A randomly initialised model ties often.  So the script records the checker's margin (largest
minus second largest logit) at every step and walks the weight seeds given on the command line
(default 0..7; seed 1 is the one the committed fixture uses) until one keeps the margin of each of the first 32 steps above MIN_MARGIN and emits at
least MIN_DISTINCT different ids in those steps (a sequence that repeats one id says less); the fixture
says which seed that was and lists the margins.  Without such a seed the last one that kept its
margins is written.

A second fixture, `python tests/golden/make_qwen3_tokens.py --varied`, writes qwen3_0p6b_greedy_varied.json:
the same shapes and prompt with weights N(0, 0.035) and norm gains 1 +- 0.1.  With the configuration's N(0, 0.02)
and gains of one the layers add little to the residual stream, the tied unembedding hands back the token that
went in, and the greedy sequence repeats one id: a fixed point that a kernel far outside tolerance would still
reproduce.  The larger weights make nearly every step produce a new id, so an error anywhere in the stack moves the
sequence.  (Larger still is no better: at N(0, 0.05) the random stack amplifies bf16 rounding so much that two
correct implementations differ by 3e-2 of the largest logit after 28 layers.)  Its rule is plain: the first seed
whose first 32 margins all exceed 1e-2, no search beyond that.
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


def oracle_weights(cfg, seed, gains="ones", std=0.02):
    w = {k: [] for k in ("q", "k", "v", "o", "gate", "up", "down", "ln1", "ln2", "q_norm", "k_norm")}
    for name, a in synth.decoder_weights(cfg, seed, std=std, gains=gains):
        if name in ("embed", "norm"):
            w[name] = a
        else:
            w[name.split(".", 2)[2].replace("mlp.", "")].append(a)
    return w


MIN_MARGIN = 5e-2   # logits are O(1); a bf16 rounding moved by summation order shifts them by up to ~1e-2
MIN_DISTINCT = 3


def _margin(logits_row):
    top2 = np.partition(logits_row, -2)[-2:]
    return float(top2[1] - top2[0])


def probe_ids(vocab, count=32, seed=11):
    """The vocabulary ids whose logits the fixture records at every step (a fixed, seeded sample)."""
    return np.sort(np.random.default_rng(seed).choice(vocab, size=count, replace=False)).astype(np.int64)


def greedy(cfg, seed, prompt, new, context, stop_below=None, probes=None, gains="ones", std=0.02):
    """Returns (tokens, margins); stops early (None, margins) once one of the first 32 margins is too small.
    With `probes` (a dict), also records per step the winning logit and the logits at `probe_ids`."""
    dec = O.Decoder(dict(cfg, context=context, slots=1), oracle_weights(cfg, seed, gains, std))
    n = len(prompt)
    at = probe_ids(cfg["vocab"])

    def note(row):
        if probes is not None:
            probes.setdefault("top", []).append(round(float(row.max()), 5))
            probes.setdefault("at", []).append([round(float(v), 5) for v in row[at]])

    ids, logits, _ = dec.step(prompt, [0] * n, list(range(n)), want_logits=True)
    out, margins = [int(ids[-1])], [_margin(logits[-1])]
    note(logits[-1])
    for t in range(1, new):
        if stop_below is not None and t <= 32 and margins[-1] < stop_below:
            return None, margins
        ids, logits, _ = dec.step([out[-1]], [0], [n + t - 1], want_logits=True)
        out.append(int(ids[0]))
        margins.append(_margin(logits[0]))
        note(logits[0])
    return out, margins


VARIED = dict(std=0.035, gains="near_one", min_margin=1e-2, min_distinct=16)


def write_varied(seeds):
    cfg = synth.QWEN3_0_6B
    prompt = synth.prompt_tokens(cfg["vocab"], 128, seed=0)
    t0 = time.time()
    for seed in seeds:
        probes = {}
        tokens, margins = greedy(cfg, seed, prompt.tolist(), 64, 192, stop_below=VARIED["min_margin"], probes=probes,
                                 gains=VARIED["gains"], std=VARIED["std"])
        print(f"seed {seed}: {'kept' if tokens else 'near tie at step %d' % (len(margins) - 1)}, "
              f"smallest margin {min(margins[:32]):.4g}, {time.time() - t0:.0f}s", flush=True)
        if tokens:
            break
    else:
        raise SystemExit("no seed kept its margins")
    distinct = len(set(tokens[:32]))
    if distinct < VARIED["min_distinct"]:
        raise SystemExit(f"only {distinct} distinct ids in the first 32")
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "qwen3_0p6b_greedy_varied.json")
    with open(path, "w") as f:
        json.dump({"config": cfg, "seed": seed, "std": VARIED["std"], "gains": VARIED["gains"], "prompt_seed": 0,
                   "prompt_len": 128, "new": 64, "prompt_head": prompt[:8].tolist(), "tokens": tokens,
                   "min_margin": VARIED["min_margin"], "distinct_in_first_32": distinct,
                   "margins": [round(m, 5) for m in margins], "probe_ids": probe_ids(cfg["vocab"]).tolist(),
                   "top_logit": probes["top"], "probe_logits": probes["at"], "numpy": np.__version__,
                   "seconds": round(time.time() - t0, 1)}, f, indent=1)
    print(path, tokens[:8], f"{distinct} distinct, {time.time() - t0:.0f}s")


if __name__ == "__main__":
    if "--varied" in sys.argv:
        write_varied([int(a) for a in sys.argv[1:] if a.isdigit()] or list(range(8)))
        raise SystemExit(0)
    cfg = synth.QWEN3_0_6B
    prompt = synth.prompt_tokens(cfg["vocab"], 128, seed=0)
    seeds = [int(a) for a in sys.argv[1:]] or list(range(8))
    t0 = time.time()
    for seed in seeds:
        probes = {}
        tokens, margins = greedy(cfg, seed, prompt.tolist(), 64, 192, stop_below=MIN_MARGIN, probes=probes)
        print(f"seed {seed}: {'kept' if tokens else 'near tie at step %d' % (len(margins) - 1)}, "
              f"smallest margin {min(margins[:32]):.4g}, {time.time() - t0:.0f}s", flush=True)
        if tokens:
            kept = (seed, tokens, margins, probes)
            if len(set(tokens[:32])) >= MIN_DISTINCT:
                break
            print(f"  only {len(set(tokens[:32]))} distinct ids", flush=True)
    if "kept" not in dir():
        raise SystemExit("no seed kept its margins")
    seed, tokens, margins, probes = kept
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "qwen3_0p6b_greedy.json")
    with open(path, "w") as f:
        json.dump({"config": cfg, "seed": seed, "prompt_seed": 0, "prompt_len": 128, "new": 64,
                   "prompt_head": prompt[:8].tolist(), "tokens": tokens, "min_margin": MIN_MARGIN,
                   "margins": [round(m, 5) for m in margins],
                   "probe_ids": probe_ids(cfg["vocab"]).tolist(), "top_logit": probes["top"], "probe_logits": probes["at"],
                   "numpy": np.__version__,
                   "seconds": round(time.time() - t0, 1)}, f, indent=1)
    print(path, tokens[:8], f"{time.time() - t0:.0f}s")
