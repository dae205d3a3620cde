"""The bidirectional embedding encoder against the CPU checker's ops composed in the same order, with
bf16 at the same storage points.  Embeddings are unit-length f32 rows: within 1e-2 of the checker
relative to the largest component, and cosine above 0.999 per text."""
import numpy as np
import pytest
import torch

import oracle as O
from tessera_b200 import synth
from tests.util import dev_u32

pytestmark = pytest.mark.gpu

CFG = dict(layers=2, hidden=256, heads=2, kv_heads=1, head_dim=256, ffn=384, vocab=500, eps=1e-6, theta=1e4)


def _oracle_encode(cfg, w, tokens, lens):
    h_, d, heads, kvh = cfg["hidden"], cfg["head_dim"], cfg["heads"], cfg["kv_heads"]
    out = []
    at = 0
    for n in lens:
        ids = tokens[at:at + n]
        at += n
        pos = np.arange(n)
        x = O.bf16_widen(O.gather(w["embed"], ids))
        for l in range(cfg["layers"]):
            g = lambda f: w[f"layers.{l}.{f}"]
            h = O.bf16_round(O.rms_norm(x, g("ln1"), cfg["eps"]))
            q = O.bf16_round(O.matmul(h, g("q"))).reshape(n, heads, d)
            k = O.bf16_round(O.matmul(h, g("k"))).reshape(n, kvh, d)
            v = O.bf16_round(O.matmul(h, g("v"))).reshape(n, kvh, d)
            q = O.bf16_round(O.rope(O.rms_norm(q, g("q_norm"), cfg["eps"]), pos, cfg["theta"], "halves"))
            k = O.bf16_round(O.rope(O.rms_norm(k, g("k_norm"), cfg["eps"]), pos, cfg["theta"], "halves"))
            a = O.bf16_round(O.attend(q[None], k[None], v[None], "bidirectional", d ** -0.5)[0]).reshape(n, heads * d)
            x = O.matmul(a, g("o")) + x
            h = O.bf16_round(O.rms_norm(x, g("ln2"), cfg["eps"]))
            act = O.bf16_round(O.act(O.matmul(h, g("mlp.gate")), "gelu_tanh") * O.matmul(h, g("mlp.up")))
            x = O.matmul(act, g("mlp.down")) + x
        hid = O.rms_norm(x, w["norm"], cfg["eps"])
        mean = O.mean(hid, 0)
        out.append(mean / max(float(np.sqrt((mean * mean).sum())), 1e-12))
    return np.stack(out)


def test_embeddings_match_oracle():
    from tessera_b200.encoder import Encoder
    cfg = CFG
    weights = list(synth.decoder_weights(cfg, seed=21, gains="near_one", std=0.05))
    enc = Encoder(cfg, weights)
    rng = np.random.default_rng(2)
    lens = [5, 130, 64, 1, 33]
    tokens = rng.integers(0, cfg["vocab"], size=sum(lens)).astype(np.uint32)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
    got = enc.forward(dev_u32(tokens), dev_u32(cu), max(lens))
    torch.cuda.synchronize()
    got = got.cpu().numpy()
    want = _oracle_encode(cfg, dict(weights), tokens, lens)
    assert np.allclose(np.linalg.norm(got, axis=1), 1.0, atol=1e-4)
    assert np.max(np.abs(got - want)) <= 1e-2 * np.max(np.abs(want))
    assert np.all((got * want).sum(axis=1) > 0.999)
