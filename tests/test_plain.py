"""The plain implementation itself: anchored once against the reference's compiled CPU code
(tests/golden), and checked for the properties the engine tests rely on."""
import json
import sys
from pathlib import Path

import numpy as np
import torch

import plain_qwen3 as P
from conftest import TINY, random_tokens

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_matches_the_compiled_reference():
    """Last-position logits of laik/vllm-cpp's forward_cpu (tests/golden/make_golden.py made them) equal the
    plain implementation's with the reference's three departures switched on."""
    sys.path.insert(0, str(GOLDEN))
    import make_golden as G
    d = json.loads((GOLDEN / "reference_logits.json").read_text())
    w = {k: torch.from_numpy(v.astype(np.float64)) for k, v in G.make_weights(d["spec"]).items()}
    cfg = G.make_config(d["spec"])
    for n, ref in d["logits"].items():
        lg = P.forward(cfg, w, d["tokens"][:int(n)], qk_norm=False, rope_interleaved_lanes=True, down_in_place=True)[-1]
        assert np.abs(lg.numpy() - np.array(ref)).max() < 5e-6
    # and the switches matter: the intended model gives other logits
    lg = P.forward(cfg, w, d["tokens"][:5])[-1].numpy()
    assert np.abs(lg - np.array(d["logits"]["5"])).max() > 1e-3


def test_causal_prefixes_agree(plain_models):
    """Logits at position p do not depend on later tokens."""
    for name in TINY:
        cfg, w = plain_models[name]
        toks = random_tokens(cfg["vocab_size"], 40, 9)
        full = P.forward(cfg, w, toks)
        part = P.forward(cfg, w, toks[:17])
        assert torch.allclose(full[:17], part, atol=1e-12)


def test_window_limits_what_a_position_sees():
    q = torch.randn(30, 2, 16, dtype=torch.float64)
    k = torch.randn(30, 1, 16, dtype=torch.float64)
    v = torch.randn(30, 1, 16, dtype=torch.float64)
    full, win = P.attention(q, k, v), P.attention(q, k, v, window=8)
    assert torch.allclose(full[:8], win[:8]) and not torch.allclose(full[8:], win[8:])
    # position p with window W equals plain attention over keys p-W+1..p
    p = 20
    alone = P.attention(q[p - 7:p + 1], k[p - 7:p + 1], v[p - 7:p + 1])[-1]
    assert torch.allclose(alone, win[p])
    assert P.layer_windows({"num_hidden_layers": 3, "sliding_window": 24, "use_sliding_window": True, "max_window_layers": 1}) == [None, 24, 24]
    assert P.layer_windows(TINY["B"]) == [None, 24, 24]


def test_rope_is_a_rotation_by_position_differences():
    cos, sin = P.rope_angles(32, 1e4, [3, 10])
    x, y = torch.randn(1, 1, 32, dtype=torch.float64), torch.randn(1, 1, 32, dtype=torch.float64)
    for rope in (P.rope_half_split, P.rope_interleaved):
        a = rope(x.repeat(2, 1, 1), cos, sin)
        assert torch.allclose(a.norm(dim=-1), x.norm(dim=-1).expand(2, 1))
        cos2, sin2 = P.rope_angles(32, 1e4, [13, 20])
        d1 = (rope(x, cos[:1], sin[:1]) * rope(y, cos[1:], sin[1:])).sum()
        d2 = (rope(x, cos2[:1], sin2[:1]) * rope(y, cos2[1:], sin2[1:])).sum()
        assert torch.allclose(d1, d2)


def test_sampling_rules():
    lg = np.array([0.5, 2.0, 2.0, -1.0, 1.9], dtype=np.float32)
    assert P.sample(lg, temperature=0.0) == 1                      # lowest index among ties
    assert P.sample(lg, temperature=0.0, repeat_penalty=1.5, history=[1, 2]) == 4
    assert list(P.penalise([2.0, -2.0, 0.0], [0, 0, 1, 2], 2.0)) == [0.5, -4.0, 0.0]   # once per occurrence
    keep = P.nucleus(np.log(np.array([0.5, 0.3, 0.15, 0.05])), 0.79)
    assert list(keep) == [True, True, False, False]
    keep = P.nucleus(np.log(np.array([0.5, 0.3, 0.15, 0.05])), 0.81)
    assert list(keep) == [True, True, True, False]
    draws = [P.sample(lg, temperature=1.0, seed=3, step=s) for s in range(300)]
    assert draws == [P.sample(lg, temperature=1.0, seed=3, step=s) for s in range(300)]   # a function of (seed, step)
    freq = np.bincount(draws, minlength=5) / 300
    want = np.exp(lg - lg.max()); want /= want.sum()
    assert np.abs(freq - want).max() < 0.1
    us = [P.uniform(1, 2, i) for i in range(1000)]
    assert 0 < min(us) and max(us) < 1 and abs(np.mean(us) - 0.5) < 0.05
