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


def test_half_split_rotation_is_the_interleaved_one_on_permuted_lanes():
    """The reference's CPU path rotates lanes (2i, 2i+1) (src/model.cpp:983-985) and is what the compiled-reference
    anchor pins; the model as intended pairs lanes (i, i + head_dim/2) (src/mlx_backend.cpp:411-412).  The two are
    the same rotation up to the lane permutation 2i -> i, 2i+1 -> i + head_dim/2, so the half-split function
    inherits the anchored one's angles and signs."""
    hd = 32
    cos, sin = P.rope_angles(hd, 1e4, [0, 1, 7, 100])
    x = torch.randn(4, 3, hd, dtype=torch.float64)
    perm = torch.cat([torch.arange(0, hd, 2), torch.arange(1, hd, 2)])     # interleaved lane that sits at each half-split lane
    inter = P.rope_interleaved(x, cos, sin)
    # put x's half-split lanes where the interleaved function pairs them, rotate, and bring them back
    y = torch.empty_like(x)
    y[..., perm] = x
    back = P.rope_interleaved(y, cos, sin)[..., perm]
    assert torch.allclose(P.rope_half_split(x, cos, sin), back, atol=1e-15)
    assert not torch.allclose(P.rope_half_split(x, cos, sin), inter)


def test_one_head_by_hand():
    """A pin that does not come from the same hand as the code: head_dim 4, theta 100, two positions, gains other
    than one, every number below worked out with pencil and the formulas alone
    (norm: x * w / sqrt(mean(x^2) + eps), cuda/attention.cu:169-182; angle = pos * theta^(-2i/hd),
    src/model.cpp:979-982; pairs (i, i + hd/2), src/mlx_backend.cpp:411-412; norm before rotation).

    x = (3, 4, 0, 0), eps = 0: mean(x^2) = 25/4, 1/rms = 2/5, normalised (1.2, 1.6, 0, 0); gains (2, 1, 3, 0.5)
    give (2.4, 1.6, 0, 0).  At position 1 the angles are 1 * 100^0 = 1 and 1 * 100^(-1/2) = 0.1: lane pair (0, 2)
    turns by 1 rad, pair (1, 3) by 0.1 rad: (2.4 cos 1, 1.6 cos 0.1, 2.4 sin 1, 1.6 sin 0.1).  At position 0
    nothing turns."""
    import math
    x = torch.tensor([[[3.0, 4.0, 0.0, 0.0]], [[3.0, 4.0, 0.0, 0.0]]], dtype=torch.float64)   # [T=2, heads=1, hd=4]
    w = torch.tensor([2.0, 1.0, 3.0, 0.5], dtype=torch.float64)
    n = P.head_rms_norm(x, w, 0.0)
    assert torch.allclose(n[0, 0], torch.tensor([2.4, 1.6, 0.0, 0.0], dtype=torch.float64), atol=1e-15)
    cos, sin = P.rope_angles(4, 100.0, [0, 1])
    assert torch.allclose(cos[1], torch.tensor([math.cos(1.0), math.cos(0.1)], dtype=torch.float64))
    r = P.rope_half_split(n, cos, sin)
    assert torch.allclose(r[0, 0], n[0, 0])
    want = torch.tensor([2.4 * math.cos(1.0), 1.6 * math.cos(0.1), 2.4 * math.sin(1.0), 1.6 * math.sin(0.1)], dtype=torch.float64)
    assert torch.allclose(r[1, 0], want, atol=1e-15)
    # a second vector with weight in the upper half, so that the sign of the sine term is pinned as well:
    # x = (0, 0, 1, 0) at position 1 -> pair (0, 2) = (0, 1) turned by 1 rad = (-sin 1, cos 1)
    e = torch.tensor([[[0.0, 0.0, 1.0, 0.0]]], dtype=torch.float64)
    r = P.rope_half_split(e, cos[1:], sin[1:])
    assert torch.allclose(r[0, 0], torch.tensor([-math.sin(1.0), 0.0, math.cos(1.0), 0.0], dtype=torch.float64), atol=1e-15)
    # eps enters under the root: x = (1, 1, 1, 1), eps = 3 -> 1 / sqrt(1 + 3) = 1/2
    one = torch.ones(1, 1, 4, dtype=torch.float64)
    assert torch.allclose(P.head_rms_norm(one, torch.ones(4, dtype=torch.float64), 3.0), 0.5 * one)
    # and the whole attention of two positions, scores scaled by 1/sqrt(hd) = 1/2: q = k, |k0| = |k1| = 2 would
    # need more arithmetic than a pencil likes; take q1 = (2, 0, 0, 0), k0 = (2, 0, 0, 0), k1 = (0, 0, 0, 0):
    # scores (2, 0), weights e^2/(e^2+1) and 1/(e^2+1); v0 = (1, 0, 0, 0), v1 = (0, 1, 0, 0)
    q = torch.tensor([[[0.0, 0, 0, 0]], [[2.0, 0, 0, 0]]], dtype=torch.float64)
    k = torch.tensor([[[2.0, 0, 0, 0]], [[0.0, 0, 0, 0]]], dtype=torch.float64)
    v = torch.tensor([[[1.0, 0, 0, 0]], [[0.0, 1, 0, 0]]], dtype=torch.float64)
    a = P.attention(q, k, v)
    e2 = math.exp(2.0)
    assert torch.allclose(a[1, 0], torch.tensor([e2 / (e2 + 1), 1 / (e2 + 1), 0, 0], dtype=torch.float64), atol=1e-15)
    assert torch.allclose(a[0, 0], v[0, 0])     # position 0 sees itself only
