"""Plain, slow Qwen3-dense decoder used as the oracle of the test-suite.

Whole sequences, no cache, no batching, one function per part, float64 by
default.  It shares no code with the package under test: it reads config.json
and model.safetensors itself and restates every formula from the reference's
sources (laik/vllm-cpp; file:line given per function, paths relative to that
project).  Where the reference's CPU forward departs from the intended Qwen3
model (per-head q/k norm never applied, interleaved RoPE lanes, constant RoPE
base), the intended model is the default and the reference's behaviour is
kept behind switches (``qk_norm=False``, ``rope_interleaved_lanes=True``,
``down_in_place=True``) so the
oracle itself can be anchored against the compiled reference
(tests/golden/make_golden.py).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# --------------------------------------------------------------------------
# reading a model folder (independent of the package's loader)
# --------------------------------------------------------------------------

_ST_DTYPES = {"F32": (np.float32, 4), "F16": (np.float16, 2), "BF16": (np.uint16, 2), "I32": (np.int32, 4)}


def read_safetensors(path, max_rows=None) -> dict[str, torch.Tensor]:
    """File layout as src/model.cpp:169-219 reads it: 8-byte little-endian header
    length, JSON header {name: {dtype, shape, data_offsets}}, then raw data;
    bf16 widened as src/model.cpp:262-275 does (bits << 16).
    ``max_rows`` {tensor name: n} keeps only the first n rows of those tensors (a
    vocabulary too large to hold in 64-bit; the rest of the file is not read)."""
    path = Path(path)
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
    base = 8 + hlen
    raw = np.memmap(path, dtype=np.uint8, mode="r")
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        npdt, size = _ST_DTYPES[meta["dtype"]]
        b, e = meta["data_offsets"]
        shape = list(meta["shape"])
        if max_rows and name in max_rows and shape and shape[0] > max_rows[name]:
            shape[0] = max_rows[name]
            e = b + int(np.prod(shape)) * size
        arr = np.frombuffer(raw[base + b : base + e], dtype=npdt).reshape(shape)
        if meta["dtype"] == "BF16":
            arr = (arr.astype(np.uint32) << 16).view(np.float32)
        out[name] = torch.from_numpy(np.array(arr, dtype=np.float64 if arr.dtype != np.int32 else np.int32))
    return out


def read_model(model_dir, vocab_rows=None):
    """``vocab_rows``: keep only that many rows of the embedding table and the LM head (token ids and logits
    below that number are then all the oracle can speak about)."""
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    limit = {"model.embed_tokens.weight": vocab_rows, "lm_head.weight": vocab_rows} if vocab_rows else None
    weights = read_safetensors(model_dir / "model.safetensors", limit)
    return cfg, weights


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------


def embed(ids, table):
    """x[t,:] = E[id_t,:] (src/model.cpp:1157-1163)."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def rms_norm(x, weight, eps):
    """y = w * x / sqrt(mean(x^2) + eps) over the last axis (src/model.cpp:924-930)."""
    inv = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return weight * x * inv


def linear(x, w):
    """y = x . W^T with W stored [out, in] (src/model.cpp:932-944)."""
    return x @ w.T


def head_rms_norm(x, weight, eps):
    """RMSNorm over each head's head_dim lanes, one gain vector shared by all
    heads (cuda/attention.cu:169-182; gains loaded at src/model.cpp:501-504).
    x: [T, heads, head_dim]."""
    return rms_norm(x, weight, eps)


def rope_angles(head_dim, theta, positions):
    """inv_freq_i = 1 / theta^(2i/head_dim), angle = inv_freq_i * pos
    (src/model.cpp:582-589, 979-982).  Returns cos, sin of shape [T, head_dim/2]."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    inv_freq = 1.0 / (float(theta) ** (2.0 * i / head_dim))
    ang = torch.as_tensor(positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
    return torch.cos(ang), torch.sin(ang)


def rope_half_split(x, cos, sin):
    """Rotation on lanes (i, i + head_dim/2): the pairing of the reference's
    MLX path (src/mlx_backend.cpp:411-412, traditional=false) and of its CUDA
    rope_kernel (cuda/attention_kernels.cuh:275-287).  x: [T, heads, head_dim]."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def rope_interleaved(x, cos, sin):
    """Rotation on lanes (2i, 2i+1): the pairing of the reference's CPU path
    (src/model.cpp:983-985).  Kept only to anchor this file against it."""
    x0, x1 = x[..., 0::2], x[..., 1::2]
    c, s = cos[:, None, :], sin[:, None, :]
    out = torch.empty_like(x)
    out[..., 0::2] = x0 * c - x1 * s
    out[..., 1::2] = x0 * s + x1 * c
    return out


def attention(q, k, v, window=None):
    """Causal softmax attention of whole sequences with grouped KV heads.

    Query head h reads KV head h // (heads / kv_heads); scores (q.k)/sqrt(head_dim);
    position p sees keys 0..p (src/model.cpp:1000-1052, causal by truncation at
    :1214-1220); exact softmax (the reference's +1e-9 guard is not kept).
    ``window`` W restricts position p to keys p-W+1..p.
    q: [T, heads, hd]; k, v: [T, kv_heads, hd] -> [T, heads, hd]."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty_like(q)
    pos = torch.arange(T)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > pos[:, None] - int(window)
    for h in range(nh):
        kh = h // g
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        w = torch.softmax(s, dim=-1)
        out[:, h, :] = w @ v[:, kh, :]
    return out


def silu(z):
    """z / (1 + exp(-z)) (src/model.cpp:964-966)."""
    return z / (1.0 + torch.exp(-z))


def swiglu_mlp(y, w_gate, w_up, w_down, down_in_place=False):
    """down(silu(gate(y)) * up(y)) (src/model.cpp:1237-1244).  The reference computes the
    down projection in place -- output j is stored over input j before output j+1 is
    summed (:1243-1244) -- which the intended model does not do; ``down_in_place`` repeats
    that only so this file can be anchored against the reference's output."""
    a = silu(linear(y, w_gate)) * linear(y, w_up)
    if not down_in_place:
        return linear(a, w_down)
    out = torch.empty(a.shape[0], w_down.shape[0], dtype=a.dtype)
    for t in range(a.shape[0]):
        buf = a[t].clone()
        for j in range(w_down.shape[0]):
            v = buf @ w_down[j]
            out[t, j] = v
            if j < buf.shape[0]:
                buf[j] = v
    return out


# --------------------------------------------------------------------------
# whole model
# --------------------------------------------------------------------------


def layer_windows(cfg):
    """Per-layer attention window from Qwen3's config.json keys: ``layer_types``
    if given ("sliding_attention" -> ``sliding_window``), else
    ``use_sliding_window`` with layers >= ``max_window_layers`` windowed."""
    L = cfg["num_hidden_layers"]
    sw = cfg.get("sliding_window")
    lt = cfg.get("layer_types")
    if lt is not None:
        return [int(sw) if t == "sliding_attention" else None for t in lt]
    if cfg.get("use_sliding_window", False) and sw is not None:
        mwl = cfg.get("max_window_layers", L)
        return [int(sw) if i >= mwl else None for i in range(L)]
    return [None] * L


def forward(cfg, weights, ids, *, qk_norm=True, rope_interleaved_lanes=False, down_in_place=False, return_hidden=False):
    """Logits [T, vocab] at every position of one whole sequence
    (the layer order of src/model.cpp:1176-1263)."""
    W = {k: v.double() for k, v in weights.items()}
    H = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim", H // nh)
    eps = cfg.get("rms_norm_eps", 1e-6)
    theta = cfg.get("rope_theta", 1e6)
    T = len(ids)
    windows = layer_windows(cfg)
    cos, sin = rope_angles(hd, theta, list(range(T)))
    rope = rope_interleaved if rope_interleaved_lanes else rope_half_split

    x = embed(ids, W["model.embed_tokens.weight"])
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        y = rms_norm(x, W[p + "input_layernorm.weight"], eps)
        q = linear(y, W[p + "self_attn.q_proj.weight"]).view(T, nh, hd)
        k = linear(y, W[p + "self_attn.k_proj.weight"]).view(T, nkv, hd)
        v = linear(y, W[p + "self_attn.v_proj.weight"]).view(T, nkv, hd)
        if qk_norm:
            q = head_rms_norm(q, W[p + "self_attn.q_norm.weight"], eps)
            k = head_rms_norm(k, W[p + "self_attn.k_norm.weight"], eps)
        q, k = rope(q, cos, sin), rope(k, cos, sin)
        a = attention(q, k, v, windows[l]).reshape(T, nh * hd)
        x = x + linear(a, W[p + "self_attn.o_proj.weight"])
        y = rms_norm(x, W[p + "post_attention_layernorm.weight"], eps)
        x = x + swiglu_mlp(y, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"], W[p + "mlp.down_proj.weight"],
                           down_in_place)
    if return_hidden:
        return x
    y = rms_norm(x, W["model.norm.weight"], eps)
    head = W["lm_head.weight"] if "lm_head.weight" in W else W["model.embed_tokens.weight"]
    return linear(y, head)


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------

_M64 = (1 << 64) - 1


def _mix64(z):
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform(seed, step, index):
    """Counter-based uniform in (0,1): two rounds of a 64-bit finaliser over
    (seed, step) then the element index; the top 23 bits give (k + 0.5) / 2^23,
    which a 32-bit float holds exactly."""
    key = _mix64(((seed & 0xFFFFFFFF) << 32) | (step & 0xFFFFFFFF))
    bits = _mix64(key ^ (index & _M64))
    return ((bits >> 41) + 0.5) / float(1 << 23)


def penalise(logits, history, penalty):
    """Repetition penalty, once per occurrence in the history: positive scores
    are divided, negative multiplied (src/model.cpp:1299-1307)."""
    s = np.array(logits, dtype=np.float64)
    for t in history:
        if 0 <= t < len(s):
            if s[t] > 0:
                s[t] /= penalty
            elif s[t] < 0:
                s[t] *= penalty
    return s


def nucleus(scores, top_p):
    """Mask of the shortest descending-probability prefix whose mass reaches
    top_p (src/model.cpp:1314-1334); ties at the cut are all kept."""
    p = np.exp(scores - scores.max())
    p /= p.sum()
    order = np.argsort(-p, kind="stable")
    cum = np.cumsum(p[order])
    keep = int(np.searchsorted(cum, top_p, side="left")) + 1
    keep = min(keep, len(p))
    cut = p[order[keep - 1]]
    return p >= cut


def sample(logits, *, temperature, top_p=1.0, repeat_penalty=1.0, history=(), seed=0, step=0):
    """Next token from one row of logits.  temperature <= 0: argmax, lowest
    index on ties (src/mlx_backend.cpp:516-524).  Else the categorical draw of
    src/model.cpp:1309-1351 from softmax(scores / temperature) cut to the nucleus,
    drawn as argmax(scores/T + Gumbel(u_i)) with counter-based u_i."""
    s = penalise(logits, history, repeat_penalty) if repeat_penalty != 1.0 else np.array(logits, dtype=np.float64)
    if temperature <= 0:
        return int(np.argmax(s))
    s = s / temperature
    keep = nucleus(s, top_p) if top_p < 1.0 else np.ones(len(s), dtype=bool)
    u = np.array([uniform(seed, step, i) for i in range(len(s))])
    z = s - np.log(-np.log(u))
    z[~keep] = -np.inf
    return int(np.argmax(z))


def generate(cfg, weights, prompt, max_new, *, temperature=0.0, top_p=1.0, repeat_penalty=1.0, seed=0, stop_ids=()):
    """Whole-sequence recompute per token (src/model.cpp:1358-1384), with the
    engine path's history = prompt + generated (src/paged_engine.cpp:544-549)."""
    toks = list(prompt)
    out = []
    for step in range(max_new):
        logits = forward(cfg, weights, toks)[-1].numpy()
        t = sample(logits.astype(np.float32), temperature=temperature, top_p=top_p, repeat_penalty=repeat_penalty,
                   history=toks, seed=seed, step=step)
        out.append(t)
        toks.append(t)
        if t in stop_ids:
            break
    return out
