"""Shared fixtures: tiny model folders with random weights (made in a temporary folder), the
plain implementation's logits for them, and the ``gpu`` marker."""
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Tiny configurations that differ in every size and option.
TINY = {
    # 2 layers, tied head, no window, page 4
    "A": dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=1e4,
              tie_word_embeddings=True),
    # 3 layers, untied head, heads*head_dim != hidden, GQA ratio 3, odd intermediate size, two windowed layers, page 8
    "B": dict(vocab_size=384, hidden_size=96, intermediate_size=200, num_hidden_layers=3, num_attention_heads=6,
              num_key_value_heads=2, head_dim=32, max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=1e6,
              tie_word_embeddings=False, sliding_window=24,
              layer_types=("full_attention", "sliding_attention", "sliding_attention")),
    # head_dim 64 with pages of 16 tokens: in bfloat16 the tensor-core attention kernels (tcgen05 for prompt
    # portions, mma.sync for decoded tokens); four query heads on one KV head, one windowed layer
    "C": dict(vocab_size=320, hidden_size=128, intermediate_size=176, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=1, head_dim=64, max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=5e4,
              tie_word_embeddings=False, sliding_window=40, layer_types=("sliding_attention", "full_attention")),
    # head_dim 128, the serving models' head size (its own norm-rotate-store kernel, 128-lane attention tiles),
    # two query heads a KV head, an intermediate size that is no multiple of 64
    "D": dict(vocab_size=512, hidden_size=256, intermediate_size=344, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=128, max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=1e6,
              tie_word_embeddings=False),
}
TINY_SEED = {"A": 0, "B": 2, "C": 4, "D": 6}
TINY_PAGE = {"A": 4, "B": 8, "C": 16, "D": 16}


def tiny_config(name):
    from vllm_cpp_b200 import Qwen3Config
    return Qwen3Config(**TINY[name])


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (bfloat16-stored random weights)."""
    from vllm_cpp_b200 import write_random_model
    out = {}
    for name in TINY:
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(tiny_config(name), TINY_SEED[name], d, dtype="bfloat16")
        out[name] = d
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    """name -> (config dict, weights) as the plain implementation reads them."""
    import plain_qwen3
    return {name: plain_qwen3.read_model(d) for name, d in model_dirs.items()}


class PlainLogits:
    """Caches the plain implementation's logits of whole sequences."""

    def __init__(self, plain_models):
        self.models = plain_models
        self.cache = {}

    def __call__(self, name, tokens):
        import plain_qwen3
        key = (name, tuple(tokens))
        if key not in self.cache:
            cfg, w = self.models[name]
            self.cache[key] = plain_qwen3.forward(cfg, w, list(tokens)).numpy()
        return self.cache[key]


@pytest.fixture(scope="session")
def plain_logits(plain_models):
    return PlainLogits(plain_models)


def random_tokens(vocab, n, seed):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
