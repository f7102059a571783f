"""Random-weights mode: a model folder from a configuration and a seed.

The reference has no such mode.  Matrices and the embedding are N(0, 0.02), all
norm gains 1 + N(0, 0.1); each tensor has a generator of its own, seeded from
(seed, tensor name), so the values do not depend on the order of generation.
``write_random_model`` writes config.json and model.safetensors;
``RandomWeightStore`` hands out the same kinds of tensors straight on the device
for benchmarks of shapes too large to be worth a file.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .loader import TensorSpec, WeightStore
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
GAIN_STD = 0.1


def _tensor_seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") & ((1 << 63) - 1)


def _generate(spec: TensorSpec, seed: int, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    if spec.role == "vector":
        return 1.0 + GAIN_STD * torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
    if spec.role == "table":
        if spec.high < 1:
            raise ValueError(f"integer table '{spec.name}' does not say what range its entries have (TensorSpec.high)")
        return torch.randint(0, spec.high, tuple(spec.shape), generator=g, dtype=torch.int32, device=device)
    return MATRIX_STD * torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)


def write_random_model(config, seed: int, out_dir, dtype: str = "bfloat16") -> Path:
    """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors`` for a typed configuration.

    ``dtype`` is the stored precision: "bfloat16" (values are rounded once, so the
    32-bit and the bfloat16 engine read the same numbers) or "float32"."""
    from ..models import expected_tensors  # late: models imports weights

    store_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    cfg = config.to_dict()
    cfg["torch_dtype"] = dtype
    (out_dir / "config.json").write_text(json.dumps(cfg, indent=2))
    tensors = {s.name: (_generate(s, seed) if s.role == "table" else _generate(s, seed).to(store_dtype))
               for s in expected_tensors(config)}
    write_safetensors(out_dir / "model.safetensors", tensors, {"format": "pt", "seed": str(seed)})
    return out_dir


class RandomWeightStore(WeightStore):
    """A WeightStore whose tensors are drawn on the device when asked for (no file)."""

    def __init__(self, specs: list[TensorSpec], seed: int, compute_dtype: torch.dtype, device):
        super().__init__({}, compute_dtype, device)
        self._specs = {s.name: s for s in specs}
        self._seed = seed

    def names(self):
        return self._specs.keys()

    def __contains__(self, name):
        return name in self._specs

    def check(self, specs):
        return None

    def stored_dtype(self, name):
        return torch.bfloat16

    def _draw(self, name: str) -> torch.Tensor:
        # rounded through bfloat16 like a stored checkpoint would be
        return _generate(self._specs[name], self._seed, self.device).to(torch.bfloat16)

    def matrix(self, name):
        return self._draw(name).to(self.compute_dtype)

    def matrices(self, names, interleave=False):
        parts = [self.matrix(n) for n in names]
        if interleave:
            return torch.stack(parts, dim=1).reshape(-1, parts[0].shape[1]).contiguous()
        return torch.cat(parts, dim=0)

    def vector(self, name):
        t = self._draw(name)
        return t.float() if self.compute_dtype == torch.float32 else t

    def table(self, name):
        return _generate(self._specs[name], self._seed, self.device)
