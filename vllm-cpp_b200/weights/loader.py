"""Weights by tensor name, checked against what the model expects.

The reference binds per-layer tensors by exact key and leaves a null pointer
where one is missing, checks no shapes, and finds ``model.norm.weight`` by
substring (src/model.cpp:392-400, 457-523, 569-572).  Here the model states every
tensor it expects (name, shape, role) and one error lists everything that is
missing, unexpected or mis-shaped.

What is stored is kept: bfloat16 stays bfloat16 and a tensor stored in 32-bit
stays 32-bit; integer tables become int32.  Only the consumer decides otherwise:
a *matrix* bound for a tensor-core product is handed out in the engine's compute
dtype, and in the float32 engine everything is widened (exactly) to 32-bit.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

import torch

from .safetensors_io import read_safetensors


class WeightError(ValueError):
    pass


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple
    role: str = "matrix"     # "matrix" (operand of a matrix product), "vector" (gains), "table" (integers)
    optional: bool = False
    high: int = 0            # role "table": entries lie in [0, high) (what the random-weights mode draws from)


class WeightStore:
    """Hands out device tensors by checkpoint name."""

    def __init__(self, tensors: dict[str, torch.Tensor], compute_dtype: torch.dtype, device):
        self._tensors = tensors
        self.compute_dtype = compute_dtype
        self.device = torch.device(device)
        self._cache: dict[tuple, torch.Tensor] = {}

    def names(self):
        return self._tensors.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._tensors

    def check(self, specs: list[TensorSpec]) -> None:
        expected = {s.name: s for s in specs}
        missing = [n for n, s in expected.items() if n not in self._tensors and not s.optional]
        unexpected = sorted(n for n in self._tensors if n not in expected)
        wrong = []
        for n, s in expected.items():
            if n in self._tensors and tuple(self._tensors[n].shape) != tuple(s.shape):
                wrong.append(f"{n}: expected {tuple(s.shape)}, found {tuple(self._tensors[n].shape)}")
        if missing or unexpected or wrong:
            def show(items):
                return "".join(f"\n    {i}" for i in items[:40]) + (f"\n    ... and {len(items) - 40} more" if len(items) > 40 else "")
            msg = "the checkpoint does not match the model:"
            if missing:
                msg += f"\n  missing tensors ({len(missing)}):" + show(sorted(missing))
            if unexpected:
                msg += f"\n  unexpected tensors ({len(unexpected)}):" + show(unexpected)
            if wrong:
                msg += f"\n  wrong shapes ({len(wrong)}):" + show(wrong)
            raise WeightError(msg)

    def _raw(self, name: str) -> torch.Tensor:
        try:
            return self._tensors[name]
        except KeyError:
            raise WeightError(f"tensor '{name}' is not in the checkpoint") from None

    def stored_dtype(self, name: str) -> torch.dtype:
        return self._raw(name).dtype

    def _to_device(self, t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        # .to() copies out of the read-only memory map
        return t.to(device=self.device, dtype=dtype).contiguous()

    def matrix(self, name: str) -> torch.Tensor:
        """Operand of a matrix product, in the engine's compute dtype."""
        key = ("m", name)
        if key not in self._cache:
            self._cache[key] = self._to_device(self._raw(name), self.compute_dtype)
        return self._cache[key]

    def matrices(self, names: list[str], interleave: bool = False) -> torch.Tensor:
        """Several matrices with equal inner size stacked along the output axis (q,k,v -> qkv).  With
        ``interleave`` their rows alternate instead (row n*i + j is row i of matrix j; gate,up -> gate_up)."""
        parts = [self._raw(n) for n in names]
        rows = sum(p.shape[0] for p in parts)
        out = torch.empty((rows, parts[0].shape[1]), dtype=self.compute_dtype, device=self.device)
        if interleave:
            if any(p.shape != parts[0].shape for p in parts):
                raise WeightError(f"tensors {names} must have one shape to be interleaved")
            view = out.view(parts[0].shape[0], len(parts), parts[0].shape[1])
            for j, p in enumerate(parts):
                view[:, j].copy_(p.to(self.device), non_blocking=False)
            return out
        r = 0
        for p in parts:
            out[r: r + p.shape[0]].copy_(p.to(self.device), non_blocking=False)
            r += p.shape[0]
        return out

    def vector(self, name: str) -> torch.Tensor:
        """Gains: bfloat16 stays bfloat16, 32-bit stays 32-bit; everything is 32-bit in the float32 engine."""
        t = self._raw(name)
        if self.compute_dtype == torch.float32 or t.dtype == torch.float16:
            dtype = torch.float32
        else:
            dtype = t.dtype
        if dtype not in (torch.float32, torch.bfloat16):
            raise WeightError(f"tensor '{name}' is stored as {t.dtype}; gains must be floating point")
        return self._to_device(t, dtype)

    def table(self, name: str) -> torch.Tensor:
        t = self._raw(name)
        if t.dtype not in (torch.int32, torch.int64):
            raise WeightError(f"tensor '{name}' is stored as {t.dtype}; an integer table was expected")
        return self._to_device(t, torch.int32)

    def release(self) -> None:
        """Drops host references (memory maps) once every part is bound."""
        self._tensors = {}
        self._cache = {}


def open_model_weights(model_dir, compute_dtype: torch.dtype, device) -> WeightStore:
    """All ``*.safetensors`` of a folder, in name order (src/model.cpp:289-304)."""
    model_dir = Path(model_dir)
    files = sorted(model_dir.glob("*.safetensors"))
    if not files:
        raise WeightError(f"{model_dir}: no .safetensors file in the model folder")
    index = model_dir / "model.safetensors.index.json"
    if index.is_file():
        # a sharded checkpoint says which file holds which tensor: every file it names must be there
        import json
        try:
            named = set(json.loads(index.read_text()).get("weight_map", {}).values())
        except (json.JSONDecodeError, AttributeError):
            raise WeightError(f"{index}: not a valid shard index") from None
        gone = sorted(n for n in named if not (model_dir / n).is_file())
        if gone:
            raise WeightError(f"{model_dir}: the shard index names files that are missing: {gone}")
    tensors: dict[str, torch.Tensor] = {}
    for f in files:
        for name, t in read_safetensors(f).items():
            if name in tensors:
                raise WeightError(f"tensor '{name}' appears in more than one file of {model_dir}")
            tensors[name] = t
    return WeightStore(tensors, compute_dtype, device)
