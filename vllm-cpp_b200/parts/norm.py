"""RMSNorm: y = w * x / sqrt(mean(x^2) + eps), the gain multiplying directly
(src/model.cpp:924-930), fused with the addition of the pending delta into the
32-bit residual stream (the reference adds separately, src/model.cpp:1226-1227, 1248-1250)."""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .base import Norm


class RMSNorm(Norm):
    """params: ``size``, ``eps``.  Tensor: ``<prefix>weight`` [size]."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = None

    def tensor_specs(self):
        return [TensorSpec(self.prefix + "weight", (self.size,), "vector")]

    def bind(self, store):
        self.weight = store.vector(self.prefix + "weight")

    def forward(self, resid, delta, rows=None):
        n = resid.shape[0] if rows is None else rows.numel()
        out = workspace.empty((n, self.size), self.build.compute_dtype, resid.device)
        ops.add_rmsnorm(resid, delta, self.weight, self.eps, out, rows)
        return out
