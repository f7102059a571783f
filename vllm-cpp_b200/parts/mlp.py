"""SwiGLU feed-forward: down(silu(gate(y)) * up(y)), silu(z) = z / (1 + exp(-z))
(src/model.cpp:964-966, 1237-1244), with separate input and output buffers for the
down projection.  gate and up become one [2I, H] matrix at load, gate_i in row 2i
and up_i in row 2i+1, so that one product yields both side by side: in the
tensor-core kernel the two land in adjacent accumulator lanes and the SiLU-gate
is a shuffle away in its epilogue."""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .base import FeedForward
import os

from .linear import choose_splits, matmul_tn

# The SiLU-gate runs in the gate-and-up product's epilogue when that product is not cut into k-slices (whose sums must
# exist before the SiLU): always where its units fill the SMs anyway (the 14B sizes, 272 feature tiles: 8 tokens
# 58.6 -> 56.5 us, 64 tokens 67.6 -> 60.1 against product and SiLU-gate kernel), and above this many tokens, from where
# the one kernel without slices is as fast as the two with them (8B sizes, 64 tokens: 45.8 against 45.7 us; 128: 51.1
# against 52.8; 32: 44.0 against 40.8) and the step has a kernel boundary less.
FUSE_ABOVE_TOKENS = int(os.environ.get("VLLM_CPP_B200_SWIGLU_FUSE_ABOVE", "63"))


class SwiGLUMLP(FeedForward):
    """params: ``hidden_size``, ``intermediate_size``.
    Tensors: ``<prefix>gate_proj.weight`` [I,H], ``up_proj.weight`` [I,H], ``down_proj.weight`` [H,I]."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.w_gate_up = None
        self.w_down = None

    def tensor_specs(self):
        p, H, I = self.prefix, self.hidden, self.inter
        return [TensorSpec(p + "gate_proj.weight", (I, H)), TensorSpec(p + "up_proj.weight", (I, H)),
                TensorSpec(p + "down_proj.weight", (H, I))]

    def bind(self, store):
        p = self.prefix
        self.w_gate_up = store.matrices([p + "gate_proj.weight", p + "up_proj.weight"], interleave=True)
        self.w_down = store.matrix(p + "down_proj.weight")

    def forward(self, x, ctx):
        act = workspace.empty((x.shape[0], self.inter), x.dtype, x.device)
        T, K = x.shape
        if x.dtype == torch.bfloat16 and ops.gemm_tma_ok(x, self.w_gate_up) and (
                T > FUSE_ABOVE_TOKENS or ops.gemm_effective_splits(K, choose_splits(self.w_gate_up.shape[0], T, K)) == 1):
            # no k-slices are needed, or they no longer pay: the SiLU-gate runs in the product's epilogue
            ops.gemm_bf16_swiglu(self.w_gate_up, x, act, ctx.status, after_small_kernel=True)   # (after a norm)
        else:
            gate_up = matmul_tn(x, self.w_gate_up, ctx.status, allow_partials=True, after_small_kernel=True)   # (after a norm)
            ops.swiglu(gate_up, act)
            return matmul_tn(act, self.w_down, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        return matmul_tn(act, self.w_down, ctx.status, out_dtype=torch.float32, allow_partials=True)
