"""Dense projections y = x . W^T with W stored [out, in] as in the checkpoint
(src/model.cpp:932-944).

float32 engine: the package's FFMA kernel, true 32-bit.  bfloat16 engine: a
tensor-core product with 32-bit accumulation; where the reference's own CUDA
path calls a library for its products (cublasGemmEx, cuda/tp_model.cu:259-269)
a library product stands here too.
"""
from __future__ import annotations

import torch

from .. import ops


def matmul_tn(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x [T,K], w [N,K] -> [T,N] in ``out_dtype`` (default: x's dtype)."""
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32:
        if w.dtype != torch.float32:
            raise ops.KernelError("float32 activations need float32 weights")
        out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=x.device)
        ops.sgemm_tn(x, w, out)
        return out
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ops.KernelError(f"matmul_tn: unsupported operand types {x.dtype} x {w.dtype}")
    if out_dtype == torch.float32:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    return torch.mm(x, w.t())
