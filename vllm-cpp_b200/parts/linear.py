"""Dense projections y = x . W^T with W stored [out, in] as in the checkpoint
(src/model.cpp:932-944).

float32 engine: the package's FFMA kernel, true 32-bit.  bfloat16 engine: the
package's tcgen05/TMA kernel, bfloat16 operands and 32-bit accumulation in TMEM.
With few tokens the product is a stream of weights from HBM; the inner dimension
is then cut into slices so that enough blocks are in flight to fill the GPU, each
slice writes a 32-bit partial sum, and whichever kernel reads the result next adds
the slices in order.  The reference calls cublasGemmEx for these products
(cuda/tp_model.cu:259-269); ``VLLM_CPP_B200_LIBRARY_GEMM=1`` swaps a library
product in for comparison runs.
"""
from __future__ import annotations

import os

import torch

from .. import ops

NUM_SMS = 148
LIBRARY_GEMM = os.environ.get("VLLM_CPP_B200_LIBRARY_GEMM", "0") == "1"


def token_tile(T: int) -> int:
    for bn in (16, 32, 64, 128, 256):
        if T <= bn:
            return bn
    return 256


def choose_splits(M: int, T: int, K: int, max_splits: int = 8) -> int:
    """Number of k-slices for a product that streams weights (few tokens): the kernel's persistent blocks, one
    per SM, walk (feature tile x token tile x k-slice) units round robin, so the slices are chosen to spread
    the k-blocks evenly over the SMs; each extra slice costs one more partial sum to write and add."""
    if T > 128:
        return 1      # enough tokens per weight tile: the product is compute bound and partial sums only cost traffic
    tiles = -(-M // 128) * -(-T // token_tile(T))
    total_kb = -(-K // 64)
    best, best_cost = 1, None
    for s in range(1, max_splits + 1):
        kb = -(-total_kb // s)
        if s > 1 and kb < 8:
            break
        s_eff = -(-total_kb // kb)
        units = tiles * s_eff
        busiest = -(-units // NUM_SMS) * kb                      # k-blocks the busiest SM streams
        cost = busiest + 3 * -(-units // NUM_SMS) + 0.02 * total_kb * s_eff   # + per-unit and per-partial overheads
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def matmul_tn(x: torch.Tensor, w: torch.Tensor, status: torch.Tensor | None = None, *, out_dtype=None,
              allow_partials: bool = False) -> torch.Tensor:
    """x [T,K], w [N,K] -> [T,N] in ``out_dtype`` (default: x's dtype).  With ``allow_partials`` the result may
    come back as [S,T,N] 32-bit partial sums, which the caller's next kernel adds."""
    out_dtype = out_dtype or x.dtype
    T, N = x.shape[0], w.shape[0]
    if x.dtype == torch.float32:
        if w.dtype != torch.float32:
            raise ops.KernelError("float32 activations need float32 weights")
        out = torch.empty((T, N), dtype=torch.float32, device=x.device)
        ops.sgemm_tn(x, w, out)
        return out
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ops.KernelError(f"matmul_tn: unsupported operand types {x.dtype} x {w.dtype}")
    if LIBRARY_GEMM:
        return torch.mm(x, w.t(), out_dtype=torch.float32) if out_dtype == torch.float32 else torch.mm(x, w.t())
    K = x.shape[1]
    if not ops.gemm_tma_ok(x, w):
        # rows that are not 16-byte multiples (an inner size like 100): the plain kernel takes them
        out = torch.empty((T, N), dtype=out_dtype, device=x.device)
        ops.gemm_bf16_plain(x, w, out)
        return out
    splits = choose_splits(N, T, K) if allow_partials else 1
    splits = ops.gemm_effective_splits(K, splits)
    if splits > 1:
        out = torch.empty((splits, T, N), dtype=torch.float32, device=x.device)
    else:
        out = torch.empty((T, N), dtype=out_dtype, device=x.device)
    ops.gemm_bf16_tn(w, x, out, splits, status)
    return out
