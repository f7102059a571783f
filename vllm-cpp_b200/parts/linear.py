"""Dense projections y = x . W^T with W stored [out, in] as in the checkpoint
(src/model.cpp:932-944).

float32 engine: the package's FFMA kernel, true 32-bit.  bfloat16 engine: the
package's tcgen05/TMA kernel, bfloat16 operands and 32-bit accumulation in TMEM.
With few tokens the product is a stream of weights from HBM; the inner dimension
is then cut into slices so that enough blocks are in flight to fill the GPU, each
slice writes a 32-bit partial sum, and whichever kernel reads the result next adds
the slices in order.  The reference calls cublasGemmEx for these products
(cuda/tp_model.cu:259-269); no library product stands on this path.
"""
from __future__ import annotations

import functools

import torch

from .. import ops, workspace

MAX_SPLIT_TOKENS = 1024     # above this many tokens a product is never cut into k-slices


def token_tile(T: int) -> int:
    for bn in (16, 32, 64, 128, 256):
        if T <= bn:
            return bn
    return 256


@functools.lru_cache(maxsize=4096)
def choose_splits(M: int, T: int, K: int, max_splits: int = 8, num_sms: int | None = None) -> int:
    """Number of k-slices of a product whose units (feature tile x token tile) do not fill the SMs by themselves.
    The kernel's persistent blocks, one per SM, walk (feature tile x token tile x k-slice) units round robin, so
    the slices are chosen to spread the k-blocks evenly over the SMs in whole rounds; each extra slice costs one
    more 32-bit partial sum to write and to add."""
    NUM_SMS = num_sms or ops.num_sms()
    total_kb = -(-K // 64)
    if T > MAX_SPLIT_TOKENS:
        return 1      # units in plenty: partial sums would only cost traffic
    if T > 128:
        # 128 x 256 units (the shape the kernel uses for sliced products of more than 128 tokens).  Times in us,
        # fitted to measurements at 160 to 1,024 tokens: half a microsecond per k-block of a unit, two per unit,
        # and the partial sums written and read back at about 5 TB/s.
        tiles = -(-M // 128) * -(-T // 256)
        best, best_cost = 1, None
        for s in range(1, max_splits + 1):
            kb = -(-total_kb // s)
            if s > 1 and kb < 8:
                break
            s_eff = -(-total_kb // kb)
            rounds = -(-tiles * s_eff // NUM_SMS)
            cost = rounds * (0.5 * kb + 2.0) + (s_eff * T * M * 8 / 5e6 if s_eff > 1 else 0.0)
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = s, cost
        return best
    tiles = -(-M // 128) * -(-T // token_tile(T))
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
              allow_partials: bool = False, after_small_kernel: bool = False) -> torch.Tensor:
    """x [T,K], w [N,K] -> [T,N] in ``out_dtype`` (default: x's dtype).  With ``allow_partials`` the result may
    come back as [S,T,N] 32-bit partial sums, which the caller's next kernel adds.  ``after_small_kernel``: what made
    ``x`` was a short kernel (see ops.gemm_bf16_tn)."""
    out_dtype = out_dtype or x.dtype
    T, N = x.shape[0], w.shape[0]
    if x.dtype == torch.float32:
        if w.dtype != torch.float32:
            raise ops.KernelError("float32 activations need float32 weights")
        out = workspace.empty((T, N), torch.float32, x.device)
        ops.sgemm_tn(x, w, out)
        return out
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ops.KernelError(f"matmul_tn: unsupported operand types {x.dtype} x {w.dtype}")
    K = x.shape[1]
    if not ops.gemm_tma_ok(x, w):
        # rows that are not 16-byte multiples (an inner size like 100): the plain kernel takes them
        out = workspace.empty((T, N), out_dtype, x.device)
        ops.gemm_bf16_plain(x, w, out)
        return out
    splits = choose_splits(N, T, K) if allow_partials else 1
    splits = ops.gemm_effective_splits(K, splits)
    if splits > 1:
        out = workspace.empty((splits, T, N), torch.float32, x.device)
    else:
        out = workspace.empty((T, N), out_dtype, x.device)
    ops.gemm_bf16_tn(w, x, out, splits, status, after_small_kernel=after_small_kernel)
    return out
