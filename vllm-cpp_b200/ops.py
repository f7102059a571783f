"""Python face of the CUDA kernels in ``csrc/kernels`` (loaded through ctypes).

Each function takes torch CUDA tensors, checks shapes and dtypes, and launches
on torch's current stream.  There is no CPU fallback and no library fallback:
if the kernel library cannot be built or loaded, importing a kernel raises.
"""
from __future__ import annotations

import ctypes
import functools
import math
import struct
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
STATUS_BITS = {1: "token id outside the vocabulary", 2: "page id outside the pool",
               4: "a bounded wait inside a kernel gave up", 8: "position outside the rotary table",
               16: "shared memory did not start on the boundary a kernel's tiles need",
               32: "a work item names a partial-result row outside the buffer it was given"}
ITEM_INTS = 6

_lib = None


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {t.dtype} (float32 or bfloat16)")


def lib():
    """The loaded kernel library; built on first use."""
    global _lib
    if _lib is None:
        path = _build.build_kernels()
        try:
            L = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelError(f"cannot load the CUDA kernel library {path}: {e}") from e
        L.vcb_last_error.restype = ctypes.c_char_p
        _declare(L)
        _lib = L
    return _lib


def _declare(L):
    P, I, LL, F = c_void_p, c_int, c_longlong, c_float
    sigs = {
        "vcb_embed_gather": [P, I, P, P, I, I, I, P, P],
        "vcb_add_rmsnorm": [P, P, I, I, LL, P, I, F, P, I, P, I, I, P],
        "vcb_swiglu": [P, I, I, LL, P, I, I, I, P],
        "vcb_qknorm_rope_kvwrite": [P, I, I, LL, I, P, P, I, I, F, P, I, P, P, P, P, LL, I, I, I, I, I, I, I, I, I, P, P],
        "vcb_gemm_bf16_tn": [P, P, P, I, I, I, I, LL, LL, LL, I, LL, P, P],
        "vcb_gemm_bf16_tn_shape": [P, P, P, I, I, I, I, LL, LL, LL, I, LL, I, I, P, P],
        "vcb_gemm_effective_splits": [I, I],
        "vcb_gemm_set_pairs": [I],
        "vcb_gemm_bf16_swiglu": [P, P, P, I, I, I, LL, LL, LL, I, I, P, P],
        "vcb_gemm_bf16_qkv": [P, P, I, I, LL, LL, P, P, LL, I, I, P, P, P, I, P, P, I, I, F, I, I, P, P],
        "vcb_sgemm_tn": [P, P, P, I, I, I, LL, LL, LL, P],
        "vcb_gemm_bf16_plain": [P, P, P, I, I, I, I, LL, LL, LL, P],
        "vcb_attn_paged": [P, P, I, P, LL, P, P, I, P, P, P, P, I, I, P, P, I, I, I, I, I, I, F, P, P],
        "vcb_scatter_i32": [P, P, P, P, I, LL, P],
        "vcb_selftest_wait_timeout": [LL, P, P, P],
        "vcb_state_reset": [P, I, LL, LL, LL, I, I, P, P, P, I, ctypes.c_uint, P, P],
        "vcb_attn_mma": [P, P, P, LL, P, P, I, P, P, P, P, I, I, P, P, P, P, I, I, I, I, I, I, F, P, I, I, P],
        "vcb_attn_mma_supported": [I, I],
        "vcb_attn_mma_max_clusters": [I, I, I],
        "vcb_attn_mma_fused_supported": [I, I, I],
        "vcb_attn_mma_decode_fused": [P, I, LL, P, P, I, I, F, P, I, P, P, P, LL, P, P, I, P, P, P, P, I, P, P, P, P, I, I,
                                      I, I, I, I, F, P, I, P],
        "vcb_attn_tc": [P, P, P, LL, P, P, I, P, P, P, P, I, I, I, I, I, I, I, F, P, P, P],
        "vcb_attn_tc_supported": [I, I, I],
        "vcb_attn_stream": [P, P, P, LL, P, P, I, P, P, P, I, P, I, I, I, I, I, I, F, P, I, P],
        "vcb_attn_stream_supported": [I, I, I, I, I],
        "vcb_attn_merge": [P, P, P, P, I, I, I, I, I, P],
        "vcb_sample": [P, LL, I, I, P, P, P, P],
        "vcb_sample_split": [P, LL, I, I, P, P, P, P, I, P, P],
        "vcb_count_tokens": [P, P, P, I, I, I, P],
    }
    for name, args in sigs.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = c_int


_num_sms = None


def num_sms() -> int:
    """Streaming multiprocessors of the current device, asked once (148 on a B200); where there is no device
    -- the host-side tests of the planning arithmetic -- the B200's count."""
    global _num_sms
    if _num_sms is None:
        _num_sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count \
            if torch.cuda.is_available() else 148
    return _num_sms


launch_count = 0   # kernels of this library launched so far (every launcher starts exactly one)


def _call(name: str, *args):
    global launch_count
    L = lib()
    launch_count += 1
    fn = getattr(L, name)
    # ctypes takes arguments beyond the declared ones without a word and passes them as 32-bit integers: a pointer or
    # a stream handle would lose its upper half
    if fn.argtypes is None or len(fn.argtypes) != len(args):
        raise KernelError(f"{name}: {len(args)} arguments for a declaration of {0 if fn.argtypes is None else len(fn.argtypes)}")
    rc = fn(*args)
    if rc != 0:
        raise KernelError(L.vcb_last_error().decode() or f"{name} failed with code {rc}")


_held_stream: int | None = None   # the stream handle for the launches inside hold_stream(), asked for once


def _stream() -> int:
    return _held_stream if _held_stream is not None else torch.cuda.current_stream().cuda_stream


class hold_stream:
    """Within this context every launch goes to the stream that is current on entry, without asking torch for it
    again (three microseconds a launch, a quarter of a launch's host time).  Not to be held across a change of
    the current stream: a graph capture, for one, must start outside it."""

    def __enter__(self):
        global _held_stream
        self._outer = _held_stream
        _held_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _held_stream
        _held_stream = self._outer
        return False


def _p(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, contiguous=True):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def check_status(status: torch.Tensor, where: str = "step") -> None:
    """Reads the device status word (a synchronising copy) and raises on any set bit."""
    v = int(status.item())
    if v:
        status.zero_()
        what = [msg for bit, msg in STATUS_BITS.items() if v & bit]
        raise KernelError(f"{where}: a kernel reported: " + "; ".join(what))


# --------------------------------------------------------------------------


def embed_gather(table, ids, out, status):
    _need(table, "table"); _need(ids, "ids", torch.int32); _need(out, "out", torch.float32)
    T, H = out.shape
    V = table.shape[0]
    assert table.shape[1] == H and ids.numel() >= T
    _call("vcb_embed_gather", _p(table), _dt(table), _p(ids), _p(out), T, H, V, _p(status), _stream())


def add_rmsnorm(resid, delta, weight, eps, out, rows=None):
    """resid [T,H] f32 (updated in place with the deltas unless ``rows`` is given);
    delta None, [T,H] or [S,T,H]; out [n,H] in the activation dtype."""
    _need(resid, "resid", torch.float32); _need(weight, "weight"); _need(out, "out")
    T, H = resid.shape
    S, stride, dptr, ddt = 0, 0, None, F32
    if delta is not None:
        _need(delta, "delta")
        if delta.dim() == 2:
            delta = delta.unsqueeze(0)
        S = delta.shape[0]
        assert delta.shape[1] >= T and delta.shape[2] == H, (delta.shape, resid.shape)
        stride, dptr, ddt = delta.stride(0), delta.data_ptr(), _dt(delta)
    n = T if rows is None else rows.numel()
    if rows is not None:
        _need(rows, "rows", torch.int32)
    assert out.shape[0] >= n and out.shape[1] == H and weight.numel() == H
    _call("vcb_add_rmsnorm", _p(resid), dptr, ddt, S, stride, _p(weight), _dt(weight), float(eps), _p(out), _dt(out),
          _p(rows), n, H, _stream())


def _partials(t: torch.Tensor, name: str):
    """[T, W] or [S, T, W] (S partial sums to be added) -> (S, stride between partials)."""
    _need(t, name)
    if t.dim() == 2:
        return 1, 0
    return t.shape[0], t.stride(0)


def swiglu(gate_up, out):
    """out[t, i] = silu(gate_up[t, 2i]) * gate_up[t, 2i+1]: gate and up alternate along a row.
    gate_up [T, 2I] or [S, T, 2I] (32-bit partial sums); out [T, I]."""
    S, stride = _partials(gate_up, "gate_up"); _need(out, "out")
    T, I2 = gate_up.shape[-2:]
    assert out.shape == (T, I2 // 2)
    _call("vcb_swiglu", _p(gate_up), _dt(gate_up), S, stride, _p(out), _dt(out), T, I2 // 2, _stream())


def qknorm_rope_kvwrite(qkv, q_weight, k_weight, eps, cos_sin, positions, slot_map, q_out, pages, nh, nkv, hd,
                        status, has_kv=True, use_norm=True, rotary_dim=None, interleaved=False):
    """qkv [T, W] or [S, T, W] (32-bit partial sums); pages: one layer's [num_pages, 2, nkv, page_size, hd];
    slot_map int32 [T] = page * page_size + offset or -1.  ``rotary_dim`` (default: hd) lanes of a head are
    rotated, paired (i, i + rotary_dim/2) or, with ``interleaved``, (2i, 2i+1); cos_sin is [positions, rotary_dim]."""
    rotary_dim = hd if rotary_dim is None else int(rotary_dim)
    S, stride = _partials(qkv, "qkv")
    _need(cos_sin, "cos_sin", torch.float32); _need(positions, "positions", torch.int32); _need(q_out, "q_out")
    T = qkv.shape[-2]
    width = (nh + (2 * nkv if has_kv else 0)) * hd
    assert qkv.shape[-1] == width, (qkv.shape, width)
    if cos_sin.shape[1] != rotary_dim:
        raise KernelError(f"the table of angles has {cos_sin.shape[1]} columns, {rotary_dim} lanes are to be rotated")
    wdt = F32
    if use_norm:
        _need(q_weight, "q_norm weight"); wdt = _dt(q_weight)
        if has_kv:
            _need(k_weight, "k_norm weight", q_weight.dtype)
    page_stride = page_size = num_pages = 0
    if has_kv:
        _need(pages, "pages", q_out.dtype); _need(slot_map, "slot_map", torch.int32)
        num_pages, two, nkv_p, page_size, hd_p = pages.shape
        assert two == 2 and nkv_p == nkv and hd_p == hd
        page_stride = pages.stride(0)
    _call("vcb_qknorm_rope_kvwrite", _p(qkv), _dt(qkv), S, stride, _dt(q_out), _p(q_weight), _p(k_weight), wdt,
          int(use_norm), float(eps), _p(cos_sin), cos_sin.shape[0], _p(positions), _p(slot_map), _p(q_out), _p(pages),
          page_stride, max(page_size, 1), num_pages, nh, nkv, hd, T, int(has_kv), rotary_dim, int(bool(interleaved)),
          _p(status), _stream())


def gemm_bf16_plain(x, w, out):
    """out[T,N] = x[T,K] . w[N,K]^T for bfloat16 operands of any inner size (no TMA alignment needed)."""
    _need(x, "x", torch.bfloat16, contiguous=False); _need(w, "w", torch.bfloat16, contiguous=False); _need(out, "out")
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (T, N) and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _call("vcb_gemm_bf16_plain", _p(x), _p(w), _p(out), _dt(out), T, N, K, x.stride(0), w.stride(0), out.stride(0), _stream())


def gemm_tma_ok(x, w) -> bool:
    """Whether the tcgen05/TMA product can address these operands (16-byte rows and bases)."""
    K = x.shape[1]
    return (K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def gemm_effective_splits(K: int, splits: int) -> int:
    """The number of k-slices the kernel makes of ``splits`` asked for: whole 64-wide k-blocks, none empty
    (the arithmetic of vcb_gemm_effective_splits, here without a call into the library)."""
    total_kb = -(-K // 64)
    splits = max(1, min(int(splits), total_kb))
    per = -(-total_kb // splits)
    return -(-total_kb // per)


GEMM_SHAPES = ("n16", "n32", "n64", "n128", "n256", "m256_n192", "m256_n256", "pair", "m256_n160")   # unit shapes of the kernel, by index


def gemm_set_pairs(mode: int) -> None:
    """Which products of more than 128 tokens without k-slices run on pairs of blocks (``cta_group::2``: one MMA
    spans 256 features on two SMs, each block loads its half of the token tile): 0 none, 1 those whose units fill
    the pairs' rounds no worse than the single-block kernel's fill the SMs' (the default, which
    ``VLLM_CPP_B200_GEMM_PAIRS`` overrides), 2 all that can.  Process-wide."""
    lib().vcb_gemm_set_pairs(int(mode))


def gemm_bf16_tn(w, x, out, splits, status, shape=-1, after_small_kernel=False):
    """out[z, t, m] = sum over k-slice z of w[m, k] x[t, k]   (tcgen05 + TMA; w [M,K], x [T,K] bfloat16).
    out: [T, M] (bfloat16 or float32, one slice) or [S, T, M] float32 with S = gemm_effective_splits(K, splits).
    ``shape`` forces one of GEMM_SHAPES (an index) whatever the sizes; -1 lets the kernel choose.
    ``after_small_kernel``: the kernel before this one in the stream is a short one (a norm, the SiLU-gate): a decode
    product then asks further weight tiles into L2 while it waits for it (VLLM_CPP_B200_GEMM_PREFETCH)."""
    _need(w, "w", torch.bfloat16, contiguous=False); _need(x, "x", torch.bfloat16, contiguous=False); _need(out, "out")
    M, K = w.shape
    T = x.shape[0]
    assert x.shape[1] == K and w.stride(1) == 1 and x.stride(1) == 1
    S = gemm_effective_splits(K, splits)
    if out.dim() == 2:
        assert S == 1 and out.shape == (T, M)
        ldc, sstride = out.stride(0), 0
    else:
        assert out.shape == (S, T, M) and out.dtype == torch.float32
        ldc, sstride = out.stride(1), out.stride(0)
    _call("vcb_gemm_bf16_tn_shape", _p(w), _p(x), _p(out), _dt(out), M, T, K, w.stride(0), x.stride(0), ldc, S, sstride,
          int(shape), int(bool(after_small_kernel)), _p(status), _stream())


def gemm_bf16_swiglu(w_gate_up, x, out, status, shape=-1, after_small_kernel=False):
    """out[t, i] = silu(gate_i . x_t) * (up_i . x_t) with gate_i in row 2i and up_i in row 2i+1 of w_gate_up: the
    product and the SiLU-gate in one kernel (adjacent accumulator lanes are paired in the epilogue).
    ``shape`` and ``after_small_kernel`` as in gemm_bf16_tn."""
    _need(w_gate_up, "w_gate_up", torch.bfloat16); _need(x, "x", torch.bfloat16, contiguous=False)
    _need(out, "out", torch.bfloat16)
    I2, K = w_gate_up.shape
    T = x.shape[0]
    assert I2 % 2 == 0 and x.shape[1] == K and x.stride(1) == 1 and out.shape == (T, I2 // 2)
    _call("vcb_gemm_bf16_swiglu", _p(w_gate_up), _p(x), _p(out), I2 // 2, T, K, w_gate_up.stride(0), x.stride(0),
          out.stride(0), int(shape), int(bool(after_small_kernel)), _p(status), _stream())


def gemm_qkv_rope(w_qkv, x, q_out, pages, slot_map, positions, cos_sin, q_weight, k_weight, eps, nh, nkv, status,
                  use_norm=True):
    """The stacked q, k, v projection of a prompt portion with what :func:`qknorm_rope_kvwrite` does in its epilogue
    (head_dim 128, the whole head rotated in half-split pairs): per-head norm of queries and keys, rotation, queries to
    ``q_out`` [T, nh * 128], keys and values to the tokens' slots of ``pages`` (None: a layer that stores none; then
    ``w_qkv`` holds the query rows only).  No k-slices, so for more than 128 tokens; 32-bit from the product's sums on."""
    _need(w_qkv, "w_qkv", torch.bfloat16); _need(x, "x", torch.bfloat16, contiguous=False); _need(q_out, "q_out", torch.bfloat16)
    _need(cos_sin, "cos_sin", torch.float32); _need(positions, "positions", torch.int32)
    M, K = w_qkv.shape
    T = x.shape[0]
    assert x.shape[1] == K and x.stride(1) == 1 and q_out.shape == (T, nh * 128) and cos_sin.shape[1] == 128
    page_stride = page_size = num_pages = 0
    if pages is not None:
        _need(pages, "pages", torch.bfloat16); _need(slot_map, "slot_map", torch.int32)
        num_pages, two, nkv_p, page_size, hd_p = pages.shape
        assert two == 2 and nkv_p == nkv and hd_p == 128 and M == (nh + 2 * nkv) * 128
        page_stride = pages.stride(0)
    else:
        assert M == nh * 128
    wdt = F32
    if use_norm:
        _need(q_weight, "q_norm weight")
        wdt = _dt(q_weight)
        if pages is not None:
            _need(k_weight, "k_norm weight", q_weight.dtype)
    _call("vcb_gemm_bf16_qkv", _p(w_qkv), _p(x), T, K, w_qkv.stride(0), x.stride(0), _p(q_out), _p(pages), page_stride,
          page_size, num_pages, _p(slot_map), _p(positions), _p(cos_sin), cos_sin.shape[0], _p(q_weight), _p(k_weight), wdt,
          int(use_norm), float(eps), nh, nkv, _p(status), _stream())


def sgemm_tn(a, b, out):
    """out[M,N] = a[M,K] . b[N,K]^T in true 32-bit."""
    _need(a, "a", torch.float32, contiguous=False); _need(b, "b", torch.float32, contiguous=False)
    _need(out, "out", torch.float32, contiguous=False)
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and b.stride(1) == 1 and out.stride(1) == 1
    _call("vcb_sgemm_tn", _p(a), _p(b), _p(out), M, N, K, a.stride(0), b.stride(0), out.stride(0), _stream())


def attn_paged(q, out, pages, block_table, q_start, q_len, ctx_len, items, n_items, rows_max, part_o, part_ml,
               nh, nkv, hd, window, status, table_row=None):
    """block_table int32 [rows, max_blocks]; entry e reads row ``table_row[e]`` (row e when table_row is None)."""
    _need(q, "q"); _need(out, "out", q.dtype); _need(pages, "pages", q.dtype)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_len", q_len), ("ctx_len", ctx_len),
                    ("items", items)):
        _need(t, name, torch.int32)
    num_pages, two, nkv_p, page_size, hd_p = pages.shape
    assert two == 2 and nkv_p == nkv and hd_p == hd
    _call("vcb_attn_paged", _p(q), _p(out), _dt(q), _p(pages), pages.stride(0), _p(block_table), _p(table_row), block_table.shape[1],
          _p(q_start), _p(q_len), _p(ctx_len), _p(items), n_items, rows_max, _p(part_o), _p(part_ml), nh, nkv, hd,
          page_size, num_pages, int(window or 0), 1.0 / math.sqrt(hd), _p(status), _stream())


def attn_merge(part_o, part_ml, dec_rows, out, n_dec, nh, hd, nslices):
    _need(part_o, "part_o", torch.float32); _need(part_ml, "part_ml", torch.float32)
    _need(dec_rows, "dec_rows", torch.int32); _need(out, "out")
    _call("vcb_attn_merge", _p(part_o), _p(part_ml), _p(dec_rows), _p(out), _dt(out), n_dec, nh, hd, nslices, _stream())


def sample(logits, params, counts, out, no_nucleus=False):
    """logits [R,V] f32; params [R,8] int32 records (see sampling.cu); counts [slots,V] int32 or None.
    ``no_nucleus``: no row has top_p < 1, so the vocabulary can be dealt to several blocks per row."""
    _need(logits, "logits", torch.float32, contiguous=False); _need(params, "params", torch.int32)
    _need(out, "out", torch.int32)
    R, V = logits.shape
    assert logits.stride(1) == 1 and params.shape == (R, 8) and out.numel() >= R
    if counts is not None:
        _need(counts, "counts", torch.int32)
        assert counts.shape[1] == V
    nb = max(1, min(64, 2 * num_sms() // max(R, 1), V // 2048))
    if no_nucleus and nb > 1:
        global launch_count
        from . import workspace
        part_v = workspace.empty((R * nb,), torch.float32, logits.device)
        part_i = workspace.empty((R * nb,), torch.int32, logits.device)
        _call("vcb_sample_split", _p(logits), logits.stride(0), R, V, _p(params), _p(counts), _p(part_v), _p(part_i),
              nb, _p(out), _stream())
        launch_count += 1   # two kernels
        return
    _call("vcb_sample", _p(logits), logits.stride(0), R, V, _p(params), _p(counts), _p(out), _stream())


def count_tokens(ids, slots, counts, n, slot_bias=0):
    """counts[slots[t] - slot_bias, ids[t]] += 1 for tokens whose slot entry less the bias is >= 0."""
    _need(ids, "ids", torch.int32); _need(slots, "slots", torch.int32); _need(counts, "counts", torch.int32)
    _call("vcb_count_tokens", _p(ids), _p(slots), _p(counts), n, counts.shape[1], slot_bias, _stream())


def scatter_i32(dst, idx, val, count, capacity):
    """dst.flat[idx[i]] = val[i] for i < min(count[0], capacity); count is a device int32."""
    _need(dst, "dst", torch.int32); _need(idx, "idx", torch.int32); _need(val, "val", torch.int32)
    _need(count, "count", torch.int32)
    _call("vcb_scatter_i32", _p(dst), _p(idx), _p(val), _p(count), capacity, dst.numel(), _stream())


def state_reset(state, slots, q_len, ctx_len, n_entries, value, status):
    """state [caches, slots, ...]: the rows of the requests whose entries start at position 0 (ctx_len == q_len > 0)
    are filled with ``value``; all on the device (a captured step includes it)."""
    _need(state, "state"); _need(slots, "slots", torch.int32); _need(q_len, "q_len", torch.int32); _need(ctx_len, "ctx_len", torch.int32)
    if state.dim() < 2:
        raise KernelError("a state tensor is [caches, slots, ...]")
    n_caches, num_slots = state.shape[0], state.shape[1]
    row = state[0, 0].numel()
    if state.dtype == torch.float32:
        bits = struct.unpack("<I", struct.pack("<f", float(value)))[0]
    elif state.dtype == torch.bfloat16:
        bits = struct.unpack("<I", struct.pack("<f", float(torch.tensor(float(value)).to(torch.bfloat16).float())))[0] >> 16
    elif state.dtype == torch.int32:
        bits = int(value) & 0xFFFFFFFF
    else:
        raise KernelError(f"state of type {state.dtype} (float32, bfloat16 or int32)")
    _call("vcb_state_reset", _p(state), state.element_size(), state.stride(0), state.stride(1), row, n_caches, num_slots,
          _p(slots), _p(q_len), _p(ctx_len), n_entries, bits, _p(status), _stream())


def selftest_wait_timeout(limit_clocks: int, status: torch.Tensor) -> list[int]:
    """Lets the kernels' bounded mbarrier wait run out on a barrier nothing arrives at (see csrc/kernels/selftest.cu)
    and returns [the wait's answer, the abort flag seen by another warp, a later wait's answer, whether that one
    returned at once]; the status word gets the wait-timeout bit."""
    _need(status, "status", torch.int32)
    out = torch.full((4,), -1, dtype=torch.int32, device=status.device)
    _call("vcb_selftest_wait_timeout", int(limit_clocks), _p(status), _p(out), _stream())
    return out.tolist()


def attn_mma_supported(dtype: torch.dtype, hd: int) -> bool:
    """Whether the tensor-core attention kernel takes this element type and head size."""
    return bool(lib().vcb_attn_mma_supported(BF16 if dtype == torch.bfloat16 else F32, hd))


def attn_mma_fused_supported(dtype: torch.dtype, hd: int, page_size: int) -> bool:
    """Whether decoded tokens can be attended straight from the stacked q, k, v projection (attn_mma_decode_fused)."""
    return bool(lib().vcb_attn_mma_fused_supported(BF16 if dtype == torch.bfloat16 else F32, hd, page_size))


def attn_mma_decode_fused(qkv, q_weight, k_weight, eps, cos_sin, slot_map, out, pages, block_table, q_start,
                          q_len, ctx_len, items, n_items, part_o, part_ml, slice_counters, dec_rows, nh, nkv, hd, window,
                          status, table_row=None, use_norm=True, cluster=0):
    """Attention of single decoded tokens straight from the stacked projection ``qkv`` [S, T, (nh + 2 nkv) hd]
    (32-bit k-slice partial sums): each block norms and rotates its own query heads, and the blocks that read the
    token's own position store its key and value in the cache first -- what qknorm_rope_kvwrite and attn_mma do
    in two kernels.  Items: one token each, as for :func:`attn_mma` with rows_max 16; a token's position is its
    entry's context length less one."""
    _need(qkv, "qkv", torch.float32); _need(out, "out", torch.bfloat16); _need(pages, "pages", torch.bfloat16)
    _need(cos_sin, "cos_sin", torch.float32); _need(slot_map, "slot_map", torch.int32)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_len", q_len), ("ctx_len", ctx_len), ("items", items)):
        _need(t, name, torch.int32)
    assert qkv.dim() == 3 and qkv.shape[2] == (nh + 2 * nkv) * hd and cos_sin.shape[1] == hd
    num_pages, two, nkv_p, page_size, hd_p = pages.shape
    assert two == 2 and nkv_p == nkv and hd_p == hd
    wdt = F32
    if use_norm:
        _need(q_weight, "q_norm weight"); _need(k_weight, "k_norm weight", q_weight.dtype)
        wdt = _dt(q_weight)
    _call("vcb_attn_mma_decode_fused", _p(qkv), qkv.shape[0], qkv.stride(0), _p(q_weight), _p(k_weight), wdt, int(use_norm),
          float(eps), _p(cos_sin), cos_sin.shape[0], _p(slot_map), _p(out), _p(pages), pages.stride(0),
          _p(block_table), _p(table_row), block_table.shape[1], _p(q_start), _p(q_len), _p(ctx_len), _p(items), n_items,
          _p(part_o), _p(part_ml), _p(slice_counters), _p(dec_rows), nh, nkv, hd, page_size, num_pages, int(window or 0),
          1.0 / math.sqrt(hd), _p(status), int(cluster), _stream())


@functools.lru_cache(maxsize=None)
def attn_mma_max_clusters(hd: int, cluster: int, deep: bool) -> int:
    """How many clusters of ``cluster`` blocks of the decode attention kernel run at once on this device (``deep``: the
    variant with the ring of six stages, which has an SM to itself).  -1 when the driver does not say."""
    return int(lib().vcb_attn_mma_max_clusters(hd, cluster, int(deep)))


def attn_tc_supported(dtype: torch.dtype, hd: int, page_size: int) -> bool:
    """Whether the tcgen05 attention kernel for prompt portions takes this element type, head size and page size."""
    return bool(lib().vcb_attn_tc_supported(BF16 if dtype == torch.bfloat16 else F32, hd, page_size))


def attn_tc(q, out, pages, block_table, q_start, q_len, ctx_len, items, n_items, nh, nkv, hd, window, status,
            table_row=None, work=None):
    """Attention of prompt portions on tcgen05 tensor cores (bfloat16, head_dim 64 or 128, pages of 8 to 64
    tokens).  Items as for :func:`attn_paged` with one key slice and at most 128 rows each.  ``work``: two int32
    zeros, zero again when the kernel is through (the queue its blocks take their units from); launches that share
    them must follow one another on a stream.  Made on the spot when not given."""
    if work is None:
        work = torch.zeros(2, dtype=torch.int32, device=q.device)
    _need(work, "work", torch.int32)
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(pages, "pages", torch.bfloat16)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_len", q_len), ("ctx_len", ctx_len),
                    ("items", items)):
        _need(t, name, torch.int32)
    num_pages, two, nkv_p, page_size, hd_p = pages.shape
    assert two == 2 and nkv_p == nkv and hd_p == hd
    _call("vcb_attn_tc", _p(q), _p(out), _p(pages), pages.stride(0), _p(block_table), _p(table_row),
          block_table.shape[1], _p(q_start), _p(q_len), _p(ctx_len), _p(items), n_items, nh, nkv, hd, page_size,
          num_pages, int(window or 0), 1.0 / math.sqrt(hd), _p(status), _p(work), _stream())


def attn_mma(q, out, pages, block_table, q_start, q_len, ctx_len, items, n_items, rows_max, part_o, part_ml,
             nh, nkv, hd, window, status, table_row=None, allow_tma=True, slice_counters=None, dec_rows=None,
             cluster=0):
    """Tensor-core variant of :func:`attn_paged` (bfloat16, head_dim 64 or 128; rows_max 16 or 128).
    With ``slice_counters`` (int32 zeros, one per decoded token and KV head group, left at zero again) and
    ``dec_rows``, the block that finishes a token's last key slice merges the slices itself; with ``cluster`` = the
    number of slices per token (2 to 8) as well, the slices' blocks run as a cluster and merge through shared memory."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(pages, "pages", torch.bfloat16)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_len", q_len), ("ctx_len", ctx_len),
                    ("items", items)):
        _need(t, name, torch.int32)
    num_pages, two, nkv_p, page_size, hd_p = pages.shape
    assert two == 2 and nkv_p == nkv and hd_p == hd
    _call("vcb_attn_mma", _p(q), _p(out), _p(pages), pages.stride(0), _p(block_table), _p(table_row),
          block_table.shape[1], _p(q_start), _p(q_len), _p(ctx_len), _p(items), n_items, rows_max, _p(part_o),
          _p(part_ml), _p(slice_counters), _p(dec_rows), nh, nkv, hd, page_size, num_pages, int(window or 0),
          1.0 / math.sqrt(hd), _p(status), int(allow_tma), int(cluster), _stream())


def attn_stream_supported(dtype: torch.dtype, hd: int, page_size: int, nh: int, nkv: int) -> bool:
    """Whether :func:`attn_stream` takes these sizes (bfloat16, head_dim 64 or 128, pages of 8 to 64 tokens, at
    most 16 query heads a KV head)."""
    return bool(lib().vcb_attn_stream_supported(BF16 if dtype == torch.bfloat16 else F32, hd, page_size, nh, nkv))


def attn_stream(q, out, pages, block_table, q_len, ctx_len, items, n_dec, dec_rows, nh, nkv, hd, window, status,
                table_row=None, blocks=0):
    """Single decoded tokens, many of them: persistent blocks walk the (token, KV head) pairs, all keys of a pair in
    one block, the loading warp running ahead from pair to pair.  ``items`` [n_dec, 6] as for :func:`attn_mma` with
    one slice; ``dec_rows`` [n_dec] the tokens' rows of ``q`` and ``out``; entries with q_len 0 are skipped.
    ``blocks``: how many blocks to run on (0: two an SM, or one where the head group is large)."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(pages, "pages", torch.bfloat16)
    for name, t in (("block_table", block_table), ("q_len", q_len), ("ctx_len", ctx_len), ("items", items),
                    ("dec_rows", dec_rows)):
        _need(t, name, torch.int32)
    num_pages, two, nkv_p, page_size, hd_p = pages.shape
    assert two == 2 and nkv_p == nkv and hd_p == hd
    _call("vcb_attn_stream", _p(q), _p(out), _p(pages), pages.stride(0), _p(block_table), _p(table_row),
          block_table.shape[1], _p(q_len), _p(ctx_len), _p(items), n_dec, _p(dec_rows), nh, nkv, hd, page_size,
          num_pages, int(window or 0), 1.0 / math.sqrt(hd), _p(status), int(blocks), _stream())


# --------------------------------------------------------------------------  a look at a step from inside
_timeline = None
_TL_ROLE_EVERY, _TL_ROLE_BLOCKS, _TL_ROLES, _TL_ROLE_MARKS = 37, 8, 3, 2048     # as in kernels/common.cuh
_TL_ROLE_WORDS = _TL_ROLE_BLOCKS * _TL_ROLES * _TL_ROLE_MARKS * 2
TIMELINE_KERNELS = {1: "gemm", 2: "attn_decode", 3: "add_rmsnorm", 4: "qknorm_rope", 5: "swiglu", 6: "attn_tc", 7: "other"}


def timeline_begin(capacity: int = 1 << 18) -> None:
    """Starts recording the kernels' timeline marks (a library built with VLLM_CPP_B200_TIMELINE=1 only): thread 0 of
    every block notes when the block starts, when its wait for the kernel before it ends, and when it ends."""
    global _timeline
    L = lib()
    if not hasattr(L, "vcb_timeline_set_gemm"):
        raise KernelError("this kernel library was built without timeline marks (build with VLLM_CPP_B200_TIMELINE=1)")
    _timeline = torch.zeros(2 + 4 * capacity + _TL_ROLE_WORDS, dtype=torch.int64, device="cuda")
    _timeline[1] = capacity
    torch.cuda.synchronize()
    for unit in ("gemm", "attn_mma", "attn_tc", "attn_stream", "elementwise"):
        fn = getattr(L, f"vcb_timeline_set_{unit}")
        fn.argtypes, fn.restype = [c_void_p], c_int
        if fn(_timeline.data_ptr()) != 0:
            raise KernelError("could not hand the timeline buffer to the kernels")


def timeline_end():
    """Stops recording; returns the records as a list of dicts (t_ns, clock, kernel, phase, sm, tile, block, grid), by
    time.  The marks of the roles inside a block (phases from 10 on; they have a ``role``, a tile number and the SM's
    clock, but no time: t_ns 0) come first."""
    global _timeline
    L = lib()
    torch.cuda.synchronize()
    for unit in ("gemm", "attn_mma", "attn_tc", "attn_stream", "elementwise"):
        getattr(L, f"vcb_timeline_set_{unit}")(None)
    buf = _timeline.cpu().numpy()
    _timeline = None
    n = int(min(buf[0], buf[1]))
    rec = buf[2:2 + 4 * n].reshape(n, 4)
    out = [dict(t_ns=int(r[0]), clock=int(r[1]), kernel=TIMELINE_KERNELS.get(int(r[2]) >> 32, "?"), phase=(int(r[2]) >> 24) & 0xFF,
                sm=int(r[2]) & 0xFF, tile=0, block=int(r[3]) & 0xFFFFFFFF, grid=int(r[3]) >> 32) for r in rec]
    # the logs of the roles inside a block: (clock, tag) pairs per (recording block, role)
    logs = buf[2 + 4 * int(buf[1]):].reshape(_TL_ROLE_BLOCKS, _TL_ROLES, _TL_ROLE_MARKS, 2)
    for b in range(_TL_ROLE_BLOCKS):
        for role in range(_TL_ROLES):
            for clock, tag in logs[b, role]:
                tag = int(tag) & 0xFFFFFFFFFFFFFFFF
                if tag >> 63:
                    out.append(dict(t_ns=0, clock=int(clock), kernel=TIMELINE_KERNELS.get((tag >> 48) & 0xFF, "?"), phase=(tag >> 32) & 0xFFFF,
                                    sm=-1, tile=tag & 0xFFFFFFFF, block=b * _TL_ROLE_EVERY, grid=0, role=role))
    out.sort(key=lambda d: d["t_ns"])
    return out
