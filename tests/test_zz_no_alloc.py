"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

It serves hosts that cannot allocate device memory when they call in (all memory already given to their own
pools, or a phase in which cudaMalloc's locks and device-wide synchronisation are not acceptable); the partial
results of the key slices then live in an array built into the library.  Checked here against the regular entry
points (which take caller-allocated partial buffers), on two calls in a row with different inputs, so that
whatever the first call left in the shared array must not leak into the second.
Collected last on purpose: if it fails, a run that stops at the first failure has run everything else.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def declare(L):
    P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    fn = L.vcb_attn_decode_no_alloc
    fn.argtypes = [P, P, I, P, LL, P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P, P]
    fn.restype = I
    return fn


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_entry_point_matches_the_allocating_one(dtype):
    from vllm_cpp_b200 import ops
    L = ops.lib()
    fn = declare(L)
    dev = torch.device("cuda:0")
    nh, nkv, hd, ps, S = 8, 2, 64, 16, 4
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    for call, ctxs in enumerate([[700, 33, 1500], [64, 2049]]):         # two calls in a row, other shapes the second time
        torch.manual_seed(call)
        B = len(ctxs)
        blocks = [-(-c // ps) for c in ctxs]
        num_pages = sum(blocks) + 2
        pages = torch.randn(num_pages, 2, nkv, ps, hd, device=dev).to(dtype)
        perm = torch.randperm(num_pages).tolist()
        bt = torch.full((B, max(blocks)), -1, dtype=torch.int32)
        for b, n in enumerate(blocks):
            bt[b, :n] = torch.tensor([perm.pop() for _ in range(n)])
        bt = bt.to(dev)
        q = torch.randn(B, nh * hd, device=dev).to(dtype)
        items = i32([[b, 0, 1, s, S, b] for b in range(B) for s in range(S)])
        q_start, q_len, ctx_len, dec_rows = i32(list(range(B))), i32([1] * B), i32(ctxs), i32(list(range(B)))
        # the existing entry points, partials in buffers allocated here
        want = torch.full_like(q, float("nan"))
        po = torch.empty(B * nh * S, hd, device=dev)
        pm = torch.empty(B * nh * S, 2, device=dev)
        ops.attn_paged(q, want, pages, bt, q_start, q_len, ctx_len, items, B * S, 8, po, pm, nh, nkv, hd, 0, status)
        ops.attn_merge(po, pm, dec_rows, want, B, nh, hd, S)
        # the new one, through the C symbol
        got = torch.full_like(q, float("nan"))
        before = torch.cuda.memory_allocated()
        rc = fn(q.data_ptr(), got.data_ptr(), ops._dt(q), pages.data_ptr(), pages.stride(0), bt.data_ptr(), None,
                bt.shape[1], q_start.data_ptr(), q_len.data_ptr(), ctx_len.data_ptr(), items.data_ptr(),
                dec_rows.data_ptr(), B, S, nh, nkv, hd, ps, num_pages, 0, 1.0 / math.sqrt(hd), status.data_ptr(),
                torch.cuda.current_stream().cuda_stream)
        assert rc == 0, L.vcb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert status.item() == 0 and not torch.isnan(got.float()).any()
        tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(got.float(), want.float(), **tol)
    # a call beyond the built-in scratch is refused with a clear error and launches nothing
    rc = fn(None, None, 1, None, 0, None, None, 1, None, None, None, None, None, 4096, 64, 64, 8, 128, 16, 1, 0, 0.1,
            None, None)
    assert rc != 0 and b"exceed" in L.vcb_last_error()
