"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

It serves hosts that cannot allocate device memory when they call in (all memory already given to their own
pools, or a phase in which cudaMalloc's locks and device-wide synchronisation are not acceptable); the partial
results of the key slices then live in an array built into the library.  Checked here against the regular entry
points (which take caller-allocated partial buffers) and against a plain 64-bit attention, on two calls in a
row with different inputs, so that whatever the first call left in the shared array must not leak into the
second: the second call has an entry without tokens (its row must come out as zeros, not as the first call's
result), a row that is to be skipped (it must stay untouched) and a window.
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


def plain_attention(q, k, v, window):
    """One query at the last position of k, v [n, nkv, hd]; q [nh, hd]; 64-bit (src/model.cpp:1000-1052)."""
    nh, hd = q.shape
    n, nkv, _ = k.shape
    lo = max(0, n - window) if window else 0
    out = torch.empty(nh, hd, dtype=torch.float64)
    for h in range(nh):
        s = (k[lo:, h // (nh // nkv)] @ q[h]) / math.sqrt(hd)
        out[h] = torch.softmax(s, 0) @ v[lo:, h // (nh // nkv)]
    return out


def make_case(seed, ctxs, nh, nkv, hd, ps, S, dtype, dev):
    """Keys and values of each request scattered over shuffled pages (NaN everywhere else), one query each."""
    g = torch.Generator().manual_seed(seed)
    B = len(ctxs)
    blocks = [-(-c // ps) for c in ctxs]
    num_pages = sum(blocks) + 2
    pages = torch.full((num_pages, 2, nkv, ps, hd), float("nan"), dtype=dtype)
    perm = torch.randperm(num_pages, generator=g).tolist()
    bt = torch.full((B, max(blocks + [1])), -1, dtype=torch.int32)
    kv = []
    for b, c in enumerate(ctxs):
        k = torch.randn(c, nkv, hd, generator=g).to(dtype)
        v = torch.randn(c, nkv, hd, generator=g).to(dtype)
        kv.append((k.double(), v.double()))
        tab = [perm.pop() for _ in range(blocks[b])]
        bt[b, :blocks[b]] = torch.tensor(tab, dtype=torch.int32)
        for p0 in range(0, c, ps):
            n = min(ps, c - p0)
            pages[tab[p0 // ps], 0, :, :n] = k[p0:p0 + n].transpose(0, 1)
            pages[tab[p0 // ps], 1, :, :n] = v[p0:p0 + n].transpose(0, 1)
    q = torch.randn(B, nh * hd, generator=g).to(dtype)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    items = i32([[b, 0, 1, s, S, b] for b in range(B) for s in range(S)])
    return dict(pages=pages.to(dev), bt=bt.to(dev), q=q.to(dev), kv=kv, items=items, q_start=i32(list(range(B))),
                q_len=i32([1 if c else 0 for c in ctxs]), ctx_len=i32(ctxs), num_pages=num_pages)


def call(fn, L, c, got, dec_rows, B, S, nh, nkv, hd, ps, window, status, items=None):
    from vllm_cpp_b200 import ops
    items = c["items"] if items is None else items
    rc = fn(c["q"].data_ptr(), got.data_ptr(), ops._dt(c["q"]), c["pages"].data_ptr(), c["pages"].stride(0),
            c["bt"].data_ptr(), None, c["bt"].shape[1], c["q_start"].data_ptr(), c["q_len"].data_ptr(),
            c["ctx_len"].data_ptr(), items.data_ptr(), dec_rows.data_ptr(), B, S, nh, nkv, hd, ps, c["num_pages"],
            window, 1.0 / math.sqrt(hd), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.vcb_last_error().decode()
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_entry_point_matches_the_allocating_one(dtype):
    from vllm_cpp_b200 import ops
    L = ops.lib()
    fn = declare(L)
    dev = torch.device("cuda:0")
    nh, nkv, hd, ps, S = 8, 2, 64, 16, 4
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    # two calls in a row; the second time other shapes, a window, an entry without tokens (index 1) and a row
    # that is to be skipped (index 3)
    for n_call, (ctxs, window, rows) in enumerate([([700, 33, 1500, 90], 0, [0, 1, 2, 3]),
                                                   ([64, 0, 2049, 300], 200, [0, 1, 2, -1])]):
        B = len(ctxs)
        c = make_case(n_call, ctxs, nh, nkv, hd, ps, S, dtype, dev)
        dec_rows = i32(rows)
        # the existing entry points, partials in buffers allocated here
        want = torch.full_like(c["q"], 7.0)
        po = torch.empty(B * nh * S, hd, device=dev)
        pm = torch.empty(B * nh * S, 2, device=dev)
        ops.attn_paged(c["q"], want, c["pages"], c["bt"], c["q_start"], c["q_len"], c["ctx_len"], c["items"], B * S,
                       8, po, pm, nh, nkv, hd, window, status)
        ops.attn_merge(po, pm, dec_rows, want, B, nh, hd, S)
        # the new one, through the C symbol: warmed up once, then watched for device memory it might take
        got = torch.full_like(c["q"], 7.0)
        call(fn, L, c, got, dec_rows, B, S, nh, nkv, hd, ps, window, status)
        got.fill_(7.0)
        free_before = torch.cuda.mem_get_info()[0]        # the driver's count: sees cudaMalloc, not just torch's pool
        torch_before = torch.cuda.memory_allocated()
        call(fn, L, c, got, dec_rows, B, S, nh, nkv, hd, ps, window, status)
        assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == torch_before
        assert status.item() == 0 and not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want.float(), **tol)
        # ... and against plain 64-bit attention
        for b, (ctx, row) in enumerate(zip(ctxs, rows)):
            if row < 0:
                assert (got[b] == 7.0).all(), "a row that was to be skipped was written"
            elif ctx == 0:
                assert (got[row] == 0).all(), "an entry without tokens must give zeros, whatever the array held"
            else:
                k, v = c["kv"][b]
                ref = plain_attention(c["q"][b].double().cpu().view(nh, hd), k, v, window)
                torch.testing.assert_close(got[row].double().cpu().view(nh, hd), ref, **tol)
    # a call beyond the built-in scratch is refused with a clear error and launches nothing
    rc = fn(None, None, 1, None, 0, None, None, 1, None, None, None, None, None, 4096, 64, 64, 8, 128, 16, 1, 0, 0.1,
            status.data_ptr(), None)
    assert rc != 0 and b"exceed" in L.vcb_last_error()


def test_no_alloc_entry_point_refuses_items_outside_its_array():
    """Items that name a token index, a slice or a slice count other than the call's would address the built-in
    array outside the part that the call laid out.  The kernel leaves such an item out, reports it in the status
    word and writes nothing for it; the other tokens of the call are still right."""
    from vllm_cpp_b200 import ops
    L = ops.lib()
    fn = declare(L)
    dev = torch.device("cuda:0")
    nh, nkv, hd, ps, S, dtype = 8, 2, 64, 16, 4, torch.float32
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ctxs = [130, 500, 77]
    B = len(ctxs)
    c = make_case(5, ctxs, nh, nkv, hd, ps, S, dtype, dev)
    dec_rows = torch.tensor([0, 1, -1], dtype=torch.int32, device=dev)    # the token whose items are bad is skipped by the merge
    good = torch.full_like(c["q"], 7.0)
    call(fn, L, c, good, dec_rows, B, S, nh, nkv, hd, ps, 0, status)
    assert status.item() == 0
    for bad in ([2, 0, 1, 0, S, B + 1000000],        # token index far beyond n_dec
                [2, 0, 1, S + 3, S, 2],              # slice beyond the slice count
                [2, 0, 1, 0, S + 60, 2]):            # another slice count than the call's
        items = c["items"].clone()
        items[2 * S] = torch.tensor(bad, dtype=torch.int32, device=dev)
        got = torch.full_like(c["q"], 7.0)
        call(fn, L, c, got, dec_rows, B, S, nh, nkv, hd, ps, 0, status)
        call(fn, L, c, got, dec_rows, B, S, nh, nkv, hd, ps, 0, status, items=items)
        assert status.item() == 32, "the bad item was not reported"
        status.zero_()
        assert torch.equal(got[:2], good[:2]) and (got[2] == 7.0).all()
    # the array is intact for the next caller
    got = torch.full_like(c["q"], 7.0)
    call(fn, L, c, got, dec_rows, B, S, nh, nkv, hd, ps, 0, status)
    assert status.item() == 0 and torch.equal(got, good)
