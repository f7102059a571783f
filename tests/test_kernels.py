"""Each CUDA kernel alone against a plain PyTorch 32/64-bit restatement of the same op, at
sizes other than the engine's tiny models (odd widths, head sizes in steps of 16, MQA/MHA/GQA)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def dev():
    return torch.device("cuda:0")


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("table_dtype", DTYPES)
def test_embed_gather(table_dtype):
    from vllm_cpp_b200 import ops
    V, H, T = 301, 72, 19
    table = torch.randn(V, H, device=dev()).to(table_dtype)
    ids = torch.randint(0, V, (T,), device=dev(), dtype=torch.int32)
    out = torch.empty(T, H, device=dev())
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.embed_gather(table, ids, out, status)
    assert torch.equal(out, table.float()[ids.long()])
    assert status.item() == 0
    ids[3] = V  # outside the vocabulary: reported, row zeroed, nothing read out of bounds
    ops.embed_gather(table, ids, out, status)
    assert status.item() == 1 and out[3].abs().max().item() == 0
    status.zero_()


@pytest.mark.parametrize("H", [72, 1000, 4096, 14000])
@pytest.mark.parametrize("S", [0, 1, 3])
@pytest.mark.parametrize("out_dtype,w_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                               (torch.bfloat16, torch.float32)])
def test_add_rmsnorm(H, S, out_dtype, w_dtype):
    from vllm_cpp_b200 import ops
    T, eps = 7, 1e-5
    resid = torch.randn(T, H, device=dev())
    delta = torch.randn(S, T, H, device=dev()) if S else None
    w = (1 + 0.1 * torch.randn(H, device=dev())).to(w_dtype)
    out = torch.empty(T, H, device=dev(), dtype=out_dtype)
    x = resid.double() + (delta.double().sum(0) if S else 0)
    want = w.double() * x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    r = resid.clone()
    ops.add_rmsnorm(r, delta, w, eps, out)
    torch.testing.assert_close(out.double(), want, **tol(out_dtype))
    torch.testing.assert_close(r.double(), x, rtol=1e-6, atol=1e-6)
    # gathered rows: stream untouched
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=dev())
    r2 = resid.clone()
    out2 = torch.empty(3, H, device=dev(), dtype=out_dtype)
    ops.add_rmsnorm(r2, delta, w, eps, out2, rows)
    torch.testing.assert_close(out2.double(), want[rows.long()], **tol(out_dtype))
    assert torch.equal(r2, resid)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    from vllm_cpp_b200 import ops
    T, I = 5, 200
    gu = (3 * torch.randn(T, 2 * I, device=dev())).to(dtype)
    out = torch.empty(T, I, device=dev(), dtype=dtype)
    ops.swiglu(gu, out)
    g, u = gu[:, 0::2].double(), gu[:, 1::2].double()     # gate and up alternate along a row
    torch.testing.assert_close(out.double(), g / (1 + torch.exp(-g)) * u, **tol(dtype))
    # the 16-byte path (I a multiple of 8), far-out gate values included
    gu = (30 * torch.randn(T, 2 * I, device=dev())).to(dtype)
    ops.swiglu(gu, out)
    g, u = gu[:, 0::2].double(), gu[:, 1::2].double()
    torch.testing.assert_close(out.double(), g / (1 + torch.exp(-g)) * u, **tol(dtype))
    gu = gu[:, :2 * 37].contiguous()
    out = torch.empty(T, 37, device=dev(), dtype=dtype)
    ops.swiglu(gu, out)
    g, u = gu[:, 0::2].double(), gu[:, 1::2].double()
    torch.testing.assert_close(out.double(), g / (1 + torch.exp(-g)) * u, **tol(dtype))


@pytest.mark.parametrize("T,I,S", [(8, 12288, 3), (64, 200, 1), (257, 1004, 5), (3, 36, 9)])
def test_swiglu_of_k_slice_partial_sums(T, I, S):
    """32-bit partial sums of a stacked gate/up product in, bfloat16 out (what follows a sliced product in the
    bfloat16 engine): the slices are added in order, then the SiLU-gate."""
    from vllm_cpp_b200 import ops
    torch.manual_seed(T + I + S)
    gu = 2 * torch.randn(S, T, 2 * I, device=dev())
    out = torch.empty(T, I, device=dev(), dtype=torch.bfloat16)
    ops.swiglu(gu, out)
    x = gu.double().sum(0)
    g, u = x[:, 0::2], x[:, 1::2]
    torch.testing.assert_close(out.double(), g / (1 + torch.exp(-g)) * u, **tol(torch.bfloat16))


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (3, 200, 96), (17, 384, 200), (130, 67, 33), (64, 64, 1)])
def test_sgemm_tn(M, N, K):
    from vllm_cpp_b200 import ops
    a, b = torch.randn(M, K, device=dev()), torch.randn(N, K, device=dev())
    out = torch.empty(M, N, device=dev())
    ops.sgemm_tn(a, b, out)
    # 32-bit accumulation of K products of unit-scale numbers: error bound about K * 2^-24 * |a||b|
    torch.testing.assert_close(out.double(), a.double() @ b.double().T, rtol=1e-5, atol=K * 2.0 ** -24 * 16)
    # a row's result does not depend on what else is in the batch
    out1 = torch.empty(1, N, device=dev())
    ops.sgemm_tn(a[M - 1:M].contiguous(), b, out1)
    assert torch.equal(out1[0], out[M - 1])


@pytest.mark.parametrize("M,N,K", [(5, 300, 4096), (3, 136, 12288), (7, 200, 17408), (130, 264, 5120)])
def test_sgemm_tn_at_serving_inner_sizes(M, N, K):
    """The inner sizes of the 4B, 8B and 14B layer shapes (the 32-bit engine at those sizes is the oracle of the
    bfloat16 engine): operands of the scale activations and weights have there, against a 64-bit product."""
    from vllm_cpp_b200 import ops
    g = torch.Generator(device=dev()).manual_seed(K)
    a = torch.randn(M, K, device=dev(), generator=g)
    b = 0.02 * torch.randn(N, K, device=dev(), generator=g)
    out = torch.empty(M, N, device=dev())
    ops.sgemm_tn(a, b, out)
    want = a.double() @ b.double().T
    # K products summed one after the other in 32-bit: the rounding errors of the running sum add up like a random
    # walk, about sqrt(K) * 2^-24 of its size (K = 12288: 7e-6 of the largest result; a dropped term would be 3e-3)
    scale = want.abs().max().item()
    assert (out.double() - want).abs().max().item() < 2 * math.sqrt(K) * 2.0 ** -24 * scale
    out1 = torch.empty(1, N, device=dev())
    ops.sgemm_tn(a[M - 1:M].contiguous(), b, out1)
    assert torch.equal(out1[0], out[M - 1])


def rope_table(hd, theta, n):
    i = torch.arange(hd // 2, dtype=torch.float64)
    ang = torch.arange(n, dtype=torch.float64)[:, None] * theta ** (-2 * i / hd)[None]
    return torch.cat([ang.cos(), ang.sin()], 1).float().to(dev())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (6, 2, 32), (5, 5, 48), (8, 1, 128), (3, 1, 256)])
def test_qknorm_rope_kvwrite(dtype, nh, nkv, hd):
    from vllm_cpp_b200 import ops
    T, ps, num_pages, eps, max_pos = 11, 4, 9, 1e-5, 64
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=dev()).to(dtype)
    qw = (1 + 0.1 * torch.randn(hd, device=dev())).to(dtype)
    kw = (1 + 0.1 * torch.randn(hd, device=dev())).to(dtype)
    table = rope_table(hd, 1e4, max_pos)
    pos = torch.randint(0, max_pos, (T,), device=dev(), dtype=torch.int32)
    slots = torch.randperm(num_pages * ps, device=dev())[:T].to(torch.int32)
    slots[4] = -1  # a padded token stores nothing
    pages = torch.zeros(num_pages, 2, nkv, ps, hd, device=dev(), dtype=dtype)
    q_out = torch.empty(T, nh * hd, device=dev(), dtype=dtype)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.qknorm_rope_kvwrite(qkv, qw, kw, eps, table, pos, slots, q_out, pages, nh, nkv, hd, status)
    assert status.item() == 0
    x = qkv.double().view(T, nh + 2 * nkv, hd)

    def norm_rope(h, w):
        h = w.double() * h / torch.sqrt((h * h).mean(-1, keepdim=True) + eps)
        c, s = table[pos.long(), :hd // 2].double()[:, None], table[pos.long(), hd // 2:].double()[:, None]
        a, b = h[..., :hd // 2], h[..., hd // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    q_want, k_want, v_want = norm_rope(x[:, :nh], qw), norm_rope(x[:, nh:nh + nkv], kw), x[:, nh + nkv:]
    torch.testing.assert_close(q_out.double().view(T, nh, hd), q_want, **tol(dtype))
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        torch.testing.assert_close(pages[s // ps, 0, :, s % ps].double(), k_want[t], **tol(dtype))
        torch.testing.assert_close(pages[s // ps, 1, :, s % ps].double(), v_want[t], **tol(dtype))
    written = {int(s) for s in slots if s >= 0}
    for s in range(num_pages * ps):
        if s not in written:
            assert pages[s // ps, :, :, s % ps].abs().max().item() == 0


@pytest.mark.parametrize("pairs", [1, 2])
@pytest.mark.parametrize("nh,nkv,T,K,norm,kv", [(4, 2, 300, 192, True, True), (5, 1, 129, 64, True, True), (3, 3, 521, 320, False, True),
                                                (32, 8, 1024, 256, True, True), (6, 2, 200, 128, True, False)])
def test_qkv_projection_with_norm_rotation_and_store_in_its_epilogue(nh, nkv, T, K, norm, kv, pairs):
    """gemm_qkv_rope (prompt portions, head_dim 128): the stacked projection whose epilogue norms each query and key
    head, rotates it and stores queries, keys and values -- against 64-bit arithmetic on the same bfloat16 operands,
    and against the two kernels it replaces.  Token counts that end inside a unit and inside a chunk of 32, a token
    that stores nowhere, positions all over the table, pages in any order; with and without the norms; a layer that
    stores no keys (query rows only).  pairs 2: on pairs of blocks wherever they take the sizes (an odd number of heads
    leaves the second block of the last pair without one)."""
    from vllm_cpp_b200 import ops
    ops.gemm_set_pairs(pairs)
    try:
        _qkv_projection_case(nh, nkv, T, K, norm, kv)
    finally:
        ops.gemm_set_pairs(1)


def _qkv_projection_case(nh, nkv, T, K, norm, kv):
    from vllm_cpp_b200 import ops
    hd, ps, eps, max_pos = 128, 16, 1e-6, 700
    torch.manual_seed(nh * 7 + T)
    heads = nh + (2 * nkv if kv else 0)
    w = (0.05 * torch.randn(heads * hd, K, device=dev())).to(torch.bfloat16)
    x = torch.randn(T, K, device=dev()).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(hd, device=dev())).to(torch.bfloat16) if norm else None
    kw = (1 + 0.1 * torch.randn(hd, device=dev())).to(torch.bfloat16) if norm and kv else None
    table = rope_table(hd, 1e4, max_pos)
    pos = torch.randint(0, max_pos, (T,), device=dev(), dtype=torch.int32)
    num_pages = T // ps + 3
    slots = torch.randperm(num_pages * ps, device=dev())[:T].to(torch.int32)
    slots[T // 2] = -1
    pages = torch.zeros(num_pages, 2, nkv, ps, hd, device=dev(), dtype=torch.bfloat16) if kv else None
    q_out = torch.full((T, nh * hd), float("nan"), device=dev(), dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.gemm_qkv_rope(w, x, q_out, pages, slots if kv else None, pos, table, qw, kw, eps, nh, nkv, status, use_norm=norm)
    torch.cuda.synchronize()
    assert status.item() == 0
    h = (x.double() @ w.double().t()).view(T, heads, hd)
    c, s = table[pos.long(), :hd // 2].double()[:, None], table[pos.long(), hd // 2:].double()[:, None]

    def norm_rope(v, g):
        if norm:
            v = g.double() * v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
        a, b = v[..., :hd // 2], v[..., hd // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    close = dict(rtol=1e-2, atol=2e-2)      # bfloat16 results of sums of up to 320 products
    torch.testing.assert_close(q_out.double().view(T, nh, hd), norm_rope(h[:, :nh], qw), **close)
    if kv:
        k_want, v_want = norm_rope(h[:, nh:nh + nkv], kw), h[:, nh + nkv:]
        idx = torch.nonzero(slots >= 0).flatten()
        sl = slots[idx].long()
        torch.testing.assert_close(pages[sl // ps, 0, :, sl % ps].double(), k_want[idx], **close)
        torch.testing.assert_close(pages[sl // ps, 1, :, sl % ps].double(), v_want[idx], **close)
        untouched = torch.ones(num_pages * ps, dtype=torch.bool, device=dev())
        untouched[sl] = False
        rest = torch.nonzero(untouched).flatten()
        assert pages[rest // ps, :, :, rest % ps].abs().max().item() == 0
        # the two kernels it replaces give the same up to the rounding of the projection to bfloat16 in between
        qkv = torch.empty(T, heads * hd, device=dev(), dtype=torch.bfloat16)
        ops.gemm_bf16_tn(w, x, qkv, 1, status)
        pages2, q2 = torch.zeros_like(pages), torch.empty_like(q_out)
        ops.qknorm_rope_kvwrite(qkv, qw, kw, eps, table, pos, slots, q2, pages2, nh, nkv, hd, status, use_norm=norm)
        torch.testing.assert_close(q_out.float(), q2.float(), rtol=2e-2, atol=4e-2)
        torch.testing.assert_close(pages.float(), pages2.float(), rtol=2e-2, atol=4e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,rot,interleaved", [(16, 8, True), (32, 32, True), (64, 16, False), (128, 64, False), (48, 2, True), (128, 128, True)])
def test_qknorm_rope_kvwrite_partial_and_interleaved(dtype, hd, rot, interleaved):
    """Only the first ``rot`` lanes of a head turn (the norm still covers the whole head), paired (i, i + rot/2) or
    (2i, 2i+1); three k-slices of partial sums in 32-bit where the input is."""
    from vllm_cpp_b200 import ops
    nh, nkv, T, ps, num_pages, eps, max_pos = 3, 1, 9, 4, 5, 1e-6, 40
    S = 3 if dtype == torch.float32 else 1
    parts = torch.randn(S, T, (nh + 2 * nkv) * hd, device=dev()).to(dtype)
    qkv = parts if S > 1 else parts[0]
    qw = (1 + 0.1 * torch.randn(hd, device=dev())).to(dtype)
    kw = (1 + 0.1 * torch.randn(hd, device=dev())).to(dtype)
    table = rope_table(rot, 300.0, max_pos)
    pos = torch.randint(0, max_pos, (T,), device=dev(), dtype=torch.int32)
    slots = torch.randperm(num_pages * ps, device=dev())[:T].to(torch.int32)
    pages = torch.zeros(num_pages, 2, nkv, ps, hd, device=dev(), dtype=dtype)
    q_out = torch.empty(T, nh * hd, device=dev(), dtype=dtype)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.qknorm_rope_kvwrite(qkv, qw, kw, eps, table, pos, slots, q_out, pages, nh, nkv, hd, status,
                            rotary_dim=rot, interleaved=interleaved)
    assert status.item() == 0
    x = parts.double().sum(0).view(T, nh + 2 * nkv, hd)
    c, sn = table[pos.long(), :rot // 2].double()[:, None], table[pos.long(), rot // 2:].double()[:, None]

    def norm_rope(h, w):
        h = w.double() * h / torch.sqrt((h * h).mean(-1, keepdim=True) + eps)
        out = h.clone()
        if interleaved:
            a, b = h[..., 0:rot:2], h[..., 1:rot:2]
            out[..., 0:rot:2], out[..., 1:rot:2] = a * c - b * sn, b * c + a * sn
        else:
            a, b = h[..., :rot // 2], h[..., rot // 2:rot]
            out[..., :rot // 2], out[..., rot // 2:rot] = a * c - b * sn, b * c + a * sn
        return out

    torch.testing.assert_close(q_out.double().view(T, nh, hd), norm_rope(x[:, :nh], qw), **tol(dtype))
    k_want = norm_rope(x[:, nh:nh + nkv], kw)
    for t in range(T):
        s = int(slots[t])
        torch.testing.assert_close(pages[s // ps, 0, :, s % ps].double(), k_want[t], **tol(dtype))
        torch.testing.assert_close(pages[s // ps, 1, :, s % ps].double(), x[t, nh + nkv:], **tol(dtype))
    with pytest.raises(ops.KernelError):       # a table of another width than the lanes to turn
        ops.qknorm_rope_kvwrite(qkv, qw, kw, eps, rope_table(hd + 2, 300.0, max_pos), pos, slots, q_out, pages, nh, nkv, hd,
                                status, rotary_dim=rot, interleaved=interleaved)


@pytest.mark.parametrize("sdtype,value", [(torch.float32, 0.25), (torch.bfloat16, -1.5), (torch.int32, 7)])
def test_state_reset(sdtype, value):
    """The state rows of requests whose entries start at position 0 take the initial value, in every cache of the
    group; entries further on, empty entries and other slots keep what they hold; a slot outside the table is
    reported and nothing is written for it."""
    from vllm_cpp_b200 import ops
    caches, slots_n, shape = 3, 6, (5, 7)
    state = torch.full((caches, slots_n) + shape, 9, dtype=sdtype, device=dev())
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev())
    # entry: (slot, q_len, ctx_len): starts, is further on, starts, is empty
    slots, q_len, ctx_len = i32([4, 1, 0, 2]), i32([3, 1, 1, 0]), i32([3, 10, 1, 0])
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.state_reset(state, slots, q_len, ctx_len, 4, value, status)
    assert status.item() == 0
    for s in range(slots_n):
        want = value if s in (4, 0) else 9
        assert (state[:, s] == torch.tensor(want, dtype=sdtype)).all(), s
    ops.state_reset(state, i32([77]), i32([2]), i32([2]), 1, value, status)
    assert status.item() == 32
    assert (state[:, 1] == 9).all()


def build_paged(seqs_kv, nkv, hd, ps, dtype, num_pages, shuffle_seed=0):
    """Scatters per-request K/V [len, nkv, hd] into shuffled pages; returns pages and block tables."""
    g = torch.Generator().manual_seed(shuffle_seed)
    perm = torch.randperm(num_pages, generator=g).tolist()
    pages = torch.full((num_pages, 2, nkv, ps, hd), float("nan"), device=dev(), dtype=dtype)
    tables = []
    for k, v in seqs_kv:
        n = k.shape[0]
        tab = [perm.pop() for _ in range(-(-n // ps))]
        for p in range(n):
            pages[tab[p // ps], 0, :, p % ps] = k[p].to(dtype)
            pages[tab[p // ps], 1, :, p % ps] = v[p].to(dtype)
        tables.append(tab)
    return pages, tables


def attention_reference(q, k, v, start, window):
    """q [n, nh, hd] at positions start..start+n-1 over k, v [start+n, nkv, hd] (64-bit)."""
    n, nh, hd = q.shape
    nkv = k.shape[1]
    out = torch.empty(n, nh, hd, dtype=torch.float64)
    kpos = torch.arange(k.shape[0])
    for i in range(n):
        p = start + i
        ok = kpos <= p
        if window:
            ok &= kpos > p - window
        for h in range(nh):
            s = (k[:, h // (nh // nkv)] @ q[i, h]) / math.sqrt(hd)
            s = s.masked_fill(~ok, float("-inf"))
            out[i, h] = torch.softmax(s, 0) @ v[:, h // (nh // nkv)]
    return out


def run_attention(dtype, nh, nkv, hd, ps, window, shapes, craft=None):
    """Runs the plain kernel, and the tensor-core kernel too where it takes the type and head size."""
    from vllm_cpp_b200 import ops
    plan = _run_attention(dtype, nh, nkv, hd, ps, window, shapes, craft, mma=False)
    if ops.attn_mma_supported(dtype, hd):
        plan = _run_attention(dtype, nh, nkv, hd, ps, window, shapes, craft, mma=True)           # TMA tile loads where the page size allows
        plan = _run_attention(dtype, nh, nkv, hd, ps, window, shapes, craft, mma="no_tma")      # cp.async tile loads
        plan = _run_attention(dtype, nh, nkv, hd, ps, window, shapes, craft, mma="cluster")     # a token's key slices merged within a cluster of blocks
    if ops.attn_tc_supported(dtype, hd, ps):
        plan = _run_attention(dtype, nh, nkv, hd, ps, window, shapes, craft, mma="tc")           # tcgen05 for the prompt portions
    return plan


def _run_attention(dtype, nh, nkv, hd, ps, window, shapes, craft, mma):
    """shapes: list of (cached tokens before the step, query tokens of the step)."""
    from vllm_cpp_b200 import ops
    from vllm_cpp_b200.parts import attention as A
    DECODE_ROWS, SPAN_ROWS = (A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS) if mma else (A.DECODE_ROWS, A.SPAN_ROWS)
    AttentionPlan = lambda c, h, k: A.AttentionPlan(c, h, k, DECODE_ROWS, SPAN_ROWS, hd if mma == "cluster" else None)
    import functools
    kernel = (functools.partial(ops.attn_mma, allow_tma=(mma in (True, "cluster"))) if mma else ops.attn_paged)
    torch.manual_seed(1)
    seqs, qs = [], []
    for start, n in shapes:
        k = torch.randn(start + n, nkv, hd, dtype=torch.float64)
        v = torch.randn(start + n, nkv, hd, dtype=torch.float64)
        q = torch.randn(n, nh, hd, dtype=torch.float64)
        if craft:
            craft(q, k, v, start, n)
        # what the kernel sees is rounded to its storage type
        k, v, q = k.to(dtype).double(), v.to(dtype).double(), q.to(dtype).double()
        seqs.append((k, v))
        qs.append(q)
    num_pages = sum(-(-(s + n) // ps) for s, n in shapes) + 3
    pages, tables = build_paged(seqs, nkv, hd, ps, dtype, num_pages)

    class Ctx:
        pass
    ctx = Ctx()
    ctx.device = dev()
    ctx.host_q_len = [n for _, n in shapes]
    ctx.host_ctx_len = [s + n for s, n in shapes]
    ctx.host_q_start = list(np.cumsum([0] + ctx.host_q_len[:-1]))
    plan = AttentionPlan(ctx, nh, nkv)
    E, T = len(shapes), sum(ctx.host_q_len)
    mb = max(len(t) for t in tables)
    bt = torch.full((E, mb), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    q_flat = torch.cat(qs).to(dtype).to(dev()).view(T, nh * hd)
    out = torch.full_like(q_flat, float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    args = (pages, bt.to(dev()), i32(ctx.host_q_start), i32(ctx.host_q_len), i32(ctx.host_ctx_len))
    if plan.n_dec:
        S = plan.nslices
        po = torch.empty(plan.n_dec * nh * S, hd, device=dev()) if S > 1 else None
        pm = torch.empty(plan.n_dec * nh * S, 2, device=dev()) if S > 1 else None
        fused = mma in (True, "cluster") and S > 1      # the last-arriving block, or the slices' cluster, merges the key slices
        extra = dict(slice_counters=plan.slice_counters, dec_rows=plan.dec_rows, cluster=plan.cluster) if fused else {}
        if mma == "cluster" and S > 1:
            assert plan.cluster == S                    # short contexts: the slices were chosen to fit clusters
            po = pm = None                              # nothing goes through global memory
        kernel(q_flat, out, *args, plan.dec_items, plan.n_dec * S, DECODE_ROWS, po, pm, nh, nkv, hd, window, status, **extra)
        if fused:
            assert int(plan.slice_counters.abs().sum()) == 0        # left ready for the next launch
        elif S > 1:
            ops.attn_merge(po, pm, plan.dec_rows, out, plan.n_dec, nh, hd, S)
    if plan.n_span_items and mma == "tc":
        ops.attn_tc(q_flat, out, *args, plan.span_items, plan.n_span_items, nh, nkv, hd, window, status)
    elif plan.n_span_items:
        kernel(q_flat, out, *args, plan.span_items, plan.n_span_items, SPAN_ROWS, None, None, nh, nkv, hd, window, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    got = out.double().cpu().view(T, nh, hd)
    t = 0
    for (start, n), q, (k, v) in zip(shapes, qs, seqs):
        want = attention_reference(q, k, v, start, window)
        torch.testing.assert_close(got[t:t + n], want, **tol(dtype))
        t += n
    return plan


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,ps", [(4, 2, 16, 4), (6, 2, 32, 8), (8, 8, 64, 16), (4, 1, 128, 16),
                                          (12, 1, 48, 16), (2, 1, 256, 32), (40, 2, 16, 8), (6, 2, 64, 8),
                                          (32, 8, 128, 16), (40, 2, 128, 4), (5, 1, 64, 5)])
def test_attention_mixed_batch(dtype, nh, nkv, hd, ps):
    # prompt portions of several sizes beside single decoded tokens, page edges on both sides
    run_attention(dtype, nh, nkv, hd, ps, 0, [(0, 7), (31, 1), (0, 1), (13, 34), (63, 2), (200, 1), (16, 16)])


@pytest.mark.parametrize("nh,nkv,hd,ps,window,blocks", [(32, 8, 128, 16, 0, 0), (8, 2, 128, 16, 0, 3), (4, 1, 64, 8, 0, 2),
                                                        (6, 2, 64, 32, 40, 3), (16, 1, 128, 64, 100, 1), (10, 2, 64, 16, 0, 5)])
def test_attention_of_many_decoded_tokens_on_persistent_blocks(nh, nkv, hd, ps, window, blocks):
    """attn_stream (blocks that walk the (token, KV head) pairs, the loading warp running ahead from pair to pair)
    against 64-bit attention: 75 single tokens whose contexts end at every place of a page and reach from one key to
    forty pages, empty entries in between (their rows stay untouched), so few blocks that each takes more than one
    batch of 32 pairs, every pair's first keys from its description and the later ones from page ids read ahead."""
    from vllm_cpp_b200 import ops
    assert ops.attn_stream_supported(torch.bfloat16, hd, ps, nh, nkv)
    torch.manual_seed(nh + hd + ps)
    dtype = torch.bfloat16
    rng = np.random.default_rng(hd + ps)
    ctxs = [1, 2, ps - 1, ps, ps + 1, 63, 64, 65, 127, 128, 129, 8 * ps, 8 * ps + 1, 40 * ps - 3, 700] + rng.integers(1, 400, 60).tolist()
    empty = {4, 17, 40}                                   # entries without a token this step
    B = len(ctxs)
    seqs = [(torch.randn(c, nkv, hd, dtype=torch.float64).to(dtype).double(),
             torch.randn(c, nkv, hd, dtype=torch.float64).to(dtype).double()) for c in ctxs]
    num_pages = sum(-(-c // ps) for c in ctxs) + 3
    pages, tables = build_paged(seqs, nkv, hd, ps, dtype, num_pages)
    mb = max(len(t) for t in tables)
    bt = torch.full((B, mb), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    q = torch.randn(B, nh, hd, dtype=torch.float64).to(dtype)
    q_flat = q.to(dev()).view(B, nh * hd)
    out = torch.full_like(q_flat, float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    items = np.zeros((B, ops.ITEM_INTS), dtype=np.int32)
    for n in range(B):
        items[n] = (n, 0, 1, 0, 1, n)
    q_len = [0 if e in empty else 1 for e in range(B)]
    for _ in range(2):      # twice: nothing is left behind by a launch
        ops.attn_stream(q_flat, out, pages, bt.to(dev()), i32(q_len), i32(ctxs), i32(items), B, i32(list(range(B))),
                        nh, nkv, hd, window, status, blocks=blocks)
    torch.cuda.synchronize()
    assert status.item() == 0
    got = out.double().cpu().view(B, nh, hd)
    for e, (c, (k, v)) in enumerate(zip(ctxs, seqs)):
        if e in empty:
            assert torch.isnan(got[e]).all()
            continue
        want = attention_reference(q[e:e + 1].double(), k, v, c - 1, window)
        torch.testing.assert_close(got[e:e + 1], want, **tol(dtype))


@pytest.mark.parametrize("nh,nkv,hd,ps,window,S,norm", [(8, 2, 128, 16, 0, 3, True), (4, 1, 64, 8, 0, 1, True), (32, 8, 128, 16, 0, 4, True),
                                                       (6, 2, 64, 32, 40, 2, True), (16, 1, 128, 64, 100, 5, False)])
def test_attention_of_decoded_tokens_straight_from_the_projection(nh, nkv, hd, ps, window, S, norm):
    """attn_mma_decode_fused (per-head norm, rotation, cache store and attention of single tokens in one kernel, from
    the projection's k-slice partial sums) against the two kernels it replaces: the same bits in the output and in
    the cache, whose contexts end at every place of a page, and against 64-bit attention over the stored keys."""
    from vllm_cpp_b200 import ops
    from vllm_cpp_b200.parts import attention as A
    torch.manual_seed(hd + ps + S)
    dtype = torch.bfloat16
    ctxs = [1, ps, ps + 1, 3 * ps - 1, 200, 64, 777, 5 * ps]       # context lengths including the new token
    B = len(ctxs)
    seqs = [(torch.randn(c, nkv, hd, dtype=torch.float64).to(dtype).double(),
             torch.randn(c, nkv, hd, dtype=torch.float64).to(dtype).double()) for c in ctxs]
    num_pages = sum(-(-c // ps) for c in ctxs) + 3
    pages, tables = build_paged(seqs, nkv, hd, ps, dtype, num_pages)
    # the newest position of every request is still to be written: poison it
    slots = []
    for c, tab in zip(ctxs, tables):
        slot = tab[(c - 1) // ps] * ps + (c - 1) % ps
        slots.append(slot)
        pages[slot // ps, :, :, slot % ps] = float("nan")
    W = (nh + 2 * nkv) * hd
    qkv = torch.randn(S, B, W, device=dev())
    qw = (1 + 0.1 * torch.randn(hd, device=dev())).to(dtype) if norm else None
    kw = (1 + 0.1 * torch.randn(hd, device=dev())).to(dtype) if norm else None
    max_pos = 1024
    table = rope_table(hd, 1e4, max_pos)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    positions, slot_map = i32([c - 1 for c in ctxs]), i32(slots)

    class Ctx:
        pass
    ctx = Ctx()
    ctx.device, ctx.host_q_len, ctx.host_ctx_len, ctx.host_q_start = dev(), [1] * B, ctxs, list(range(B))
    plan = A.AttentionPlan(ctx, nh, nkv, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    assert plan.decode_only
    NS = plan.nslices
    mb = max(len(t) for t in tables)
    bt = torch.full((B, mb), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t)
    bt = bt.to(dev())
    qs, ql, cl = i32(list(range(B))), i32([1] * B), i32(ctxs)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    eps = 1e-6

    def partials():
        if NS == 1:
            return None, None
        return torch.empty(B * nh * NS, hd, device=dev()), torch.empty(B * nh * NS, 2, device=dev())

    # the two kernels
    pages_a = pages.clone()
    q = torch.empty(B, nh * hd, device=dev(), dtype=dtype)
    ops.qknorm_rope_kvwrite(qkv, qw, kw, eps, table, positions, slot_map, q, pages_a, nh, nkv, hd, status, use_norm=norm)
    out_a = torch.full_like(q, float("nan"))
    po, pm = partials()
    ops.attn_mma(q, out_a, pages_a, bt, qs, ql, cl, plan.dec_items, B * NS, A.MMA_DECODE_ROWS, po, pm, nh, nkv, hd, window, status,
                 slice_counters=plan.slice_counters if NS > 1 else None, dec_rows=plan.dec_rows)
    # the one
    pages_b = pages.clone()
    out_b = torch.full_like(q, float("nan"))
    po, pm = partials()
    ops.attn_mma_decode_fused(qkv, qw, kw, eps, table, slot_map, out_b, pages_b, bt, qs, ql, cl, plan.dec_items,
                              B * NS, po, pm, plan.slice_counters if NS > 1 else None, plan.dec_rows, nh, nkv, hd, window,
                              status, use_norm=norm)
    # and the one with a token's key slices as a cluster of blocks that merge through shared memory
    plan_c = A.AttentionPlan(ctx, nh, nkv, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS, hd)
    pages_c = pages.clone()
    out_c = torch.full_like(q, float("nan"))
    if plan_c.cluster:
        ops.attn_mma_decode_fused(qkv, qw, kw, eps, table, slot_map, out_c, pages_c, bt, qs, ql, cl, plan_c.dec_items,
                                  B * plan_c.nslices, None, None, plan_c.slice_counters, plan_c.dec_rows, nh, nkv, hd,
                                  window, status, use_norm=norm, cluster=plan_c.cluster)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert torch.equal(pages_a.view(torch.int16), pages_b.view(torch.int16)), "the cache differs"
    assert not torch.isnan(out_b.float()).any()
    assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16)), "the attention output differs"
    if plan_c.cluster:
        assert torch.equal(pages_a.view(torch.int16), pages_c.view(torch.int16)), "the cache differs (clusters)"
        if plan_c.nslices == NS:     # the same slices, merged in the same order: the same bits
            assert torch.equal(out_b.view(torch.int16), out_c.view(torch.int16)), "the attention output differs (clusters)"
        else:
            torch.testing.assert_close(out_c.float(), out_b.float(), **tol(dtype))
    # and what came out is attention of the rotated query over the stored keys
    got = out_b.double().cpu().view(B, nh, hd)
    for b, (c, tab) in enumerate(zip(ctxs, tables)):
        k = torch.stack([pages_b[tab[p // ps], 0, :, p % ps] for p in range(c)]).double().cpu()
        v = torch.stack([pages_b[tab[p // ps], 1, :, p % ps] for p in range(c)]).double().cpu()
        want = attention_reference(q[b].double().cpu().view(1, nh, hd), k, v, c - 1, window)
        torch.testing.assert_close(got[b:b + 1], want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 24, 100])
@pytest.mark.parametrize("hd", [32, 64])
def test_attention_window(dtype, window, hd):
    run_attention(dtype, 6, 2, hd, 8, window, [(0, 40), (57, 1), (23, 3), (130, 1), (300, 70)])


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(8, 2, 128, 16, 0), (3, 3, 128, 64, 0), (10, 2, 64, 8, 0), (4, 1, 128, 32, 0),
                                                 (8, 2, 128, 16, 100), (2, 1, 64, 16, 7), (130, 1, 64, 16, 0),
                                                 (4, 2, 128, 8, 0), (6, 2, 64, 64, 33), (5, 1, 64, 32, 0)])
def test_attention_long_prompt_portions(nh, nkv, hd, ps, window):
    """Prompt portions over many key tiles (what the tcgen05 kernel pipelines): from an empty cache, behind a long
    prefix, a prefix that ends inside a page and inside a tile, group sizes that do not divide 128 rows."""
    run_attention(torch.bfloat16, nh, nkv, hd, ps, window, [(0, 300), (517, 130), (1000, 2), (63, 65), (64, 64), (0, 64)])


def test_attention_tcgen05_many_blocks_many_launches():
    """Two thousand tokens on 32 heads: 512 blocks of up to 32 key tiles, launched over and over, against the
    mma.sync kernel on the same inputs.  (Warps of a block may run a tile apart; a hand-off that counted on their
    staying together showed only here, once in a few hundred launches.)"""
    from vllm_cpp_b200 import ops
    from vllm_cpp_b200.parts import attention as A
    nh, nkv, hd, ps, T = 32, 8, 128, 16, 2048
    torch.manual_seed(3)
    npages = T // ps
    pages = torch.randn(npages, 2, nkv, ps, hd, device=dev()).to(torch.bfloat16)
    bt = torch.randperm(npages, device=dev()).to(torch.int32).view(1, -1)
    q = torch.randn(T, nh * hd, device=dev()).to(torch.bfloat16)

    class Ctx:
        pass
    c = Ctx()
    c.device, c.host_q_len, c.host_ctx_len, c.host_q_start = dev(), [T], [T], [0]
    plan = A.AttentionPlan(c, nh, nkv, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev())
    qs, ql, cl = i32([0]), i32([T]), i32([T])
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    want = torch.empty_like(q)
    ops.attn_mma(q, want, pages, bt, qs, ql, cl, plan.span_items, plan.n_span_items, A.MMA_SPAN_ROWS, None, None,
                 nh, nkv, hd, 0, status)
    outs = [torch.full_like(q, float("nan")) for _ in range(4)]
    for i in range(200):
        ops.attn_tc(q, outs[i % 4], pages, bt, qs, ql, cl, plan.span_items, plan.n_span_items, nh, nkv, hd, 0, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    for o in outs:
        torch.testing.assert_close(o.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(o, outs[0])      # and the same bits every time


@pytest.mark.parametrize("hd,ps,nh,nkv", [(128, 16, 32, 8), (64, 8, 24, 8)])
def test_attention_tcgen05_units_from_the_queue(hd, ps, nh, nkv):
    """The tcgen05 kernel's blocks take their work units from a queue.  Here there are more units than blocks that
    run at once (so most come through the queue), the items are laid out for longer portions than are there (units
    with nothing to do, at the front and in the middle of the queue), and launch follows launch on the same two
    counters, eagerly and in a captured graph: every output equals 64-bit attention, and the counters are back at
    zero."""
    from vllm_cpp_b200 import ops
    from vllm_cpp_b200.parts import attention as A
    torch.manual_seed(hd + ps)
    planned = [(0, 1400), (300, 40), (16, 900), (1000, 700)]        # (keys before the portion, tokens the items are for)
    actual = [(0, 1400), (300, 11), (16, 0), (1000, 333)]           # what is there: whole, cut, nothing, cut
    seqs, qs = [], []
    for start, n in actual:
        k = torch.randn(start + n, nkv, hd, dtype=torch.float64).to(torch.bfloat16).double()
        v = torch.randn(start + n, nkv, hd, dtype=torch.float64).to(torch.bfloat16).double()
        seqs.append((k, v))
        qs.append(torch.randn(n, nh, hd, dtype=torch.float64).to(torch.bfloat16).double())
    num_pages = sum(-(-(s + n) // ps) for s, n in planned) + 3
    pages, tables = build_paged(seqs, nkv, hd, ps, torch.bfloat16, num_pages)

    class Ctx:
        pass
    c = Ctx()
    c.device = dev()
    c.host_q_len = [n for _, n in planned]
    c.host_ctx_len = [s + n for s, n in planned]
    q_start = [int(x) for x in np.cumsum([0] + [n for _, n in actual[:-1]])]
    c.host_q_start = q_start
    plan = A.AttentionPlan(c, nh, nkv, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    assert plan.n_span_items * nkv > 2 * ops.num_sms()
    mb = max(-(-(s + n) // ps) for s, n in planned)
    bt = torch.full((len(planned), mb), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    T = sum(n for _, n in actual)
    q = torch.cat(qs).to(torch.bfloat16).to(dev()).view(T, nh * hd)
    args = (pages, bt.to(dev()), i32(q_start), i32([n for _, n in actual]), i32([s + n for s, n in actual]))
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    work = torch.zeros(2, dtype=torch.int32, device=dev())
    outs = [torch.full_like(q, float("nan")) for _ in range(6)]
    launch = lambda o: ops.attn_tc(q, o, *args, plan.span_items, plan.n_span_items, nh, nkv, hd, 0, status, work=work)
    for o in outs[:3]:
        launch(o)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for o in outs[3:]:
            launch(o)
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    assert status.item() == 0 and work.tolist() == [0, 0]
    want = torch.cat([attention_reference(qq, k, v, start, 0) for (start, n), qq, (k, v) in zip(actual, qs, seqs) if n])
    for o in outs:
        torch.testing.assert_close(o.double().cpu().view(T, nh, hd), want, **tol(torch.bfloat16))
        assert torch.equal(o, outs[0])


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_long_decode_is_sliced(dtype):
    plan = run_attention(dtype, 8, 2, 64, 16, 0, [(3000, 1), (1025, 1)])
    assert plan.nslices > 1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 3, 511, 512, 1777])
def test_attention_far_key_stands_out(dtype, far):
    """One key among two thousand carries nearly all the weight: a kernel that skips or misplaces it shows."""
    def craft(q, k, v, start, n):
        q[:] = q / q.norm(dim=-1, keepdim=True) * 8
        k[far] = q[0, 0] * 4
        v[far] = 50.0
    run_attention(dtype, 4, 4, 64, 16, 0, [(2047, 1)], craft)
    run_attention(dtype, 4, 4, 64, 16, 0, [(2040, 8)], craft)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("offset", [0, 1])
@pytest.mark.parametrize("hd", [32, 128])
def test_attention_window_edge(dtype, offset, hd):
    """A dominant key exactly at the window's first position must count; one position earlier it must not."""
    W, start = 24, 100
    def craft(q, k, v, s, n):
        q[:] = q / q.norm(dim=-1, keepdim=True) * 8
        edge = (s + n - 1) - W + 1 - offset      # offset 0: last key inside; 1: first key outside
        k[edge] = q[-1, 0] * 4
        v[edge] = 50.0
    run_attention(dtype, 2, 2, hd, 8, W, [(start, 1)], craft)
    run_attention(dtype, 2, 2, hd, 8, W, [(start - 5, 6)], craft)


def plain_sample(*a, **k):
    import plain_qwen3
    return plain_qwen3.sample(*a, **k)


@pytest.mark.parametrize("V", [50, 1000, 20011])
def test_sampling_matches_plain(V):
    from vllm_cpp_b200.sampling import Sampler, SamplingOptions
    rng = np.random.default_rng(V)
    logits = torch.tensor(rng.normal(0, 2, size=(6, V)), dtype=torch.float32)
    logits[1, 7] = logits[1].max() + 0.0   # a tie for greedy: lowest index wins
    logits[1, 3] = logits[1, 7]
    opts = [SamplingOptions(0.0, 1.0, 1.0, 0), SamplingOptions(0.0, 0.8, 1.0, 0), SamplingOptions(0.8, 1.0, 1.0, 4),
            SamplingOptions(1.3, 0.8, 1.0, 5), SamplingOptions(0.7, 0.5, 1.2, 6), SamplingOptions(0.0, 1.0, 1.5, 7)]
    steps = [0, 1, 2, 3, 4, 5]
    slots = [0, 1, 2, 3, 4, 5]
    s = Sampler(V, 6, dev())
    history = {4: rng.integers(0, V, 30).tolist() + [int(logits[4].argmax())] * 3, 5: [int(logits[5].argmax())] * 4}
    s._need_counts()
    for slot, h in history.items():
        for t in h:
            s.counts[slot, t] += 1
    got = s.sample(logits.to(dev()), opts, steps, slots).cpu().tolist()
    for i, o in enumerate(opts):
        want = plain_sample(logits[i].numpy(), temperature=o.temperature, top_p=o.top_p, repeat_penalty=o.repeat_penalty,
                            history=history.get(i, ()), seed=o.seed, step=steps[i])
        assert got[i] == want, (i, got[i], want)
    assert got[1] == 3


def test_sampling_distribution():
    """Empirical frequencies of seeded draws follow softmax(logits / T) cut to the nucleus."""
    from vllm_cpp_b200.sampling import Sampler, SamplingOptions
    V, N = 12, 4000
    logits = torch.tensor([2.0, 1.5, 1.0, 0.5, 0.0, -0.5, -1.0, -1.5, -2.0, -2.5, -3.0, -9.0])
    rows = logits[None].repeat(N, 1).to(dev())
    s = Sampler(V, 1, dev())
    for top_p in (1.0, 0.7):
        toks = s.sample(rows, [SamplingOptions(0.9, top_p, 1.0, 123)] * N, list(range(N)), [0] * N).cpu().numpy()
        p = torch.softmax(logits.double() / 0.9, 0).numpy()
        if top_p < 1:
            order = np.argsort(-p)
            keep = order[:int(np.searchsorted(np.cumsum(p[order]), top_p)) + 1]
            mask = np.zeros(V, bool); mask[keep] = True
            p = np.where(mask, p, 0); p /= p.sum()
            assert set(np.unique(toks)) <= set(keep.tolist())
        freq = np.bincount(toks, minlength=V) / N
        assert np.abs(freq - p).max() < 0.03


def test_count_tokens():
    from vllm_cpp_b200 import ops
    V = 37
    ids = torch.tensor([1, 1, 5, 36, 1, 2], dtype=torch.int32, device=dev())
    slots = torch.tensor([0, 0, 1, 1, -1, 0], dtype=torch.int32, device=dev())
    counts = torch.zeros(2, V, dtype=torch.int32, device=dev())
    ops.count_tokens(ids, slots, counts, 6)
    assert counts[0, 1] == 2 and counts[0, 2] == 1 and counts[1, 5] == 1 and counts[1, 36] == 1 and counts.sum() == 5


def test_kernels_refuse_what_they_cannot_do():
    from vllm_cpp_b200 import ops
    with pytest.raises(ops.KernelError, match="CUDA tensor"):
        ops.swiglu(torch.zeros(2, 4), torch.zeros(2, 2))
    q = torch.zeros(1, 24, device=dev())
    pages = torch.zeros(2, 2, 1, 4, 24, device=dev())
    z = torch.zeros(1, dtype=torch.int32, device=dev())
    items = torch.zeros(1, 6, dtype=torch.int32, device=dev())
    with pytest.raises(ops.KernelError, match="multiple of 16"):
        ops.attn_paged(q, q.clone(), pages, z.view(1, 1), z, z, z, items, 1, 8, None, None, 1, 1, 24, 0, z)


@pytest.mark.parametrize("M,T,K,splits", [
    (128, 16, 64, 1), (128, 1, 64, 1), (64, 3, 96, 1), (200, 17, 200, 1), (384, 8, 4096, 4), (6144, 8, 4096, 3),
    (4096, 64, 1024, 2), (1000, 33, 520, 2), (256, 100, 256, 1), (384, 256, 512, 1), (300, 700, 328, 1),
    (4096, 2048, 512, 1), (128, 130, 8, 1), (6144, 2048, 256, 1), (6144, 700, 128, 1),
    (4096, 256, 1024, 4), (600, 513, 2048, 3), (1000, 160, 1536, 8)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_bf16_tn(M, T, K, splits, out_dtype):
    """The tcgen05/TMA product against 64-bit: tile edges in every dimension, k tails, k-slices, 1 to 2048 tokens."""
    from vllm_cpp_b200 import ops
    if splits > 1 and out_dtype != torch.float32:
        pytest.skip("k-slices write 32-bit partial sums")
    torch.manual_seed(M + T + K)
    w = torch.randn(M, K, device=dev()).to(torch.bfloat16)
    x = torch.randn(T, K, device=dev()).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    S = ops.gemm_effective_splits(K, splits)
    out = torch.full((S, T, M) if S > 1 else (T, M), float("nan"), dtype=out_dtype, device=dev())
    ops.gemm_bf16_tn(w, x, out, splits, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    got = out.double().sum(0) if S > 1 else out.double()
    want = x.double() @ w.double().T
    if out_dtype == torch.float32:
        torch.testing.assert_close(got, want, rtol=1e-4, atol=K * 2.0 ** -24 * 64)
    else:
        torch.testing.assert_close(got, want, rtol=1e-2, atol=1e-2 * K ** 0.5)
    # a token's result does not depend on what else is in the batch
    if T > 1 and S == 1:
        one = torch.empty((1, M), dtype=out_dtype, device=dev())
        ops.gemm_bf16_tn(w, x[T - 1:T].contiguous(), one, 1, status)
        assert torch.equal(one[0], out[T - 1])


@pytest.mark.parametrize("shape", range(9))
@pytest.mark.parametrize("M,T,K,splits", [(300, 5, 200, 1), (520, 300, 1096, 1), (520, 300, 1096, 3), (128, 700, 64, 1)])
def test_gemm_bf16_tn_every_unit_shape(shape, M, T, K, splits):
    """Each unit shape of the kernel, forced, at sizes that are not the ones it is chosen for: many token tiles
    of a small shape, one ragged tile of a large one, k-slices."""
    from vllm_cpp_b200 import ops
    torch.manual_seed(shape + M + T)
    w = torch.randn(M, K, device=dev()).to(torch.bfloat16)
    x = torch.randn(T, K, device=dev()).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    S = ops.gemm_effective_splits(K, splits)
    out = torch.full((S, T, M) if S > 1 else (T, M), float("nan"), dtype=torch.float32, device=dev())
    if ops.GEMM_SHAPES[shape] == "pair" and M < 256:
        with pytest.raises(ops.KernelError, match="at least 256 features"):
            ops.gemm_bf16_tn(w, x, out, splits, status, shape=shape)
        return
    ops.gemm_bf16_tn(w, x, out, splits, status, shape=shape)
    torch.cuda.synchronize()
    assert status.item() == 0
    got = out.double().sum(0) if S > 1 else out.double()
    torch.testing.assert_close(got, x.double() @ w.double().T, rtol=1e-4, atol=K * 2.0 ** -24 * 64)
    with pytest.raises(ops.KernelError, match="no unit shape"):
        ops.gemm_bf16_tn(w, x, out, splits, status, shape=9)


@pytest.mark.parametrize("M,T,K", [(256, 129, 64), (512, 300, 256), (1000, 700, 328), (6144, 512, 1024), (4096, 2048, 512),
                                   (300, 257, 1096), (24576, 160, 128)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_bf16_tn_on_pairs_of_blocks(M, T, K, out_dtype):
    """The two-block kernel (cta_group::2, 256 x 256 units, each block half of the token tile), forced, against
    64-bit and against the single-block kernel: ragged feature, token and k edges, one unit and many."""
    from vllm_cpp_b200 import ops
    torch.manual_seed(M + T + K)
    w = torch.randn(M, K, device=dev()).to(torch.bfloat16)
    x = torch.randn(T, K, device=dev()).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    outs = []
    try:
        for mode in (2, 0):
            ops.gemm_set_pairs(mode)
            out = torch.full((T, M), float("nan"), dtype=out_dtype, device=dev())
            ops.gemm_bf16_tn(w, x, out, 1, status)
            torch.cuda.synchronize()
            assert status.item() == 0
            outs.append(out)
    finally:
        ops.gemm_set_pairs(1)
    want = x.double() @ w.double().T
    if out_dtype == torch.float32:
        torch.testing.assert_close(outs[0].double(), want, rtol=1e-4, atol=K * 2.0 ** -24 * 64)
    else:
        torch.testing.assert_close(outs[0].double(), want, rtol=1e-2, atol=1e-2 * K ** 0.5)
    assert torch.equal(outs[0], outs[1])      # the same k order, the same bits


@pytest.mark.parametrize("I,T,K", [(128, 256, 64), (200, 300, 96), (1536, 2048, 512), (264, 160, 128)])
def test_gemm_bf16_swiglu_on_pairs_of_blocks(I, T, K):
    from vllm_cpp_b200 import ops
    torch.manual_seed(I + T)
    w = (torch.randn(2 * I, K, device=dev()) * 0.2).to(torch.bfloat16)
    x = torch.randn(T, K, device=dev()).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    outs = []
    try:
        for mode in (2, 0):
            ops.gemm_set_pairs(mode)
            out = torch.full((T, I), float("nan"), dtype=torch.bfloat16, device=dev())
            ops.gemm_bf16_swiglu(w, x, out, status)
            torch.cuda.synchronize()
            assert status.item() == 0
            outs.append(out)
    finally:
        ops.gemm_set_pairs(1)
    gu = x.double() @ w.double().T
    g, u = gu[:, 0::2], gu[:, 1::2]
    torch.testing.assert_close(outs[0].double(), g / (1 + torch.exp(-g)) * u, rtol=2e-2, atol=2e-2)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("M,T,K,splits", [(6144, 256, 4096, 3), (4096, 512, 12288, 4), (1000, 300, 1096, 5), (512, 130, 640, 2)])
def test_gemm_k_slices_on_pairs_of_blocks(M, T, K, splits):
    """k-slices on the two-block kernel: every slice's 32-bit partial equals the single-block kernel's to the bit
    (the same k-blocks in the same order), and their sum is the product."""
    from vllm_cpp_b200 import ops
    torch.manual_seed(M + T + K)
    w = torch.randn(M, K, device=dev()).to(torch.bfloat16)
    x = torch.randn(T, K, device=dev()).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    S = ops.gemm_effective_splits(K, splits)
    assert S > 1
    pair = torch.full((S, T, M), float("nan"), dtype=torch.float32, device=dev())
    single = torch.full((S, T, M), float("nan"), dtype=torch.float32, device=dev())
    ops.gemm_bf16_tn(w, x, pair, splits, status, shape=ops.GEMM_SHAPES.index("pair"))
    ops.gemm_bf16_tn(w, x, single, splits, status, shape=ops.GEMM_SHAPES.index("n256"))
    torch.cuda.synchronize()
    assert status.item() == 0
    assert torch.equal(pair, single)
    torch.testing.assert_close(pair.double().sum(0), x.double() @ w.double().T, rtol=1e-4, atol=K * 2.0 ** -24 * 64)


def test_choose_splits_fills_the_sms():
    from vllm_cpp_b200.parts.linear import choose_splits
    assert choose_splits(6144, 256, 4096) == 3      # 48 units of 128 x 256 -> 144
    assert choose_splits(4096, 256, 12288) == 4     # 32 units -> 128
    assert choose_splits(4096, 512, 4096) == 2      # 64 units -> 128
    assert choose_splits(4096, 1024, 4096) == 1     # 128 units already
    assert choose_splits(24576, 2048, 4096) == 1
    assert choose_splits(6144, 8, 4096) == 3


def test_gemm_bf16_tn_refuses_unaligned_rows():
    from vllm_cpp_b200 import ops
    w = torch.zeros(128, 100, device=dev(), dtype=torch.bfloat16)
    x = torch.zeros(4, 100, device=dev(), dtype=torch.bfloat16)
    out = torch.zeros(4, 128, device=dev())
    with pytest.raises(ops.KernelError, match="multiples of 8"):
        ops.gemm_bf16_tn(w, x, out, 1, torch.zeros(1, dtype=torch.int32, device=dev()))


@pytest.mark.parametrize("out_dtype", DTYPES)
def test_partial_sum_inputs(out_dtype):
    """The kernels that read a product cut into k-slices add the slices themselves."""
    from vllm_cpp_b200 import ops
    T, I, S = 5, 72, 3
    parts = torch.randn(S, T, 2 * I, device=dev())
    out = torch.empty(T, I, device=dev(), dtype=out_dtype)
    ops.swiglu(parts, out)
    tot = parts.double().sum(0)
    g, u = tot[:, 0::2], tot[:, 1::2]
    torch.testing.assert_close(out.double(), g / (1 + torch.exp(-g)) * u, **tol(out_dtype))

    nh, nkv, hd, ps, num_pages, eps = 4, 2, 32, 4, 6, 1e-6
    qkv = torch.randn(S, T, (nh + 2 * nkv) * hd, device=dev())
    one = qkv.sum(0)
    w = torch.ones(hd, device=dev())
    table = rope_table(hd, 1e4, 64)
    pos = torch.arange(T, device=dev(), dtype=torch.int32)
    slots = torch.arange(T, device=dev(), dtype=torch.int32)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    res = []
    for inp in (qkv, one):
        pages = torch.zeros(num_pages, 2, nkv, ps, hd, device=dev(), dtype=out_dtype)
        q = torch.empty(T, nh * hd, device=dev(), dtype=out_dtype)
        ops.qknorm_rope_kvwrite(inp, w, w, eps, table, pos, slots, q, pages, nh, nkv, hd, status)
        res.append((q.double(), pages.double()))
    torch.testing.assert_close(res[0][0], res[1][0], **tol(out_dtype))
    torch.testing.assert_close(res[0][1], res[1][1], **tol(out_dtype))


def test_sampling_split_over_blocks_matches_plain():
    """Rows without a nucleus cut are dealt to several blocks per row; the token is the same."""
    from vllm_cpp_b200.sampling import Sampler, SamplingOptions
    V = 50021
    rng = np.random.default_rng(5)
    logits = torch.tensor(rng.normal(0, 2, size=(5, V)), dtype=torch.float32)
    logits[0, 40000] = logits[0, 17] = logits[0].max() + 1   # greedy tie across blocks: lowest index
    opts = [SamplingOptions(0.0, 1.0, 1.0, 0), SamplingOptions(0.0, 0.5, 1.0, 0), SamplingOptions(0.8, 1.0, 1.0, 4),
            SamplingOptions(1.3, 1.0, 1.0, 5), SamplingOptions(0.7, 1.0, 1.3, 6)]
    s = Sampler(V, 5, dev())
    s._need_counts()
    hist = rng.integers(0, V, 40).tolist() + [int(logits[4].argmax())] * 2
    for t in hist:
        s.counts[4, t] += 1
    got = s.sample(logits.to(dev()), opts, [3, 4, 5, 6, 7], [0, 1, 2, 3, 4]).cpu().tolist()
    for i, o in enumerate(opts):
        want = plain_sample(logits[i].numpy(), temperature=o.temperature, top_p=o.top_p, repeat_penalty=o.repeat_penalty,
                            history=hist if i == 4 else (), seed=o.seed, step=3 + i)
        assert got[i] == want, (i, got[i], want)
    assert got[0] == 17


@pytest.mark.parametrize("I,T,K", [(128, 256, 64), (200, 300, 96), (12288 // 8, 2048, 512), (72, 130, 264), (264, 160, 128),
                                   (1024, 385, 64), (100, 7, 64)])
@pytest.mark.parametrize("shape", [-1, 0, 2, 3, 4, 5, 6, 8])
def test_gemm_bf16_swiglu(I, T, K, shape):
    """The product with the SiLU-gate in its epilogue against 64-bit, for the chosen and for forced unit shapes.
    Gate values reach far below -87, where silu is zero to every precision."""
    from vllm_cpp_b200 import ops
    if shape >= 0 and T * I > 1 << 20:
        pytest.skip("the large case runs with the chosen shape only")
    torch.manual_seed(I + T)
    w = (torch.randn(2 * I, K, device=dev()) * 0.2).to(torch.bfloat16)
    w[0::2][:: 5] *= 40          # some gates far out on both sides
    x = torch.randn(T, K, device=dev()).to(torch.bfloat16)
    out = torch.full((T, I), float("nan"), dtype=torch.bfloat16, device=dev())
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.gemm_bf16_swiglu(w, x, out, status, shape=shape)
    torch.cuda.synchronize()
    assert status.item() == 0
    gu = x.double() @ w.double().T
    g, u = gu[:, 0::2], gu[:, 1::2]
    assert g.min() < -100 and g.max() > 100
    want = g / (1 + torch.exp(-g)) * u
    torch.testing.assert_close(out.double(), want, rtol=2e-2, atol=2e-2)
    # and the same numbers as the product followed by the SiLU-gate kernel, to bfloat16 rounding
    full = torch.empty(T, 2 * I, dtype=torch.float32, device=dev())
    ops.gemm_bf16_tn(w, x, full, 1, status)
    two = torch.empty_like(out)
    ops.swiglu(full, two)
    torch.testing.assert_close(out.float(), two.float(), rtol=2 ** -7, atol=1e-30)


def test_qknorm_fast_path_matches_general_path():
    """head_dim 128 in bfloat16 takes a vectorised kernel; the same inputs as 32-bit partial sums take the general one."""
    from vllm_cpp_b200 import ops
    T, nh, nkv, hd, ps, num_pages = 9, 6, 2, 128, 4, 5
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=dev()).to(torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(hd, device=dev())).to(torch.bfloat16)
    kw = (1 + 0.1 * torch.randn(hd, device=dev())).to(torch.bfloat16)
    table = rope_table(hd, 1e6, 64)
    pos = torch.randint(0, 64, (T,), device=dev(), dtype=torch.int32)
    slots = torch.randperm(num_pages * ps, device=dev())[:T].to(torch.int32)
    slots[2] = -1
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    res = []
    for inp in (qkv, qkv.float().unsqueeze(0)):
        pages = torch.zeros(num_pages, 2, nkv, ps, hd, device=dev(), dtype=torch.bfloat16)
        q = torch.zeros(T, nh * hd, device=dev(), dtype=torch.bfloat16)
        ops.qknorm_rope_kvwrite(inp, qw, kw, 1e-6, table, pos, slots, q, pages, nh, nkv, hd, status)
        res.append((q.float(), pages.float()))
    assert status.item() == 0
    torch.testing.assert_close(res[0][0], res[1][0], rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(res[0][1], res[1][1], rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_bf16_product_of_unaligned_inner_size(out_dtype):
    """An inner size that is no multiple of 8 cannot be addressed by TMA; the projection falls back to the plain kernel."""
    from vllm_cpp_b200.parts.linear import matmul_tn
    T, N, K = 5, 70, 100
    x = torch.randn(T, K, device=dev()).to(torch.bfloat16)
    w = torch.randn(N, K, device=dev()).to(torch.bfloat16)
    y = matmul_tn(x, w, torch.zeros(1, dtype=torch.int32, device=dev()), out_dtype=out_dtype, allow_partials=True)
    assert y.shape == (T, N) and y.dtype == out_dtype
    torch.testing.assert_close(y.double(), x.double() @ w.double().T, rtol=1e-2, atol=1e-1)


def test_a_bounded_wait_that_runs_out_is_reported_and_harmless():
    """Every TMA and tcgen05 kernel of the library waits on mbarriers through one helper whose waits are bounded by
    the clock.  Here that helper waits, for a millisecond at most, on a barrier that nothing arrives at: the wait
    answers false, the status word gets the wait-timeout bit, the block's abort flag is up (a later wait in the block
    gives up at once), check_status raises with the bit's text and clears it, and the next ordinary kernels run."""
    from vllm_cpp_b200 import ops
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    got = ops.selftest_wait_timeout(2_000_000, status)
    assert got == [0, 1, 0, 1], got
    assert status.item() == 4
    with pytest.raises(ops.KernelError, match="bounded wait"):
        ops.check_status(status)
    assert status.item() == 0
    # the context is as usable as before: a TMA / tcgen05 product right after
    x = torch.randn(8, 256, device=dev()).to(torch.bfloat16)
    w = torch.randn(128, 256, device=dev()).to(torch.bfloat16)
    out = torch.empty(8, 128, device=dev(), dtype=torch.float32)
    ops.gemm_bf16_tn(w, x, out, 1, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    torch.testing.assert_close(out.double(), x.double() @ w.double().T, rtol=1e-3, atol=1e-3)
    with pytest.raises(ops.KernelError):
        ops.selftest_wait_timeout(10 ** 12, status)       # no long waits on request
