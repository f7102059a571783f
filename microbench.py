#!/usr/bin/env python3
"""Per-kernel timings at a model's layer sizes, on one GPU.

    python microbench.py [--model 8b|4b|14b|CONFIG.json] [--peaks FILE] gemm [T ...]   the four projections (and lm_head) at T tokens
    python microbench.py [...] attention        decode attention over a paged cache; prompt attention
    python microbench.py [...] small            add+norm, norm-rotate-store, SiLU-gate
    python microbench.py [...] gemm --library   the products beside the library's (torch.mm), for comparison
    VLLM_CPP_B200_TIMELINE=1 VLLM_CPP_B200_BUILD_DIR=/tmp/vcb_timeline python microbench.py [--layers L] [--batch B]
        [--context C] timeline              one captured decode step seen from inside: when the blocks of each kernel
                                            start, when their wait for the kernel before ends, when they end
    VLLM_CPP_B200_TIMELINE=1 VLLM_CPP_B200_BUILD_DIR=/tmp/vcb_timeline python microbench.py attention-roles [T]
                                            the roles inside a block of the tcgen05 prompt attention kernel over a
                                            prompt of T tokens (default 8192): clocks from mark to mark, per tile

The sizes come from a Qwen3 configuration: one of the three serving shapes by name (default 8b) or a config.json.

How it times: every launch is captured ``reps`` times in a CUDA graph (so that launch overhead does not set the
floor), the graph is replayed ten times between CUDA events, and the median replay divided by ``reps`` is reported.
Products rotate over copies of their weights that together exceed L2, so that weights come from HBM as in a step.
``VCB_MICROBENCH_PAGE`` sets the page size of the attention runs (default 16).
Each line also gives the time the same bytes or flops take at the peaks of ``--peaks FILE`` (JSON with ``hbm_gbs``
and ``bf16_tflops``; default: MEASURED_PEAKS.json in the current folder if there is one, else 6650 GB/s and
1590 TFLOP/s) and, with ``--library``, the library's time for the same product.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch

from vllm_cpp_b200 import Qwen3Config, ops
from vllm_cpp_b200.parts import attention as A
from vllm_cpp_b200.parts.linear import choose_splits

NAMED = {
    "8b": dict(hidden_size=4096, intermediate_size=12288, num_attention_heads=32, num_key_value_heads=8, head_dim=128),
    "14b": dict(hidden_size=5120, intermediate_size=17408, num_attention_heads=40, num_key_value_heads=8, head_dim=128),
    "4b": dict(hidden_size=2560, intermediate_size=9728, num_attention_heads=32, num_key_value_heads=8, head_dim=128),
}
PAGE = int(os.environ.get("VCB_MICROBENCH_PAGE", "16"))
# set from the command line in main()
SHAPES: dict = {}
NH = NKV = HD = 0
PEAKS = (6650.0, 1590.0)
LIBRARY = False


def set_model(cfg: Qwen3Config) -> None:
    global SHAPES, NH, NKV, HD
    NH, NKV, HD = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    H, I = cfg.hidden_size, cfg.intermediate_size
    SHAPES = {"qkv": ((NH + 2 * NKV) * HD, H), "o": (H, NH * HD), "gate_up": (2 * I, H), "down": (H, I), "lm_head": (cfg.vocab_size, H)}


def peaks():
    return PEAKS


def timeit(fn, reps: int = 20, iters: int = 10) -> float:
    """fn(k) launches once, using buffer set k.  Microseconds per launch."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for k in range(3):
            fn(k)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for k in range(reps):
            fn(k)
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) / reps)
    ts.sort()
    return ts[len(ts) // 2] * 1e3


def bench_gemm(tokens, dev, status):
    hbm, tc = peaks()
    for T in tokens:
        for name, (M, K) in SHAPES.items():
            if name == "lm_head" and T > 256:
                continue
            ncopy = max(1, min(8, (300 << 20) // (M * K * 2) + 1))
            ws = [(0.02 * torch.randn(M, K, device=dev)).to(torch.bfloat16) for _ in range(ncopy)]
            x = torch.randn(T, K, device=dev).to(torch.bfloat16)
            s = choose_splits(M, T, K)
            S = ops.gemm_effective_splits(K, s)
            out = torch.empty((S, T, M) if S > 1 else (T, M), dtype=torch.float32 if S > 1 else torch.bfloat16, device=dev)
            ours = timeit(lambda k: ops.gemm_bf16_tn(ws[k % ncopy], x, out, s, status))
            extra = ""
            if name == "gate_up" and T > 128:
                act = torch.empty(T, M // 2, dtype=torch.bfloat16, device=dev)
                extra = f"  with SiLU-gate {timeit(lambda k: ops.gemm_bf16_swiglu(ws[k % ncopy], x, act, status)):.1f}"
            lib = timeit(lambda k: torch.mm(x, ws[k % ncopy].t())) if LIBRARY else float("nan")
            print(f"product {name:8s} T={T:5d} k-slices {S}: {ours:7.1f} us{extra}   library {lib:7.1f}   "
                  f"at HBM peak {M * K * 2 / hbm / 1e3:6.1f}   at bf16 peak {2.0 * M * K * T / tc / 1e6:6.1f}", flush=True)
            del ws, x


class _Ctx:
    pass


def bench_attention(dev, status, only=None):
    """``only``: one (requests, context) pair of decode attention instead of the list (and no prompt attention)."""
    hbm, tc = peaks()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    cases = ((1, 4096), (8, 4096), (64, 4096), (32, 2048), (64, 512), (128, 256), (256, 128), (256, 1024))
    for B, ctx_len in ((only,) if only else cases):
        npages = B * (ctx_len // PAGE + 1)
        pages = torch.randn(npages, 2, NKV, PAGE, HD, device=dev).to(torch.bfloat16)
        bt = torch.arange(npages, dtype=torch.int32, device=dev).view(B, -1)
        q = torch.randn(B, NH * HD, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        c = _Ctx()
        c.device, c.host_q_len, c.host_ctx_len, c.host_q_start = dev, [1] * B, [ctx_len] * B, list(range(B))
        plan = A.AttentionPlan(c, NH, NKV, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS, HD if A.CLUSTER_MERGE else None)
        S = plan.nslices
        po = torch.empty(B * NH * S, HD, device=dev) if S > 1 else None
        pm = torch.empty(B * NH * S, 2, device=dev) if S > 1 else None
        qs, ql, cl = i32(c.host_q_start), i32(c.host_q_len), i32(c.host_ctx_len)
        us = timeit(lambda k: ops.attn_mma(q, out, pages, bt, qs, ql, cl, plan.dec_items, B * S, A.MMA_DECODE_ROWS, po, pm,
                                           NH, NKV, HD, 0, status, slice_counters=plan.slice_counters if S > 1 else None,
                                           dec_rows=plan.dec_rows, cluster=plan.cluster))
        kv_bytes = B * ctx_len * 2 * NKV * HD * 2
        walk = ""
        if B * NKV > ops.num_sms() and ops.attn_stream_supported(torch.bfloat16, HD, PAGE, NH, NKV):
            one = A.AttentionPlan(c, NH, NKV, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
            items = one.dec_items if one.nslices == 1 else i32([[e, 0, 1, 0, 1, e] for e in range(B)])
            us_w = timeit(lambda k: ops.attn_stream(q, out, pages, bt, ql, cl, items, B, one.dec_rows, NH, NKV, HD, 0, status))
            walk = f"   on blocks that walk the pairs {us_w:7.1f} us"
        print(f"decode attention  batch {B:3d} context {ctx_len:5d} key slices {S:2d}{' in clusters' if plan.cluster else ''}: {us:7.1f} us{walk}   at HBM peak {kv_bytes / hbm / 1e3:6.1f}", flush=True)
        del pages
    for T in (() if only else (2048, 8192)):
        npages = T // PAGE
        pages = torch.randn(npages, 2, NKV, PAGE, HD, device=dev).to(torch.bfloat16)
        bt = torch.arange(npages, dtype=torch.int32, device=dev).view(1, -1)
        q = torch.randn(T, NH * HD, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        c = _Ctx()
        c.device, c.host_q_len, c.host_ctx_len, c.host_q_start = dev, [T], [T], [0]
        plan = A.AttentionPlan(c, NH, NKV, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
        qs, ql, cl = i32([0]), i32([T]), i32([T])
        flops = 4.0 * NH * HD * T * (T + 1) / 2
        mma = timeit(lambda k: ops.attn_mma(q, out, pages, bt, qs, ql, cl, plan.span_items, plan.n_span_items, A.MMA_SPAN_ROWS,
                                            None, None, NH, NKV, HD, 0, status))
        tcg = timeit(lambda k: ops.attn_tc(q, out, pages, bt, qs, ql, cl, plan.span_items, plan.n_span_items, NH, NKV, HD, 0, status, work=plan.span_work))
        print(f"prompt attention  {T} tokens: mma.sync {mma:7.1f} us ({flops / mma / 1e6:5.0f} TFLOP/s)   tcgen05 {tcg:7.1f} us "
              f"({flops / tcg / 1e6:5.0f} TFLOP/s)   at bf16 peak {flops / tc / 1e6:6.1f}", flush=True)


def bench_small(dev, status):
    hbm, _ = peaks()
    H, I = SHAPES["o"][0], SHAPES["down"][1]
    for T in (8, 64, 2048):
        resid = torch.randn(T, H, device=dev)
        w = torch.ones(H, device=dev).to(torch.bfloat16)
        out = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
        for S in ((4,) if T <= 128 else (1,)):
            d = torch.randn(S, T, H, device=dev)
            us = timeit(lambda k: ops.add_rmsnorm(resid, d, w, 1e-6, out))
            print(f"add+norm          T={T:5d} slices {S}: {us:7.1f} us   at HBM peak {(T * H * (8 + 4 * S + 2)) / hbm / 1e3:6.1f}", flush=True)
        S = 3 if T <= 128 else 1
        gu = torch.randn(S, T, 2 * I, device=dev) if S > 1 else torch.randn(T, 2 * I, device=dev).to(torch.bfloat16)
        act = torch.empty(T, I, device=dev, dtype=torch.bfloat16)
        print(f"SiLU-gate         T={T:5d} slices {S}: {timeit(lambda k: ops.swiglu(gu, act)):7.1f} us", flush=True)
        width = (NH + 2 * NKV) * HD
        qkv = torch.randn(S, T, width, device=dev) if S > 1 else torch.randn(T, width, device=dev).to(torch.bfloat16)
        gain = torch.ones(HD, device=dev, dtype=torch.bfloat16)
        table = torch.randn(8192, HD, device=dev)
        pos = torch.arange(T, device=dev, dtype=torch.int32)
        pages = torch.zeros(T // PAGE + 2, 2, NKV, PAGE, HD, device=dev, dtype=torch.bfloat16)
        qo = torch.empty(T, NH * HD, device=dev, dtype=torch.bfloat16)
        us = timeit(lambda k: ops.qknorm_rope_kvwrite(qkv, gain, gain, 1e-6, table, pos, pos, qo, pages, NH, NKV, HD, status))
        print(f"norm-rotate-store T={T:5d} slices {S}: {us:7.1f} us", flush=True)


def bench_attention_roles(dev, status, tokens: int):
    """The roles inside one block of the tcgen05 prompt attention kernel (a library built with VLLM_CPP_B200_TIMELINE=1):
    a prompt of ``tokens`` tokens, one launch; for the block that works on the longest unit, the median clocks from one
    mark of a role to its next, tile by tile, and the clocks a tile takes each role."""
    import statistics
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    T = tokens
    npages = T // PAGE
    pages = torch.randn(npages, 2, NKV, PAGE, HD, device=dev).to(torch.bfloat16)
    bt = torch.arange(npages, dtype=torch.int32, device=dev).view(1, -1)
    q = torch.randn(T, NH * HD, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    c = _Ctx()
    c.device, c.host_q_len, c.host_ctx_len, c.host_q_start = dev, [T], [T], [0]
    plan = A.AttentionPlan(c, NH, NKV, A.MMA_DECODE_ROWS, A.MMA_SPAN_ROWS)
    qs, ql, cl = i32([0]), i32([T]), i32([T])
    run = lambda: ops.attn_tc(q, out, pages, bt, qs, ql, cl, plan.span_items, plan.n_span_items, NH, NKV, HD, 0, status,
                              work=plan.span_work)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    ops.timeline_begin()
    run()
    rec = [r for r in ops.timeline_end() if r["kernel"] == "attn_tc" and "role" in r and r["block"] == 0]
    names = {10: "load: asks", 11: "load: stages free", 12: "load: copies sent", 20: "products: asks for K", 21: "products: K there",
             22: "products: Q.K^T issued", 23: "products: weights and V there", 24: "products: P.V issued", 30: "row: asks for scores",
             31: "row: scores there", 32: "row: scores loaded", 33: "row: weights computed", 34: "row: handed over"}
    print(f"prompt attention, {T} tokens, block 0: {len(rec)} marks of its roles")
    for role, phases in (("loading warp", (10, 11, 12)), ("product thread", (20, 21, 22, 23, 24)), ("softmax row", (30, 31, 32, 33, 34))):
        by = {ph: {r["tile"]: r["clock"] for r in rec if r["phase"] == ph} for ph in phases}
        last = sorted(by[phases[-1]].items())
        period = [b[1] - a[1] for a, b in zip(last, last[1:]) if b[0] == a[0] + 1]
        print(f"  {role}: a tile every {statistics.median(period):.0f} clocks (median of {len(period)})" if period else f"  {role}: too few tiles")
        for a, b in zip(phases, phases[1:]):
            d = [by[b][t] - by[a][t] for t in by[a] if t in by[b]]
            if d:
                print(f"    {names[a]:30s} -> {names[b]:30s} {statistics.median(d):7.0f}")


def bench_timeline(cfg, batch: int, context: int, layers: int, first: int, count: int):
    """One captured decode step of ``layers`` layers, recorded by the kernels' own timeline marks (a library built with
    VLLM_CPP_B200_TIMELINE=1), printed launch by launch: the times (us from the step's first mark) at which the first
    and the last block of a launch started, left their wait for the kernel before, and ended."""
    import numpy as np
    from vllm_cpp_b200 import EngineConfig, LLM
    from vllm_cpp_b200.engine.step import StepEntry
    from vllm_cpp_b200.runtime import runtime
    from vllm_cpp_b200.sampling import Sampler, SamplingOptions
    import dataclasses
    cfg = dataclasses.replace(cfg, num_hidden_layers=layers, layer_types=())     # (the kinds of the layers follow from the window)
    max_tokens = batch * (-(-(context + 128) // 64) * 64)
    llm = LLM(config=cfg, random_seed=0, engine=EngineConfig(dtype="bfloat16", page_size=PAGE, max_tokens=max_tokens,
                                                            max_num_seqs=batch, max_step_tokens=256, max_model_len=context + 128))
    runner, rt = llm.runner, runtime()
    cm = rt.CacheManager(runner.layout.runtime_groups(rt, PAGE, max_tokens // PAGE), batch)
    for t in runner.cache.tensors:
        t.normal_(0, 1)
    for r in range(batch):
        cm.open(r)
        assert cm.reserve(r, context + 100)
        cm.commit(r, context)
    greedy = SamplingOptions(0.0, 1.0, 1.0, 0)
    rng = np.random.default_rng(0)

    def post(ctx, logits):
        return llm.sampler.sample_records(logits, ctx.user[:8 * logits.shape[0]].view(-1, 8), False, True)

    def step():
        entries = [StepEntry(cm.slot(r), cm.num_tokens(r), [int(rng.integers(0, 1000))], [cm.block_table(r, 0)], [0]) for r in range(batch)]
        flat, _, _ = Sampler.records([greedy] * batch, [0] * batch, [e.slot for e in entries])
        runner.step(entries, check=False, user=flat, post=post, post_key=("sample", False, True))
        for r in range(batch):
            cm.commit(r, cm.num_tokens(r) + 1)

    for _ in range(10):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); step(); e1.record(); e1.synchronize()
    plain_ms = e0.elapsed_time(e1)
    ops.timeline_begin()
    e0.record(); step(); e1.record(); e1.synchronize()
    rec = [r for r in ops.timeline_end() if "role" not in r]     # the block-wide marks; roles inside blocks are another view
    print(f"decode step, batch {batch}, context {context}, {layers} layers: {plain_ms:.3f} ms; with the marks recorded {e0.elapsed_time(e1):.3f} ms; "
          f"{len(rec)} marks")
    # marks -> launches: a launch of a kernel takes every (block, phase) once
    t0 = rec[0]["t_ns"]
    launches, open_by = [], {}
    for r in rec:
        lst = open_by.setdefault((r["kernel"], r["grid"]), [])
        tag = (r["block"], r["phase"])
        target = next((c for c in lst[-3:] if tag not in c["tags"] and (r["phase"] == 0 or (r["block"], 0) in c["tags"])), None)
        if target is None:
            target = dict(kernel=r["kernel"], tags=set(), recs=[])
            lst.append(target)
            launches.append(target)
        target["tags"].add(tag)
        target["recs"].append(r)
    launches.sort(key=lambda c: min(x["t_ns"] for x in c["recs"]))

    def span(rs, ph):
        ts = [(x["t_ns"] - t0) / 1e3 for x in rs if x["phase"] == ph]
        return (f"{min(ts):9.2f} {max(ts):9.2f}" if ts else "        -         -")
    if os.environ.get("VCB_TIMELINE_DUMP"):
        json.dump(rec, open(os.environ["VCB_TIMELINE_DUMP"], "w"))
    print(f"{'kernel':12s} {'blocks':>6s}   {'start: first':>9s} {'last':>9s}   {'wait over: first':>9s} {'last':>6s}   {'end: first':>9s} {'last':>9s}")
    for c in launches[first:first + count]:
        print(f"{c['kernel']:12s} {len({t[0] for t in c['tags']}):6d}   {span(c['recs'], 0)}   {span(c['recs'], 1)}   {span(c['recs'], 2)}")


def main(argv):
    global PEAKS, LIBRARY
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="8b", help="8b, 4b, 14b, or a config.json of the Qwen3 architecture")
    ap.add_argument("--peaks", default=None, help="JSON file with hbm_gbs and bf16_tflops")
    ap.add_argument("--library", action="store_true", help="time the library's product (torch.mm) beside each of ours")
    ap.add_argument("--layers", type=int, default=12, help="timeline: layers of the model")
    ap.add_argument("--batch", type=int, default=None, help="timeline: requests decoding (default 8); attention: with --context, that one case only")
    ap.add_argument("--context", type=int, default=None, help="timeline: tokens each request holds (default 4096)")
    ap.add_argument("--first", type=int, default=18, help="timeline: first launch to print")
    ap.add_argument("--count", type=int, default=30, help="timeline: launches to print")
    ap.add_argument("what", nargs="?", default="gemm", choices=["gemm", "attention", "attention-roles", "small", "timeline"])
    ap.add_argument("tokens", nargs="*", type=int)
    args = ap.parse_args(argv)
    if args.model in NAMED:
        cfg = Qwen3Config(vocab_size=151936, num_hidden_layers=1, max_position_embeddings=40960, **NAMED[args.model])
    else:
        cfg = Qwen3Config.from_dict(json.loads(Path(args.model).read_text()))
    set_model(cfg)
    pfile = Path(args.peaks) if args.peaks else Path("MEASURED_PEAKS.json")
    if pfile.is_file():
        d = json.loads(pfile.read_text())
        PEAKS = (float(d["hbm_gbs"]), float(d["bf16_tflops"]))
    elif args.peaks:
        print(f"microbench: {pfile} not found", file=sys.stderr)
        return 2
    LIBRARY = args.library
    if not torch.cuda.is_available():
        print("microbench: needs a CUDA device", file=sys.stderr)
        return 2
    dev = torch.device("cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    what = args.what
    if what == "gemm":
        bench_gemm(args.tokens or [8, 64, 256, 2048], dev, status)
    elif what == "attention":
        bench_attention(dev, status, (args.batch, args.context) if args.batch and args.context else None)
    elif what == "attention-roles":
        bench_attention_roles(dev, status, (args.tokens or [8192])[0])
    elif what == "small":
        bench_small(dev, status)
    elif what == "timeline":
        bench_timeline(cfg, args.batch or 8, args.context or 4096, args.layers, args.first, args.count)
    else:
        print(__doc__)
        return 2
    ops.check_status(status, "microbench")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
