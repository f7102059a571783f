#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens/s (batch 8 at the stated context; batch 1 and 64
as extra points), prefill tokens/s at 2,048 tokens, each with its roofline fraction.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

Shapes: the Qwen3-8B layer sizes of the baseline's third configuration, random weights drawn on the
device, synthetic token ids.  One "step" is one decode step of the whole batch.  Weights (16 GB) are
far larger than L2, so no flush is needed between timed iterations.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
             num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
             rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = 16


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def mark(self):
        return time.time()

    def stop(self):
        if self.proc:
            self.proc.terminate()

    def summary(self, windows):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, r in self.rows:
            if not any(a <= t <= b for a, b in windows) or len(r) < 6:
                continue
            try:
                sm.append(float(r[0])); mx = max(mx, float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (for profiling runs)")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel (for profiling runs)")
    ap.add_argument("--mode", default="all", choices=["all", "decode", "prefill"], help="what to run (profiling runs)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "laik/vllm-cpp has no Python package or installable build (pip finds no setup.py/pyproject.toml), "
                          "its CUDA sources do not compile with nvcc 12.9, and its CUDA forward has attention stubbed out"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import numpy as np
    import torch
    from vllm_cpp_b200 import EngineConfig, LLM, Qwen3Config, ops
    from vllm_cpp_b200.engine.step import StepEntry
    from vllm_cpp_b200.runtime import runtime

    pk = peaks()
    cfgd = dict(MODEL, num_hidden_layers=args.layers)
    cfg = Qwen3Config(**cfgd)
    B_MAX = 64
    points = [args.batch] if args.skip_points else sorted({1, args.batch, B_MAX})
    max_seqs = max(points)
    # room for the end-to-end run, whose requests start decoding up to two steps apart each
    steps_total = args.steps + args.warmup + 2 * args.batch + 24
    per_req = -(-(args.context + steps_total) // 64) * 64
    max_tokens = max(max(points) * per_req, 8192)
    t0 = time.time()
    llm = LLM(config=cfg, random_seed=0, engine=EngineConfig(dtype="bfloat16", page_size=PAGE, max_tokens=max_tokens,
                                                            max_num_seqs=max(points), max_step_tokens=PREFILL_TOKENS,
                                                            max_model_len=args.context + steps_total + 8,
                                                            cuda_graphs=not args.no_graphs))
    runner = llm.runner
    dev = runner.device
    load_s = time.time() - t0
    rt = runtime()
    rng = np.random.default_rng(0)
    V = cfg.vocab_size

    # bytes and flops of the model
    H, I, nh, nkv, hd, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.num_hidden_layers
    layer_params = (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * I * H
    weight_bytes = 2 * (L * layer_params + V * H) + 2 * L * (2 * H + 2 * hd) + 2 * H
    kv_bytes_per_token = L * 2 * nkv * hd * 2

    clocks = ClockSampler()
    clocks.start()
    windows = []

    def fresh_cache():
        runner.reset_tables()
        return rt.CacheManager(runner.layout.runtime_groups(rt, PAGE, max_tokens // PAGE), max_seqs)

    # the cache of requests that "hold" a context: random keys and values stand for a processed prompt
    for t in runner.cache.tensors:
        for i in range(t.shape[0]):
            t[i].normal_(0, 1)

    def decode_point(B, steps, warmup):
        cm = fresh_cache()
        for r in range(B):
            cm.open(r)
            assert cm.reserve(r, args.context + steps + warmup + 1)
            cm.commit(r, args.context)
        times = []
        launches = 0
        for it in range(warmup + steps):
            entries = []
            for r in range(B):
                pos = cm.num_tokens(r)
                entries.append(StepEntry(cm.slot(r), pos, [int(rng.integers(0, V))], [cm.block_table(r, 0)], [0]))
            timed = it >= warmup
            if it == warmup:
                torch.cuda.synchronize()
                windows.append([clocks.mark(), None])
            l0 = ops.launch_count
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            flat, use_counts, no_nucleus = Sampler.records([GREEDY] * B, [0] * B, [e.slot for e in entries])
            toks = runner.step(entries, check=False, user=flat, post=sample_post, post_key=("sample", False, True))
            e1.record()
            e1.synchronize()
            if timed:
                times.append(e0.elapsed_time(e1))
                launches += ops.launch_count - l0
            for r in range(B):
                cm.commit(r, cm.num_tokens(r) + 1)
        windows[-1][1] = clocks.mark()
        ops.check_status(runner.status)
        ms = sum(times) / len(times)
        return dict(ms=ms, tok_s=B * 1000.0 / ms, launches=launches,
                    bytes=weight_bytes + B * (args.context + warmup + steps / 2) * kv_bytes_per_token)

    from vllm_cpp_b200.sampling import Sampler, SamplingOptions
    GREEDY = SamplingOptions(0.0, 1.0, 1.0, 0)

    def sample_post(ctx, logits):   # what LLM.step runs after the model, captured with the step
        return llm.sampler.sample_records(logits, ctx.user[:8 * logits.shape[0]].view(-1, 8), False, True)

    if args.mode == "prefill":
        points = []
    results = {}
    for B in points:
        st = args.steps if B == args.batch else max(8, args.steps // 4)
        results[B] = decode_point(B, st, args.warmup)
    if args.mode == "decode":
        print(json.dumps({"mode": "decode", "ms_per_step": {b: results[b]["ms"] for b in points}}))
        return 0
    head = results.get(args.batch)

    # prefill: one prompt of 2,048 tokens in one step, logits of the last token only
    def prefill_once():
        cm = fresh_cache()
        cm.open(0)
        assert cm.reserve(0, PREFILL_TOKENS)
        ent = [StepEntry(cm.slot(0), 0, rng.integers(0, V, PREFILL_TOKENS).tolist(), [cm.block_table(0, 0)], [PREFILL_TOKENS - 1])]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step(ent, check=False)
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1)

    for _ in range(3):
        prefill_once()
    windows.append([clocks.mark(), None])
    pf = [prefill_once() for _ in range(5)]
    windows[-1][1] = clocks.mark()
    pf_ms = statistics.median(pf)
    T = PREFILL_TOKENS
    pf_flops = 2.0 * T * L * layer_params + 2.0 * V * H + L * 4.0 * nh * hd * (T * (T + 1) / 2)
    if args.mode == "prefill":
        print(json.dumps({"mode": "prefill", "ms": pf_ms, "tokens_per_s": T * 1000.0 / pf_ms}))
        return 0
    # frac: against the library's burst rate (one product timed alone); the eight back-to-back steps timed here run
    # under the power cap like the library's seconds-long loop, whose rate frac_of_sustained is taken against
    prefill = {"value": T * 1000.0 / pf_ms, "tokens": T, "ms": pf_ms, "frac": pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12),
               "frac_of_sustained": pf_flops / (pf_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12)}

    # end to end through the Python entry point: host token lists in, host tokens out, every step
    B = args.batch
    e2e_steps = args.steps
    for r in range(B):
        llm.submit_tokens(rng.integers(0, V, args.context - args.warmup).tolist(), args.warmup + e2e_steps + 2 * B + 8, 0.0, 1.0,
                          repeat_penalty=1.0, ignore_eos=True)
    while True:   # feed the prompts; stop when every request is decoding
        o = llm.step()
        if len(o.new_token_ids) == B:
            break
    for _ in range(args.warmup - 1):
        llm.step()
    torch.cuda.synchronize()
    h0, d0 = llm.h2d_bytes, llm.d2h_bytes
    windows.append([clocks.mark(), None])
    t0 = time.perf_counter()
    n_tok = 0
    for _ in range(e2e_steps):
        n_tok += len(llm.step().new_token_ids)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    windows[-1][1] = clocks.mark()
    e2e = {"value": n_tok / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": (llm.h2d_bytes - h0) / e2e_steps,
           "d2h_bytes_per_step": (llm.d2h_bytes - d0) / e2e_steps, "ms_per_step": 1000 * e2e_s / e2e_steps}
    clocks.stop()

    achieved = head["bytes"] / (head["ms"] * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s, Qwen3-8B shape, batch %d, context %d" % (args.batch, args.context),
        "value": head["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform random token ids, random cache contents for the held context)",
        "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": cfg.num_hidden_layers, "layers_of_named_config": MODEL["num_hidden_layers"],
                   "hidden": H, "heads": nh, "kv_heads": nkv, "head_dim": hd, "intermediate": I, "vocab": V,
                   "global_batch": args.batch, "seq_len": args.context, "page_size": PAGE, "parallelism": "single GPU",
                   "l2": "inputs (16 GB of weights) larger than L2", "peaks": pk["source"]},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"]},
        "points": {"decode_b%d" % b: results[b]["tok_s"] for b in points if b != args.batch},
        "e2e": e2e,
        "gpu_launches": head["launches"],
        "clocks": clocks.summary(windows),
        "load_s": load_s,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
