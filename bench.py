#!/usr/bin/env python3
"""Benchmark of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--workloads all|headline] [--impl reference]

Headline: decode tokens/s of the Qwen3-8B layer sizes (the baseline's third configuration) at batch 8 and context
4,096, the median of K device-timed steps after W warm-up steps; beside it batch 1 and 64, batch 8 at context 2,176
(a 2,048-token prompt half-way through 256 decoded tokens), batch 8 launched kernel by kernel instead of from a
captured graph, the prefill of one 2,048-token prompt, and the same decode loop end to end through ``LLM.step()``
(host token lists in, host tokens out).  Each with its fraction of the measured roofline.

Two more workloads run after it unless ``--workloads headline`` is given, both through ``LLM.step()`` and the scheduler:
* Qwen3-14B layer sizes, 8 prompts of 8,192 tokens fed in portions of 2,048, then 256 greedy tokens each;
* Qwen3-4B layer sizes, 32 requests with prompts of 128 to 4,096 tokens (seed 5) under a step budget of 2,048
  tokens, 128 new tokens each: prompt portions beside decoding.

Random weights drawn on the device, synthetic token ids.  One "step" is one decode step of the whole batch.  The
weights (8 to 28 GB) are far larger than L2, so no flush is needed between timed iterations.
"""
import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL_8B = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
MODEL_14B = dict(MODEL_8B, hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40)
MODEL_4B = dict(MODEL_8B, hidden_size=2560, intermediate_size=9728, tie_word_embeddings=True)
CONTEXT = 4096
WORKLOAD_CONTEXT = 2176     # a 2,048-token prompt half-way through its 256 decoded tokens
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
    """Samples the SM clock and the throttle reasons of the GPU that the benchmark runs on (asked for by UUID:
    nvidia-smi's own indices ignore CUDA_VISIBLE_DEVICES) while the timed regions run.  Read-only."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_id: str = "0"):
        self.rows, self.proc, self.gpu_id = [], None, gpu_id

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu_id, f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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
            if not any(a <= t <= (b or t) for a, b in windows) or len(r) < 6:
                continue
            try:
                sm.append(float(r[0])); mx = max(mx, float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm), "gpu": self.gpu_id}


def gpu_id_for_nvidia_smi(torch) -> str:
    """'GPU-<uuid>' of the CUDA device in use if nvidia-smi knows it under that name, else index 0."""
    try:
        uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
        name = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        r = subprocess.run(["nvidia-smi", "-i", name, "--query-gpu=uuid", "--format=csv,noheader"],
                           capture_output=True, text=True, timeout=20)
        if r.returncode == 0 and r.stdout.strip():
            return name
    except Exception:
        pass
    return "0"


def model_numbers(cfg):
    H, I, nh, nkv, hd, L, V = (cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                               cfg.head_dim, cfg.num_hidden_layers, cfg.vocab_size)
    layer_params = (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * I * H
    tables = 1 if cfg.tie_word_embeddings else 2
    # a decode step reads every layer matrix, the LM head and the norm gains once; of the embedding table only the
    # rows of its tokens (a tied table is the LM head, read whole)
    weight_bytes = 2 * (L * layer_params + V * H) + 2 * L * (2 * H + 2 * hd) + 2 * H
    return dict(layer_params=layer_params, weight_bytes=weight_bytes, kv_bytes_per_token=L * 2 * nkv * hd * 2,
                stored_bytes=2 * (L * layer_params + tables * V * H))


def prefill_flops(cfg, T, past=0):
    """Products over T tokens, the LM head on one row, causal attention of T queries over past + their own keys."""
    n = model_numbers(cfg)
    L, nh, hd = cfg.num_hidden_layers, cfg.num_attention_heads, cfg.head_dim
    return 2.0 * T * L * n["layer_params"] + 2.0 * cfg.vocab_size * cfg.hidden_size + L * 4.0 * nh * hd * (T * past + T * (T + 1) / 2)


def release(*objs):
    import torch
    gc.collect()
    torch.cuda.empty_cache()


# ------------------------------------------------------------------------------------------------ headline: 8B
def run_headline(args, pk, clocks, windows):
    import numpy as np
    import torch
    from vllm_cpp_b200 import EngineConfig, LLM, Qwen3Config, ops
    from vllm_cpp_b200.engine.step import StepEntry
    from vllm_cpp_b200.runtime import runtime
    from vllm_cpp_b200.sampling import Sampler, SamplingOptions

    cfg = Qwen3Config(**dict(MODEL_8B, num_hidden_layers=args.layers))
    nums = model_numbers(cfg)
    points = [args.batch] if args.skip_points else sorted({1, args.batch, 64})
    max_seqs = max(points)
    # room for the end-to-end run, whose requests start decoding up to two steps apart each
    steps_total = args.steps + args.warmup + 2 * args.batch + 24
    per_req = -(-(args.context + steps_total) // 64) * 64
    max_tokens = max(max_seqs * per_req, 8192)
    t0 = time.time()
    llm = LLM(config=cfg, random_seed=0, engine=EngineConfig(dtype="bfloat16", page_size=PAGE, max_tokens=max_tokens,
                                                            max_num_seqs=max_seqs, max_step_tokens=PREFILL_TOKENS,
                                                            max_model_len=args.context + steps_total + 8,
                                                            cuda_graphs=not args.no_graphs))
    runner = llm.runner
    load_s = time.time() - t0
    rt = runtime()
    rng = np.random.default_rng(0)
    V = cfg.vocab_size
    GREEDY = SamplingOptions(0.0, 1.0, 1.0, 0)

    def fresh_cache():
        runner.reset_tables()
        return rt.CacheManager(runner.layout.runtime_groups(rt, PAGE, max_tokens // PAGE), max_seqs)

    # the cache of requests that "hold" a context: random keys and values stand for a processed prompt
    for t in runner.cache.tensors:
        for i in range(t.shape[0]):
            t[i].normal_(0, 1)

    def sample_post(ctx, logits):   # what LLM.step runs after the model, captured with the step
        return llm.sampler.sample_records(logits, ctx.user[:8 * logits.shape[0]].view(-1, 8), False, True)

    def decode_point(B, context, steps, warmup, graphs=True):
        runner.cuda_graphs = graphs and not args.no_graphs
        cm = fresh_cache()
        for r in range(B):
            cm.open(r)
            assert cm.reserve(r, context + steps + warmup + 1)
            cm.commit(r, context)
        times, launches = [], 0
        for it in range(warmup + steps):
            entries = []
            for r in range(B):
                pos = cm.num_tokens(r)
                entries.append(StepEntry(cm.slot(r), pos, [int(rng.integers(0, V))], [cm.block_table(r, 0)], [0]))
            if it == warmup:
                torch.cuda.synchronize()
                windows.append([clocks.mark(), None])
            l0 = ops.launch_count
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            flat, _, _ = Sampler.records([GREEDY] * B, [0] * B, [e.slot for e in entries])
            runner.step(entries, check=False, user=flat, post=sample_post, post_key=("sample", False, True))
            e1.record()
            e1.synchronize()
            if it >= warmup:
                times.append(e0.elapsed_time(e1))
                launches += ops.launch_count - l0
            for r in range(B):
                cm.commit(r, cm.num_tokens(r) + 1)
        windows[-1][1] = clocks.mark()
        ops.check_status(runner.status)
        runner.cuda_graphs = not args.no_graphs
        ms = statistics.median(times)
        nbytes = nums["weight_bytes"] + B * (context + warmup + steps / 2) * nums["kv_bytes_per_token"]
        gbs = nbytes / (ms * 1e-3) / 1e9
        return dict(ms=ms, mean_ms=sum(times) / len(times), tok_s=B * 1000.0 / ms, launches=launches, bytes=nbytes,
                    gbs=gbs, frac=gbs / pk["hbm_gbs"])

    results = {}
    if args.mode != "prefill":
        for B in points:
            results[("b", B)] = decode_point(B, args.context, args.steps, args.warmup)
        if not args.skip_points:
            results[("ctx", WORKLOAD_CONTEXT)] = decode_point(args.batch, WORKLOAD_CONTEXT, args.steps, args.warmup)
            results[("eager", args.batch)] = decode_point(args.batch, args.context, args.steps, args.warmup, graphs=False)
    if args.mode == "decode":
        print(json.dumps({"mode": "decode", "batch": args.batch, "context": args.context, "layers": args.layers,
                          "ms_per_step": {f"{k[0]}{k[1]}": v["ms"] for k, v in results.items()},
                          "roofline_frac": {f"{k[0]}{k[1]}": round(v["frac"], 4) for k, v in results.items()}}))
        return None
    head = results.get(("b", args.batch))

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
    pf = [prefill_once() for _ in range(9)]
    windows[-1][1] = clocks.mark()
    pf_ms = statistics.median(pf)
    T = PREFILL_TOKENS
    pf_flops = prefill_flops(cfg, T)
    if args.mode == "prefill":
        print(json.dumps({"mode": "prefill", "ms": pf_ms, "tokens_per_s": T * 1000.0 / pf_ms}))
        return None
    # frac: against the library's burst rate (one product timed alone); the back-to-back steps timed here run
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
    step_s, n_tok = [], 0
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        t1 = time.perf_counter()
        n_tok += len(llm.step().new_token_ids)     # returns host tokens: the step has run when it comes back
        step_s.append(time.perf_counter() - t1)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    windows[-1][1] = clocks.mark()
    e2e_ms = 1000 * statistics.median(step_s)
    e2e = {"value": B * 1000.0 / e2e_ms, "unit": "tokens/s", "h2d_bytes_per_step": (llm.h2d_bytes - h0) / e2e_steps,
           "d2h_bytes_per_step": (llm.d2h_bytes - d0) / e2e_steps, "ms_per_step": e2e_ms,
           "mean_tokens_per_s": n_tok / e2e_s}

    name = {("b", 1): "decode_b1", ("b", 64): "decode_b64", ("ctx", WORKLOAD_CONTEXT): f"decode_b{args.batch}_ctx{WORKLOAD_CONTEXT}",
            ("eager", args.batch): f"decode_b{args.batch}_kernel_by_kernel"}
    line = {
        "metric": "decode tokens/s, Qwen3-8B shape, batch %d, context %d" % (args.batch, args.context),
        "value": head["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform random token ids, random cache contents for the held context)",
        "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": cfg.num_hidden_layers, "layers_of_named_config": MODEL_8B["num_hidden_layers"],
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": V,
                   "global_batch": args.batch, "seq_len": args.context, "page_size": PAGE, "parallelism": "single GPU",
                   "l2": "inputs (16 GB of weights) larger than L2", "peaks": pk["source"], "timing": "median of steps, CUDA events"},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": head["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": head["frac"]},
        "points": {name[k]: v["tok_s"] for k, v in results.items() if k in name},
        "points_ms": {name[k]: v["ms"] for k, v in results.items() if k in name},
        "points_roofline_frac": {name[k]: v["frac"] for k, v in results.items() if k in name},
        "mean_ms_per_step": head["mean_ms"],
        "e2e": e2e,
        "gpu_launches": head["launches"],
        "workspace_mb": runner.workspace.bytes() / 2 ** 20,
        "load_s": load_s,
    }
    del llm, runner
    release()
    return line


# ------------------------------------------------------------------------------------------------ 14B: long prompts, then decode
class GcPauses:
    """Seconds the Python collector ran inside a timed region (its pauses are the host's, so they belong to the
    end-to-end numbers; reported so that a slow run can be told from a slow engine)."""

    def __enter__(self):
        import gc
        self.total, self.count, self._t = 0.0, 0, 0.0
        gc.callbacks.append(self._cb)
        return self

    def _cb(self, phase, info):
        if phase == "start":
            self._t = time.perf_counter()
        else:
            self.total += time.perf_counter() - self._t
            self.count += 1

    def __exit__(self, *exc):
        import gc
        gc.callbacks.remove(self._cb)


def run_14b(args, pk, clocks, windows):
    """8 prompts of 8,192 tokens in portions of 2,048, then 256 greedy tokens each, through LLM.step()."""
    import numpy as np
    import torch
    from vllm_cpp_b200 import EngineConfig, LLM, Qwen3Config
    layers = args.layers_14b
    cfg = Qwen3Config(**dict(MODEL_14B, num_hidden_layers=layers))
    nums = model_numbers(cfg)
    B, P, NEW = 8, 8192, 256
    rng = np.random.default_rng(6)
    prompts = [rng.integers(0, cfg.vocab_size, P).tolist() for _ in range(B)]
    llm = LLM(config=cfg, random_seed=0, engine=EngineConfig(dtype="bfloat16", page_size=PAGE, max_tokens=B * (P + 320),
                                                            max_num_seqs=B, max_step_tokens=2048, max_model_len=P + 320))
    llm.warm_up(0.0, 1.0, 1.0)       # the captured decoding steps are made before the clock starts, as at a server's start
    for p in prompts:
        llm.submit_tokens(p, NEW, 0.0, 1.0, repeat_penalty=1.0, ignore_eos=True)
    torch.cuda.synchronize()
    windows.append([clocks.mark(), None])
    t0 = time.perf_counter()
    prefill_steps, decode_s, first_decode = 0, [], None
    flops = 0.0
    with GcPauses() as pauses:
        while llm.has_requests():
            t1 = time.perf_counter()
            o = llm.step()
            dt = time.perf_counter() - t1
            if o.num_prompt_tokens:
                prefill_steps += 1
            else:
                if first_decode is None:
                    torch.cuda.synchronize()
                    first_decode = t1
                decode_s.append(dt)
        torch.cuda.synchronize()
    windows[-1][1] = clocks.mark()
    prefill_s = first_decode - t0
    for _ in range(B):     # each prompt: four portions of 2,048 over what came before
        flops += sum(prefill_flops(cfg, 2048, past) for past in range(0, P, 2048))
    ms = 1000 * statistics.median(decode_s)
    nbytes = nums["weight_bytes"] + B * (P + NEW / 2) * nums["kv_bytes_per_token"]
    out = {"model": "Qwen3-14B shape", "layers": layers, "layers_of_named_config": MODEL_14B["num_hidden_layers"],
           "requests": B, "prompt_tokens_each": P, "portion": 2048, "new_tokens_each": NEW,
           "prefill_tokens_per_s": B * P / prefill_s, "prefill_s": prefill_s, "prefill_steps": prefill_steps,
           "prefill_frac_of_sustained": flops / prefill_s / (pk["bf16_tflops_sustained"] * 1e12),
           "decode_tokens_per_s": B * 1000.0 / ms, "decode_ms_per_step": ms, "decode_steps": len(decode_s),
           "decode_roofline_frac": nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"],
           "preemptions": llm.stats().preemptions, "python_gc_s": round(pauses.total, 4), "python_gc_runs": pauses.count,
           "through": "LLM.step() and the scheduler, host tokens in and out"}
    del llm
    release()
    return out


# ------------------------------------------------------------------------------------------------ 4B: a mixed batch
def run_4b(args, pk, clocks, windows):
    """32 requests, prompts of 128 to 4,096 tokens (seed 5), step budget 2,048 tokens, 128 new tokens each."""
    import numpy as np
    import torch
    from vllm_cpp_b200 import EngineConfig, LLM, Qwen3Config
    layers = args.layers_4b
    cfg = Qwen3Config(**dict(MODEL_4B, num_hidden_layers=layers))
    rng = np.random.default_rng(5)
    lens = rng.integers(128, 4097, 32).tolist()
    prompts = [rng.integers(0, cfg.vocab_size, n).tolist() for n in lens]
    total = sum(lens)
    NEW = 128
    max_tokens = -(-(total + 32 * (NEW + 64)) // 64) * 64
    llm = LLM(config=cfg, random_seed=0, engine=EngineConfig(dtype="bfloat16", page_size=PAGE, max_tokens=max_tokens,
                                                            max_num_seqs=32, max_step_tokens=2048, max_model_len=4096 + NEW + 128))
    warmed = llm.warm_up(0.0, 1.0, 1.0)       # the captured decoding steps are made before the clock starts, as at a server's start
    for p in prompts:
        llm.submit_tokens(p, NEW, 0.0, 1.0, repeat_penalty=1.0, ignore_eos=True)
    cache = llm.scheduler.cache()
    torch.cuda.synchronize()
    windows.append([clocks.mark(), None])
    t0 = time.perf_counter()
    steps = gen = mixed_steps = 0
    fewest_free = cache.free_pages(0)
    while llm.has_requests():
        o = llm.step()
        fewest_free = min(fewest_free, cache.free_pages(0))     # read after each step: the pool's high-water mark
        steps += 1
        gen += len(o.new_token_ids)
        mixed_steps += bool(o.num_prompt_tokens and o.num_generation_tokens)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    windows[-1][1] = clocks.mark()
    st = llm.stats()
    out = {"model": "Qwen3-4B shape", "layers": layers, "layers_of_named_config": MODEL_4B["num_hidden_layers"],
           "requests": 32, "prompt_tokens": total, "new_tokens_each": NEW, "step_token_budget": 2048,
           "total_tokens_per_s": (total + gen) / dt, "generated_tokens_per_s": gen / dt, "seconds": dt, "steps": steps,
           "steps_with_portions_beside_decoding": mixed_steps, "mean_step_ms": 1000 * dt / steps,
           "pages_high_water": max_tokens // PAGE - fewest_free, "pages_in_pool": max_tokens // PAGE, "preemptions": st.preemptions,
           "graph_replays": llm.runner.graph_replays, "decoding_steps_captured_before_the_clock": warmed,
           "through": "LLM.step() and the scheduler, host tokens in and out"}
    del llm
    release()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--layers", type=int, default=MODEL_8B["num_hidden_layers"])
    ap.add_argument("--layers-14b", type=int, default=MODEL_14B["num_hidden_layers"])
    ap.add_argument("--layers-4b", type=int, default=MODEL_4B["num_hidden_layers"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workloads", default="all", choices=["all", "headline", "14b", "4b"],
                    help="headline: the 8B numbers only; 14b / 4b: that workload alone (prints its own JSON line)")
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

    import torch
    pk = peaks()
    clocks = ClockSampler(gpu_id_for_nvidia_smi(torch))
    clocks.start()
    windows = []
    try:
        if args.workloads in ("14b", "4b"):
            out = (run_14b if args.workloads == "14b" else run_4b)(args, pk, clocks, windows)
            out["clocks"] = clocks.summary(windows)
            print(json.dumps(out))
            return 0
        line = run_headline(args, pk, clocks, windows)
        if line is None:
            return 0
        line["clocks"] = clocks.summary(windows)      # of the 8B runs; the other workloads carry their own
        if args.workloads == "all" and args.mode == "all" and not args.skip_points:
            extra = {}
            for key, fn in (("qwen3_14b_long_prompts", run_14b), ("qwen3_4b_mixed_batch", run_4b)):
                w = []
                try:
                    extra[key] = fn(args, pk, clocks, w)
                    extra[key]["clocks"] = clocks.summary(w)
                except Exception as e:   # the headline stands even if a further workload cannot run (memory, time)
                    extra[key] = {"error": f"{type(e).__name__}: {e}"[:300]}
                    release()
            line["workloads"] = extra
        print(json.dumps(line))
        return 0
    finally:
        clocks.stop()


if __name__ == "__main__":
    sys.exit(main())
