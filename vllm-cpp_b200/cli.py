"""Command line in the manner of the reference's cpu_runner (src/cpu_runner.cpp:9-26, 51-64):

    vllm_cpp_run <model_path> --tokens IDs [--tokens IDs ...] [--max-new N] [--temp T] [--top-p P]
                 [--paged] [--max-batch N] [--max-tokens N] [--debug]

Same option names, meanings and defaults (max-new 2048, temp 0.7, top-p 0.8, max-batch 4,
max-tokens 8192 as in its code, :48).  There is no tokenizer here, so input is raw token ids
(``--tokens``, comma-separated, repeatable: one request each) and output is token ids.
``--paged`` is accepted for compatibility: the paged engine is the only engine.  Added options:
``--repeat-penalty`` (the reference's fixed 1.1), ``--seed``, ``--dtype``, ``--page-size``,
``--max-step-tokens``, ``--stop-id``, ``--ignore-eos``, and ``--random CONFIG.json --random-seed S``
to write a folder of random weights into <model_path> first.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def parse_token_ids(text: str) -> list[int]:
    return [int(t) for t in text.split(",") if t.strip()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="vllm_cpp_run", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model_path", help="model directory (config.json and .safetensors files)")
    ap.add_argument("prompt", nargs="?", default=None, help="text prompts need a tokenizer, which this engine has not")
    ap.add_argument("--tokens", action="append", default=[], metavar="IDs", help="input as raw token ids (comma-separated)")
    ap.add_argument("--max-new", type=int, default=2048, metavar="N", help="max new tokens (default: 2048)")
    ap.add_argument("--temp", type=float, default=0.7, metavar="T", help="temperature (default: 0.7; <= 0 is greedy)")
    ap.add_argument("--top-p", type=float, default=0.8, metavar="P", help="top-p (default: 0.8)")
    ap.add_argument("--paged", action="store_true", help="use the paged engine (always on)")
    ap.add_argument("--max-batch", type=int, default=4, metavar="N", help="max concurrent requests (default: 4)")
    ap.add_argument("--max-tokens", type=int, default=8192, metavar="N", help="tokens the cache pool holds (default: 8192)")
    ap.add_argument("--debug", action="store_true", help="print id and time per token")
    ap.add_argument("--repeat-penalty", type=float, default=1.1)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-step-tokens", type=int, default=2048)
    ap.add_argument("--stop-id", type=int, action="append", default=None)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--profile", action="store_true",
                    help="time the groups of kernels of every step (steps then run kernel by kernel); printed at the end, and per step with --debug")
    ap.add_argument("--random", metavar="CONFIG.json", default=None,
                    help="write random weights for this configuration into <model_path> first")
    ap.add_argument("--random-seed", type=int, default=0)
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.prompt is not None:
        print("error: a text prompt needs a tokenizer; give token ids with --tokens", file=sys.stderr)
        return 1
    if not args.tokens:
        print("error: no input; give token ids with --tokens IDs", file=sys.stderr)
        return 1
    prompts = [parse_token_ids(t) for t in args.tokens]

    from . import EngineConfig, LLM
    if args.random:
        from .models import qwen3  # noqa: F401
        from .registry import architecture_of
        from .weights import write_random_model
        data = json.loads(open(args.random).read())
        write_random_model(architecture_of(data).config_cls.from_dict(data), args.random_seed, args.model_path)

    print("=== vllm_cpp_b200 runner ===", file=sys.stderr)
    t0 = time.time()
    max_tokens = -(-args.max_tokens // args.page_size) * args.page_size
    llm = LLM(args.model_path, engine=EngineConfig(dtype=args.dtype, page_size=args.page_size, max_tokens=max_tokens,
                                                   max_num_seqs=args.max_batch, max_step_tokens=args.max_step_tokens,
                                                   profile=args.profile))
    llm.debug = args.debug
    print(f"Model loaded in {int((time.time() - t0) * 1000)} ms", file=sys.stderr)
    for i, p in enumerate(prompts):
        print(f"Input tokens (raw) [{i}]: {len(p)} tokens", file=sys.stderr)

    last = [time.time()]
    count = [0]

    def on_token(rid, tok):
        count[0] += 1
        if args.debug:
            now = time.time()
            print(f"  Token {count[0]}: request={rid} id={tok} time={int((now - last[0]) * 1000)}ms", file=sys.stderr)
            last[0] = now

    t0 = time.time()
    outs = llm.generate(prompts, args.max_new, args.temp, args.top_p, repeat_penalty=args.repeat_penalty,
                        seed=args.seed, stop_ids=args.stop_id, ignore_eos=args.ignore_eos, on_token=on_token)
    dt = time.time() - t0
    for o in outs:
        print(",".join(str(t) for t in o))
    n = sum(len(o) for o in outs)
    print(f"\n--- Generation complete ---\nTokens generated: {n}\nTotal time: {int(dt * 1000)} ms", file=sys.stderr)
    if n:
        print(f"Speed: {dt * 1000 / n:.2f} ms/token", file=sys.stderr)
    st = llm.stats()
    if st.kernel_ms:
        total = sum(st.kernel_ms.values())
        print(f"Kernel groups over {st.profiled_steps} steps ({total:.1f} ms on the device):", file=sys.stderr)
        for k, v in sorted(st.kernel_ms.items(), key=lambda kv: -kv[1]):
            print(f"  {k:14s} {v:10.2f} ms  {100 * v / total:5.1f} %", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
