"""The Python entry point: load a model folder, submit token lists, step, collect tokens.

Names follow the reference's PagedEngine (src/paged_engine.h:24-47): ``submit_tokens``,
``step`` returning request ids / new token ids / finished flags and the two token
counts, ``get_request``, ``remove_request``, ``has_requests``; ``generate`` is the
loop of its cpu_runner (src/cpu_runner.cpp:85-114) for a list of prompts.  There
is no tokenizer: prompts are token ids, as with the runner's ``--tokens``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..config import EngineConfig
from ..models import build_model, expected_tensors, load_config
from ..runtime import runtime
from ..sampling import Sampler, SamplingOptions
from ..weights import RandomWeightStore, open_model_weights
from .step import ModelRunner, StepEntry

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}

# the reference's generation defaults (src/config.h:97-100)
TEMPERATURE, TOP_P, REPEAT_PENALTY, MAX_NEW_TOKENS = 0.7, 0.8, 1.1, 2048


@dataclass
class EngineOutput:
    request_ids: list = field(default_factory=list)
    new_token_ids: list = field(default_factory=list)
    finished: list = field(default_factory=list)
    num_prompt_tokens: int = 0
    num_generation_tokens: int = 0
    preempted: list = field(default_factory=list)


class EngineStats:
    """The scheduler's counters by attribute, plus the profile of the kernel groups when it is switched on."""

    def __init__(self, scheduler_stats, kernel_ms: dict, profiled_steps: int):
        self._scheduler = scheduler_stats
        self.kernel_ms = kernel_ms
        self.profiled_steps = profiled_steps

    def __getattr__(self, name):
        return getattr(self._scheduler, name)


class LLM:
    """One model on one GPU with its cache, scheduler and sampler."""

    def __init__(self, model=None, *, config=None, random_seed: int | None = None, engine: EngineConfig | None = None,
                 **engine_options):
        """``model``: a folder with config.json and *.safetensors.  Or ``config`` (a typed
        configuration) with ``random_seed``: random weights drawn on the device, no file."""
        self.engine_config = engine or EngineConfig(**engine_options)
        ec = self.engine_config
        if not torch.cuda.is_available():
            raise RuntimeError("vllm_cpp_b200 runs on a CUDA device (sm_100a); none is available")
        self.device = torch.device(ec.device)
        torch.cuda.set_device(self.device)
        dtype = TORCH_DTYPES[ec.dtype]
        if model is not None:
            self.config = load_config(model)
            store = open_model_weights(model, dtype, self.device)
        else:
            if config is None or random_seed is None:
                raise ValueError("give a model folder, or a configuration and random_seed")
            self.config = config
            store = RandomWeightStore(expected_tensors(config), random_seed, dtype, self.device)
        self.model = build_model(self.config, dtype, self.device)
        self.model.load(store)
        store.release()
        self.max_model_len = min(ec.max_model_len or self.model.spec.max_positions, self.model.spec.max_positions)
        self.runner = ModelRunner(self.model, ec.page_size, ec.num_pages, ec.max_num_seqs, dtype, self.device,
                                  cuda_graphs=ec.cuda_graphs, max_model_len=self.max_model_len,
                                  max_step_tokens=ec.max_step_tokens, profile=ec.profile)
        rt = runtime()
        self.scheduler = rt.Scheduler(self.runner.layout.runtime_groups(rt, ec.page_size, ec.num_pages),
                                      ec.max_num_seqs, ec.max_step_tokens, self.max_model_len)
        self.sampler = Sampler(self.model.spec.vocab_size, ec.max_num_seqs, self.device)
        self.default_stop_ids = list(self.model.spec.stop_ids)
        self._options: dict[int, SamplingOptions] = {}
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._pinned = None
        self.debug = False   # one structured line per step on standard error
        self._step_index = 0

    # ---- the reference's engine surface ----
    def submit_tokens(self, prompt_tokens, max_new_tokens: int = MAX_NEW_TOKENS, temperature: float = TEMPERATURE,
                      top_p: float = TOP_P, *, repeat_penalty: float = REPEAT_PENALTY, seed: int = 0,
                      stop_ids=None, ignore_eos: bool = False) -> int:
        rt = runtime()
        prompt = [int(t) for t in prompt_tokens]
        for t in prompt:
            if not 0 <= t < self.model.spec.vocab_size:
                raise ValueError(f"token id {t} is outside the vocabulary of {self.model.spec.vocab_size}")
        stops = [] if ignore_eos else list(self.default_stop_ids if stop_ids is None else stop_ids)
        opts = SamplingOptions(float(temperature), float(top_p), float(repeat_penalty), int(seed))
        rid = self.scheduler.submit(prompt, int(max_new_tokens),
                                    rt.SamplingParams(opts.temperature, opts.top_p, opts.repeat_penalty,
                                                      opts.seed & 0xFFFFFFFFFFFFFFFF), stops)
        self._options[rid] = opts
        return rid

    def has_requests(self) -> bool:
        return self.scheduler.has_unfinished()

    def get_request(self, request_id: int):
        return self.scheduler.request(request_id) if self.scheduler.knows(request_id) else None

    def remove_request(self, request_id: int) -> None:
        if self.scheduler.knows(request_id):
            self.scheduler.abort(request_id)
            self.scheduler.forget(request_id)
        self._options.pop(request_id, None)

    def step(self) -> EngineOutput:
        import time
        t0 = time.perf_counter()
        out = self._step()
        if self.debug:
            import sys
            c = self.scheduler.cache()
            free = [c.free_pages(g) for g in range(c.num_groups())]
            print(f"[step {self._step_index}] prompt_tokens={out.num_prompt_tokens} generation_tokens={out.num_generation_tokens} "
                  f"sampled={len(out.new_token_ids)} finished={sum(out.finished)} preempted={len(out.preempted)} "
                  f"waiting={self.scheduler.num_waiting()} running={self.scheduler.num_running()} free_pages={free} "
                  f"ms={(time.perf_counter() - t0) * 1e3:.2f}"
                  + ("".join(f" {k}_ms={v:.3f}" for k, v in sorted(self.runner.profile.items())) if self.runner.profile else ""),
                  file=sys.stderr, flush=True)
        self._step_index += 1
        return out

    def _step(self) -> EngineOutput:
        out = EngineOutput()
        sched = self.scheduler.schedule()
        out.preempted = list(sched.preempted)
        out.num_prompt_tokens, out.num_generation_tokens = sched.num_prompt_tokens, sched.num_generation_tokens
        if not sched.entries:
            return out
        cache = self.scheduler.cache()
        n_groups = cache.num_groups()
        entries, sampled_entries = [], []
        # single tokens first, then prompt portions (each kind in the scheduler's order): the order in which a
        # captured step of both takes them; the tokens go back to the scheduler in its own order
        ordered = sorted(sched.entries, key=lambda e: len(e.tokens) != 1)
        for e in ordered:
            tables = [cache.block_table(e.request, g) for g in range(n_groups)]
            n = len(e.tokens)
            entries.append(StepEntry(e.slot, e.start_pos, list(e.tokens), tables, [n - 1] if e.sample else []))
            if e.sample:
                sampled_entries.append(e)
        penalised = {e.slot for e in ordered if self._options[e.request].repeat_penalty not in (0.0, 1.0)}
        if penalised:
            self.sampler._need_counts()
            self.sampler.forget([e.slot for e in ordered if e.start_pos == 0 and e.slot in penalised])
        # Beside the model's own numbers the step carries 8 per sampled row and then, where occurrences are
        # counted, one per token (its request's slot + 1, 0 for none).  A captured step pads rows and tokens to
        # its own size, so the per-token part starts after the padded rows.
        flat, use_counts, no_nucleus = Sampler.records([self._options[e.request] for e in sampled_entries],
                                                       [e.gen_step for e in sampled_entries],
                                                       [e.slot for e in sampled_entries])
        n_rows = len(sampled_entries)
        rows_pad = self.runner.rows_capacity(entries)
        user = flat + [0] * (8 * (rows_pad - n_rows))
        if penalised:
            user += Sampler.token_slots(entries, penalised)
        counting = bool(penalised)
        toks = self.runner.step(entries, check=False, user=user, post=self._sampling_after(rows_pad, counting, use_counts, no_nucleus),
                                post_key=("sample", counting, use_counts, no_nucleus))
        tokens: list[int] = []
        if sampled_entries:
            host = self._readback(toks[:n_rows])
            if host[-1]:
                from .. import ops
                ops.check_status(self.runner.status)
            tokens = host[:-1]
        self.h2d_bytes += self.runner.last_h2d_bytes
        by_request = {e.request: t for e, t in zip(sampled_entries, tokens)}
        in_order = [e for e in sched.entries if e.sample]
        finished = set(self.scheduler.update([by_request[e.request] for e in in_order]))
        for e in in_order:
            out.request_ids.append(e.request)
            out.new_token_ids.append(by_request[e.request])
            out.finished.append(e.request in finished)
        return out

    def _sampling_after(self, rows_pad: int, counting: bool, use_counts: bool, no_nucleus: bool):
        """What a step runs on its own stream right after the model: the occurrence counts of the step's tokens where a
        request has a repetition penalty, then one sampled token per row of logits.  (A captured step includes it.)"""
        def post(ctx, logits):
            if counting:
                self.sampler.observe(ctx.token_ids, ctx.user[8 * rows_pad:8 * rows_pad + ctx.T], ctx.T)
            if logits is None:
                return None
            return self.sampler.sample_records(logits, ctx.user[:8 * logits.shape[0]].view(-1, 8), use_counts, no_nucleus)
        return post

    def warm_up(self, temperature: float = TEMPERATURE, top_p: float = TOP_P, repeat_penalty: float = REPEAT_PENALTY,
                batch_sizes=None) -> int:
        """Captures the decoding steps that requests with these sampling options will replay, before any request is
        there: one per padded batch size up to ``max_num_seqs`` (or those that ``batch_sizes`` round up to), for
        contexts of the short class.  Without it a run captures each such step when it first meets the size, 0.1 to
        0.2 s each at serving sizes, in the middle of serving.  Returns the number of steps captured now."""
        runner = self.runner
        if not runner.cuda_graphs:
            return 0
        options = SamplingOptions(temperature, top_p, repeat_penalty, 0)
        _, use_counts, no_nucleus = Sampler.records([options], [0], [0])
        counting = repeat_penalty not in (0.0, 1.0)
        if counting:
            self.sampler._need_counts()
        post_key = ("sample", counting, use_counts, no_nucleus)
        limit = next((b for b in runner.GRAPH_BUCKETS if b >= self.engine_config.max_num_seqs), runner.GRAPH_BUCKETS[-1])
        if batch_sizes is None:
            buckets = [b for b in runner.GRAPH_BUCKETS if b <= limit]
        else:
            buckets = sorted({next((b for b in runner.GRAPH_BUCKETS if b >= n), None) for n in batch_sizes} - {None})
        made = 0
        for bucket in buckets:
            key = (bucket, post_key, runner.GRAPH_CONTEXT_BOUNDS[0])
            if key not in runner._graphs and len(runner._graphs) < runner.MAX_GRAPHS:
                runner._capture(key, self._sampling_after(bucket, counting, use_counts, no_nucleus))
                made += 1
        return made

    def _readback(self, toks: torch.Tensor) -> list[int]:
        """The sampled tokens and the status word in one pinned buffer, one synchronisation."""
        n = toks.numel()
        if self._pinned is None or self._pinned.numel() < n + 1:
            self._pinned = torch.empty(max(n + 1, 257), dtype=torch.int32).pin_memory()
        self._pinned[:n].copy_(toks, non_blocking=True)
        self._pinned[n:n + 1].copy_(self.runner.status, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += (n + 1) * 4
        return self._pinned[:n + 1].tolist()

    # ---- convenience ----
    def generate(self, prompts, max_new_tokens: int = MAX_NEW_TOKENS, temperature: float = TEMPERATURE,
                 top_p: float = TOP_P, *, repeat_penalty: float = REPEAT_PENALTY, seed: int = 0, stop_ids=None,
                 ignore_eos: bool = False, on_token=None) -> list[list[int]]:
        """Generates for every prompt (a list of token ids each); request i samples with seed + i."""
        rids = [self.submit_tokens(p, max_new_tokens, temperature, top_p, repeat_penalty=repeat_penalty,
                                   seed=seed + i, stop_ids=stop_ids, ignore_eos=ignore_eos)
                for i, p in enumerate(prompts)]
        results = {r: [] for r in rids}
        while self.has_requests():
            o = self.step()
            for rid, tok in zip(o.request_ids, o.new_token_ids):
                if rid in results:
                    results[rid].append(tok)
                    if on_token:
                        on_token(rid, tok)
        for r in rids:
            self.scheduler.forget(r)
            self._options.pop(r, None)
        return [results[r] for r in rids]

    def stats(self):
        """The scheduler's counters (requests, tokens, steps, preemptions, ...) and, with ``EngineConfig(profile=True)``,
        ``kernel_ms``: milliseconds per group of kernels (embedding, mixer, feed_forward, head, sampling, tables),
        summed over ``profiled_steps`` steps."""
        return EngineStats(self.scheduler.stats(), dict(self.runner.profile or {}), self.runner.profile_steps)
