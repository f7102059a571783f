"""Generation through the Python entry point and the command line against the plain implementation:
greedy and seeded sampling, portions under a token budget, preemption by recompute, long decoding."""
import subprocess
import sys

import pytest

from conftest import ROOT, TINY_PAGE, random_tokens

pytestmark = pytest.mark.gpu


def make_llm(model_dir, name, dtype="float32", **kw):
    from vllm_cpp_b200 import LLM, EngineConfig
    opts = dict(dtype=dtype, page_size=TINY_PAGE[name], max_tokens=1024, max_num_seqs=4, max_step_tokens=16)
    opts.update(kw)
    return LLM(model_dir, engine=EngineConfig(**opts))


def plain_generate(plain_models, name, prompt, n, **kw):
    import plain_qwen3
    cfg, w = plain_models[name]
    return plain_qwen3.generate(cfg, w, prompt, n, **kw)


def test_greedy_config_a(model_dirs, plain_models):
    """3 requests with prompts of 5, 11 and 17 tokens, 8 greedy tokens each, pages of 4."""
    prompts = [random_tokens(256, n, 1 + i) for i, n in enumerate((5, 11, 17))]
    llm = make_llm(model_dirs["A"], "A")
    got = llm.generate(prompts, 8, 0.0, 1.0, repeat_penalty=1.0)
    assert got == [plain_generate(plain_models, "A", p, 8) for p in prompts]


def test_sampled_config_b(model_dirs, plain_models):
    """4 requests (1, 7, 33, 64 tokens), portions of 16 beside decoding, temperature 0.8 seed 4, 12 tokens."""
    prompts = [random_tokens(384, n, 3 + i) for i, n in enumerate((1, 7, 33, 64))]
    llm = make_llm(model_dirs["B"], "B")
    got = llm.generate(prompts, 12, 0.8, 1.0, repeat_penalty=1.0, seed=4)
    want = [plain_generate(plain_models, "B", p, 12, temperature=0.8, seed=4 + i) for i, p in enumerate(prompts)]
    assert got == want


def test_captured_steps_are_dropped_and_made_again(model_dirs, plain_models):
    """With room for two captured steps only, the steps of this run (lone portions, portions beside single tokens,
    one to four single tokens) push one another out and are captured again: the tokens stay those of the plain
    implementation."""
    prompts = [random_tokens(384, n, 3 + i) for i, n in enumerate((1, 7, 33, 64))]
    llm = make_llm(model_dirs["B"], "B")
    llm.runner.MAX_GRAPHS = 2
    got = llm.generate(prompts, 12, 0.8, 1.0, repeat_penalty=1.0, seed=4)
    got += llm.generate(prompts[:1], 5, 0.0, 1.0, repeat_penalty=1.0)
    want = [plain_generate(plain_models, "B", p, 12, temperature=0.8, seed=4 + i) for i, p in enumerate(prompts)]
    want.append(plain_generate(plain_models, "B", prompts[0], 5))
    assert got == want
    assert len(llm.runner._graphs) <= 2 and llm.runner.graph_replays > 10


@pytest.mark.parametrize("name", ["B", "C"])
def test_captured_and_kernel_by_kernel_steps_give_the_same_tokens(name, model_dirs):
    """Forty requests arriving a few at a time, sampled with the reference's defaults (temperature, nucleus,
    repetition penalty), in a pool so small that requests are preempted: in 32-bit the tokens do not depend on
    whether steps replay captured graphs (padded, slots left empty) or run kernel by kernel."""
    import numpy as np
    from conftest import TINY
    vocab = TINY[name]["vocab_size"]
    streams = []
    for graphs in (True, False):
        llm = make_llm(model_dirs[name], name, cuda_graphs=graphs, max_tokens=320, max_num_seqs=6, max_step_tokens=48)
        rng = np.random.default_rng(11)
        pending = [random_tokens(vocab, int(n), 500 + i) for i, n in enumerate(rng.integers(1, 90, 40))]
        ids, out, steps = [], {}, 0
        while pending or llm.has_requests():
            if pending and steps % 3 == 0:
                for _ in range(min(int(rng.integers(1, 4)), len(pending))):
                    ids.append(llm.submit_tokens(pending.pop(), int(rng.integers(1, 24)), seed=len(ids), ignore_eos=True))
            o = llm.step()
            steps += 1
            for rid, tok in zip(o.request_ids, o.new_token_ids):
                out.setdefault(rid, []).append(tok)
        streams.append([out[r] for r in ids])
        if graphs:
            assert llm.runner.graph_replays > steps // 2
            kinds = {k[0] if isinstance(k[0], str) else "single tokens" for k in llm.runner._graphs}
            assert kinds == {"single tokens", "portion", "mixed"}, kinds
        assert llm.stats().preemptions > 0
    assert streams[0] == streams[1]


def test_reference_defaults_top_p_and_penalty(model_dirs, plain_models):
    """The reference's own defaults: temperature 0.7, top-p 0.8, repetition penalty 1.1 over prompt + output."""
    prompts = [random_tokens(256, n, 20 + i) for i, n in enumerate((9, 30))]
    llm = make_llm(model_dirs["A"], "A")
    got = llm.generate(prompts, 10, seed=11)
    want = [plain_generate(plain_models, "A", p, 10, temperature=0.7, top_p=0.8, repeat_penalty=1.1, seed=11 + i)
            for i, p in enumerate(prompts)]
    assert got == want


def test_bfloat16_greedy_mostly_agrees(model_dirs, plain_models):
    prompts = [random_tokens(384, n, 40 + i) for i, n in enumerate((12, 50, 100))]
    llm = make_llm(model_dirs["B"], "B", dtype="bfloat16")
    got = llm.generate(prompts, 16, 0.0, 1.0, repeat_penalty=1.0)
    want = [plain_generate(plain_models, "B", p, 16) for p in prompts]
    first = sum(g[0] == w[0] for g, w in zip(got, want))
    agree = sum(a == b for g, w in zip(got, want) for a, b in zip(g, w))
    assert first == 3 and agree >= 36, (got, want)


@pytest.mark.parametrize("name", ["C", "D"])
def test_bfloat16_generation_on_the_tensor_core_kernels(name, model_dirs, plain_models):
    """Six requests on the configurations with head sizes 64 and 128 in bfloat16: prompt portions of 64 tokens
    through the tcgen05 attention kernel beside decoded tokens through the mma.sync one, captured steps.  Greedy
    tokens of a bfloat16 engine may leave the plain implementation's at a near tie, so each chosen token is judged
    where it was chosen: the plain implementation's logits over the engine's own sequence must hold that token
    within the bfloat16 tolerance of their largest, and most tokens must be the plain implementation's choice."""
    import plain_qwen3
    cfg, w = plain_models[name]
    vocab, top = cfg["vocab_size"], cfg["max_position_embeddings"]
    lengths = (3, 40, 64, 97, 130, 150)
    prompts = [random_tokens(vocab, n, 500 + i) for i, n in enumerate(lengths)]
    llm = make_llm(model_dirs[name], name, dtype="bfloat16", max_tokens=2048, max_num_seqs=6, max_step_tokens=64)
    got = llm.generate(prompts, 24, 0.0, 1.0, repeat_penalty=1.0, ignore_eos=True)
    assert llm.runner.graph_replays > 20
    same = total = 0
    for p, g in zip(prompts, got):
        assert len(g) == 24 and len(p) + 24 <= top
        logits = plain_qwen3.forward(cfg, w, p + g[:-1])[len(p) - 1:]
        assert logits.shape[0] == 24
        scale = float(logits.abs().max())
        for t, tok in enumerate(g):
            best = float(logits[t].max())
            assert float(logits[t, tok]) >= best - 3e-2 * scale, (len(p), t, tok, int(logits[t].argmax()))
            same += int(logits[t].argmax()) == tok
            total += 1
    assert same >= 0.9 * total, (same, total)


def test_preemption_recomputes_to_the_same_tokens(model_dirs, plain_models):
    """A pool too small for all requests at their full length: the youngest is preempted, recomputed
    later, and every request still produces the tokens it produces alone."""
    prompts = [random_tokens(256, n, 60 + i) for i, n in enumerate((30, 28, 26, 20))]
    llm = make_llm(model_dirs["A"], "A", max_tokens=128, max_step_tokens=32)
    got = llm.generate(prompts, 24, 0.9, 1.0, repeat_penalty=1.0, seed=3)
    assert llm.stats().preemptions > 0
    want = [plain_generate(plain_models, "A", p, 24, temperature=0.9, seed=3 + i) for i, p in enumerate(prompts)]
    assert got == want
    cache = llm.scheduler.cache()
    cache.check_invariants()
    assert cache.free_pages(0) == 128 // TINY_PAGE["A"] and cache.free_slots() == 4


def test_long_decoding_and_stop(model_dirs, plain_models):
    """One request decoding up to the model's last position; then one that stops on a stop id."""
    prompt = random_tokens(384, 3, 77)
    llm = make_llm(model_dirs["B"], "B")
    got = llm.generate([prompt], 253, 0.0, 1.0, repeat_penalty=1.0)[0]
    want = plain_generate(plain_models, "B", prompt, 253)
    assert len(got) == 253 and got == want
    stop = want[5]
    first = want.index(stop)
    got2 = llm.generate([prompt], 50, 0.0, 1.0, repeat_penalty=1.0, stop_ids=[stop])[0]
    assert got2 == want[:first + 1]


def test_engine_surface(model_dirs):
    """submit_tokens / step / get_request / remove_request / has_requests, as the reference's engine has them."""
    llm = make_llm(model_dirs["A"], "A")
    rid = llm.submit_tokens([1, 2, 3], 4, 0.0, 1.0, repeat_penalty=1.0)
    assert llm.has_requests()
    out = llm.step()
    assert out.request_ids == [rid] and len(out.new_token_ids) == 1 and out.num_prompt_tokens == 3
    assert llm.get_request(rid).generated == out.new_token_ids
    llm.remove_request(rid)
    assert not llm.has_requests() and llm.get_request(rid) is None
    with pytest.raises(ValueError):
        llm.submit_tokens([], 4)
    with pytest.raises(ValueError):
        llm.submit_tokens([999], 4)
    with pytest.raises(ValueError):
        llm.submit_tokens([1] * 120, 20)   # beyond the model's 128 positions


def test_command_line(model_dirs, plain_models):
    prompt = random_tokens(256, 6, 5)
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "vllm_cpp_run"), str(model_dirs["A"]), "--tokens",
                        ",".join(map(str, prompt)), "--max-new", "5", "--temp", "0", "--top-p", "1", "--repeat-penalty", "1",
                        "--dtype", "float32", "--page-size", "4", "--max-tokens", "256", "--debug"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    got = [int(t) for t in r.stdout.strip().splitlines()[-1].split(",")]
    assert got == plain_generate(plain_models, "A", prompt, 5)


def test_sizes_that_fit_no_fast_path(tmp_path, plain_models):
    """Hidden size 100 (rows no multiple of 16 bytes), head_dim 48, 5 heads over 1 KV head, odd vocabulary:
    both precisions still run, through the plain kernels where the tensor-core ones cannot."""
    import plain_qwen3
    from vllm_cpp_b200 import LLM, EngineConfig, Qwen3Config, write_random_model
    cfg = Qwen3Config(vocab_size=211, hidden_size=100, intermediate_size=108, num_hidden_layers=2, num_attention_heads=5,
                      num_key_value_heads=1, head_dim=48, max_position_embeddings=96, rms_norm_eps=1e-5, rope_theta=5e4,
                      tie_word_embeddings=False)
    d = write_random_model(cfg, 9, tmp_path / "odd")
    pc, pw = plain_qwen3.read_model(d)
    prompts = [random_tokens(211, n, 90 + n) for n in (3, 20, 41)]
    want = [plain_qwen3.generate(pc, pw, p, 10) for p in prompts]
    llm = LLM(d, engine=EngineConfig(dtype="float32", page_size=8, max_tokens=512, max_num_seqs=4, max_step_tokens=16))
    assert llm.generate(prompts, 10, 0.0, 1.0, repeat_penalty=1.0) == want
    llm = LLM(d, engine=EngineConfig(dtype="bfloat16", page_size=8, max_tokens=512, max_num_seqs=4, max_step_tokens=16))
    got = llm.generate(prompts, 10, 0.0, 1.0, repeat_penalty=1.0)
    assert sum(a == b for g, w in zip(got, want) for a, b in zip(g, w)) >= 24


def test_host_running_ahead_of_the_gpu_does_not_mix_up_steps(model_dirs, plain_models):
    """A prompt cut into many portions samples nothing until its last portion, so nothing makes the host wait for
    the GPU between those steps: with the GPU held back (a bounded sleep kernel in front of every step) the host
    fills the buffers of several steps before the first of them has been copied.  Each step must still get its own
    tokens, positions and cache slots."""
    import torch
    prompts = [random_tokens(384, 150, 91), random_tokens(384, 97, 92)]
    want = [plain_generate(plain_models, "B", p, 4) for p in prompts]
    for graphs in (True, False):
        llm = make_llm(model_dirs["B"], "B", cuda_graphs=graphs, max_step_tokens=16, max_num_seqs=1)
        inner = llm.runner.step

        def lagging_step(*a, **kw):
            torch.cuda._sleep(30_000_000)      # some 15 ms during which the host goes on to the next steps
            return inner(*a, **kw)

        llm.runner.step = lagging_step
        got = llm.generate(prompts, 4, 0.0, 1.0, repeat_penalty=1.0)
        assert got == want, f"captured steps {graphs}"
        if graphs:
            assert llm.runner.graph_replays >= 150 // 16 + 97 // 16


def test_many_live_requests_through_the_large_captured_steps(model_dirs, plain_models):
    """More than 130 requests decoding at once: the captured steps of 128 and 256 single tokens, and the captured
    mixed step with 64 single-token slots (forty requests decoding beside a newcomer's prompt), against the plain
    implementation's greedy tokens, in 32-bit."""
    first = [random_tokens(256, 3 + i % 7, 300 + i) for i in range(40)]
    late = [random_tokens(256, 2 + i % 9, 700 + i) for i in range(101)]
    llm = make_llm(model_dirs["A"], "A", max_tokens=8192, max_num_seqs=256, max_step_tokens=256)
    out = {}

    def step():
        o = llm.step()
        for rid, tok in zip(o.request_ids, o.new_token_ids):
            out.setdefault(rid, []).append(tok)

    ids = [llm.submit_tokens(p, 20, 0.0, 1.0, repeat_penalty=1.0, ignore_eos=True) for p in first]
    while llm.scheduler.num_waiting() or len(out) < 40:
        step()                                    # all forty are decoding now
    ids.append(llm.submit_tokens(late[0], 9, 0.0, 1.0, repeat_penalty=1.0, ignore_eos=True))
    step()                                        # forty single tokens beside one portion
    assert any(k[0] == "mixed" and k[1] == 64 for k in llm.runner._graphs), list(llm.runner._graphs)
    ids += [llm.submit_tokens(p, 5 + i % 5, 0.0, 1.0, repeat_penalty=1.0, ignore_eos=True) for i, p in enumerate(late[1:])]
    most = 0
    while llm.has_requests():
        most = max(most, llm.scheduler.num_running())
        step()
    assert most > 130
    buckets = {k[0] for k in llm.runner._graphs if not isinstance(k[0], str)}
    assert {128, 256} <= buckets, buckets
    new = [20] * 40 + [9] + [5 + i % 5 for i in range(100)]
    for rid, p, n in zip(ids, first + late, new):
        assert out[rid] == plain_generate(plain_models, "A", p, n), f"request {rid}"


def test_steps_take_their_buffers_from_the_workspace(model_dirs):
    """Kernel by kernel, a step asks the device allocator for nothing once the scratch memory has its size: fifty
    mixed steps (portions beside single tokens, requests coming and going), the allocator's count of allocations
    unchanged from the tenth step on."""
    import numpy as np
    import torch
    llm = make_llm(model_dirs["C"], "C", dtype="bfloat16", cuda_graphs=False, max_tokens=2048, max_num_seqs=6, max_step_tokens=48)
    rng = np.random.default_rng(5)
    steps, counts, overflows = 0, [], []
    pending = [random_tokens(320, int(n), 900 + i) for i, n in enumerate(rng.integers(2, 120, 30))]
    while steps < 50:
        if pending and steps % 2 == 0:
            llm.submit_tokens(pending.pop(), int(rng.integers(4, 30)), seed=steps, ignore_eos=True)
        llm.step()
        steps += 1
        counts.append(torch.cuda.memory_stats()["allocation.all.allocated"])
        overflows.append(llm.runner.workspace.overflows)     # requests the scratch could not serve (torch.empty did)
    assert llm.runner.graph_replays == 0
    assert counts[49] == counts[9], (counts[9], counts[49], overflows[9], overflows[49])
    assert overflows[49] == overflows[9]


def test_profile_of_kernel_groups(model_dirs, plain_models):
    """EngineConfig(profile=True): the same tokens, every step kernel by kernel, and the time of each group of
    kernels (embedding, each layer's mixer and feed-forward, head, sampling) summed in the engine's statistics."""
    prompts = [random_tokens(384, n, 40 + i) for i, n in enumerate((12, 50))]
    llm = make_llm(model_dirs["B"], "B", profile=True)
    got = llm.generate(prompts, 6, 0.0, 1.0, repeat_penalty=1.0)
    assert got == [plain_generate(plain_models, "B", p, 6) for p in prompts]
    st = llm.stats()
    assert llm.runner.graph_replays == 0 and 0 < st.profiled_steps <= st.steps
    assert {"embedding", "mixer", "feed_forward", "head", "sampling", "tables"} <= set(st.kernel_ms)
    assert all(v > 0 for v in st.kernel_ms.values())
    assert st.preemptions == 0                       # the scheduler's own counters are still there
    assert make_llm(model_dirs["B"], "B").stats().kernel_ms == {}


def test_nothing_is_finalised_while_a_step_is_captured(model_dirs, plain_models):
    """An engine that is dropped leaves captured graphs behind, in reference cycles that only the collector frees;
    destroying one while another capture is open makes that capture invalid.  So the runner keeps the collector off
    until a capture is closed: seen here from inside the model's forward pass, with a dropped engine's graphs as the
    garbage and a collector set to run at every opportunity."""
    import gc
    import weakref

    import torch
    prompts = [random_tokens(256, n, 1 + i) for i, n in enumerate((5, 11, 17))]
    old = make_llm(model_dirs["A"], "A")
    old.generate(prompts, 4, 0.0, 1.0, repeat_penalty=1.0)
    assert len(old.runner._graphs) > 0
    ring = [old]
    ring.append(ring)                      # garbage that reference counting alone does not free

    llm = make_llm(model_dirs["A"], "A")
    seen = []
    forward = llm.runner.model.forward

    def watched(ctx, views):
        if torch.cuda.is_current_stream_capturing():
            seen.append(gc.isenabled())
            _ = [[i] for i in range(2000)]   # container allocations: what sets an enabled collector off
        return forward(ctx, views)

    llm.runner.model.forward = watched
    gone = weakref.ref(old.runner)
    del old, ring
    thresholds = gc.get_threshold()
    gc.set_threshold(1, 1, 1)
    try:
        assert gc.isenabled()
        got = llm.generate(prompts, 8, 0.0, 1.0, repeat_penalty=1.0)
    finally:
        gc.set_threshold(*thresholds)
    assert seen and not any(seen)
    assert gc.isenabled()
    gc.collect()
    assert gone() is None
    assert got == [plain_generate(plain_models, "A", p, 8) for p in prompts]


def test_warm_up_captures_the_decoding_steps_beforehand(model_dirs, plain_models):
    """LLM.warm_up captures the decoding steps of every padded batch size up to max_num_seqs for the given sampling
    options; the run after it captures none of them again and gives the plain implementation's tokens."""
    prompts = [random_tokens(256, n, 1 + i) for i, n in enumerate((5, 11, 17))]
    llm = make_llm(model_dirs["A"], "A")
    made = llm.warm_up(0.0, 1.0, 1.0)
    assert made == 3 and llm.warm_up(0.0, 1.0, 1.0) == 0            # batch sizes 1, 2, 4 for max_num_seqs 4
    decoding = {k for k in llm.runner._graphs if isinstance(k[0], int)}
    assert {k[0] for k in decoding} == {1, 2, 4}
    got = llm.generate(prompts, 8, 0.0, 1.0, repeat_penalty=1.0)
    assert {k for k in llm.runner._graphs if isinstance(k[0], int)} == decoding     # replayed, none made anew
    assert got == [plain_generate(plain_models, "A", p, 8) for p in prompts]
    # other sampling options are other steps; batch sizes can be named
    assert llm.warm_up(0.8, 0.9, 1.1, batch_sizes=[3]) == 1
