"""The serving kernels at the layer sizes of the benchmark model (Qwen3-8B shape: hidden 4096, 32/8 heads of 128,
intermediate 12288, vocabulary 151936; two layers to keep it short) against the engine's own true-32-bit path,
whose kernels the other tests tie to the plain implementation at small sizes.  Same random weights, a prompt fed
in portions, then decoding through captured steps."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bf16_engine_follows_the_32_bit_engine_at_8b_layer_sizes():
    from vllm_cpp_b200 import LLM, EngineConfig, Qwen3Config
    from vllm_cpp_b200.engine.step import StepEntry
    from vllm_cpp_b200.runtime import runtime
    cfg = Qwen3Config(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=2,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=4096,
                      rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
    rng = np.random.default_rng(0)
    tokens = {0: rng.integers(0, cfg.vocab_size, 1000).tolist(), 1: rng.integers(0, cfg.vocab_size, 150).tolist()}
    # portions: a long one (fused feed-forward path, 256-token tiles), short ones (k-sliced products), then single tokens
    # and portions of one request alone, which run as captured steps padded to 16, 256, 64 and 256 tokens
    plan = ([[(0, 300), (1, 17)], [(0, 300), (1, 100)], [(0, 90), (1, 25)]] + [[(0, 1), (1, 1)]] * 8
            + [[(0, 2)], [(0, 130)], [(0, 33)], [(0, 137)]])
    rows = {}
    for dtype in ("float32", "bfloat16"):
        llm = LLM(config=cfg, random_seed=1, engine=EngineConfig(dtype=dtype, page_size=16, max_tokens=2048, max_num_seqs=2,
                                                                 max_step_tokens=512))
        runner = llm.runner
        rt = runtime()
        cm = rt.CacheManager(runner.layout.runtime_groups(rt, 16, 128), 2)
        pos = {0: 0, 1: 0}
        for r in pos:
            cm.open(r)
        got = []
        for step in plan:
            entries = []
            for r, n in step:
                assert cm.reserve(r, pos[r] + n)
                entries.append(StepEntry(cm.slot(r), pos[r], tokens[r][pos[r]:pos[r] + n], [cm.block_table(r, 0)], [n - 1]))
                pos[r] += n
            got.append(runner.step(entries).float().cpu().clone())
            for r, _ in step:
                cm.commit(r, pos[r])
        rows[dtype] = torch.cat(got)
        if dtype == "bfloat16":
            # all but the first two steps (317 and 400 tokens side by side: too many for a captured mixed step) ran
            # from captured graphs: portions side by side, single tokens, lone portions
            assert runner.graph_replays == len(plan) - 2
        del llm, runner
        torch.cuda.empty_cache()
    ref, got = rows["float32"], rows["bfloat16"]
    err = ((got - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max().item()
    assert err < 3e-2, err
    assert (got.argmax(dim=1) == ref.argmax(dim=1)).float().mean().item() >= 0.8


@pytest.mark.parametrize("page_size,window,hd,nh,nkv,hidden,inter", [
    (8, 0, 128, 32, 8, 4096, 12288),          # eight pages a key tile
    (64, 256, 128, 32, 8, 4096, 12288),       # one page a key tile, a windowed layer before a full one
    (16, 100, 64, 14, 2, 896, 4864),          # head_dim 64, seven query heads a KV head, sizes that are no power of two
    (4, 0, 128, 16, 2, 2048, 6144),           # pages too small for TMA boxes: the cp.async loaders
    (16, 0, 128, 40, 8, 5120, 17408),         # the 14B shape: five query heads a KV head, 136 feature tiles of 128
    (16, 0, 128, 32, 8, 2560, 9728),          # the 4B shape: heads x head_dim wider than the hidden size
])
def test_bf16_engine_follows_the_32_bit_engine_at_other_serving_sizes(page_size, window, hd, nh, nkv, hidden, inter):
    """Two requests fed in large and small portions, then decoded, in bfloat16 against the true-32-bit engine: other
    page sizes, group sizes and head sizes than the benchmark model's, with and without a window."""
    from vllm_cpp_b200 import LLM, EngineConfig, Qwen3Config
    from vllm_cpp_b200.engine.step import StepEntry
    from vllm_cpp_b200.runtime import runtime
    kw = dict(sliding_window=window, layer_types=("sliding_attention", "full_attention")) if window else {}
    cfg = Qwen3Config(vocab_size=32000, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=2,
                      num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, max_position_embeddings=4096,
                      rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False, **kw)
    rng = np.random.default_rng(0)
    tokens = {0: rng.integers(0, cfg.vocab_size, 900).tolist(), 1: rng.integers(0, cfg.vocab_size, 200).tolist()}
    plan = [[(0, 300), (1, 17)], [(0, 500), (1, 100)], [(0, 90), (1, 60)]] + [[(0, 1), (1, 1)]] * 6 + [[(0, 4)]]
    rows = {}
    for dtype in ("float32", "bfloat16"):
        llm = LLM(config=cfg, random_seed=1, engine=EngineConfig(dtype=dtype, page_size=page_size, max_tokens=2048,
                                                                 max_num_seqs=2, max_step_tokens=1024))
        runner = llm.runner
        rt = runtime()
        cm = rt.CacheManager(runner.layout.runtime_groups(rt, page_size, 2048 // page_size), 2)
        pos = {0: 0, 1: 0}
        for r in pos:
            cm.open(r)
        got = []
        for step in plan:
            entries = []
            for r, n in step:
                assert cm.reserve(r, pos[r] + n)
                tables = [cm.block_table(r, g) for g in range(len(runner.layout.groups))]
                entries.append(StepEntry(cm.slot(r), pos[r], tokens[r][pos[r]:pos[r] + n], tables, [n - 1]))
                pos[r] += n
            got.append(runner.step(entries).float().cpu().clone())
            for r, _ in step:
                cm.commit(r, pos[r])
        rows[dtype] = torch.cat(got)
        del llm, runner
        torch.cuda.empty_cache()
    ref, got = rows["float32"], rows["bfloat16"]
    err = ((got - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max().item()
    assert err < 3e-2, err
    assert (got.argmax(dim=1) == ref.argmax(dim=1)).float().mean().item() >= 0.8


def test_long_context_decoding_at_8b_layer_sizes():
    """A prompt of 12,000 tokens in portions of 2,048, then single tokens at a context beyond the 8,192 of the first
    class of captured steps (other key slicing, other graph), in bfloat16 against the true-32-bit engine."""
    from vllm_cpp_b200 import LLM, EngineConfig, Qwen3Config
    from vllm_cpp_b200.engine.step import StepEntry
    from vllm_cpp_b200.runtime import runtime
    cfg = Qwen3Config(vocab_size=32000, hidden_size=4096, intermediate_size=12288, num_hidden_layers=2,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=16384,
                      rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
    rng = np.random.default_rng(3)
    n_prompt, n_decode = 12000, 5
    tokens = rng.integers(0, cfg.vocab_size, n_prompt + n_decode).tolist()
    rows = {}
    for dtype in ("float32", "bfloat16"):
        llm = LLM(config=cfg, random_seed=2, engine=EngineConfig(dtype=dtype, page_size=16, max_tokens=12288, max_num_seqs=1,
                                                                 max_step_tokens=2048, max_model_len=16384))
        runner = llm.runner
        rt = runtime()
        cm = rt.CacheManager(runner.layout.runtime_groups(rt, 16, 12288 // 16), 1)
        cm.open(0)
        got, pos = [], 0
        steps = [2048] * (n_prompt // 2048) + [n_prompt % 2048] + [1] * n_decode
        for n in steps:
            assert cm.reserve(0, pos + n)
            out = runner.step([StepEntry(cm.slot(0), pos, tokens[pos:pos + n], [cm.block_table(0, 0)], [n - 1])])
            got.append(out.float().cpu().clone())
            pos += n
            cm.commit(0, pos)
        rows[dtype] = torch.cat(got)
        if dtype == "bfloat16":
            assert runner.graph_replays >= n_decode
        del llm, runner
        torch.cuda.empty_cache()
    ref, got = rows["float32"], rows["bfloat16"]
    err = ((got - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max().item()
    assert err < 3e-2, err


def test_single_tokens_beside_portions_at_8b_layer_sizes():
    """Twelve requests decoding beside the prompt portions of newcomers, the kind of step that is captured with slots
    for single tokens and for portions, in bfloat16 against the true-32-bit engine."""
    from vllm_cpp_b200 import LLM, EngineConfig, Qwen3Config
    from vllm_cpp_b200.engine.step import StepEntry
    from vllm_cpp_b200.runtime import runtime
    cfg = Qwen3Config(vocab_size=32000, hidden_size=4096, intermediate_size=12288, num_hidden_layers=2,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=4096,
                      rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
    rng = np.random.default_rng(4)
    lengths = [int(n) for n in rng.integers(40, 700, 12)] + [190, 130]
    tokens = [rng.integers(0, cfg.vocab_size, n + 8).tolist() for n in lengths]
    rows = {}
    for dtype in ("float32", "bfloat16"):
        llm = LLM(config=cfg, random_seed=3, engine=EngineConfig(dtype=dtype, page_size=16, max_tokens=8192, max_num_seqs=14,
                                                                 max_step_tokens=1024))
        runner = llm.runner
        rt = runtime()
        cm = rt.CacheManager(runner.layout.runtime_groups(rt, 16, 512), 14)
        pos = [0] * 14
        for r in range(14):
            cm.open(r)

        def entry(r, n):
            assert cm.reserve(r, pos[r] + n)
            e = StepEntry(cm.slot(r), pos[r], tokens[r][pos[r]:pos[r] + n], [cm.block_table(r, 0)], [n - 1])
            pos[r] += n
            return e

        def run(entries):
            out = runner.step(entries).float().cpu().clone()
            for r in range(14):
                cm.commit(r, pos[r])
            return out

        got = [run([entry(r, lengths[r])]) for r in range(12)]                    # the twelve prompts, one at a time
        got.append(run([entry(r, 1) for r in range(12)] + [entry(12, 100)]))          # single tokens beside one portion
        got.append(run([entry(r, 1) for r in range(12)] + [entry(12, 90), entry(13, 70)]))   # beside two
        got.append(run([entry(r, 1) for r in range(5)] + [entry(13, 60)]))            # fewer single tokens: a smaller step
        got.append(run([entry(r, 1) for r in range(14)]))                             # all fourteen decode
        rows[dtype] = torch.cat(got)
        if dtype == "bfloat16":
            # two captured kinds of mixed step served the three: 32 single-token slots in 192 rows (twice), 8 in 96
            assert sorted(k[1:3] for k in runner._graphs if k[0] == "mixed") == [(8, 96), (32, 192)]
        del llm, runner
        torch.cuda.empty_cache()
    ref, got = rows["float32"], rows["bfloat16"]
    err = ((got - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)).max().item()
    assert err < 3e-2, err
    assert (got.argmax(dim=1) == ref.argmax(dim=1)).float().mean().item() >= 0.8
