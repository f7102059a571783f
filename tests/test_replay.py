"""bin/trace_run against the plain implementation: the same requests whole, with the last 32
tokens one by one, in portions of changing size down to two tokens (all logits wanted, or the last one's), and mixed (up to four live
requests, pages used again) -- in 32-bit and in bfloat16, on the four tiny configurations (head sizes 16, 32, 64
and 128: each has kernels of its own)."""
import numpy as np
import pytest

import replay_util as R
from conftest import TINY, TINY_PAGE, random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [40, 75, 128, 33, 90, 64, 17, 2], "B": [1, 7, 33, 64, 150, 256, 97, 130],
           "C": [200, 65, 256, 3, 129, 64, 48, 100], "D": [300, 64, 17, 500, 129, 33, 256, 2]}
# largest |difference| allowed, as a fraction of the largest |logit| of the reference row set
REL_TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def make_requests(name):
    vocab = TINY[name]["vocab_size"]
    return {f"r{i}": random_tokens(vocab, n, 100 * i + len(name)) for i, n in enumerate(LENGTHS[name])}


def compare(name, dtype, trace, out_dir, requests, plain_logits):
    vocab = TINY[name]["vocab_size"]
    worst = 0.0
    for step, want in enumerate(trace.wanted):
        got = R.read_step(out_dir, step, vocab)
        if not want:
            assert got is None
            continue
        assert got is not None and got.shape == (len(want), vocab), f"step {step}: {None if got is None else got.shape}"
        ref = np.stack([plain_logits(name, requests[rid])[pos] for rid, pos in want])
        scale = np.abs(ref).max()
        err = np.abs(got - ref).max(axis=1) / scale
        bad = np.nonzero(err > REL_TOL[dtype])[0]
        assert len(bad) == 0, (f"{name} {dtype}: step {step}, first wrong row {want[bad[0]]} (request, position): "
                               f"relative error {err[bad[0]]:.3e} > {REL_TOL[dtype]}")
        worst = max(worst, err.max())
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "portions_last", "mixed", "mixed_last"])
def test_replay(name, dtype, mode, model_dirs, plain_logits, tmp_path):
    """``portions_last`` and ``mixed_last`` ask for the last token's logits only, as serving does: such steps run
    as captured steps padded to the next size (a lone portion; single tokens beside portions), here also over a
    NaN-filled cache."""
    requests = make_requests(name)
    trace = {"whole": R.whole, "tail": R.tail_one_by_one, "portions": R.portions, "portions_last": R.portions_last,
             "mixed": R.mixed, "mixed_last": R.mixed_last}[mode](requests)
    out = R.run_trace(model_dirs[name], dtype, trace, tmp_path / "out", TINY_PAGE[name],
                      extra_args=["--poison"] if mode.endswith("_last") else [])
    worst = compare(name, dtype, trace, out, requests, plain_logits)
    print(f"{name} {dtype} {mode}: worst relative error {worst:.3e}, pool {trace.max_tokens} tokens, {len(trace.steps)} steps")


@pytest.mark.parametrize("mode", ["whole", "portions"])
def test_replay_with_norm_rotation_and_store_in_the_projection(mode, model_dirs, plain_logits, tmp_path):
    """Configuration D (head_dim 128) in bfloat16 with the q, k, v projection doing the per-head norm, the rotation and
    the cache store in its epilogue for every portion of more than 32 tokens (serving does from about 1,300 on): the
    prompts whole -- 500, 300, 256, 129 tokens end in the middle of a unit and of a chunk -- and in portions, over a
    NaN-filled cache, against the plain implementation."""
    requests = make_requests("D")
    trace = {"whole": R.whole, "portions": R.portions}[mode](requests)
    out = R.run_trace(model_dirs["D"], "bfloat16", trace, tmp_path / "out", TINY_PAGE["D"], extra_args=["--poison"],
                      extra_env={"VLLM_CPP_B200_QKV_EPILOGUE_ABOVE": "32"})
    worst = compare("D", "bfloat16", trace, out, requests, plain_logits)
    print(f"D bfloat16 {mode}, projection epilogue: worst relative error {worst:.3e}")


@pytest.mark.parametrize("name", ["C", "D"])
@pytest.mark.parametrize("mode", ["tail", "mixed"])
def test_replay_with_decoded_tokens_on_persistent_attention_blocks(name, mode, model_dirs, plain_logits, tmp_path):
    """Head sizes 64 (one layer with a window) and 128 in bfloat16 with every step's single tokens on the attention
    kernel whose blocks walk the (token, KV head) pairs (serving takes it for more pairs than resident blocks): the
    last 32 tokens decoded one by one, and the mixed trace in which pages are used again, over a NaN-filled cache,
    against the plain implementation."""
    requests = make_requests(name)
    trace = {"tail": R.tail_one_by_one, "mixed": R.mixed}[mode](requests)
    out = R.run_trace(model_dirs[name], "bfloat16", trace, tmp_path / "out", TINY_PAGE[name], extra_args=["--poison"],
                      extra_env={"VLLM_CPP_B200_ATTN_STREAM": "2"})
    worst = compare(name, "bfloat16", trace, out, requests, plain_logits)
    print(f"{name} bfloat16 {mode}, single tokens on persistent attention blocks: worst relative error {worst:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_modes_agree_with_each_other(dtype, model_dirs, tmp_path):
    """Cutting and batching change the logits by rounding only (far below the distance to the reference)."""
    name = "B"
    requests = make_requests(name)
    vocab = TINY[name]["vocab_size"]
    rows = {}
    for mode, build in (("whole", R.whole), ("mixed", R.mixed)):
        trace = build(requests)
        out = R.run_trace(model_dirs[name], dtype, trace, tmp_path / mode, TINY_PAGE[name])
        for step, want in enumerate(trace.wanted):
            got = R.read_step(out, step, vocab)
            for i, key in enumerate(want):
                rows.setdefault(key, {})[mode] = got[i]
    worst = max(np.abs(v["whole"] - v["mixed"]).max() / np.abs(v["whole"]).max() for v in rows.values())
    assert worst < (1e-5 if dtype == "float32" else 2e-2), worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_mixed_with_poisoned_pages(name, dtype, model_dirs, plain_logits, tmp_path):
    """The mixed trace again with the cache NaN-filled at the start and every returned page NaN-filled again:
    a key read from a page's unwritten tail, from a page a window has passed, or from a previous owner's
    leftovers would turn the logits into NaN."""
    requests = make_requests(name)
    trace = R.mixed(requests, seed=1)
    out = R.run_trace(model_dirs[name], dtype, trace, tmp_path / "out", TINY_PAGE[name], extra_args=["--poison"])
    compare(name, dtype, trace, out, requests, plain_logits)
