"""The true-32-bit engine against the plain implementation at the layer sizes of the serving models.

Every other comparison with the plain implementation runs on tiny configurations; at real layer sizes the
bfloat16 engine is compared with the engine's own 32-bit path (test_real_shapes.py), which makes that path an
oracle.  Here it is tied down itself: two layers of the 8B, 14B and 4B shapes with weights from a file, replayed
through bin/trace_run --dtype float32 in mixed steps (up to four live requests, portions beside single tokens,
pages used again, more than 64 steps) and in portions of changing size, against tests/plain_qwen3.py in 64-bit
at 2e-5 of the largest logit.

What is cut, and why: the 8B case keeps the real vocabulary of 151,936 in the model and in the engine, and the
plain implementation reads the first 4,096 rows of the embedding table and of the LM head only (token ids are
drawn below 4,096 and the logits of those rows are compared): two 64-bit tables of 151,936 x 4,096 would need
10 GB.  The 14B and 4B cases have a vocabulary of 8,200 in the model itself.  The layer sizes are whole.
"""
import numpy as np
import pytest

import replay_util as R
from conftest import random_tokens

pytestmark = pytest.mark.gpu

SHAPES = {
    # name: (config keys, vocabulary rows the oracle reads, page size)
    "8B": (dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, tie_word_embeddings=False), 4096, 16),
    "14B": (dict(vocab_size=8200, hidden_size=5120, intermediate_size=17408, num_attention_heads=40,
                 num_key_value_heads=8, head_dim=128, tie_word_embeddings=False), None, 16),
    "4B": (dict(vocab_size=8200, hidden_size=2560, intermediate_size=9728, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, tie_word_embeddings=True), None, 16),
}
LENGTHS = [150, 64, 17, 200, 129, 33, 2]
REL_TOL = 2e-5


@pytest.fixture(scope="module")
def real_models(tmp_path_factory):
    from vllm_cpp_b200 import Qwen3Config, write_random_model
    import plain_qwen3
    made = {}

    def get(name):
        if name not in made:
            keys, rows, _ = SHAPES[name]
            cfg = Qwen3Config(num_hidden_layers=2, max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=1e6, **keys)
            d = tmp_path_factory.mktemp(f"real_{name}")
            write_random_model(cfg, 11, d, dtype="bfloat16")
            made[name] = (d, plain_qwen3.read_model(d, vocab_rows=rows))
        return made[name]
    return get


@pytest.mark.parametrize("name,mode", [("8B", "mixed_last"), ("14B", "mixed_last"), ("14B", "portions_last"),
                                       ("4B", "mixed_last"), ("4B", "portions")])
def test_32_bit_engine_equals_the_plain_implementation_at_real_layer_sizes(name, mode, real_models, tmp_path):
    import plain_qwen3
    keys, rows, page = SHAPES[name]
    model_dir, (pcfg, pw) = real_models(name)
    vocab = keys["vocab_size"]
    ids_below = rows or vocab
    requests = {f"r{i}": random_tokens(ids_below, n, 31 * i + len(name)) for i, n in enumerate(LENGTHS)}
    trace = {"mixed_last": lambda r: R.mixed(r, seed=2, last_only=True, decode_tail=26),
             "portions_last": R.portions_last, "portions": R.portions}[mode](requests)
    if mode == "mixed_last":
        assert len(trace.steps) >= 64
    out = R.run_trace(model_dir, "float32", trace, tmp_path / "out", page, timeout=1800)
    plain = {rid: plain_qwen3.forward(pcfg, pw, toks).numpy() for rid, toks in requests.items()}
    worst = 0.0
    for step, want in enumerate(trace.wanted):
        got = R.read_step(out, step, vocab)
        if not want:
            assert got is None
            continue
        assert got is not None and got.shape == (len(want), vocab)
        ref = np.stack([plain[rid][pos] for rid, pos in want])
        got = got[:, :ref.shape[1]]
        err = np.abs(got - ref).max(axis=1) / np.abs(ref).max()
        bad = np.nonzero(err > REL_TOL)[0]
        assert len(bad) == 0, (f"{name} {mode}: step {step}, first wrong row {want[bad[0]]} (request, position): "
                               f"relative error {err[bad[0]]:.3e} > {REL_TOL}")
        worst = max(worst, err.max())
    print(f"{name} float32 {mode}: worst relative error {worst:.3e} over {len(trace.steps)} steps")
