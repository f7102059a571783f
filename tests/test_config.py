"""Typed configuration and the architecture / part registries."""
import json

import pytest

from vllm_cpp_b200 import ConfigError, EngineConfig, Qwen3Config
from vllm_cpp_b200.config.base import load_config_dict
from vllm_cpp_b200.registry import architecture_of, get_architecture, part_class, register_part, unregister_part

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "attention_bias": False, "attention_dropout": 0.0, "bos_token_id": 151643,
    "eos_token_id": 151645, "head_dim": 128, "hidden_act": "silu", "hidden_size": 4096, "initializer_range": 0.02,
    "intermediate_size": 12288, "max_position_embeddings": 40960, "max_window_layers": 36, "model_type": "qwen3",
    "num_attention_heads": 32, "num_hidden_layers": 36, "num_key_value_heads": 8, "rms_norm_eps": 1e-06,
    "rope_scaling": None, "rope_theta": 1000000, "sliding_window": None, "tie_word_embeddings": False,
    "torch_dtype": "bfloat16", "use_cache": True, "use_sliding_window": False, "vocab_size": 151936}


def test_reads_every_size_from_the_file(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(QWEN3_8B))
    import vllm_cpp_b200.models  # noqa: F401  (registers the architecture)
    data = load_config_dict(tmp_path)
    cfg = architecture_of(data).config_cls.from_dict(data)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads) == (4096, 36, 32, 8)
    assert (cfg.head_dim, cfg.intermediate_size, cfg.vocab_size, cfg.max_position_embeddings) == (128, 12288, 151936, 40960)
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 1e6 and not cfg.tie_word_embeddings      # "1e-06" is a real number
    assert cfg.eos_token_ids == (151645,) and cfg.bos_token_id == 151643
    assert cfg.layer_types == ("full_attention",) * 36 and cfg.sliding_window is None
    assert Qwen3Config.from_dict(cfg.to_dict()) == cfg


def test_defaults_and_derived_values():
    d = dict(QWEN3_8B)
    del d["head_dim"], d["num_key_value_heads"], d["rms_norm_eps"], d["rope_theta"]
    cfg = Qwen3Config.from_dict(d)
    assert cfg.head_dim == 128 and cfg.num_key_value_heads == 32 and cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 1e6
    d = dict(QWEN3_8B, hidden_size=2560, head_dim=128)      # heads * head_dim != hidden_size is allowed (the 4B shape)
    assert Qwen3Config.from_dict(d).head_dim == 128
    d = dict(QWEN3_8B, eos_token_id=[1, 2])
    assert Qwen3Config.from_dict(d).eos_token_ids == (1, 2)


def test_window_keys():
    d = dict(QWEN3_8B, num_hidden_layers=4, use_sliding_window=True, sliding_window=1024, max_window_layers=2)
    cfg = Qwen3Config.from_dict(d)
    assert cfg.layer_types == ("full_attention", "full_attention", "sliding_attention", "sliding_attention")
    assert [cfg.layer_window(i) for i in range(4)] == [None, None, 1024, 1024]
    d = dict(QWEN3_8B, num_hidden_layers=2, sliding_window=64, layer_types=["sliding_attention", "full_attention"])
    assert [Qwen3Config.from_dict(d).layer_window(i) for i in range(2)] == [64, None]
    d = dict(QWEN3_8B, num_hidden_layers=2, sliding_window=64, use_sliding_window=False)   # window given but unused
    assert Qwen3Config.from_dict(d).sliding_window is None


@pytest.mark.parametrize("change,word", [
    ({"hidden_size": None}, "hidden_size"), ({"vocab_size": "many"}, "vocab_size"), ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"num_key_value_heads": 5}, "num_key_value_heads"), ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_experts": 64}, "num_experts"), ({"use_sliding_window": True}, "sliding_window"),
    ({"layer_types": ["full_attention"]}, "layer_types"), ({"layer_types": ["conv"] * 36}, "conv"),
    ({"rms_norm_eps": -1}, "rms_norm_eps"), ({"tie_word_embeddings": "no"}, "tie_word_embeddings"),
    ({"head_dim": 127}, "head_dim")])
def test_errors_name_the_key(change, word):
    d = dict(QWEN3_8B)
    d.update(change)
    if change.get("hidden_size", 0) is None:
        del d["hidden_size"]
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(d)


def test_registry(tmp_path):
    import vllm_cpp_b200.models  # noqa: F401
    assert get_architecture("Qwen3ForCausalLM").config_cls is Qwen3Config
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        get_architecture("LlamaForCausalLM")               # the error lists what is registered
    with pytest.raises(ConfigError, match="architectures"):
        architecture_of({"hidden_size": 1})
    with pytest.raises(ConfigError, match="no config.json"):
        load_config_dict(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config_dict(tmp_path)
    import vllm_cpp_b200.parts  # noqa: F401
    assert part_class("mixer", "gqa_attention").__name__ == "GQAAttention"
    with pytest.raises(ConfigError, match="gqa_attention"):
        part_class("mixer", "nothing")
    register_part("norm", "toy", dict)
    assert part_class("norm", "toy") is dict
    unregister_part("norm", "toy")


def test_model_description_is_data():
    """The description names parts and numbers layer by layer, and the order of execution is a list."""
    import vllm_cpp_b200.models  # noqa: F401
    cfg = Qwen3Config.from_dict(dict(QWEN3_8B, num_hidden_layers=3, use_sliding_window=True, sliding_window=512, max_window_layers=1))
    spec = get_architecture(cfg.architecture).describe(cfg)
    assert [r.layer for r in spec.order] == [0, 1, 2] and [r.cache for r in spec.order] == [0, 1, 2]
    mixers = [l.parts["mixer"][0] for l in spec.layers]
    assert [m.kind for m in mixers] == ["gqa_attention"] * 3
    assert [m.params["window"] for m in mixers] == [0, 512, 512]
    assert mixers[0].params["position"].params == {"head_dim": 128, "theta": 1e6, "max_positions": 40960}
    assert spec.lm_head_tensor == "lm_head.weight" and spec.stop_ids == (151645,)


def test_engine_config():
    e = EngineConfig(dtype="bf16", page_size=16, max_tokens=4096)
    assert e.dtype == "bfloat16" and e.num_pages == 256
    with pytest.raises(ConfigError, match="dtype"):
        EngineConfig(dtype="fp8")
    with pytest.raises(ConfigError, match="multiple"):
        EngineConfig(page_size=16, max_tokens=100)
