"""Qwen3 dense decoder: from its typed configuration to a model description.

Layer order and tensor names as the reference binds them (src/model.cpp:483-523:
input_layernorm, self_attn.{q,k,v,o}_proj, self_attn.{q,k}_norm,
post_attention_layernorm, mlp.{gate,up,down}_proj; :403 model.embed_tokens.weight,
:560-566 lm_head.weight or the tied embedding, :569 model.norm.weight), without
projection biases.  This file only writes data: which part with which numbers in
which layer, and the order the layers run in.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..registry import LayerRun, LayerSpec, ModelSpec, PartSpec, register_architecture


def describe_qwen3(cfg: Qwen3Config) -> ModelSpec:
    rope = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                             "max_positions": cfg.max_position_embeddings})
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
    layers = []
    for l in range(cfg.num_hidden_layers):
        mixer = PartSpec("gqa_attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "eps": cfg.rms_norm_eps,
            "qk_norm": True, "window": cfg.layer_window(l) or 0, "has_kv": True, "position": rope})
        layers.append(LayerSpec(
            prefix=f"model.layers.{l}.", block=PartSpec("prenorm"),
            parts={"norm1": (norm, "input_layernorm."), "mixer": (mixer, "self_attn."),
                   "norm2": (norm, "post_attention_layernorm."), "feed_forward": (ffn, "mlp.")}))
    return ModelSpec(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
        embed_tensor="model.embed_tokens.weight", layers=tuple(layers),
        order=tuple(LayerRun(layer=l, cache=l, writes=True) for l in range(cfg.num_hidden_layers)),
        final_norm=norm, final_norm_prefix="model.norm.",
        lm_head_tensor=None if cfg.tie_word_embeddings else "lm_head.weight",
        stop_ids=tuple(cfg.eos_token_ids))


register_architecture("Qwen3ForCausalLM", Qwen3Config, describe_qwen3)
