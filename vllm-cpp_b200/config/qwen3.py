"""Qwen3 dense decoder configuration, from the keys of its config.json.

Key list and meanings follow what the reference reads or derives
(src/model.cpp:366-379 for the parsed keys, :412-431 head_dim / head-count
inference, :519 intermediate size from the gate matrix, :560-566 tied LM head)
with the departures that the intended model needs: ``rope_theta`` and
``rms_norm_eps`` are honoured (the reference's CPU path uses the constant
ROPE_BASE, src/config.h:43, and mis-parses 1e-06), ``head_dim`` may differ
from hidden/heads, and the per-layer attention kind (all keys or a sliding
window) is part of the configuration.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .base import ConfigError, KeyReader, ModelConfig

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    tie_word_embeddings: bool = False
    sliding_window: int | None = None
    layer_types: tuple[str, ...] = ()
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    architecture: str = "Qwen3ForCausalLM"
    extra: dict = field(default_factory=dict, compare=False)

    def __post_init__(self):
        # a configuration made in code (not read from a file) may leave the per-layer kinds out
        if not self.layer_types:
            kind = SLIDING_ATTENTION if self.sliding_window else FULL_ATTENTION
            object.__setattr__(self, "layer_types", (kind,) * self.num_hidden_layers)
        object.__setattr__(self, "layer_types", tuple(self.layer_types))
        object.__setattr__(self, "eos_token_ids", tuple(self.eos_token_ids))
        if len(self.layer_types) != self.num_hidden_layers:
            raise ConfigError(f"layer_types has {len(self.layer_types)} entries for {self.num_hidden_layers} layers")
        if SLIDING_ATTENTION in self.layer_types and not self.sliding_window:
            raise ConfigError("a layer is 'sliding_attention' but sliding_window is not set")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("num_key_value_heads must divide num_attention_heads")

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "Qwen3Config":
        r = KeyReader(data)
        archs = r.string_list("architectures", ("Qwen3ForCausalLM",))
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", heads, minimum=1)
        if heads % kv_heads:
            raise ConfigError(f"config.json: num_key_value_heads={kv_heads} must divide num_attention_heads={heads}")
        head_dim = r.integer("head_dim", None, minimum=1)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError("config.json: head_dim is absent and hidden_size is not a multiple of num_attention_heads")
            head_dim = hidden // heads
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim={head_dim} must be even (rotary pairs)")
        layers = r.integer("num_hidden_layers", minimum=1)

        if r.boolean("attention_bias", False):
            raise ConfigError("config.json: attention_bias=true is unsupported (Qwen3 dense has no projection biases)")
        if data.get("rope_scaling") is not None:
            raise ConfigError("config.json: rope_scaling is unsupported (only plain rotary positions)")
        act = r.string("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act='{act}' is unsupported (only 'silu')")
        for moe_key in ("num_experts", "num_local_experts"):
            if data.get(moe_key):
                raise ConfigError(f"config.json: '{moe_key}' is set; the expert variant is another architecture")

        window = r.integer("sliding_window", None, minimum=1)
        layer_types = r.string_list("layer_types", None)
        if layer_types is None:
            if r.boolean("use_sliding_window", False):
                if window is None:
                    raise ConfigError("config.json: use_sliding_window=true needs 'sliding_window'")
                first_windowed = r.integer("max_window_layers", layers, minimum=0)
                layer_types = tuple(SLIDING_ATTENTION if i >= first_windowed else FULL_ATTENTION for i in range(layers))
            else:
                layer_types = (FULL_ATTENTION,) * layers
        if len(layer_types) != layers:
            raise ConfigError(f"config.json: layer_types has {len(layer_types)} entries for {layers} layers")
        for t in layer_types:
            if t not in (FULL_ATTENTION, SLIDING_ATTENTION):
                raise ConfigError(f"config.json: layer_types entry '{t}' is not one of "
                                  f"'{FULL_ATTENTION}', '{SLIDING_ATTENTION}'")
        if SLIDING_ATTENTION in layer_types and window is None:
            raise ConfigError("config.json: a layer is 'sliding_attention' but 'sliding_window' is absent")
        if SLIDING_ATTENTION not in layer_types:
            window = None

        return cls(
            vocab_size=r.integer("vocab_size", minimum=1),
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size", minimum=1),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=r.integer("max_position_embeddings", minimum=1),
            rms_norm_eps=r.number("rms_norm_eps", 1e-6, positive=True),
            rope_theta=r.number("rope_theta", 1e6, positive=True),
            tie_word_embeddings=r.boolean("tie_word_embeddings", False),
            sliding_window=window,
            layer_types=layer_types,
            eos_token_ids=r.int_or_int_list("eos_token_id", None),
            bos_token_id=r.integer("bos_token_id", None),
            architecture=archs[0],
        )

    def layer_window(self, layer: int) -> int | None:
        return self.sliding_window if self.layer_types[layer] == SLIDING_ATTENTION else None

    def to_dict(self) -> dict[str, Any]:
        d = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "rope_scaling": None,
            "sliding_window": self.sliding_window,
            "use_sliding_window": self.sliding_window is not None,
            "layer_types": list(self.layer_types),
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d
