"""Registries: architecture name -> (configuration class, description function),
and part kind -> class for each family of parts.

The reference has no such table ("No plugin system: Hardcoded", README.md:128-130;
dense or expert layers are told apart by which tensors exist, src/model.cpp:512,
526-529).  Here ``architectures[0]`` of config.json picks the entry, its
``describe`` turns the typed configuration into a :class:`ModelSpec` (data only),
and the generic decoder builds parts from the spec through the part registries.
Registering a new mixer, feed-forward, norm, position encoding or architecture
needs no change to the package: call ``register_part`` / ``register_architecture``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

from .config.base import ConfigError, ModelConfig

PART_FAMILIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
# the family of a layer's part when its LayerSpec names none: by the role it plays in the block
ROLE_FAMILIES = {"norm1": "norm", "norm2": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}


@dataclass(frozen=True)
class PartSpec:
    """Which part (a name in its family's registry) and with which sizes and constants."""
    kind: str
    params: dict = field(default_factory=dict)

    def key(self) -> tuple:
        return (self.kind, tuple(sorted((k, _freeze(v)) for k, v in self.params.items())))


def _freeze(v):
    if isinstance(v, PartSpec):
        return v.key()
    if isinstance(v, dict):
        return tuple(sorted((k, _freeze(x)) for k, x in v.items()))
    if isinstance(v, (list, tuple)):
        return tuple(_freeze(x) for x in v)
    return v


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (block) and the parts it arranges; ``prefix`` starts its tensor names."""
    prefix: str
    block: PartSpec
    # role -> (PartSpec, sub-prefix) or (PartSpec, sub-prefix, family), e.g. {"norm1": (…, "input_layernorm."),
    # "mixer": (…, "self_attn."), …}.  Without a family the role's usual one is taken (ROLE_FAMILIES), else the role's
    # own name: a block of another arrangement names its roles and their families as it likes.
    parts: dict

    def family_of(self, role: str) -> str:
        entry = self.parts[role]
        return entry[2] if len(entry) > 2 else ROLE_FAMILIES.get(role, role)


@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution order: run ``layer`` against cache ``cache``.

    ``writes`` False makes the mixer read a cache that an earlier run filled
    (it must then need no keys of its own).  A layer may appear in several
    runs, each with a cache of its own."""
    layer: int
    cache: int | None
    writes: bool = True


@dataclass(frozen=True)
class ModelSpec:
    """What a model is made of.  The embedding and the head are parts like the rest: ``embedding`` and ``head`` name
    them (families "embedding" and "head"); left out, they are the plain token embedding over ``embed_tensor`` and
    the plain LM head over ``lm_head_tensor`` (None: tied to the embedding table).  ``final_norm`` None: the head
    reads the residual stream as it is."""
    hidden_size: int
    vocab_size: int
    max_positions: int
    embed_tensor: str | None
    layers: tuple            # of LayerSpec
    order: tuple             # of LayerRun
    final_norm: PartSpec | None
    final_norm_prefix: str
    lm_head_tensor: str | None   # None: the embedding table is the LM head
    stop_ids: tuple = ()
    embedding: PartSpec | None = None
    head: PartSpec | None = None

    def embedding_spec(self) -> PartSpec:
        return self.embedding or PartSpec("token_embedding", {"tensor": self.embed_tensor, "vocab_size": self.vocab_size,
                                                              "hidden_size": self.hidden_size})

    def head_spec(self) -> PartSpec:
        return self.head or PartSpec("lm_head", {"tensor": self.lm_head_tensor, "vocab_size": self.vocab_size,
                                                 "hidden_size": self.hidden_size})


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type
    describe: Callable[[ModelConfig], ModelSpec]


_ARCHITECTURES: dict[str, Architecture] = {}
_PARTS: dict[str, dict[str, type]] = {f: {} for f in PART_FAMILIES}


def register_architecture(name: str, config_cls: type, describe: Callable[[Any], ModelSpec]) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_cls, describe)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def get_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture '{name}' is not registered (registered: {sorted(_ARCHITECTURES)})")
    return _ARCHITECTURES[name]


def architecture_of(config_dict: dict) -> Architecture:
    archs = config_dict.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return get_architecture(archs[0])


def register_part(family: str, kind: str, cls: type) -> None:
    if family not in _PARTS:
        raise ConfigError(f"unknown part family '{family}' (families: {PART_FAMILIES})")
    _PARTS[family][kind] = cls


def unregister_part(family: str, kind: str) -> None:
    _PARTS.get(family, {}).pop(kind, None)


def part_class(family: str, kind: str) -> type:
    try:
        return _PARTS[family][kind]
    except KeyError:
        raise ConfigError(f"no {family} part named '{kind}' (registered: {sorted(_PARTS.get(family, {}))})") from None
