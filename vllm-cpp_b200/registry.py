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

PART_FAMILIES = ("mixer", "feed_forward", "norm", "position", "block")


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
    parts: dict  # role -> (PartSpec, sub-prefix), e.g. {"norm1": (…, "input_layernorm."), "mixer": (…, "self_attn."), …}


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
    hidden_size: int
    vocab_size: int
    max_positions: int
    embed_tensor: str
    layers: tuple            # of LayerSpec
    order: tuple             # of LayerRun
    final_norm: PartSpec
    final_norm_prefix: str
    lm_head_tensor: str | None   # None: the embedding table is the LM head
    stop_ids: tuple = ()


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
