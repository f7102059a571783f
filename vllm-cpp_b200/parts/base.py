"""Interfaces of the parts a layer is put together from.

A part is built from its own parameters (sizes and constants; never a model
configuration), says which checkpoint tensors it expects under its prefix, binds
them from a :class:`WeightStore`, and runs on the tensors of one step.  No part
knows which model it is in.

Families and what each must offer (beside ``tensor_specs`` and ``bind``):

``norm``          ``forward(resid, delta, rows=None) -> normed``: adds ``delta``
                  (``None``, ``[T,H]`` or ``[S,T,H]`` partial sums) into the 32-bit
                  residual stream, returns the normalised rows in the activation
                  dtype; with ``rows`` only those rows, and the stream is left alone.
``position``      whatever its mixer asks of it (the rotary part: a ``table``).
``mixer``         ``cache_spec()`` -> what it keeps per request (a :class:`CacheSpec`
                  or ``None``); ``forward(x, ctx, cache, writes) -> delta`` where
                  ``cache`` is the view of the cache this run was given.
``feed_forward``  ``forward(x, ctx) -> delta``.
``block``         the arrangement: ``forward(resid, pending, ctx, cache, writes) ->
                  pending`` where ``pending`` is a delta not yet added to ``resid``.

Buffers: a part takes its outputs from ``workspace.empty`` (plain ``torch.empty``
works too, at the price of an allocation per step).  Such a buffer is valid until
the run after the next begins -- long enough for what a layer hands to the next
one.  What all runs of a step share is made through ``ctx.plan(key, make)`` and
``ctx.upload(array)``, which live as long as the step.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..weights.loader import TensorSpec, WeightStore


@dataclass
class BuildContext:
    compute_dtype: torch.dtype      # matrices and activations: torch.bfloat16 or torch.float32
    device: torch.device
    shared: dict = field(default_factory=dict)   # parts with equal specs share tables through this


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer keeps for a request.

    kind "kv":    keys and values per token, ``[2, num_kv_heads, head_dim]`` each
                  token, in pages; ``window`` > 0 means only the last ``window``
                  keys are ever read, so older pages may be given back;
                  ``page_size`` > 0 asks for pages of that many tokens instead of
                  the engine's (caches that differ in it get pools of their own).
    kind "state": a block of fixed size per request, ``shape`` of ``dtype``,
                  addressed by the request's slot."""
    kind: str
    num_kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    shape: tuple = ()
    dtype: str = "float32"
    page_size: int = 0
    initial_value: float = 0.0    # kind "state": what a request's state holds before its first token


class Part:
    family = ""
    # False for a part whose forward reads host-side facts of the step (ctx.entries and the like): a model with
    # such a part is run kernel by kernel instead of from a captured graph
    capturable = True

    def __init__(self, params: dict, prefix: str, build: BuildContext):
        self.params = dict(params)
        self.prefix = prefix
        self.build = build

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def bind(self, store: WeightStore) -> None:
        pass


class Norm(Part):
    family = "norm"

    def forward(self, resid, delta, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    family = "position"


class Mixer(Part):
    family = "mixer"

    def cache_spec(self) -> CacheSpec | None:
        return None

    def forward(self, x, ctx, cache, writes: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    family = "feed_forward"

    def forward(self, x, ctx):
        raise NotImplementedError


class Block(Part):
    family = "block"

    def __init__(self, params, prefix, build, parts: dict):
        super().__init__(params, prefix, build)
        self.parts = parts

    def tensor_specs(self):
        return [s for p in self.parts.values() for s in p.tensor_specs()]

    def bind(self, store):
        for p in self.parts.values():
            p.bind(store)

    @property
    def mixer(self) -> Mixer:
        return self.parts["mixer"]

    def forward(self, resid, pending, ctx, cache, writes: bool = True):
        raise NotImplementedError
