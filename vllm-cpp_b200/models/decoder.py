"""The generic decoder: embedding, a list of layers, the order they run in, final
norm, LM head -- built from a :class:`ModelSpec` through the part registries.

The forward pass follows the reference's layer loop (src/model.cpp:1176-1263)
with two generalisations that are data in the spec: the execution order is a
list of (layer, cache) runs, so a layer may run twice or read a cache another run
filled; and each layer names its own parts, so mixers and feed-forwards may
differ along the depth.  Final norm and LM head run only on the rows whose logits
were asked for (the reference: last position only, src/model.cpp:1255-1263).
"""
from __future__ import annotations

from .. import workspace
from ..parts.base import BuildContext, CacheSpec
from ..registry import ModelSpec, part_class
from ..weights.loader import TensorSpec, WeightStore


def _build_layer(lspec, build: BuildContext):
    parts = {}
    for role, entry in lspec.parts.items():
        pspec, sub = entry[0], entry[1]
        parts[role] = part_class(lspec.family_of(role), pspec.kind)(pspec.params, lspec.prefix + sub, build)
    return part_class("block", lspec.block.kind)(lspec.block.params, lspec.prefix, build, parts)


class DecoderModel:
    def __init__(self, spec: ModelSpec, build: BuildContext):
        self.spec = spec
        self.build = build
        emb, head = spec.embedding_spec(), spec.head_spec()
        self.embedding = part_class("embedding", emb.kind)(emb.params, "", build)
        self.layers = [_build_layer(l, build) for l in spec.layers]
        self.final_norm = None
        if spec.final_norm is not None:
            self.final_norm = part_class("norm", spec.final_norm.kind)(spec.final_norm.params, spec.final_norm_prefix, build)
        self.lm_head = part_class("head", head.kind)(head.params, "", build)
        self.lm_head.attach(self.embedding)
        self.order = list(spec.order)
        for run in self.order:
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"the execution order names layer {run.layer}, the model has {len(self.layers)}")

    @property
    def capturable(self) -> bool:
        """Whether a decoding step of this model can be captured as a CUDA graph."""
        parts = [p for layer in self.layers for p in layer.parts.values()] + [self.embedding, self.lm_head]
        return all(getattr(p, "capturable", True) for p in parts)

    # ---- weights ----
    def tensor_specs(self) -> list[TensorSpec]:
        specs = list(self.embedding.tensor_specs())
        for layer in self.layers:
            specs += layer.tensor_specs()
        if self.final_norm is not None:
            specs += self.final_norm.tensor_specs()
        return specs + self.lm_head.tensor_specs()

    def load(self, store: WeightStore) -> None:
        store.check(self.tensor_specs())
        self.embedding.bind(store)
        for layer in self.layers:
            layer.bind(store)
        if self.final_norm is not None:
            self.final_norm.bind(store)
        self.lm_head.bind(store)

    # ---- caches ----
    def cache_specs(self) -> dict[int, CacheSpec]:
        """cache id -> what the writing run's mixer keeps there."""
        specs: dict[int, CacheSpec] = {}
        for run in self.order:
            if run.cache is None or not run.writes:
                continue
            spec = self.layers[run.layer].mixer.cache_spec()
            if spec is None:
                raise ValueError(f"layer {run.layer} was given cache {run.cache} but its mixer keeps nothing")
            if run.cache in specs:
                raise ValueError(f"cache {run.cache} is written by more than one run")
            specs[run.cache] = spec
        for run in self.order:
            if run.cache is not None and not run.writes:
                if run.cache not in specs:
                    raise ValueError(f"layer {run.layer} reads cache {run.cache}, which no run writes")
                if self.layers[run.layer].mixer.cache_spec() != specs[run.cache]:
                    raise ValueError(f"layer {run.layer} reads cache {run.cache} of another shape than it expects")
        return specs

    # ---- one step ----
    def forward(self, ctx, caches):
        """ctx: the step's tensors; caches: cache id -> view.  Returns 32-bit logits [rows, vocab]."""
        mark = getattr(ctx, "mark", lambda label: None)     # kernel groups for the profile, where the step keeps one
        resid = self.embedding.forward(ctx.token_ids, ctx.T, ctx.status)
        mark("embedding")
        pending = None
        for i, run in enumerate(self.order):
            cache = caches[run.cache] if run.cache is not None else None
            workspace.begin_run(i)      # the run's buffers come from the scratch region that run i - 2 used
            pending = self.layers[run.layer].forward(resid, pending, ctx, cache, run.writes)
        workspace.end_runs()
        if ctx.n_rows == 0:
            return None
        if self.final_norm is None:
            # an architecture without a final norm: the head reads the wanted rows of the stream as they are
            x = resid if pending is None else resid + (pending.sum(0) if pending.dim() == 3 else pending).float()
            y = x[ctx.logit_rows.long()].to(self.build.compute_dtype)
        else:
            y = self.final_norm.forward(resid, pending, rows=ctx.logit_rows)
        logits = self.lm_head.forward(y, ctx.status)
        mark("head")
        return logits
