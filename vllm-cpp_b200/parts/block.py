"""The pre-norm arrangement of a decoder layer:
x += mixer(norm1(x)); x += feed_forward(norm2(x))   (src/model.cpp:1181-1250).

The additions are not done here: each norm adds the delta still pending from the
part before it while it normalises, so the block hands its last delta on to
whatever norm comes next (the next layer's, or the final one)."""
from __future__ import annotations

from .base import Block


class PreNormBlock(Block):
    """parts: ``norm1``, ``mixer``, ``norm2``, ``feed_forward``."""

    def forward(self, resid, pending, ctx, cache, writes=True):
        mark = getattr(ctx, "mark", lambda label: None)     # kernel groups for the profile, where the step keeps one
        y = self.parts["norm1"].forward(resid, pending)
        d = self.parts["mixer"].forward(y, ctx, cache, writes)
        mark("mixer")
        y = self.parts["norm2"].forward(resid, d)
        out = self.parts["feed_forward"].forward(y, ctx)
        mark("feed_forward")
        return out
