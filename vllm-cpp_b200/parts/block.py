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
        y = self.parts["norm1"].forward(resid, pending)
        d = self.parts["mixer"].forward(y, ctx, cache, writes)
        y = self.parts["norm2"].forward(resid, d)
        return self.parts["feed_forward"].forward(y, ctx)
