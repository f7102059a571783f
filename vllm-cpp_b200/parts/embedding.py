"""Token embedding (x[t,:] = E[id_t,:], src/model.cpp:1157-1163) and the LM head
(logits = y . W^T in 32-bit, W the head matrix or the embedding table when they
are tied, src/model.cpp:560-566, 1260-1263).

Both are parts like any other, found through the registry (families ``embedding``
and ``head``), so that an architecture whose embedding is scaled, whose head has
a bias or caps its logits, registers its own without a change here.

``embedding``  ``forward(ids, n_tokens, status) -> [n_tokens, hidden]`` 32-bit, the
               start of the residual stream; ``table`` is what a tied head shares.
``head``       ``attach(embedding)`` once after both are built, then
               ``forward(y, status) -> [rows, vocab]`` 32-bit logits.
"""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .base import Part
from .linear import matmul_tn


class Embedding(Part):
    family = "embedding"
    table = None

    def forward(self, ids, n_tokens, status):
        raise NotImplementedError


class Head(Part):
    family = "head"

    def attach(self, embedding) -> None:
        """Called once, after the model's embedding part exists (a tied head takes its table from there)."""

    def forward(self, y, status=None):
        raise NotImplementedError


class TokenEmbedding(Embedding):
    """params: ``tensor`` (checkpoint name of the table), ``vocab_size``, ``hidden_size``."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.name, self.vocab, self.hidden = str(params["tensor"]), int(params["vocab_size"]), int(params["hidden_size"])
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab, self.hidden))]

    def bind(self, store):
        self.table = store.matrix(self.name)

    def forward(self, ids, n_tokens, status):
        out = workspace.empty((n_tokens, self.hidden), torch.float32, ids.device)
        ops.embed_gather(self.table, ids, out, status)
        return out


class LMHead(Head):
    """params: ``tensor`` (checkpoint name of the head matrix, or None: the embedding table is the head),
    ``vocab_size``, ``hidden_size``."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.name = params.get("tensor")
        self.vocab, self.hidden = int(params["vocab_size"]), int(params["hidden_size"])
        self.embedding = None
        self.weight = None

    def attach(self, embedding):
        self.embedding = embedding

    def tensor_specs(self):
        return [] if self.name is None else [TensorSpec(self.name, (self.vocab, self.hidden))]

    def bind(self, store):
        if self.name is None:
            if self.embedding is None or self.embedding.table is None:
                raise ValueError("a tied LM head needs an embedding part that has a table")
            self.weight = self.embedding.table
        else:
            self.weight = store.matrix(self.name)

    def forward(self, y, status=None):
        return matmul_tn(y, self.weight, status, out_dtype=torch.float32, after_small_kernel=True)   # (after the last norm)
