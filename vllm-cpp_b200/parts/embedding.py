"""Token embedding (x[t,:] = E[id_t,:], src/model.cpp:1157-1163) and the LM head
(logits = y . W^T in 32-bit, W the head matrix or the embedding table when they
are tied, src/model.cpp:560-566, 1260-1263)."""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .linear import matmul_tn


class TokenEmbedding:
    def __init__(self, tensor_name: str, vocab_size: int, hidden_size: int):
        self.name, self.vocab, self.hidden = tensor_name, vocab_size, hidden_size
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab, self.hidden))]

    def bind(self, store):
        self.table = store.matrix(self.name)

    def forward(self, ids, n_tokens, status):
        out = workspace.empty((n_tokens, self.hidden), torch.float32, ids.device)
        ops.embed_gather(self.table, ids, out, status)
        return out


class LMHead:
    def __init__(self, tensor_name: str | None, vocab_size: int, hidden_size: int, embedding: TokenEmbedding):
        self.name, self.vocab, self.hidden, self.embedding = tensor_name, vocab_size, hidden_size, embedding
        self.weight = None

    def tensor_specs(self):
        return [] if self.name is None else [TensorSpec(self.name, (self.vocab, self.hidden))]

    def bind(self, store):
        self.weight = self.embedding.table if self.name is None else store.matrix(self.name)

    def forward(self, y, status=None):
        return matmul_tn(y, self.weight, status, out_dtype=torch.float32)
