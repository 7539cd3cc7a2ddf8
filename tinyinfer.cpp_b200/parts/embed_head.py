"""Token embedding and the output head.

Embedding: ``x[t] = float32(E[token[t]])`` without scaling (reference:
src/inference.cu:14-24).  Head: ``logits = h E_out^T`` in float32, where ``E_out``
is the embedding table when the head is tied (reference: always tied,
src/inference.cu:70-71) or a table of its own.
"""
from __future__ import annotations

import torch

from .base import MATRIX, Part, WeightSpec, register_part


class Embedding(Part):
    category = "embedding"

    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.table = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.vocab_size, self.hidden_size), MATRIX)}

    def load_weights(self, tensors, ops):
        self.table = ops.pack_linear(tensors["weight"])

    def shared_weights(self):
        return {"weight": self.table}

    def forward(self, ops, token_ids, out):
        ops.embed(self.table, token_ids, out)


class LMHead(Part):
    category = "head"

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool):
        self.vocab_size, self.hidden_size, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.table = None

    def weight_specs(self):
        if self.tied:
            return {}
        return {"weight": WeightSpec((self.vocab_size, self.hidden_size), MATRIX)}

    def load_weights(self, tensors, ops):
        if not self.tied:
            self.table = ops.pack_linear(tensors["weight"])

    def tie(self, embedding: Embedding):
        self.table = embedding.shared_weights()["weight"]

    def forward(self, ops, h):
        logits = torch.empty((h.shape[0], self.vocab_size), dtype=torch.float32, device=h.device)
        ops.linear(h, self.table, logits)
        return logits


register_part("embedding", "embedding", Embedding)
register_part("head", "lm_head", LMHead)
