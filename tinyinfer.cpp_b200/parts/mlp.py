"""SwiGLU feed-forward: ``residual += (silu(h Wgate^T) * (h Wup^T)) Wdown^T``.

``silu(g) = g / (1 + exp(-g))`` in float32 (reference: src/cuda/ffn.cu:13-15;
gate and up as one product over stacked rows, src/inference.cu:59-65).  How the
gate and up rows are stacked is the kernel set's choice (``ops.pack_gate_up``).
"""
from __future__ import annotations

import torch

from .base import MATRIX, Part, WeightSpec, register_part


class SwiGLU(Part):
    category = "ffn"

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def weight_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {
            "gate_proj.weight": WeightSpec((i, h), MATRIX),
            "up_proj.weight": WeightSpec((i, h), MATRIX),
            "down_proj.weight": WeightSpec((h, i), MATRIX),
        }

    def load_weights(self, tensors, ops):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        self.w_gate_up = ops.pack_gate_up(g, u)
        self.w_down = ops.pack_linear(tensors["down_proj.weight"])

    def forward(self, ops, h, residual, step):
        ops.swiglu_ffn(h, self.w_gate_up, self.w_down, residual, may_defer=True)


register_part("ffn", "swiglu", SwiGLU)
