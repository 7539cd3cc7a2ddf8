"""RMSNorm: ``x * rsqrt(mean(x^2) + eps) * w``, eps inside the root, weight applied directly.

Formula as in the reference's ``rms_norm_kernel`` (src/cuda/rms_norm.cu:15-25).
All arithmetic is float32; the result is rounded once to the output dtype.
"""
from __future__ import annotations

import torch

from .base import NORM_WEIGHT, Part, WeightSpec, as_float32, register_part


class RMSNorm(Part):
    category = "norm"

    def __init__(self, size: int, eps: float):
        self.size = int(size)
        self.eps = float(eps)
        self.weight: torch.Tensor | None = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.size,), NORM_WEIGHT)}

    def load_weights(self, tensors, ops):
        self.weight = as_float32(tensors["weight"]).contiguous()

    def forward(self, ops, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty((x.shape[0], self.size), dtype=out_dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, out)
        return out

    def forward_rows(self, ops, x: torch.Tensor, rows: torch.Tensor,
                     out_dtype: torch.dtype) -> torch.Tensor:
        """Norm of the rows ``x[rows]`` only (the rows whose logits are wanted)."""
        out = torch.empty((rows.shape[0], self.size), dtype=out_dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, out, rows=rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)
