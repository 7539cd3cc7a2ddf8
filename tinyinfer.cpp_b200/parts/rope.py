"""NeoX (half-split) rotary position encoding.

For pair index ``k`` in ``[0, head_dim/2)``: ``inv_freq[k] = theta ** (-2k / head_dim)``,
angle ``a = pos * inv_freq[k]``, and the pair ``(x[k], x[k + head_dim/2])`` becomes
``(x0 cos a - x1 sin a, x0 sin a + x1 cos a)`` (reference: src/cuda/attention.cu:64-74,
src/cuda/rope.cu:19-28).  ``inv_freq`` is computed once on the host in double
precision and rounded to float32; the angle, its sine and cosine are float32 on
the device.
"""
from __future__ import annotations

import torch

from .base import Part, register_part


_TABLES: dict[tuple, torch.Tensor] = {}      # layers with the same constants share one device tensor


class RopeNeox(Part):
    category = "position"

    def __init__(self, head_dim: int, theta: float):
        if head_dim % 2:
            raise ValueError(f"rotary head_dim {head_dim} must be even")
        self.head_dim = int(head_dim)
        self.theta = float(theta)

    def inv_freq(self) -> torch.Tensor:
        half = self.head_dim // 2
        k = torch.arange(half, dtype=torch.float64)
        return torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                         -2.0 * k / self.head_dim).to(torch.float32)

    def table(self, device) -> torch.Tensor:
        key = (self.head_dim, self.theta, str(device))
        if key not in _TABLES:
            _TABLES[key] = self.inv_freq().to(device)
        return _TABLES[key]


register_part("position", "rope_neox", RopeNeox)
