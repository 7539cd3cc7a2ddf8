"""Position encodings of the attention heads, and what they tell the mixer's kernels.

A position part does not rotate anything itself: it answers ``rotation(device)`` with a
``Rotation``, the contract between it and the kernel that norms, rotates and stores the heads
(``ops.qkv_rope_store``).  ``kind`` names the pairing rule; the kernel set has kernels for some
kinds and refuses the others, unless a part has registered a handler for its own kind
(``ops.register_rotation``).  The mixer passes the ``Rotation`` on without looking inside.

Kinds built in:

``neox``   half-split pairs over the first ``rotary_dim`` elements of a head: for pair index
           ``k`` in ``[0, rotary_dim/2)``, ``inv_freq[k] = theta ** (-2k / rotary_dim)``, angle
           ``a = pos * inv_freq[k]``, and ``(x[k], x[k + rotary_dim/2])`` becomes
           ``(x0 cos a - x1 sin a, x0 sin a + x1 cos a)``; elements from ``rotary_dim`` on are
           left as they are.  With ``rotary_dim = head_dim`` this is the reference's rotation
           (src/cuda/attention.cu:64-74, src/cuda/rope.cu:19-28).
``none``   no rotation (``rotary_dim = 0``).

``inv_freq`` is computed once on the host in double precision and rounded to float32; the
angle, its sine and cosine are float32 on the device.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch

from .base import Part, register_part


@dataclass(frozen=True)
class Rotation:
    """What the kernels need to encode a head's position.

    kind        the pairing rule (a key of the kernel set's table of rotations)
    rotary_dim  how many leading elements of a head take part (0: none)
    inv_freq    ``[rotary_dim / 2]`` float32 on the device, or None
    extra       anything else a kind's own handler wants
    """
    kind: str
    rotary_dim: int
    inv_freq: Optional[torch.Tensor] = None
    extra: Any = None


_TABLES: dict[tuple, torch.Tensor] = {}      # layers with the same constants share one device tensor


class RopeNeox(Part):
    category = "position"

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None):
        rotary_dim = head_dim if rotary_dim is None else int(rotary_dim)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary width {rotary_dim} must be even and lie in (0, head_dim {head_dim}]")
        self.head_dim = int(head_dim)
        self.rotary_dim = rotary_dim
        self.theta = float(theta)

    def inv_freq(self) -> torch.Tensor:
        half = self.rotary_dim // 2
        k = torch.arange(half, dtype=torch.float64)
        return torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                         -2.0 * k / self.rotary_dim).to(torch.float32)

    def rotation(self, device) -> Rotation:
        key = (self.rotary_dim, self.theta, str(device))
        if key not in _TABLES:
            _TABLES[key] = self.inv_freq().to(device)
        return Rotation("neox", self.rotary_dim, _TABLES[key])


class NoPosition(Part):
    """Heads are normed and stored without a rotation."""
    category = "position"

    def __init__(self, head_dim: int = 0):
        self.head_dim = int(head_dim)

    def rotation(self, device) -> Rotation:
        return Rotation("none", 0, None)


register_part("position", "rope_neox", RopeNeox)
register_part("position", "none", NoPosition)
