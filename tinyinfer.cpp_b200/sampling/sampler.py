"""Next-token choice on the device: argmax, or temperature / top-k / top-p sampling.

The kernels read the logits where the step left them; only the chosen token ids go to
the host.  Uniform numbers come from a counter-based generator on the host, keyed by
(seed, request number, draw number).
"""
from __future__ import annotations

from typing import Sequence

import torch

from .params import SamplingParams

_MASK = (1 << 64) - 1


def _mix(x: int) -> int:
    """One round of the splitmix64 finaliser."""
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed: int, request_number: int, draw: int) -> float:
    """A number in [0, 1) with 24 random bits that depends only on its three keys."""
    h = _mix(_mix(_mix(seed & _MASK) ^ (request_number & _MASK)) ^ (draw & _MASK))
    return (h >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, ops, device):
        self.ops = ops
        self.device = device

    def __call__(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                 request_numbers: Sequence[int], draws: Sequence[int]) -> torch.Tensor:
        """One token id per row of ``logits`` (int32, on the device)."""
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        if rows == 0:
            return out
        if all(p.greedy for p in params):
            self.ops.argmax(logits, out)
            return out
        host = torch.empty((4, rows), dtype=torch.float32)
        for i, p in enumerate(params):
            host[0, i] = max(float(p.temperature), 0.0)
            host[1, i] = float(p.top_p)
            host[2, i] = uniform(p.seed, request_numbers[i], draws[i])
        top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32)
        dev = host.to(logits.device)
        self.ops.sample(logits, dev[0], top_k.to(logits.device), dev[1], dev[2], out)
        return out
