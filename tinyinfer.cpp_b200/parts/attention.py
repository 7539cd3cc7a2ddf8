"""Causal grouped-query attention over a paged cache, with per-head q/k RMSNorm.

Reference order (src/inference.cu:41-55, src/cuda/attention.cu:12-87,107-198):
``qkv = h Wqkv^T`` (no bias; Wqkv = [Wq; Wk; Wv] on rows) -> per head RMSNorm of q
and k with one ``[head_dim]`` weight each, before the rotation -> rotation of q and k at
the token's position as the position part describes it (NeoX pairs in the reference)
-> k, v rounded to the cache dtype and written at
the token's place -> for query head ``i``, kv head ``i // (heads / kv_heads)``,
scores ``(q . k_p) * scale`` over ``p <= pos`` (and ``p > pos - window`` if the
layer has a window), float32 softmax, weighted sum of v -> ``residual += attn Wo^T``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..config.plan import PartSpec
from .base import (MATRIX, NORM_WEIGHT, PagedKVSpec, Part, WeightSpec, as_float32, build_part,
                   register_part)


class Attention(Part):
    category = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qk_norm_eps: float, position: PartSpec, window: Optional[int] = None,
                 scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} kv heads evenly")
        if window is not None and window < 1:
            raise ValueError(f"window must be positive, got {window}")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.eps = float(qk_norm_eps)
        self.window = None if window is None else int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.position = build_part("position", position)
        self.nq = self.num_heads * self.head_dim
        self.nk = self.num_kv_heads * self.head_dim
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    def weight_specs(self):
        h = self.hidden_size
        return {
            "q_proj.weight": WeightSpec((self.nq, h), MATRIX),
            "k_proj.weight": WeightSpec((self.nk, h), MATRIX),
            "v_proj.weight": WeightSpec((self.nk, h), MATRIX),
            "o_proj.weight": WeightSpec((h, self.nq), MATRIX),
            "q_norm.weight": WeightSpec((self.head_dim,), NORM_WEIGHT),
            "k_norm.weight": WeightSpec((self.head_dim,), NORM_WEIGHT),
        }

    def load_weights(self, tensors, ops):
        q, k, v = (tensors[n + "_proj.weight"] for n in "qkv")
        dtypes = {q.dtype, k.dtype, v.dtype}
        if len(dtypes) > 1:                       # mixed storage: widen, never narrow
            q, k, v = (t.to(torch.float32) for t in (q, k, v))
        self.w_qkv = ops.pack_linear(torch.cat([q, k, v], dim=0))
        self.w_o = ops.pack_linear(tensors["o_proj.weight"])
        self.q_norm = as_float32(tensors["q_norm.weight"]).contiguous()
        self.k_norm = as_float32(tensors["k_norm.weight"]).contiguous()

    def cache_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

    def forward(self, ops, h, residual, step, cache):
        t, dev, act = h.shape[0], h.device, h.dtype
        out = torch.empty((t, self.nq), dtype=act, device=dev)
        ops.qkv_attention(h, self.w_qkv, self.q_norm, self.k_norm, self.eps, self.position.rotation(dev),
                          step, cache, out, self.num_heads, self.num_kv_heads, self.head_dim,
                          self.window, self.scale)
        ops.linear(out, self.w_o, residual, accumulate=True, may_defer=True)


register_part("mixer", "attention", Attention)
