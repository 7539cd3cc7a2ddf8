"""Arrangement of a layer's parts.

``prenorm`` (reference: src/inference.cu:35-66): ``x += mixer(norm1(x))`` then
``x += ffn(norm2(x))``; both sums happen in the float32 residual stream, inside the
mixer's and the feed-forward's last product.
"""
from __future__ import annotations

from .base import Part, register_part


class PreNormBlock(Part):
    category = "block"

    def __init__(self, mixer, ffn, mixer_norm, ffn_norm):
        self.mixer, self.ffn = mixer, ffn
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm

    def forward(self, ops, x, step, cache):
        self.mixer.forward(ops, self.mixer_norm.forward(ops, x, step.act_dtype), x, step, cache)
        self.ffn.forward(ops, self.ffn_norm.forward(ops, x, step.act_dtype), x, step)


register_part("block", "prenorm", PreNormBlock)
