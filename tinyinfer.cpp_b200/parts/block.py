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
        """A mixer or feed-forward that sets ``takes_norm`` gets ``h=None, pre_norm=<the RMSNorm
        part>`` and applies the norm to the residual inside its first product; any other gets
        the normed residual."""
        if getattr(self.mixer, "takes_norm", False) and getattr(self.mixer_norm, "is_rmsnorm", False):
            self.mixer.forward(ops, None, x, step, cache, pre_norm=self.mixer_norm)
        else:
            self.mixer.forward(ops, self.mixer_norm.forward(ops, x, step.act_dtype), x, step, cache)
        if getattr(self.ffn, "takes_norm", False) and getattr(self.ffn_norm, "is_rmsnorm", False):
            self.ffn.forward(ops, None, x, step, pre_norm=self.ffn_norm)
        else:
            self.ffn.forward(ops, self.ffn_norm.forward(ops, x, step.act_dtype), x, step)


register_part("block", "prenorm", PreNormBlock)
