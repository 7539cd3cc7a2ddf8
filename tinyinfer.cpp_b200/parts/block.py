"""Arrangement of a layer's parts.

``prenorm`` (reference: src/inference.cu:35-66): ``x += mixer(norm1(x))`` then
``x += ffn(norm2(x))``; both sums happen in the float32 residual stream, inside the
mixer's and the feed-forward's last product.
"""
from __future__ import annotations

from .base import Part, register_part


class PreNormBlock(Part):
    category = "block"
    chains_norm = True       # forward takes the normed input ``h`` and may return the next block's

    def __init__(self, mixer, ffn, mixer_norm, ffn_norm):
        self.mixer, self.ffn = mixer, ffn
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm

    def forward(self, ops, x, step, cache, h=None, next_norm=None):
        """``h``: norm1(x) if the block before already computed it.  ``next_norm``: the norm that
        follows this block; if the feed-forward can compute it in its last launch, its result is
        returned (else None).  A mixer or feed-forward that sets ``fuses_norm`` accepts
        ``then_norm=<RMSNorm part>`` and returns the normed residual."""
        if h is None:
            h = self.mixer_norm.forward(ops, x, step.act_dtype)
        h2 = None
        if getattr(self.mixer, "fuses_norm", False) and getattr(self.ffn_norm, "is_rmsnorm", False):
            h2 = self.mixer.forward(ops, h, x, step, cache, then_norm=self.ffn_norm)
        else:
            self.mixer.forward(ops, h, x, step, cache)
        if h2 is None:
            h2 = self.ffn_norm.forward(ops, x, step.act_dtype)
        if (next_norm is not None and getattr(self.ffn, "fuses_norm", False)
                and getattr(next_norm, "is_rmsnorm", False)):
            return self.ffn.forward(ops, h2, x, step, then_norm=next_norm)
        self.ffn.forward(ops, h2, x, step)
        return None


register_part("block", "prenorm", PreNormBlock)
