"""Arrangement of a layer's parts.

``prenorm`` (reference: src/inference.cu:35-66): ``x += mixer(norm1(x))`` then
``x += ffn(norm2(x))``; both sums happen in the float32 residual stream, inside the
mixer's and the feed-forward's last product.  A layer without a feed-forward stops after the mixer.

``parallel``: ``h = norm(x)``, then ``x += mixer(h)`` and ``x += ffn(h)``.
"""
from __future__ import annotations

from .base import Part, register_part


class PreNormBlock(Part):
    category = "block"

    def __init__(self, mixer, mixer_norm, ffn=None, ffn_norm=None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer, self.ffn = mixer, ffn
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm

    def forward(self, ops, x, step, cache):
        self.mixer.forward(ops, self.mixer_norm.forward(ops, x, step.act_dtype), x, step, cache)
        if self.ffn is not None:
            self.ffn.forward(ops, self.ffn_norm.forward(ops, x, step.act_dtype), x, step)


class ParallelBlock(Part):
    """``x += mixer(h) + ffn(h)`` with ``h = norm(x)``: one norm, and both sublayers read its
    output.  Each adds its result to the float32 residual stream in its last product; the
    feed-forward may be absent."""
    category = "block"

    def __init__(self, mixer, mixer_norm, ffn=None, ffn_norm=None):
        if ffn_norm is not None:
            raise ValueError("a parallel block has one norm")
        self.mixer, self.ffn, self.mixer_norm = mixer, ffn, mixer_norm

    def forward(self, ops, x, step, cache):
        h = self.mixer_norm.forward(ops, x, step.act_dtype)
        self.mixer.forward(ops, h, x, step, cache)
        if self.ffn is not None:
            self.ffn.forward(ops, h, x, step)


register_part("block", "prenorm", PreNormBlock)
register_part("block", "parallel", ParallelBlock)
