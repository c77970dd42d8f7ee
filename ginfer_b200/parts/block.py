"""Arrangements of a mixer, a feed-forward and their norms into a layer.

Pre-norm decoder block of the reference (``ginfer/core/layer/transformer/encoder.cc:33-39``):
``x = norm1(h)``, ``a = mixer(x)``, ``r = h + a``, ``y = norm2(r)``, ``m = ffn(y)``,
``h' = r + m``.  The last addition is left to whoever consumes the block's output (the next
block's first norm or the final norm), which fuses it with its normalisation.
"""
from __future__ import annotations

from .base import Block, make_part, register_block


class PreNormBlock(Block):
    def __init__(self, layer_spec):
        self.spec = layer_spec
        self.mixer_norm = make_part("norm", layer_spec.mixer_norm)
        self.mixer = make_part("mixer", layer_spec.mixer)
        self.feed_forward_norm = make_part("norm", layer_spec.feed_forward_norm)
        self.feed_forward = make_part("feed_forward", layer_spec.feed_forward)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def tensor_specs(self):
        out = []
        for p in self.parts():
            out.extend(p.tensor_specs())
        return out

    def load(self, tensors, dtype, device):
        for p in self.parts():
            p.load(tensors, dtype, device)

    def forward(self, x, delta, ctx, cache):
        h, n = self.mixer_norm.forward(x, delta)            # h = x + delta
        a = self.mixer.forward(n, ctx, cache)
        r, n2 = self.feed_forward_norm.forward(h, a)        # r = h + a
        m = self.feed_forward.forward(n2, ctx)
        return r, m                                         # meaning r + m


register_block("prenorm", PreNormBlock)
