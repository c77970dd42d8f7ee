"""Arrangements of a mixer, a feed-forward and their norms into a layer.

Pre-norm decoder block of the reference (``ginfer/core/layer/transformer/encoder.cc:33-39``):
``x = norm1(h)``, ``a = mixer(x)``, ``r = h + a``, ``y = norm2(r)``, ``m = ffn(y)``,
``h' = r + m``.  The last addition is left to whoever consumes the block's output (the next
block's first norm or the final norm), which fuses it with its normalisation.
"""
from __future__ import annotations

import torch

from .base import Block, Summed, make_part, register_block

# Steps of at most this many tokens fold the additions and normalisations into the neighbouring
# products (the kernels take up to 32).  Measured on a B200 at the 1.5B shape the folded layer is
# slower than the separate norm kernels (q/k/v 6.7 us against 4.4 + 1.9, gate/up 18.2 against
# 12.2 + 1.9: each of the 140 gate/up CTAs normalises the whole operand for itself before its first
# product; the producers pay 1.7 and 3.4 us for the sums of squares), so it is off unless a caller
# raises it.
FOLD_MAX_TOKENS = 0


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
        """``x`` is a tensor (with ``delta`` still to be added) or a :class:`Summed` state.  For
        short bf16 steps the additions and normalisations are folded into the neighbouring
        products where the parts can do that: the mixer's and the feed-forward's last product
        add the residual and leave the statistics of the sum (``Summed``), and their first
        product normalises its own operand (``LazyNorm``)."""
        fold = ctx.dtype == torch.bfloat16 and ctx.num_tokens <= FOLD_MAX_TOKENS
        # the state before the mixer, and its normalisation
        n = None
        if isinstance(x, Summed):
            h = x.tensor
            if fold and self.mixer.takes_lazy_norm:
                n = self.mixer_norm.lazy(x, ctx.dtype)
            if n is None:
                _, n = self.mixer_norm.forward(h, None, out_dtype=ctx.dtype)
        else:
            h, n = self.mixer_norm.forward(x, delta)            # h = x + delta
        if fold and self.mixer.adds_residual:
            a = self.mixer.forward(n, ctx, cache, residual=h if h.dtype == torch.float32
                                   else h.float())
        else:
            a = self.mixer.forward(n, ctx, cache)
        # the state before the feed-forward, and its normalisation
        n2 = None
        if isinstance(a, Summed):
            r = a.tensor
            if fold and self.feed_forward.takes_lazy_norm:
                n2 = self.feed_forward_norm.lazy(a, ctx.dtype)
            if n2 is None:
                _, n2 = self.feed_forward_norm.forward(r, None, out_dtype=ctx.dtype)
        else:
            r, n2 = self.feed_forward_norm.forward(h, a)        # r = h + a
        if fold and self.feed_forward.adds_residual and r.dtype == torch.float32:
            m = self.feed_forward.forward(n2, ctx, residual=r)
        else:
            m = self.feed_forward.forward(n2, ctx)
        if isinstance(m, Summed):
            return m, None
        return r, m                                             # meaning r + m


register_block("prenorm", PreNormBlock)
