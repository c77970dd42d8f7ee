"""Arrangements of a mixer, a feed-forward and their norms into a layer.

Pre-norm decoder block of the reference (``ginfer/core/layer/transformer/encoder.cc:33-39``):
``x = norm1(h)``, ``a = mixer(x)``, ``r = h + a``, ``y = norm2(r)``, ``m = ffn(y)``,
``h' = r + m``.  The last addition is left to whoever consumes the block's output (the next
block's first norm or the final norm), which fuses it with its normalisation.
"""
from __future__ import annotations

import os

import torch

from .base import Block, Summed, make_part, register_block

# Steps of at most this many tokens (bfloat16) fold the additions and normalisations into the
# neighbouring products: the product before a norm leaves the sum, its product with the norm's
# weight and partial sums of squares, the product behind it divides by the rms, and a layer of a
# decode step is 5 kernels (q/k/v, attention, output, gate/up, down) instead of 7.  Off (0) by
# default: on a B200 at the 1.5B shape, batch 8, the step takes 1.245 ms with it against 1.213 ms
# without.  The kernels of a step overlap (each starts, and loads its weights, while the one
# before still runs): the two norm kernels cost 3.1 us each, but they are also 6 us in which the
# products behind them fetch weights, and the epilogues that replace them lengthen the products
# (+0.9 us the output product, +2.4 us q/k/v) on the path every token waits for.
FOLD_MAX_TOKENS = int(os.environ.get("GINFER_B200_FOLD_MAX_TOKENS", "0"))


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

    takes_next_norm = True

    def first_norm(self):
        return self.mixer_norm

    def load(self, tensors, dtype, device):
        for p in self.parts():
            p.load(tensors, dtype, device)

    def forward(self, x, delta, ctx, cache, then=None):
        """``x`` is a tensor (with ``delta`` still to be added) or a :class:`Summed` state.  For
        short bf16 steps the additions and normalisations are folded into the neighbouring
        products where the parts can do that: the mixer's and the feed-forward's last product
        add the residual, leave the statistics of the sum and its product with the next norm's
        weight (``Summed``), and their first product divides by the rms (``LazyNorm``).
        ``then``: the norm that consumes this block's output."""
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
            a = self.mixer.forward(n, ctx, cache, then=self.feed_forward_norm,
                                   residual=h if h.dtype == torch.float32 else h.float())
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
        if fold and then is not None and self.feed_forward.adds_residual \
                and r.dtype == torch.float32:
            m = self.feed_forward.forward(n2, ctx, residual=r, then=then)
        else:
            m = self.feed_forward.forward(n2, ctx)
        if isinstance(m, Summed):
            return m, None
        return r, m                                             # meaning r + m


register_block("prenorm", PreNormBlock)
