"""Grouped-query attention over a paged cache.

Order of work in the reference (``ginfer/core/layer/transformer/attention.cc:45-82``): q/k/v
projections (bias on q, k, v and none on o for Qwen2: ``ginfer/model/qwen2.cc:15-17``), rotary
encoding of q and k, K/V written to their cache slots, attention over the cache, output
projection.  Scores: key ``c`` is visible to the query at position ``p`` iff ``c <= p``
(``flash_gqa_varlen_kernel.cu:202,214`` writes this as ``c <= r + kv_len - q_len``), scale
``1/sqrt(head_dim)``, query head ``n`` reads kv head ``n / (heads / kv_heads)``
(``flash_gqa_varlen_kernel.cu:439``).  A sliding window, which the reference lacks, adds
``p - c < window``.

Here q, k and v come from one product over joined weights; one kernel rotates q in place,
rotates k into its page and copies v into its page; softmax statistics stay in fp32.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from .base import Mixer, PagedKVSpec, Summed, TensorSpec, make_part, register_mixer
from .plan import PartSpec


class Attention(Mixer):
    takes_lazy_norm = True        # the joined q/k/v product normalises its own operand
    adds_residual = True          # the output product adds the residual and leaves statistics

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, window: int = 0, qkv_bias: bool = True,
                 out_bias: bool = False, prefix: str = "self_attn", scale: float | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.window = int(window)
        self.qkv_bias = bool(qkv_bias)
        self.out_bias = bool(out_bias)
        self.prefix = prefix + "." if prefix else ""
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = make_part("position", position)
        self.qkv = None
        self.out = None

    # ------------------------------------------------------------------ tensors
    def _key(self, proj: str, what: str) -> str:
        return f"{self.prefix}{proj}_proj.{what}"

    def tensor_specs(self):
        h, nh, nkv, hd = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim
        specs = [TensorSpec(self._key("q", "weight"), (nh * hd, h)),
                 TensorSpec(self._key("k", "weight"), (nkv * hd, h)),
                 TensorSpec(self._key("v", "weight"), (nkv * hd, h)),
                 TensorSpec(self._key("o", "weight"), (h, nh * hd))]
        if self.qkv_bias:
            specs += [TensorSpec(self._key("q", "bias"), (nh * hd,), "bias"),
                      TensorSpec(self._key("k", "bias"), (nkv * hd,), "bias"),
                      TensorSpec(self._key("v", "bias"), (nkv * hd,), "bias")]
        if self.out_bias:
            specs.append(TensorSpec(self._key("o", "bias"), (self.hidden_size,), "bias"))
        specs += self.position.tensor_specs()
        return specs

    def load(self, tensors, dtype, device):
        w = torch.cat([tensors[self._key(p, "weight")] for p in "qkv"], dim=0)
        b = None
        if self.qkv_bias:
            bs = [tensors[self._key(p, "bias")] for p in "qkv"]
            bdt = torch.float32 if any(x.dtype == torch.float32 for x in bs) else bs[0].dtype
            b = torch.cat([x.to(bdt) for x in bs], dim=0)
        self.qkv = ops.Linear(w, b)
        self.out = ops.Linear(tensors[self._key("o", "weight")],
                              tensors[self._key("o", "bias")] if self.out_bias else None)
        self.position.load(tensors, dtype, device)

    # ------------------------------------------------------------------ cache and step
    def cache_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window)

    def forward(self, x, ctx, cache, residual=None, then=None):
        nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        fused = self.position.rotary_table()
        if fused is not None and cache.write and not hasattr(x, "materialize"):
            # many tokens: one kernel multiplies, adds the bias, rotates q and k and writes the cache
            qkv = ops.qkv_rope_write(x, self.qkv, fused[0], fused[1], ctx.positions,
                                     cache.slot_mapping, cache.pages, nh, nkv, hd)
            if qkv is not None:
                o = ops.paged_attention(qkv, cache.pages, cache.block_table, ctx, nh, nkv, hd,
                                        self.scale, cache.window, cache.page_size)
                return self._project(o, residual, then)
        qkv = self.qkv(x)                                         # [T, (nh + 2 nkv) hd]
        if fused is None:                                         # an encoding with code of its own
            q = qkv[:, :nh * hd].unflatten(1, (nh, hd))
            k = qkv[:, nh * hd:(nh + nkv) * hd].unflatten(1, (nkv, hd))
            self.position.apply(q, k, ctx)
            table, rot = None, 0
        else:
            table, rot = fused
        if fused is not None and ops.attention_fuses_rope(qkv, ctx, nh, nkv, hd):
            # decode steps: the attention kernel rotates q and k and writes the cache itself
            o = ops.paged_attention(qkv, cache.pages, cache.block_table, ctx, nh, nkv, hd,
                                    self.scale, cache.window, cache.page_size,
                                    rope=(table, rot, cache.write))
        else:
            ops.rope_kv_write(qkv, table, rot, ctx.positions,
                              cache.slot_mapping if cache.write else None,
                              cache.pages, nh, nkv, hd)
            o = ops.paged_attention(qkv, cache.pages, cache.block_table, ctx, nh, nkv, hd,
                                    self.scale, cache.window, cache.page_size)
        return self._project(o, residual, then)

    def _project(self, o, residual, then):
        if residual is not None:
            s = ops.add_to(self.out, o, residual, then.fold_weight() if then is not None else None)
            if s is not None:
                return Summed(*s)
        return self.out(o)


register_mixer("attention", Attention)
