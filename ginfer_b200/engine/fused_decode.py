"""Decode steps of a recognised stack of layers in one persistent kernel.

The kernel of ``ops/decode_layers.py`` runs one fixed sequence -- RMS norm, joined q/k/v product,
rotary table, paged attention, output product, RMS norm, SiLU-gated feed-forward -- for every
layer of a step of at most 16 requests with one token each.  :func:`recognise` looks at a built
model: if every entry of its run list is exactly that block made of exactly those parts, with one
shape, it returns a :class:`FusedDecode` that the model asks first at every step; anything else
(another mixer, another norm, a subclass that may behave differently, fp32, a longer step) keeps
the path of one kernel per operation.  The parts themselves do not know about it.
"""
from __future__ import annotations

import os

import torch

from ..ops.decode_layers import DecodeLayers, LayerTensors, NotServed
from ..parts.attention import Attention
from ..parts.base import PagedKVBinding, StepContext
from ..parts.block import PreNormBlock
from ..parts.embedding import TokenEmbedding
from ..parts.feed_forward import SwiGLU
from ..parts.norm import RMSNorm


def enabled() -> bool:
    """Off unless ``GINFER_B200_FUSED_DECODE=1``: measured on a B200 at the 1.5B shape, a layer
    takes about 110 us in the persistent kernel against 54 us as separate launches (its eight
    worker warps an SM are bound by instruction latency between the grid barriers), so the
    separate kernels stay the serving path."""
    return os.environ.get("GINFER_B200_FUSED_DECODE", "0") == "1"


class FusedDecode:
    def __init__(self, model, blocks: list[PreNormBlock]):
        self.model = model
        self.blocks = blocks                       # in run order
        a: Attention = blocks[0].mixer
        self.shape = (a.hidden_size, a.num_heads, a.num_kv_heads, a.head_dim,
                      blocks[0].feed_forward.intermediate_size)
        table = a.position.rotary_table()
        self.rope, self.rot = (None, 0) if table is None else table
        self.scale = a.scale
        self.kernel: DecodeLayers | None = None
        self._page_size = None
        self._cache_sig = None
        self.refused: str | None = None            # why the kernel does not take this model

    # ------------------------------------------------------------------ set-up
    def _build(self, page_size: int, device) -> None:
        H, nh, nkv, hd, I = self.shape
        k = DecodeLayers(len(self.blocks), H, nh, nkv, hd, I, page_size, self.rot, self.scale,
                         device)
        for i, b in enumerate(self.blocks):
            a, f = b.mixer, b.feed_forward
            k.set_layer(i, LayerTensors(
                w_qkv=a.qkv.weight, w_out=a.out.weight, w_gate_up=f.gate_up.proj.weight,
                w_down=f.down.weight, b_qkv=a.qkv._bias_f32, b_out=a.out._bias_f32,
                b_down=f.down._bias_f32, gamma_mixer=b.mixer_norm.weight,
                eps_mixer=b.mixer_norm.eps, gamma_ff=b.feed_forward_norm.weight,
                eps_ff=b.feed_forward_norm.eps))
        self.kernel, self._page_size, self._cache_sig = k, page_size, None

    def _bind(self, bindings: list[PagedKVBinding]) -> list[torch.Tensor]:
        """Tell the kernel where each layer's pages are (once: they do not move) and return this
        step's block tables, one per cache group."""
        tables: list[torch.Tensor] = []
        index: dict[int, int] = {}
        sig = []
        for b in bindings:
            key = b.block_table.data_ptr()
            if key not in index:
                index[key] = len(tables)
                tables.append(b.block_table)
            sig.append((b.pages.data_ptr(), index[key], int(b.window), bool(b.write)))
        if sig != self._cache_sig:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("fused decode: cache bindings changed during graph capture")
            for i, (b, s) in enumerate(zip(bindings, sig)):
                self.kernel.set_cache(i, b.pages[0], b.pages[1], s[1], s[2], s[3])
            self.kernel.upload()
            self._cache_sig = sig
        return tables

    # ------------------------------------------------------------------ a step
    def layers(self, ctx: StepContext, bind_cache):
        """The fp32 residual stream after the last layer, or ``None`` if this step is not one
        the kernel takes."""
        if self.refused or not enabled():
            return None
        if not ctx.decode_only or ctx.dtype != torch.bfloat16 or \
                not 1 <= ctx.num_tokens <= DecodeLayers.MAX_TOKENS or ctx.num_seqs != ctx.num_tokens:
            return None
        bindings = [bind_cache(e) for e in self.model.plan.run]
        if any(not isinstance(b, PagedKVBinding) for b in bindings):
            return None
        page_size = bindings[0].page_size
        try:
            if self.kernel is None or self._page_size != page_size:
                if torch.cuda.is_current_stream_capturing():
                    return None
                self._build(page_size, ctx.device)
            tables = self._bind(bindings)
            if len(tables) > DecodeLayers.MAX_GROUPS:
                raise NotServed(f"{len(tables)} cache groups")
        except NotServed as e:
            self.refused = str(e)
            return None
        return self.kernel.run(ctx.num_tokens, ctx.positions, self.rope, tables,
                               token_ids=ctx.token_ids, embedding=self.model.embedding.weight)


def recognise(model) -> FusedDecode | None:
    """A :class:`FusedDecode` for ``model`` if every run of its plan is the block the kernel
    implements, else ``None``.  Exact types only: a subclass may compute something else."""
    if getattr(model, "dtype", None) != torch.bfloat16 or type(model.embedding) is not TokenEmbedding:
        return None
    if model.embedding.weight.dtype != torch.bfloat16 or not model.plan.run:
        return None
    blocks = [model.blocks[e.layer] for e in model.plan.run]
    first = None
    for b in blocks:
        if type(b) is not PreNormBlock or type(b.mixer) is not Attention or \
                type(b.feed_forward) is not SwiGLU or type(b.mixer_norm) is not RMSNorm or \
                type(b.feed_forward_norm) is not RMSNorm:
            return None
        a, f = b.mixer, b.feed_forward
        if a.qkv is None or a.qkv.dtype != torch.bfloat16:
            return None
        table = a.position.rotary_table()
        shape = (a.hidden_size, a.num_heads, a.num_kv_heads, a.head_dim, f.intermediate_size,
                 a.scale, None if table is None else (tuple(table[0].shape), table[1]))
        if first is None:
            first, first_table = shape, table
        elif shape != first or (table is not None and not torch.equal(table[0], first_table[0])):
            return None                                # the kernel reads one rotary table
    return FusedDecode(model, blocks)
