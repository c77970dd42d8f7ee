"""Interfaces of the parts a layer is put together from, and one registry for each family.

A part is built from a :class:`~ginfer_b200.parts.plan.PartSpec` (``kind`` plus parameters), says
which tensors it needs (:meth:`Part.tensor_specs`), receives them (:meth:`Part.load`) and runs on
the tokens of one step.  No part knows which model it is in: sizes and constants arrive as
constructor parameters, per-step facts arrive in a :class:`StepContext`, and a mixer's cache
arrives as a binding made by the cache manager.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from .plan import PartSpec


# ----------------------------------------------------------------------------- tensors of a part
@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part needs.  ``name`` is relative to the part's scope (the layer prefix).
    ``role`` decides how it is kept and how random weights are drawn:

    * ``matrix`` / ``embedding``: operands of matrix products, kept in the compute dtype;
      drawn N(0, 0.02).
    * ``bias``: kept in the compute dtype unless stored in 32-bit, which stays; N(0, 0.02).
    * ``norm``: like ``bias`` but drawn 1 + N(0, 0.02).
    * ``int``: integer table, kept as int32; drawn uniform in ``[0, int_high)``.
    """
    name: str
    shape: tuple[int, ...]
    role: str = "matrix"
    int_high: int = 2


# ----------------------------------------------------------------------------- caches of a mixer
@dataclass(frozen=True)
class PagedKVSpec:
    """What a mixer keeps of every position (``window == 0``) or of the last ``window``
    positions, in pages.  By default keys and values of ``num_kv_heads`` heads of ``head_dim``
    each.  ``planes`` names another lay-out: one ``(heads, width)`` per tensor kept of a token
    (one latent vector: ``((1, width),)``; keys and values of different widths:
    ``((heads, k_width), (heads, v_width))``)."""
    num_kv_heads: int
    head_dim: int
    window: int = 0
    planes: tuple[tuple[int, int], ...] | None = None

    def layout(self) -> tuple[tuple[int, int], ...]:
        return self.planes or ((self.num_kv_heads, self.head_dim),) * 2


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size, kept in a slot; zeroed when a request takes the slot."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class PagedKVBinding:
    # [2, num_pages, page_size, num_kv_heads, head_dim] (0 = K, 1 = V); for a spec with ``planes``
    # a tuple of tensors [num_pages, page_size, heads, width], one per plane
    pages: torch.Tensor | tuple
    block_table: torch.Tensor    # [B, W] int32, logical page -> physical page, -1 where none
    slot_mapping: torch.Tensor   # [T] int32, physical token slot (page * page_size + offset)
    page_size: int
    window: int
    write: bool


@dataclass
class StateBinding:
    state: torch.Tensor          # [num_slots, *shape]
    write: bool


# ----------------------------------------------------------------------------- per-step facts
@dataclass
class StepContext:
    """What one step's batch looks like.  Tokens of all requests are packed: request ``b`` owns
    rows ``cu_seqlens_q[b]:cu_seqlens_q[b+1]``; its tokens sit at absolute positions
    ``q_starts[b] ...`` and after the step the request holds ``kv_lens[b]`` tokens."""
    num_tokens: int
    num_seqs: int
    dtype: torch.dtype
    device: torch.device
    token_ids: torch.Tensor       # [T] int32 (device)
    positions: torch.Tensor       # [T] int32 (device)
    seq_of_token: torch.Tensor    # [T] int32 (device)
    cu_seqlens_q: torch.Tensor    # [B+1] int32 (device)
    kv_lens: torch.Tensor         # [B] int32 (device)
    slot_ids: torch.Tensor        # [B] int32 (device): per-request state slot
    logit_rows: torch.Tensor      # [R] int32 (device): rows whose logits are wanted
    q_lens_host: list[int] = field(default_factory=list)
    q_starts_host: list[int] = field(default_factory=list)
    slot_ids_host: list[int] = field(default_factory=list)
    max_q_len: int = 0
    max_kv_len: int = 0
    decode_only: bool = False
    all_rows_wanted: bool = False  # logit_rows is every row of the step, in order
    capturing: bool = False       # inside CUDA-graph capture: no host syncs, no allocation tricks
    extras: dict[str, Any] = field(default_factory=dict)


# ----------------------------------------------------------------------------- folded norms
@dataclass
class Summed:
    """A hidden state whose last residual addition is done: ``tensor [T, H]`` in fp32, with the
    partial sums of squares of its rows that the product which formed it left behind
    (``sumsq [parts, ld]``), so that a following RMS normalisation needs no pass of its own.
    ``scaled`` is ``tensor * gamma`` in the activation dtype for the norm whose weight is
    ``scaled_by`` (the norm the producer was told comes next), or ``None``."""
    tensor: torch.Tensor
    sumsq: torch.Tensor
    scaled: torch.Tensor | None = None
    scaled_by: torch.Tensor | None = None


@dataclass
class LazyNorm:
    """The RMS normalisation of a :class:`Summed` state, not computed yet: what is there is
    ``scaled = tensor * gamma`` and the sums of squares, and ``norm = scaled / rms`` row by row.
    A product that can multiply its accumulator by ``1 / rms`` takes it as it is (``x W^T / rms``
    is the product of the normalised rows); anything else calls :meth:`materialize`."""
    summed: Summed
    gamma: torch.Tensor
    eps: float
    dtype: torch.dtype

    @property
    def scaled(self) -> torch.Tensor | None:
        s = self.summed
        return s.scaled if s.scaled_by is self.gamma else None

    def materialize(self) -> torch.Tensor:
        from .. import ops
        return ops.add_rmsnorm(self.summed.tensor, None, self.gamma, self.eps, want_sum=False,
                               out_dtype=self.dtype)[1]


# ----------------------------------------------------------------------------- part interfaces
class Part:
    """Base of every part."""

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def load(self, tensors: dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        """Receive the tensors named by :meth:`tensor_specs` (already on ``device``)."""


class Norm(Part):
    def forward(self, x: torch.Tensor, delta: torch.Tensor | None = None,
                rows: torch.Tensor | None = None, want_sum: bool = True, out_dtype=None
                ) -> tuple[torch.Tensor | None, torch.Tensor]:
        """Return ``(s, norm(s))`` with ``s = x + delta`` (``s = x`` if ``delta`` is None), the
        sum formed in 32-bit.  ``rows`` (int32) selects rows of ``x``/``delta`` first.  ``s`` is
        None when ``want_sum`` is false.  ``out_dtype``: the activation dtype of ``norm(s)`` when
        it cannot be read off ``delta`` or ``x``."""
        raise NotImplementedError

    def lazy(self, summed: Summed, dtype: torch.dtype) -> LazyNorm | None:
        """The normalisation of ``summed`` as a :class:`LazyNorm`, if this norm can be folded
        into the product that consumes it; ``None`` otherwise."""
        return None

    def fold_weight(self) -> torch.Tensor | None:
        """The weight ``gamma`` if this norm is ``x * gamma / rms(x)`` and so can be split into a
        multiplication by ``gamma`` in the product before it and one by ``1 / rms`` in the product
        behind it; ``None`` (the default) if it cannot."""
        return None


class PositionEncoding(Part):
    def rotary_table(self) -> tuple[torch.Tensor, int] | None:
        """``(table, rotary_dim)`` if the mixer's cache-write kernel can apply the encoding:
        ``table [max_positions, rotary_dim]`` fp32 holds cos in its first half of columns and sin
        in its second, and the first ``rotary_dim`` channels of every head are rotated in pairs
        ``(j, j + rotary_dim/2)``; ``(None, 0)`` means nothing is to be done.  ``None`` (the
        default) means the encoding has code of its own and :meth:`apply` is called instead."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx: StepContext) -> None:
        """Encode positions in place in ``q [T, heads, head_dim]`` and ``k``; used when
        :meth:`rotary_table` gives nothing."""
        raise NotImplementedError


class Mixer(Part):
    # A mixer (or feed-forward) that sets these takes a LazyNorm as input, and the keywords
    # ``residual`` and ``then``: given a residual it may return ``Summed(residual + output)``
    # instead of its output, with ``scaled`` made for the norm ``then`` (the one that follows).
    takes_lazy_norm = False
    adds_residual = False

    def cache_spec(self) -> PagedKVSpec | StateSpec | None:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    takes_lazy_norm = False
    adds_residual = False

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """An arrangement of a mixer, a feed-forward and norms.  The hidden state travels between
    blocks as ``(x, delta)`` meaning ``x + delta``, so that a block's last addition can be fused
    into the next norm."""

    # A block that sets this takes the keyword ``then``: the norm that will consume its output
    # (the next run's first norm), so that its last product can prepare that norm's input.
    takes_next_norm = False

    def forward(self, x: torch.Tensor, delta: torch.Tensor | None, ctx: StepContext, cache
                ) -> tuple[torch.Tensor, torch.Tensor | None]:
        raise NotImplementedError

    def first_norm(self) -> "Norm | None":
        """The norm this block applies to its input first, if another block may prepare it."""
        return None


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """``x [R, hidden]`` -> logits ``[R, vocab]`` in fp32."""
        raise NotImplementedError


# ----------------------------------------------------------------------------- registries
_FAMILIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_REGISTRY: dict[str, dict[str, Callable[..., Part]]] = {f: {} for f in _FAMILIES}


def register_part(family: str, kind: str, factory: Callable[..., Part]) -> None:
    if family not in _REGISTRY:
        raise KeyError(f"unknown part family '{family}'; families are {_FAMILIES}")
    _REGISTRY[family][kind] = factory


def make_part(family: str, spec: PartSpec, **extra) -> Part:
    try:
        factory = _REGISTRY[family][spec.kind]
    except KeyError:
        raise KeyError(f"no {family} of kind '{spec.kind}' is registered; known: "
                       f"{sorted(_REGISTRY.get(family, {}))}") from None
    return factory(**dict(spec.params), **extra)


def register_mixer(kind, factory):
    register_part("mixer", kind, factory)


def register_feed_forward(kind, factory):
    register_part("feed_forward", kind, factory)


def register_norm(kind, factory):
    register_part("norm", kind, factory)


def register_position(kind, factory):
    register_part("position", kind, factory)


def register_block(kind, factory):
    register_part("block", kind, factory)
