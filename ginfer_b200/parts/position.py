"""Position encodings.

Rotary, as the reference computes it (``ginfer/core/op/kernels/cuda/rope_kernel.cu:13-16,61-71``
for the table, ``:84-102`` for the rotation): ``inv_j = 1 / theta^(j / (hd/2))``,
``angle = pos * inv_j`` in fp32, pairs ``(j, j + hd/2)`` rotated by
``o_j = x_j cos - x_{j+hd/2} sin``, ``o_{j+hd/2} = x_j sin + x_{j+hd/2} cos``; applied to queries
and keys, not to values.  Here ``inv_j`` is computed in double and rounded once to fp32, the
product ``float(pos) * inv_j`` is an fp32 product, and cos/sin of that fp32 angle are evaluated
in double and rounded to fp32, so host and device cannot disagree on a table entry.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, register_position


class RotaryPosition(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, max_positions: int,
                 rotary_dim: int | None = None):
        self.head_dim = int(head_dim)
        self.rotary_dim = int(head_dim if rotary_dim is None else rotary_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and <= head_dim "
                             f"{self.head_dim}")
        self.theta = float(theta)
        self.max_positions = int(max_positions)
        self._table: torch.Tensor | None = None

    def load(self, tensors, dtype, device):
        half = self.rotary_dim // 2
        inv = (1.0 / np.power(np.float64(self.theta),
                              np.arange(half, dtype=np.float64) / half)).astype(np.float32)
        pos = np.arange(self.max_positions, dtype=np.float32)
        ang = (pos[:, None] * inv[None, :]).astype(np.float32)      # fp32 product
        ang64 = ang.astype(np.float64)
        table = np.concatenate([np.cos(ang64), np.sin(ang64)], axis=1).astype(np.float32)
        self._table = torch.from_numpy(table).to(device)

    def rotary_table(self):
        return self._table, self.rotary_dim


class NoPosition(PositionEncoding):
    """No position information is added to queries and keys."""

    def __init__(self, **_):
        pass

    def rotary_table(self):
        return None, 0


register_position("rotary", RotaryPosition)
register_position("none", NoPosition)
