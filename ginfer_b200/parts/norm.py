"""RMS normalisation, with the preceding residual addition fused in.

Formula as the reference computes it (``ginfer/core/op/kernels/cuda/rmsnorm_kernel.cu:27-66``):
``ss = sum_j x_j^2``, ``rms = sqrtf(ss / H + eps)``, ``out_j = x_j * gamma_j / rms``, all in fp32
with one cast at the end.  The reference adds residuals in a separate kernel
(``ginfer/core/layer/transformer/encoder.cc:35,39``); here the addition happens in the same
kernel, in fp32, and the sum is written once in the activation dtype.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import LazyNorm, Norm, TensorSpec, register_norm


class RMSNorm(Norm):
    def __init__(self, size: int, eps: float, weight_name: str = "weight"):
        self.size = int(size)
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight: torch.Tensor | None = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, (self.size,), "norm")]

    def load(self, tensors, dtype, device):
        self.weight = tensors[self.weight_name]

    def forward(self, x, delta=None, rows=None, want_sum=True, out_dtype=None):
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, rows=rows, want_sum=want_sum,
                               out_dtype=out_dtype)

    def lazy(self, summed, dtype):
        return LazyNorm(summed, self.weight, self.eps, dtype)

    def fold_weight(self):
        return self.weight


register_norm("rmsnorm", RMSNorm)
