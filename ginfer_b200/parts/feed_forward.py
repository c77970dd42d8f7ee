"""Feed-forward parts.

SwiGLU as the reference computes it (``ginfer/core/layer/transformer/feedforward.cc:22-25``,
``ginfer/core/op/kernels/cuda/swiglu_kernel.cu:24-27``): ``g = y W_g^T``, ``u = y W_u^T``,
``z = (g * 1/(1+exp(-g))) * u`` in fp32, ``m = z W_d^T``; no biases.  Gate and up weights are
joined at load into one matrix so that one product reads ``y`` once.
"""
from __future__ import annotations

from .. import ops
from .base import FeedForward, Summed, TensorSpec, register_feed_forward


class SwiGLU(FeedForward):
    takes_lazy_norm = True
    adds_residual = True

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "mlp",
                 gate_name: str = "gate_proj", up_name: str = "up_proj",
                 down_name: str = "down_proj"):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        p = prefix + "." if prefix else ""
        self.gate_key = f"{p}{gate_name}.weight"
        self.up_key = f"{p}{up_name}.weight"
        self.down_key = f"{p}{down_name}.weight"
        self.gate_up = None
        self.down = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return [TensorSpec(self.gate_key, (i, h)), TensorSpec(self.up_key, (i, h)),
                TensorSpec(self.down_key, (h, i))]

    def load(self, tensors, dtype, device):
        self.gate_up = ops.GatedLinear(tensors[self.gate_key], tensors[self.up_key])
        self.down = ops.Linear(tensors[self.down_key])

    def forward(self, x, ctx, residual=None, then=None):
        z = self.gate_up(x)            # silu(gate) * up, [T, intermediate]
        if residual is not None:
            s = ops.add_to(self.down, z, residual,
                           then.fold_weight() if then is not None else None)
            if s is not None:
                return Summed(*s)
        return self.down(z)


register_feed_forward("swiglu", SwiGLU)
