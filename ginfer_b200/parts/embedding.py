"""Token embedding and output head.

Embedding: ``h[t, :] = E[ids[t], :]`` (``ginfer/core/op/kernels/cuda/embedding_kernel.cu:16-24``).
Head: the rows that want logits are selected first and only those are projected
(``ginfer/core/layer/transformer/lmhead.cc:15-27``); a tied head shares the embedding matrix
(``ginfer/model/qwen2.cc:42-46``).  Logits leave in fp32.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Embedding, Head, TensorSpec, register_part


class TokenEmbedding(Embedding):
    def __init__(self, vocab_size: int, hidden_size: int, name: str = "model.embed_tokens.weight"):
        self.vocab_size, self.hidden_size, self.name = int(vocab_size), int(hidden_size), name
        self.weight: torch.Tensor | None = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), "embedding")]

    def load(self, tensors, dtype, device):
        self.weight = tensors[self.name]

    def forward(self, token_ids, ctx):
        return ops.embedding(token_ids, self.weight)


class LinearHead(Head):
    """``tied_to`` names the tensor of another part (the embedding) to share; otherwise the head
    has a matrix ``name`` of its own."""

    def __init__(self, vocab_size: int, hidden_size: int, name: str = "lm_head.weight",
                 tied_to: str | None = None):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.name, self.tied_to = name, tied_to
        self.proj = None

    def tensor_specs(self):
        if self.tied_to:
            return []
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size), "matrix")]

    def load(self, tensors, dtype, device):
        self.proj = ops.Linear(tensors[self.tied_to or self.name], None, out_dtype=torch.float32)

    def forward(self, x, ctx):
        return self.proj(x)


register_part("embedding", "token", TokenEmbedding)
register_part("head", "linear", LinearHead)
