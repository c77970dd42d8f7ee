"""Choosing the next token of each request from fp32 logits.

Greedy: arg-max, lowest index among equals.  Temperature: ``softmax(logits / temperature)`` in
fp32 and inverse CDF in index order with a uniform number that is a pure function of the
request's seed and the index of the token being generated, so a request's samples depend neither
on what else is in the batch nor on how its prompt was cut nor on a preemption in between.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed: int, index: int) -> float:
    """A number in [0, 1) from (seed, index); 24 bits, exact in fp32."""
    h = _splitmix64(_splitmix64(seed & _MASK) ^ (index & _MASK))
    return (h >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._host = torch.empty((2, 1024), dtype=torch.float32, pin_memory=True) \
            if self.device.type == "cuda" else None

    def sample(self, logits: torch.Tensor, temperatures: list[float], seeds: list[int],
               indices: list[int]) -> list[int]:
        """``logits [R, V]`` fp32 on the device; row ``r`` belongs to a request with
        ``temperatures[r]``, ``seeds[r]``, generating its token number ``indices[r]``."""
        R = logits.shape[0]
        if R == 0:
            return []
        if all(t <= 0 for t in temperatures):
            return ops.argmax(logits).tolist()
        if R > self._host.shape[1]:
            self._host = torch.empty((2, 2 * R), dtype=torch.float32, pin_memory=True)
        h = self._host.numpy()
        h[0, :R] = np.asarray(temperatures, dtype=np.float32)
        h[1, :R] = np.asarray([uniform(s, i) for s, i in zip(seeds, indices)], dtype=np.float32)
        d = self._host[:, :R].to(self.device, non_blocking=True)
        out = ops.sample(logits, d[0].contiguous(), d[1].contiguous()).tolist()
        return out
