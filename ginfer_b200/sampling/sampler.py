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


class Pending:
    """Tokens on their way to the host; ``result()`` waits for them."""

    def __init__(self, host: torch.Tensor, n: int, event, device_tokens=None):
        self._host, self._n, self._event = host, n, event
        self.device_tokens = device_tokens      # int32 [n] on the device, for the step behind

    def result(self) -> list[int]:
        if self._event is not None:
            self._event.synchronize()
        return self._host[:self._n].tolist()


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        cuda = self.device.type == "cuda"
        # two buffers each way, taken in turns: a step's temperatures and uniforms may still be on
        # their way to the device, and its tokens still unread, when the next step is prepared
        self._host = [torch.empty(2 * 1024, dtype=torch.float32, pin_memory=True)
                      for _ in range(2)] if cuda else None
        self._sent = [None, None]            # the copy out of each host buffer has happened
        self._out = [torch.empty(1024, dtype=torch.int32, pin_memory=True) for _ in range(2)] \
            if cuda else None
        self._turn = 0

    def sample_async(self, logits: torch.Tensor, temperatures: list[float], seeds: list[int],
                     indices: list[int]) -> Pending:
        """Launch the choice of a token per row of ``logits [R, V]`` (fp32, on the device) and
        its copy to pinned host memory; row ``r`` belongs to a request with ``temperatures[r]``,
        ``seeds[r]``, generating its token number ``indices[r]``."""
        R = logits.shape[0]
        if R == 0:
            return Pending(torch.empty(0, dtype=torch.int32), 0, None)
        self._turn ^= 1
        if all(t <= 0 for t in temperatures):
            picks = ops.argmax(logits)
        else:
            k = self._turn
            if self._sent[k] is not None:
                self._sent[k].synchronize()          # two steps back: long done
            if 2 * R > self._host[k].numel():
                self._host[k] = torch.empty(4 * R, dtype=torch.float32, pin_memory=True)
            h = self._host[k].numpy()                # [temperatures | uniforms], contiguous
            h[:R] = np.asarray(temperatures, dtype=np.float32)
            h[R:2 * R] = np.asarray([uniform(s, i) for s, i in zip(seeds, indices)],
                                    dtype=np.float32)
            d = self._host[k][:2 * R].to(self.device, non_blocking=True)
            self._sent[k] = torch.cuda.Event()
            self._sent[k].record()
            picks = ops.sample(logits, d[:R], d[R:])
        if R > self._out[self._turn].numel():
            self._out[self._turn] = torch.empty(2 * R, dtype=torch.int32, pin_memory=True)
        out = self._out[self._turn]
        out[:R].copy_(picks, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return Pending(out, R, ev, picks)

    def sample(self, logits: torch.Tensor, temperatures: list[float], seeds: list[int],
               indices: list[int]) -> list[int]:
        return self.sample_async(logits, temperatures, seeds, indices).result()
