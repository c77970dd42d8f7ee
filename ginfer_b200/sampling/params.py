"""Sampling options of a request.

The reference has ``max_tokens = 64`` and ``ignore_eos = false`` and samples by arg-max only
(``ginfer/engine/sampling_params.h:5-8``, ``ginfer/model/model.cc:219-220``).  Added here:
``temperature`` (0 means arg-max) and ``seed``.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    max_tokens: int = 64
    ignore_eos: bool = False
    temperature: float = 0.0
    seed: int | None = None

    def validate(self) -> None:
        if self.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
