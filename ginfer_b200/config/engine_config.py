"""Engine options.  Names and meanings follow the reference's ``engine::Config``
(``ginfer/engine/config.h:8-21``): ``model_path``, ``max_num_batched_tokens``, ``max_num_seqs``,
``max_seq_len``, ``gpu_memory_utilization``, ``kvcache_block_size``.  Added here: the compute
``dtype``, an explicit page count (``num_kvcache_blocks``; tests use very few so that pages are
used again) and ``enforce_eager`` (no CUDA-graph replay of decode steps).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class EngineConfig:
    model_path: str
    dtype: str = "bfloat16"               # "bfloat16" | "float32"
    max_num_batched_tokens: int = 8192    # token budget of one step
    max_num_seqs: int = 64                # live requests (= per-request state slots)
    max_seq_len: int = 4096               # longest prompt + output of one request
    gpu_memory_utilization: float = 0.8   # share of free memory given to the cache pool
    kvcache_block_size: int = 16          # tokens per cache page
    num_kvcache_blocks: int | None = None  # pages per layer group; None: from free memory
    enforce_eager: bool = False
    device: str = "cuda:0"

    def validate(self) -> None:
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {self.dtype!r}")
        for k in ("max_num_batched_tokens", "max_num_seqs", "max_seq_len", "kvcache_block_size"):
            if getattr(self, k) <= 0:
                raise ValueError(f"{k} must be positive")
        if not (0.0 < self.gpu_memory_utilization <= 1.0):
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
        if self.num_kvcache_blocks is not None and self.num_kvcache_blocks <= 0:
            raise ValueError("num_kvcache_blocks must be positive")
