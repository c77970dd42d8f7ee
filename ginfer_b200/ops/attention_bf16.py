"""bf16 attention kernels for the serving path: split-KV decode and tensor-core prefill."""
from __future__ import annotations


def try_run(qkv, pages, block_table, ctx, nh, nkv, hd, scale, window, page_size):
    """Run a bf16 kernel if one takes this head size and batch shape; ``None`` otherwise."""
    return None
