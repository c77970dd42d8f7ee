"""Device memory of the cache: page tensors per layer group and state tensors per slot.

The reference allocates one tensor ``[2, L, num_blocks, block, nkv, hd]`` sized from free memory
(``ginfer/engine/model_runner.cc:52-87``).  Here caches with the same needs (kv heads, head size,
window) form a group with one tensor ``[caches, 2, num_pages, page, nkv, hd]``; a cache's K and V
pages are ``tensor[i, 0]`` and ``tensor[i, 1]``.  Mixers with state of fixed size get a tensor
``[num_slots, *shape]`` each.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import PagedKVSpec, StateSpec


@dataclass(frozen=True)
class GroupLayout:
    num_kv_heads: int
    head_dim: int
    window: int
    cache_ids: tuple[int, ...]

    def bytes_per_page(self, page_size: int, itemsize: int) -> int:
        return len(self.cache_ids) * 2 * page_size * self.num_kv_heads * self.head_dim * itemsize


def plan_groups(cache_specs: dict[int, object]) -> tuple[list[GroupLayout], dict[int, int]]:
    """Group paged caches by their needs; returns the groups and cache id -> group index."""
    by_key: dict[tuple, list[int]] = {}
    for cid in sorted(cache_specs):
        s = cache_specs[cid]
        if isinstance(s, PagedKVSpec):
            by_key.setdefault((s.num_kv_heads, s.head_dim, s.window), []).append(cid)
    groups = [GroupLayout(k[0], k[1], k[2], tuple(v)) for k, v in by_key.items()]
    where = {cid: g for g, gl in enumerate(groups) for cid in gl.cache_ids}
    return groups, where


class CacheStorage:
    def __init__(self, cache_specs: dict[int, object], groups: list[GroupLayout],
                 num_pages: list[int], page_size: int, num_slots: int, dtype: torch.dtype,
                 device):
        self.groups = groups
        self.page_size = page_size
        self.num_pages = list(num_pages)
        # one page more than the manager hands out: page `n` of a group belongs to no request; the
        # rows that pad a step up to a CUDA graph's batch size write and read there
        self.kv = [torch.zeros((len(g.cache_ids), 2, n + 1, page_size, g.num_kv_heads,
                                g.head_dim), dtype=dtype, device=device)
                   for g, n in zip(groups, num_pages)]
        self._where = {cid: (gi, i) for gi, g in enumerate(groups)
                       for i, cid in enumerate(g.cache_ids)}
        self.state = {cid: torch.zeros((num_slots, *s.shape), dtype=s.dtype, device=device)
                      for cid, s in cache_specs.items() if isinstance(s, StateSpec)}

    def group_of(self, cache_id: int) -> int:
        return self._where[cache_id][0]

    def pages_of(self, cache_id: int) -> torch.Tensor:
        gi, i = self._where[cache_id]
        return self.kv[gi][i]

    def is_paged(self, cache_id: int) -> bool:
        return cache_id in self._where

    def reset_slot(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()
