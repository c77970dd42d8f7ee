"""Device memory of the cache: page tensors per layer group and state tensors per slot.

The reference allocates one tensor ``[2, L, num_blocks, block, nkv, hd]`` sized from free memory
(``ginfer/engine/model_runner.cc:52-87``).  Here caches with the same needs (what a token keeps,
window) form a group with one tensor ``[caches, 2, num_pages, page, nkv, hd]``; a cache's K and V
pages are ``tensor[i, 0]`` and ``tensor[i, 1]``.  A group whose spec names its own planes has one
tensor ``[caches, num_pages, page, heads, width]`` per plane instead.  Mixers with state of fixed
size get a tensor ``[num_slots + 1, *shape]`` each: the last slot belongs to no request (the rows
that pad a step up to a CUDA graph's batch size read and write there, as they do on the page
that no request owns).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import PagedKVSpec, StateSpec


@dataclass(frozen=True)
class GroupLayout:
    planes: tuple[tuple[int, int], ...]       # (heads, width) of every tensor kept of a token
    stacked: bool                             # the default lay-out: K and V in one tensor
    window: int
    cache_ids: tuple[int, ...]

    def bytes_per_page(self, page_size: int, itemsize: int) -> int:
        per_token = sum(h * w for h, w in self.planes)
        return len(self.cache_ids) * page_size * per_token * itemsize

    def pages_for(self, max_num_seqs: int, max_seq_len: int, max_step_tokens: int,
                  page_size: int) -> int:
        """The most pages this group can hold at once: every slot filled to ``max_seq_len``; for
        a windowed group what ``max_num_seqs`` requests keep live of their windows (pages that
        hold a position ``> len - window``) plus the pages of one step's new tokens."""
        full = max_num_seqs * (-(-max_seq_len // page_size))
        if self.window <= 0:
            return full
        live = max_num_seqs * (-(-max(self.window - 1, 0) // page_size) + 2)
        return min(full, live + -(-max_step_tokens // page_size))


def plan_groups(cache_specs: dict[int, object]) -> tuple[list[GroupLayout], dict[int, int]]:
    """Group paged caches by their needs; returns the groups and cache id -> group index."""
    by_key: dict[tuple, list[int]] = {}
    for cid in sorted(cache_specs):
        s = cache_specs[cid]
        if isinstance(s, PagedKVSpec):
            by_key.setdefault((s.layout(), s.planes is None, s.window), []).append(cid)
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
        self.kv = []
        for g, n in zip(groups, num_pages):
            if g.stacked:
                heads, width = g.planes[0]
                self.kv.append(torch.zeros((len(g.cache_ids), 2, n + 1, page_size, heads, width),
                                           dtype=dtype, device=device))
            else:
                self.kv.append(tuple(
                    torch.zeros((len(g.cache_ids), n + 1, page_size, heads, width), dtype=dtype,
                                device=device) for heads, width in g.planes))
        self._where = {cid: (gi, i) for gi, g in enumerate(groups)
                       for i, cid in enumerate(g.cache_ids)}
        self.num_slots = num_slots
        self.state = {cid: torch.zeros((num_slots + 1, *s.shape), dtype=s.dtype, device=device)
                      for cid, s in cache_specs.items() if isinstance(s, StateSpec)}

    def group_of(self, cache_id: int) -> int:
        return self._where[cache_id][0]

    @property
    def scratch_slot(self) -> int:
        return self.num_slots

    def pages_of(self, cache_id: int):
        gi, i = self._where[cache_id]
        if self.groups[gi].stacked:
            return self.kv[gi][i]
        return tuple(t[i] for t in self.kv[gi])

    def is_paged(self, cache_id: int) -> bool:
        return cache_id in self._where

    def reset_slot(self, slot: int) -> None:
        for t in self.state.values():
            t[slot].zero_()
