"""The step function: one batch of (request, its next tokens) through the model, from the cache.

Reference: ``ginfer/engine/model_runner.cc``.  Its ``run(seqs, is_prefill)`` takes either whole
prompts or single decode tokens, never both (``model_runner.cc:300-317``), builds ``input_ids``,
``positions``, ``cu_seqlens``, ``slot_mapping`` and ``block_tables`` on the host and copies each
separately (``:177-298``), and returns arg-max ids.  Here one step takes any mix of prompt
portions and decode tokens, packs all per-step integers into one pinned buffer copied once, runs
only the given tokens against what earlier steps left in the cache, and returns fp32 logits at the
rows asked for.  Sampling is a separate stage.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import CacheStorage, NativeCacheManager, OutOfPages, plan_groups
from ..parts.base import PagedKVBinding, StateBinding, StepContext
from ..parts.model import DecoderModel


@dataclass
class StepEntry:
    request_id: object
    tokens: list[int]
    want: list[int] = field(default_factory=list)    # indices into ``tokens``


def _align4(n: int) -> int:
    return (n + 3) & ~3


GRAPH_WIDTH_STEP = 64        # block-table widths of graph-replayed steps, in pages
# Steps with prompt portions are replayed from a graph when the same shape (portion lengths, table
# width, wanted rows) comes a second time: whole-budget portions of long prompts do.  Only steps
# of at most this many requests and at least this many tokens, and this many graphs at most.
PORTION_GRAPH_MAX_SEQS = 4
PORTION_GRAPH_MIN_TOKENS = 256
PORTION_GRAPH_LIMIT = 16


@dataclass
class _StepGraph:
    graph: object
    ints: torch.Tensor            # static device buffer the graph's kernels read
    spans: dict
    logits: torch.Tensor
    launches: int


class ModelRunner:
    def __init__(self, model: DecoderModel, *, page_size: int, max_num_seqs: int,
                 max_seq_len: int, num_pages: int | None = None,
                 gpu_memory_utilization: float = 0.8, max_num_batched_tokens: int = 8192,
                 enforce_eager: bool = True):
        if model.device is None or model.device.type != "cuda":
            raise RuntimeError("the model must be loaded on a CUDA device before a runner is made")
        self.model = model
        self.device = model.device
        self.dtype = model.dtype
        self.page_size = int(page_size)
        self.max_seq_len = min(int(max_seq_len), model.plan.max_positions)
        self.max_num_seqs = int(max_num_seqs)
        self.max_num_batched_tokens = int(max_num_batched_tokens)
        self.enforce_eager = bool(enforce_eager)
        specs = model.cache_specs()
        self.groups, self._group_of_cache = plan_groups(specs)
        itemsize = torch.empty((), dtype=self.dtype).element_size()
        counts = self._page_counts(num_pages, gpu_memory_utilization, itemsize)
        self.cache = NativeCacheManager([g.window for g in self.groups], counts, self.page_size,
                                        self.max_num_seqs, self.max_seq_len)
        self.storage = CacheStorage(specs, self.groups, counts, self.page_size,
                                    self.max_num_seqs, self.dtype, self.device)
        self.vocab_size = model.plan.vocab_size
        self._host = None            # pinned staging for the step's integers
        self._host_cap = 0
        self._graphs: dict = {}
        self._portion_seen: dict = {}     # shapes of steps with prompt portions -> times seen
        self._graph_pool = None
        self._copied = torch.cuda.Event()     # the last copy out of the staging buffer
        self._copy_pending = False
        self.steps_run = 0
        self.h2d_bytes = 0            # bytes of step integers copied to the device so far
        self.graph_launches = 0       # kernel launches replayed from CUDA graphs so far

    def _page_counts(self, num_pages, utilization: float, itemsize: int) -> list[int]:
        """Pages for every cache group.  A group never gets more than it can hold at once
        (:meth:`GroupLayout.pages_for`: a windowed group needs few).  ``num_pages``: a count for
        every group, or one per group, or ``None``: the share ``utilization`` of the free device
        memory is divided so that the groups can hold the same number of tokens, what the
        windowed groups do not need going to the others."""
        caps = [g.pages_for(self.max_num_seqs, self.max_seq_len, self.max_num_batched_tokens,
                            self.page_size) for g in self.groups]
        if num_pages is not None:
            asked = list(num_pages) if isinstance(num_pages, (list, tuple)) \
                else [num_pages] * len(self.groups)
            if len(asked) != len(self.groups):
                raise ValueError(f"{len(asked)} page counts for {len(self.groups)} cache groups")
            return [max(1, min(int(n), cap)) for n, cap in zip(asked, caps)]
        free, _total = torch.cuda.mem_get_info(self.device)
        budget = int(free * utilization)
        per_page = [g.bytes_per_page(self.page_size, itemsize) for g in self.groups]
        counts = [0] * len(self.groups)
        open_groups = list(range(len(self.groups)))
        while open_groups:          # equal counts for the groups still open; the capped ones leave
            share = budget // max(1, sum(per_page[g] for g in open_groups))
            capped = [g for g in open_groups if caps[g] <= share]
            if not capped:
                for g in open_groups:
                    counts[g] = max(1, share)
                break
            for g in capped:
                counts[g] = caps[g]
                budget -= caps[g] * per_page[g]
                open_groups.remove(g)
        return counts

    # ------------------------------------------------------------------ requests
    def end(self, request_id) -> None:
        """The request is finished: its pages and its slot are given back."""
        if self.cache.has(request_id):
            self.cache.release(request_id)

    def preempt(self, request_id) -> None:
        """Give the request's pages back but keep its slot; it will be computed again."""
        self.cache.release(request_id, keep_slot=True)

    # ------------------------------------------------------------------ the step
    def _staging(self, n_ints: int) -> torch.Tensor:
        if n_ints > self._host_cap:
            self._host_cap = max(2 * n_ints, 4096)
            self._host = torch.empty(self._host_cap, dtype=torch.int32, pin_memory=True)
        return self._host

    def prepare(self, entries: list[StepEntry]):
        """Admit new requests, take pages, and lay out the step's integers on the host.
        Returns ``(host_arrays, facts)``; nothing has touched the device yet."""
        cache, P = self.cache, self.page_size
        B = len(entries)
        if B == 0:
            raise ValueError("a step needs at least one entry")
        if B > self.max_num_seqs:
            raise ValueError(f"{B} entries in one step; max_num_seqs is {self.max_num_seqs}")
        ids = [e.request_id for e in entries]
        if len(set(ids)) != B:
            raise ValueError("a request appears twice in one step")
        q_lens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int64, count=B)
        if (q_lens <= 0).any():
            raise ValueError("an entry brings no tokens")
        T = int(q_lens.sum())
        if T > self.max_num_batched_tokens:
            raise ValueError(f"a step of {T} tokens; max_num_batched_tokens is "
                             f"{self.max_num_batched_tokens} (the cache pools are sized for it)")
        # pages: check the whole step before taking any (one call into the native manager)
        slots = np.fromiter((cache.requests[i].slot if i in cache.requests else -1 for i in ids),
                            dtype=np.int32, count=B)
        need, over = cache.step_need(slots, q_lens)
        if over >= 0:
            e = entries[over]
            have = cache.get(e.request_id).num_tokens if cache.has(e.request_id) else 0
            raise ValueError(f"request {e.request_id!r} would reach {have + int(q_lens[over])} "
                             f"tokens; the limit is {self.max_seq_len}")
        new = [e.request_id for e, sl in zip(entries, slots) if sl < 0]
        if len(new) > cache.slots.num_free:
            raise RuntimeError(f"{len(new)} new requests but {cache.slots.num_free} free slots")
        for g, (k, f) in enumerate(zip(need, cache.free_pages())):
            if k > f:
                raise OutOfPages(f"the step needs {k} pages of group {g}; {f} are free")
        for rid in new:
            cache.admit(rid)
        if new:
            slots = np.fromiter((cache.requests[i].slot for i in ids), dtype=np.int32, count=B)
        q_starts = cache.lengths(slots).astype(np.int64)
        if self.storage.state:
            for sl, n0 in zip(slots, q_starts):
                if n0 == 0:                  # a sequence starts (again): its state starts at zero
                    self.storage.reset_slot(int(sl))
        cache.reserve_step(slots, q_lens)

        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64).reshape(-1)
                                 for e in entries])
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(q_lens, out=cu[1:])
        seq_of_token = np.repeat(np.arange(B), q_lens)
        positions = np.arange(T) - np.repeat(cu[:-1] - q_starts, q_lens)
        kv_lens = q_starts + q_lens
        slot_ids = slots.astype(np.int64)
        rows = []
        for b, e in enumerate(entries):
            for w in e.want:
                if not (0 <= int(w) < q_lens[b]):
                    raise ValueError(f"request {e.request_id!r} wants logits at place {w} of "
                                     f"{q_lens[b]} tokens")
                rows.append(cu[b] + int(w))
        logit_rows = np.asarray(rows, dtype=np.int64)
        width = int(-(-int(kv_lens.max()) // P))
        decode_only = int(q_lens.max()) == 1
        graphable = decode_only or (B <= PORTION_GRAPH_MAX_SEQS and T >= PORTION_GRAPH_MIN_TOKENS)
        if graphable and not self.enforce_eager:
            # such steps are replayed from CUDA graphs, one per (shape, table width): widths come
            # in steps of GRAPH_WIDTH_STEP pages so that few graphs are needed.  Steps with
            # portions take the next power of two of such steps (the portions of one long prompt
            # then share a handful of graphs; nothing in such a step is chosen by the width, while
            # a decode step splits its keys by it).
            steps = -(-width // GRAPH_WIDTH_STEP)
            if not decode_only:
                steps = 1 << (steps - 1).bit_length()
            width = min(cache.table_width, steps * GRAPH_WIDTH_STEP)
        slots_of_token = slot_ids[seq_of_token]
        slot_maps = [cache.slot_mapping(g, slots_of_token, positions)
                     for g in range(cache.num_groups)]
        tables = [cache.block_table(g, slot_ids, width) for g in range(cache.num_groups)]
        arrays = dict(token_ids=tokens, positions=positions, seq_of_token=seq_of_token,
                      cu_seqlens_q=cu, kv_lens=kv_lens, slot_ids=slot_ids, logit_rows=logit_rows)
        for g in range(cache.num_groups):
            arrays[f"slot_mapping{g}"] = slot_maps[g]
            arrays[f"block_table{g}"] = tables[g]
        all_rows = len(rows) == T and all(int(r) == i for i, r in enumerate(rows))
        facts = dict(T=T, B=B, q_lens=q_lens, q_starts=q_starts, slot_ids=slot_ids, width=width,
                     all_rows=all_rows,
                     max_q_len=int(q_lens.max()), max_kv_len=int(kv_lens.max()))
        return arrays, facts

    def _pack(self, arrays: dict[str, np.ndarray]):
        """Lay the arrays out in the pinned staging buffer; returns (host view, spans)."""
        total = sum(_align4(a.size) for a in arrays.values())
        if self._copy_pending:                # do not overwrite what the last copy still reads
            self._copied.synchronize()
        host = self._staging(total)
        hnp = host.numpy()
        off, spans = 0, {}
        for k, a in arrays.items():
            n = a.size
            hnp[off:off + n] = a.reshape(-1)
            spans[k] = (off, n, a.shape)
            off += _align4(n)
        return host[:total], spans

    def upload(self, arrays: dict[str, np.ndarray], into: torch.Tensor | None = None
               ) -> dict[str, torch.Tensor]:
        """One pinned buffer, one host-to-device copy; returns device views by name.  ``into``:
        an existing device buffer (of a CUDA graph) to copy into instead of a new one."""
        host, spans = self._pack(arrays)
        if into is None:
            dev = host.to(self.device, non_blocking=True)
        else:
            dev = into
            dev[:host.numel()].copy_(host, non_blocking=True)
        self._copied.record()
        self._copy_pending = True
        self.h2d_bytes += 4 * host.numel()
        return {k: dev[o:o + n].view(shape) for k, (o, n, shape) in spans.items()}

    def make_context(self, dev: dict[str, torch.Tensor], facts: dict) -> StepContext:
        return StepContext(
            num_tokens=facts["T"], num_seqs=facts["B"], dtype=self.dtype, device=self.device,
            token_ids=dev["token_ids"], positions=dev["positions"],
            seq_of_token=dev["seq_of_token"], cu_seqlens_q=dev["cu_seqlens_q"],
            kv_lens=dev["kv_lens"], slot_ids=dev["slot_ids"], logit_rows=dev["logit_rows"],
            q_lens_host=[int(x) for x in facts["q_lens"]],
            q_starts_host=[int(x) for x in facts["q_starts"]],
            slot_ids_host=[int(x) for x in facts["slot_ids"]],
            max_q_len=facts["max_q_len"], max_kv_len=facts["max_kv_len"],
            decode_only=facts["max_q_len"] == 1, all_rows_wanted=facts["all_rows"])

    def binder(self, dev: dict[str, torch.Tensor]):
        def bind(entry):
            cid = entry.cache
            if self.storage.is_paged(cid):
                g = self.storage.group_of(cid)
                return PagedKVBinding(self.storage.pages_of(cid), dev[f"block_table{g}"],
                                      dev[f"slot_mapping{g}"], self.page_size,
                                      self.groups[g].window, entry.write_cache)
            if cid in self.storage.state:
                return StateBinding(self.storage.state[cid], entry.write_cache)
            return None
        return bind

    @staticmethod
    def graph_batch(B: int) -> int:
        """The batch size of the CUDA graph that serves a decode step of ``B`` requests: exact up
        to 8, then the next multiple of 8 (of 16 above 64).  The rows in between are padding."""
        if B <= 8:
            return B
        step = 8 if B <= 64 else 16
        return -(-B // step) * step

    def _pad_decode(self, arrays, facts, Bp: int):
        """A decode step of B requests as one of ``Bp``: the added rows are requests of one token
        at position 0 whose page is the scratch page of each group (no request owns it)."""
        B = facts["B"]
        extra = Bp - B
        a = dict(arrays)

        def app(key, values):
            a[key] = np.concatenate([arrays[key], np.asarray(values, dtype=arrays[key].dtype)])
        app("token_ids", [0] * extra)
        app("positions", [0] * extra)
        app("seq_of_token", range(B, Bp))
        app("cu_seqlens_q", range(B + 1, Bp + 1))
        app("kv_lens", [1] * extra)
        app("slot_ids", [self.storage.scratch_slot] * extra)
        app("logit_rows", range(B, Bp))
        for g in range(self.cache.num_groups):
            scratch = self.storage.num_pages[g]
            app(f"slot_mapping{g}", [scratch * self.page_size] * extra)
            t = arrays[f"block_table{g}"]
            a[f"block_table{g}"] = np.concatenate(
                [t, np.full((extra, t.shape[1]), scratch, dtype=t.dtype)])
        if "fb_rows" in a:                             # stays last
            a["fb_rows"], a["fb_picks"] = a.pop("fb_rows"), a.pop("fb_picks")
        f = dict(facts, B=Bp, T=Bp,
                 q_lens=np.concatenate([facts["q_lens"], np.ones(extra, dtype=np.int64)]),
                 q_starts=np.concatenate([facts["q_starts"], np.zeros(extra, dtype=np.int64)]),
                 slot_ids=np.concatenate([facts["slot_ids"], np.full(extra, self.storage.scratch_slot,
                                                                       dtype=np.int64)]))
        return a, f

    def _padding_step(self, Bp: int, width: int):
        """The arrays and facts of a decode step that consists of ``Bp`` padding rows only."""
        def z(*shape):
            return np.zeros(shape, dtype=np.int64)
        arrays = dict(token_ids=z(0), positions=z(0), seq_of_token=z(0), cu_seqlens_q=z(1),
                      kv_lens=z(0), slot_ids=z(0), logit_rows=z(0))
        for g in range(self.cache.num_groups):
            arrays[f"slot_mapping{g}"] = z(0)
            arrays[f"block_table{g}"] = z(0, width)
        facts = dict(T=0, B=0, q_lens=z(0), q_starts=z(0), slot_ids=z(0), width=width,
                     all_rows=True, max_q_len=1, max_kv_len=1)
        return self._pad_decode(arrays, facts, Bp)

    @torch.no_grad()
    def warmup(self, capture_graphs: bool = False, max_width: int | None = None) -> int:
        """One token at position 0 through the model, on the scratch page, so that every library
        the model needs is built and loaded before the first request (the reference warms its
        model up the same way: ``engine/model_runner.cc:34-50``).  ``capture_graphs``: also
        capture the CUDA graphs of decode steps now, for every batch-size bucket up to
        ``max_num_seqs`` and every table width up to ``max_width`` pages (default: four width
        steps), instead of when a step first needs one.  Returns how many graphs were captured.
        The padding rows' per-request state is the scratch slot's."""
        with torch.cuda.device(self.device):
            arrays, facts = self._padding_step(1, 1)
            dev = self.upload(arrays)
            self.model.forward(self.make_context(dev, facts), self.binder(dev))
            torch.cuda.synchronize(self.device)
            if not capture_graphs or self.enforce_eager:
                return 0
            top = self.cache.table_width
            max_width = min(top, max_width or 4 * GRAPH_WIDTH_STEP)
            widths = sorted({min(top, w) for w in
                             range(GRAPH_WIDTH_STEP, max_width + GRAPH_WIDTH_STEP, GRAPH_WIDTH_STEP)})
            sizes = sorted({self.graph_batch(b) for b in range(1, self.max_num_seqs + 1)})
            made = 0
            for width in widths:
                for Bp in sizes:
                    if (Bp, width) not in self._graphs and Bp <= self.max_num_seqs + 15:
                        a, f = self._padding_step(Bp, width)
                        self._graphs[(Bp, width)] = self._capture((Bp, width), a, f)
                        made += 1
            return made

    def _graph_key(self, entries, facts):
        """Decode steps in which every request wants its token's logits replay a CUDA graph; so
        do steps with prompt portions whose shape has come before (see PORTION_GRAPH_*)."""
        if self.enforce_eager:
            return None
        if facts["max_q_len"] == 1:
            if any(len(e.want) != 1 for e in entries):
                return None
            return (self.graph_batch(facts["B"]), facts["width"])
        if facts["B"] > PORTION_GRAPH_MAX_SEQS or facts["T"] < PORTION_GRAPH_MIN_TOKENS:
            return None
        key = ("portions", tuple(int(n) for n in facts["q_lens"]), facts["width"],
               tuple(tuple(int(w) for w in e.want) for e in entries))
        if key in self._graphs:
            return key
        seen = self._portion_seen.get(key, 0) + 1
        if len(self._portion_seen) > 4096:
            self._portion_seen.clear()
        self._portion_seen[key] = seen
        graphs = sum(1 for k in self._graphs if isinstance(k[0], str))
        return key if seen >= 2 and graphs < PORTION_GRAPH_LIMIT else None

    def _capture(self, key, arrays, facts) -> _StepGraph:
        from .. import ops
        total = sum(_align4(a.size) for a in arrays.values()) + 2 * _align4(facts["B"])
        ints = torch.empty(total, dtype=torch.int32, device=self.device)
        dev = self.upload(arrays, into=ints)
        ctx = self.make_context(dev, facts)
        # what the kernels may assume about lengths is the bucket's bound, not this step's
        ctx.max_kv_len = min(facts["width"] * self.page_size, self.max_seq_len)
        ctx.capturing = True
        bind = self.binder(dev)
        # once eagerly: libraries, handles, attributes.  Pages take the same values again when the
        # graph runs; per-request state would be advanced twice, so it is put back.
        kept = {cid: t.clone() for cid, t in self.storage.state.items()}
        self.model.forward(ctx, bind)
        for cid, t in kept.items():
            self.storage.state[cid].copy_(t)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        before = ops.launch_count()
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self.model.forward(ctx, bind)
        return _StepGraph(graph, ints, {}, logits, ops.launch_count() - before)

    @torch.no_grad()
    def launch(self, prepared, entries: list[StepEntry], token_ids=None, feedback=None
               ) -> torch.Tensor:
        """Second half of a step: copy the integers and run.  ``token_ids`` (all tokens of the
        step, packed) replaces the values the entries held when the step was prepared, for a
        caller that prepares a step before its last tokens are known.  ``feedback = (src, rows,
        picks)``: token ``rows[i]`` of this step is ``src[picks[i]]``, an int32 tensor on the
        device (the tokens the step before chose), put in place by a kernel: the host need not
        have seen those tokens."""
        arrays, facts = prepared
        arrays = dict(arrays)
        arrays.pop("fb_rows", None), arrays.pop("fb_picks", None)
        if feedback is not None and len(feedback[1]):
            arrays["fb_rows"] = np.asarray(feedback[1], dtype=np.int64)      # packed last
            arrays["fb_picks"] = np.asarray(feedback[2], dtype=np.int64)
        if token_ids is not None:
            token_ids = np.asarray(token_ids, dtype=np.int64).reshape(-1)
            if token_ids.size != facts["T"]:
                raise ValueError(f"{token_ids.size} token ids for a step of {facts['T']} tokens")
            arrays["token_ids"] = token_ids
        tokens = arrays["token_ids"]
        if tokens.min() < 0 or tokens.max() >= self.vocab_size:
            raise ValueError(f"token ids must lie in [0, {self.vocab_size})")
        with torch.cuda.device(self.device):
            key = self._graph_key(entries, facts)
            if key is not None:
                padded, pfacts = arrays, facts
                if facts["max_q_len"] == 1 and key[0] != facts["B"]:
                    padded, pfacts = self._pad_decode(arrays, facts, key[0])
                g = self._graphs.get(key)
                if g is None:
                    g = self._graphs[key] = self._capture(key, padded, pfacts)
                dev = self.upload(padded, into=g.ints)
                self._feed_back(dev, feedback)
                g.graph.replay()
                self.graph_launches += g.launches
                logits = g.logits[:len(facts["slot_ids"])] if padded is not arrays else g.logits
            else:
                dev = self.upload(arrays)
                self._feed_back(dev, feedback)
                ctx = self.make_context(dev, facts)
                logits = self.model.forward(ctx, self.binder(dev))
        self.cache.commit_step(facts["slot_ids"], facts["q_lens"])
        self.steps_run += 1
        return logits

    @staticmethod
    def _feed_back(dev, feedback) -> None:
        if feedback is not None and "fb_rows" in dev:
            from .. import ops
            ops.scatter_tokens(dev["token_ids"], dev["fb_rows"], feedback[0], dev["fb_picks"])

    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        """Run the entries' tokens as one batch; returns fp32 logits ``[wanted, vocab]`` on the
        device, in the order of the entries and of each entry's ``want``.  The tensor is valid
        until the next call of ``step``."""
        return self.launch(self.prepare(entries), entries)
