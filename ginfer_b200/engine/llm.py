"""The Python entry point: token ids in, generated token ids out.

Reference: ``ginfer/engine/engine.{h,cc}``: ``Engine(Config)``, ``generate(prompts,
SamplingParams)`` adds every prompt, loops ``step()`` until the scheduler is empty and returns the
results in request order (``engine.cc:126-151``); ``step()`` is schedule, run, post-process, with
prefill and decode throughput counted per step (``engine.cc:93-124,73-91``).  The reference
returns text; this engine consumes and returns token ids (no tokenizer).
"""
from __future__ import annotations

import time
from dataclasses import dataclass

import numpy as np
import torch

from ..config.engine_config import EngineConfig
from ..ops import gemm_bf16
from ..sampling import Sampler, SamplingParams
from .loading import load_model, random_model
from .request import Request
from .runner import ModelRunner, StepEntry
from .scheduler import Scheduler


@dataclass
class EngineStats:
    """Counted as the reference does: a step with any prompt portion is a prefill step and
    counts its tokens; other steps are decode steps and count their requests."""
    prefill_tokens: int = 0
    decode_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    steps: int = 0
    preemptions: int = 0

    def summary(self) -> dict:
        return {
            "prefill_tokens": self.prefill_tokens, "decode_tokens": self.decode_tokens,
            "prefill_tok_per_s": self.prefill_tokens / self.prefill_seconds
            if self.prefill_seconds else 0.0,
            "decode_tok_per_s": self.decode_tokens / self.decode_seconds
            if self.decode_seconds else 0.0,
            "steps": self.steps, "preemptions": self.preemptions,
        }


@dataclass
class _Flight:
    """A step that has been launched: its batch and the sampled tokens on their way."""
    batch: list
    pending: object
    err_host: object = None        # pinned int: the kernels' error word, copied behind the tokens
    err_event: object = None


class Engine:
    def __init__(self, model_path: str | None = None, *, config: dict | None = None,
                 weights_seed: int = 0, dtype: str = "bfloat16",
                 max_num_batched_tokens: int = 8192, max_num_seqs: int = 64,
                 max_seq_len: int = 4096, gpu_memory_utilization: float = 0.8,
                 kvcache_block_size: int = 16, num_kvcache_blocks: int | None = None,
                 enforce_eager: bool = False, device: str = "cuda:0", seed: int = 0,
                 pipeline: bool = True, warmup: bool = True, capture_graphs: bool = False):
        """``model_path``: a folder with ``config.json`` and ``model.safetensors``; or give
        ``config`` (a ``config.json`` as a dict) and ``weights_seed`` for random weights.
        ``pipeline``: prepare each step on the host while the device runs the one before.
        ``warmup``: run one token through the model before the first request;
        ``capture_graphs``: also capture the decode steps' CUDA graphs then, not on first use."""
        self.cfg = EngineConfig(model_path or "<random>", dtype, max_num_batched_tokens,
                                max_num_seqs, max_seq_len, gpu_memory_utilization,
                                kvcache_block_size, num_kvcache_blocks, enforce_eager, device)
        self.cfg.validate()
        self._weights_from = (model_path, int(weights_seed))
        if model_path is not None:
            self.model, self.model_config = load_model(model_path, dtype, device)
        elif config is not None:
            self.model, self.model_config = random_model(config, weights_seed, dtype, device)
        else:
            raise ValueError("give model_path or config")
        self.runner = ModelRunner(
            self.model, page_size=kvcache_block_size, max_num_seqs=max_num_seqs,
            max_seq_len=max_seq_len, num_pages=num_kvcache_blocks,
            gpu_memory_utilization=gpu_memory_utilization,
            max_num_batched_tokens=max_num_batched_tokens, enforce_eager=enforce_eager)
        if warmup:
            self.runner.warmup(capture_graphs=capture_graphs)
        self.scheduler = Scheduler(self.runner.cache, max_num_seqs, max_num_batched_tokens,
                                   self.runner.max_seq_len, self.model.plan.eos_token_ids)
        self.sampler = Sampler(device)
        self.seed = int(seed)
        self.pipeline = bool(pipeline)
        self._flight = None
        self._err_host = [torch.zeros(1, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._err_turn = 0
        self.stats = EngineStats()
        self._next_id = 0
        self.requests: dict[int, Request] = {}

    def weights(self) -> dict[str, torch.Tensor]:
        """The model's tensors by their safetensors names, as stored (a folder's) or as drawn
        (random weights: drawn again from the same seeds on the same device), for a caller that
        wants to run its own implementation of the model beside this one."""
        path, seed = self._weights_from
        if path is not None:
            from ..weights.safetensors_io import open_model_tensors
            return {name: f.get(key) for name, (f, key) in open_model_tensors(path).items()}
        from ..weights.loader import kept_dtype
        from ..weights.random_init import draw_tensor
        dt = self.runner.dtype
        return {s.name: draw_tensor(s, seed, device=self.cfg.device).to(kept_dtype(s.role, dt, dt))
                for s in self.model.tensor_specs()}

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_ids: list[int], params: SamplingParams | None = None) -> int:
        params = params or SamplingParams()
        params.validate()
        rid = self._next_id
        self._next_id += 1
        seed = params.seed if params.seed is not None else (self.seed * 1000003 + rid)
        req = Request(rid, [int(t) for t in prompt_ids], params, seed=seed,
                      arrival_time=time.perf_counter())
        v = self.model.plan.vocab_size
        if any(t < 0 or t >= v for t in req.prompt):
            raise ValueError(f"prompt token ids must lie in [0, {v})")
        self.scheduler.add(req)
        self.requests[rid] = req
        return rid

    # ------------------------------------------------------------------ one step
    def _entries(self, batch):
        """Step entries of a scheduled batch; a token not known yet stands as 0 until launch."""
        out = []
        for s in batch:
            toks = s.request.tokens(s.start, s.start + s.num_tokens)
            if toks and toks[-1] == Scheduler.PENDING:
                toks = toks[:-1] + [0]
            out.append(StepEntry(s.request.request_id, toks,
                                 [s.num_tokens - 1] if s.sample else []))
        return out

    def _launch(self, batch, prepared, entries, before: "_Flight | None" = None) -> "_Flight":
        """Launch a prepared step with the requests' tokens as they are now, and the choice of
        the next tokens behind it; nothing waits for the device.  A token that the step
        ``before`` is still choosing is taken from that step's result on the device."""
        token_ids = np.fromiter((t for s in batch
                                 for t in s.request.tokens(s.start, s.start + s.num_tokens)),
                                dtype=np.int64)
        feedback = None
        unknown = np.nonzero(token_ids == Scheduler.PENDING)[0]
        if unknown.size:
            if before is None or before.pending.device_tokens is None:
                raise RuntimeError("a step has tokens that no earlier step is choosing")
            pick_of = {s.request.request_id: i
                       for i, s in enumerate(x for x in before.batch if x.sample)}
            ends = np.cumsum([s.num_tokens for s in batch]) - 1
            row_owner = {int(r): s.request.request_id for r, s in zip(ends, batch)}
            feedback = (before.pending.device_tokens, [int(r) for r in unknown],
                        [pick_of[row_owner[int(r)]] for r in unknown])
            token_ids[unknown] = 0
        logits = self.runner.launch(prepared, entries, token_ids, feedback)
        picks = [s for s in batch if s.sample]
        pending = self.sampler.sample_async(
            logits, [s.request.params.temperature for s in picks],
            [s.request.seed for s in picks],
            [s.start + s.num_tokens - len(s.request.prompt) for s in picks])
        # the kernels' error word travels behind the tokens, so that checking it waits for this
        # step only and not for the one launched after it
        self._err_turn ^= 1
        err_host = self._err_host[self._err_turn]
        err_host.copy_(gemm_bf16.error_word(self.cfg.device), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return _Flight(batch, pending, err_host, ev)

    def is_idle(self) -> bool:
        return self._flight is None and self.scheduler.is_finished()

    def step(self) -> list[Request]:
        """Complete one step: schedule and launch it unless the previous call already did, and
        (``pipeline``) schedule and prepare the following step on the host while the device still
        runs this one; then read the sampled tokens, post-process, and launch the following step.
        Returns the requests that finished.  A request that ends on an EOS token while it is
        already part of the following step is returned one call later (its extra token is
        dropped); its output is the same either way."""
        t0 = time.perf_counter()
        finished: list[Request] = []
        if self._flight is None:
            batch, dropped = self.scheduler.schedule()
            finished += dropped
            if not batch:
                return finished
            entries = self._entries(batch)
            self._flight = self._launch(batch, self.runner.prepare(entries), entries)
        cur = self._flight
        finished += self.scheduler.advance(cur.batch)
        nxt = None
        if self.pipeline:
            batch, dropped = self.scheduler.schedule()
            finished += dropped
            if batch:
                entries = self._entries(batch)
                nxt = (batch, self.runner.prepare(entries), entries)
        # the following step goes to the device before this one's tokens are read: where it
        # needs them it takes them from this step's result on the device
        following = self._launch(*nxt, before=cur) if nxt else None
        tokens = cur.pending.result()                   # the device catches up here
        cur.err_event.synchronize()
        gemm_bf16.raise_for(int(cur.err_host[0]), self.cfg.device)
        in_next = {s.request.request_id for s in nxt[0]} if nxt else ()
        finished += self.scheduler.resolve(cur.batch, tokens, in_next)
        self._flight = following
        dt = time.perf_counter() - t0
        if any(s.num_tokens > 1 for s in cur.batch):
            self.stats.prefill_tokens += sum(s.num_tokens for s in cur.batch)
            self.stats.prefill_seconds += dt
        else:
            self.stats.decode_tokens += len(cur.batch)
            self.stats.decode_seconds += dt
        self.stats.steps += 1
        self.stats.preemptions = self.scheduler.num_preemptions
        return finished

    # ------------------------------------------------------------------ the user's call
    def generate(self, prompts: list[list[int]], sampling_params=None) -> list[list[int]]:
        """Generate for every prompt (lists of token ids); returns the generated ids of each, in
        the order of ``prompts``.  ``sampling_params``: one for all, or one per prompt."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt is needed")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        while not self.is_idle():
            self.step()
        out = [self.requests[i].output for i in ids]
        self.last_requests = [self.requests.pop(i) for i in ids]
        return out
