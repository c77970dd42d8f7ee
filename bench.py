#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B]

The default run has the layer sizes of the Qwen2-1.5B shape (28 layers, hidden 1536, 12 heads,
2 kv heads, head size 128, intermediate 8960, vocabulary 151936, untied head, q/k/v bias) with
random bf16 weights, a batch of 8 requests with 512-token prompts, cache pages of 16 tokens and a
context limit of 4096.  A "step" is one decode step of the whole batch.

It prints ONE JSON line.  ``value``: decoded tokens a second, timed on the device with CUDA events
around K steps of the engine's step function plus arg-max.  ``e2e``: the same through
``Engine.step`` (scheduler, pinned host-to-device copy of the step's integers, sampling, read-back
of the sampled ids), timed with the wall clock around synchronised steps.  ``prefill``: one
2,048-token prompt in one step.  ``roofline``: the bytes a decode step has to read (every weight
once, and the cache of the live requests) over its time, against the measured copy bandwidth.
``points``: decoding at batch 1 and 64.

``--scenario serve64|chunked [--shape 7b|32b] [--layers L]`` runs one of the serving workloads
instead (continuous batching of 64 requests; 8,192-token prompts in portions beside decoding
requests) and prints its own line.

Only one GPU is used; ``--gpus N`` with N > 1 prints a line that says so and exits with 2.
``--impl reference`` reports why the reference cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

QWEN2_1P5B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 28, "hidden_size": 1536, "num_attention_heads": 12,
    "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 8960, "vocab_size": 151936,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 4096,
    "tie_word_embeddings": False, "sliding_window": 4096, "use_sliding_window": False,
    "torch_dtype": "bfloat16",
}
# the other shapes the baseline names (layer sizes only; run them with --layers where the whole
# model would not be needed): Qwen2.5-7B and Qwen2.5-32B
SHAPES = {
    "1.5b": QWEN2_1P5B,
    "7b": dict(QWEN2_1P5B, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28,
               num_key_value_heads=4, intermediate_size=18944, vocab_size=152064,
               rope_theta=1e6, max_position_embeddings=8192),
    "32b": dict(QWEN2_1P5B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=40,
                num_key_value_heads=8, intermediate_size=27648, vocab_size=152064,
                rope_theta=1e6, max_position_embeddings=16384),
}
SHAPE_NAMES = {"1.5b": "Qwen2-1.5B shape", "7b": "Qwen2.5-7B shape", "32b": "Qwen2.5-32B shape"}
CONTEXT = 4096
PROMPT = 512
PREFILL_TOKENS = 2048
PAGE = 16

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        out = dict(FALLBACK_PEAKS)
        for k in out:
            if isinstance(d.get(k), (int, float)):
                out[k] = float(d[k])
        return out, "measured"
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS), "fallback"


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.rows: list[list[str]] = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks = sorted(int(r[0]) for r in self.rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(self.rows)}


# ----------------------------------------------------------------------------- sizes
def linear_params_per_layer(c) -> int:
    h, nh, nkv, hd, i = (c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"],
                         c["head_dim"], c["intermediate_size"])
    return (nh + 2 * nkv) * hd * h + h * nh * hd + 3 * i * h


def weight_bytes(c, layers: int, itemsize: int = 2) -> int:
    h, nh, nkv, hd = c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], \
        c["head_dim"]
    per_layer = linear_params_per_layer(c) + (nh + 2 * nkv) * hd + 2 * h
    head = c["vocab_size"] * h                      # the output head; the embedding is gathered
    return (layers * per_layer + h + head) * itemsize


def kv_bytes_per_token(c, layers: int, itemsize: int = 2) -> int:
    return layers * 2 * c["num_key_value_heads"] * c["head_dim"] * itemsize


def prefill_flops(c, layers: int, T: int, wanted_rows: int = 1) -> float:
    lin = 2.0 * T * layers * linear_params_per_layer(c)
    attn = layers * 4.0 * c["num_attention_heads"] * c["head_dim"] * (T * (T + 1) / 2)
    head = 2.0 * wanted_rows * c["vocab_size"] * c["hidden_size"]
    return lin + attn + head


# ----------------------------------------------------------------------------- timed pieces
def decode_device_timed(eng, batch: int, steps: int, warmup: int, seed: int, reps: int = 1):
    """Prefill ``batch`` prompts of PROMPT tokens, then time ``steps`` decode steps (step function
    plus arg-max) with CUDA events, ``reps`` times over (each repetition on a fresh batch of
    requests, so that every one decodes at the same context lengths).  Returns (median ms per
    step, launches in one timed region, all the per-repetition times)."""
    times, launches = [], 0
    for r in range(reps):
        ms, launches = _decode_device_timed_once(eng, batch, steps, warmup, seed + 1000 * r)
        times.append(ms)
    times.sort()
    return times[len(times) // 2], launches, times


def _decode_device_timed_once(eng, batch: int, steps: int, warmup: int, seed: int):
    import torch

    from ginfer_b200 import ops
    from ginfer_b200.engine import StepEntry
    runner = eng.runner
    g = torch.Generator().manual_seed(seed)
    V = runner.vocab_size
    ids = [f"bench-{seed}-{b}" for b in range(batch)]
    prompts = torch.randint(0, V, (batch, PROMPT), generator=g).tolist()
    feed = torch.randint(0, V, (warmup + steps, batch), generator=g).tolist()
    budget = eng.cfg.max_num_batched_tokens
    per_step = max(1, budget // PROMPT)
    for i in range(0, batch, per_step):
        runner.step([StepEntry(ids[b], prompts[b], []) for b in range(i, min(batch, i + per_step))])
    for s in range(warmup):
        ops.argmax(runner.step([StepEntry(ids[b], [feed[s][b]], [0]) for b in range(batch)]))
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = ops.launch_count() + runner.graph_launches
    start.record()
    for s in range(warmup, warmup + steps):
        ops.argmax(runner.step([StepEntry(ids[b], [feed[s][b]], [0]) for b in range(batch)]))
    stop.record()
    torch.cuda.synchronize()
    launches = ops.launch_count() + runner.graph_launches - l0
    ms = start.elapsed_time(stop) / steps
    for rid in ids:
        runner.end(rid)
    return ms, launches


def decode_end_to_end(eng, batch: int, steps: int, warmup: int, seed: int, reps: int = 1):
    """The same through the public entry point, ``reps`` times over; the median."""
    runs = [_decode_end_to_end_once(eng, batch, steps, warmup, seed + 1000 * r)
            for r in range(reps)]
    runs.sort()
    return runs[len(runs) // 2]


def _decode_end_to_end_once(eng, batch: int, steps: int, warmup: int, seed: int):
    """Requests are added with host token ids, ``Engine.step`` schedules, copies the step's
    integers from pinned memory, runs, samples and reads the ids back.  Returns (ms per step, h2d
    bytes per step, d2h bytes per step)."""
    import torch

    from ginfer_b200.sampling import SamplingParams
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, eng.runner.vocab_size, (batch, PROMPT), generator=g).tolist()
    sp = SamplingParams(max_tokens=warmup + steps + 1, ignore_eos=True)
    for p in prompts:
        eng.add_request(p, sp)
    while any(len(r.output) == 0 for r in eng.requests.values()):
        eng.step()                                   # prompts
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    h0 = eng.runner.h2d_bytes
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = (eng.runner.h2d_bytes - h0) / steps
    while not eng.is_idle():
        eng.step()
    eng.requests.clear()
    return 1e3 * dt / steps, int(h2d), 4 * batch + 4      # the tokens and the kernels' error word


def prefill_timed(eng, tokens: int, reps: int, warmup: int, seed: int):
    import torch

    from ginfer_b200.engine import StepEntry
    runner = eng.runner
    g = torch.Generator().manual_seed(seed)
    prompt = torch.randint(0, runner.vocab_size, (tokens,), generator=g).tolist()
    times = []
    for r in range(warmup + reps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry("prefill", prompt, [tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        runner.end("prefill")
        if r >= warmup:
            times.append(start.elapsed_time(stop))
    times.sort()
    return times[len(times) // 2]


# ----------------------------------------------------------------------------- small workloads
MICRO = ("gemm_gateup_m8", "gemm_down_m8", "gemm_lmhead_m8", "gemm_gateup_m2048", "gemm_qkv_m2048",
         "attn_decode_b8",
         "attn_decode_b64", "attn_decode_b1_ctx32768", "prefill_2layers")


def run_micro(name: str) -> int:
    """A few launches of one kernel at the benchmark's sizes, small enough to profile (the
    commands in ``profiles/`` run these).  Weights are rotated over copies that together exceed
    the L2 cache."""
    import math

    import torch

    from ginfer_b200.ops import attention_bf16, gemm_bf16
    c = QWEN2_1P5B
    H, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    dev = "cuda:0"
    if name == "gemm_gateup_m2048":
        # the gated product of a 2,048-token prompt on the persistent tcgen05 kernel
        from ginfer_b200.ops import gemm_prefill
        x = torch.randn(PREFILL_TOKENS, H, device=dev).to(torch.bfloat16)
        ws = [(torch.randn(2 * I, H, device=dev) * 0.05).to(torch.bfloat16) for _ in range(3)]
        for i in range(6):
            y = gemm_prefill.gemm(x, ws[i % 3], None, torch.bfloat16, epi=2)
        torch.cuda.synchronize()
        gemm_bf16.check_errors()
        print(json.dumps({"micro": name, "out": list(y.shape)}))
        return 0
    if name == "gemm_qkv_m2048":
        # the joined q/k/v product of a 2,048-token prompt: bias, rotation and cache write in its
        # epilogue
        from ginfer_b200.ops import gemm_prefill
        T, N = PREFILL_TOKENS, (nh + 2 * nkv) * hd
        x = torch.randn(T, H, device=dev).to(torch.bfloat16)
        ws = [(torch.randn(N, H, device=dev) * 0.05).to(torch.bfloat16) for _ in range(3)]
        bias = torch.randn(N, device=dev)
        table = torch.randn(CONTEXT, hd, device=dev)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        slots = torch.randperm(2 * T, device=dev)[:T].to(torch.int32)
        pages = torch.zeros(2, 2 * T // PAGE + 1, PAGE, nkv, hd, dtype=torch.bfloat16, device=dev)
        for i in range(6):
            y = gemm_prefill.qkv_rope_write(x, ws[i % 3], bias, table, hd, pos, slots, pages, nh,
                                            nkv, hd, min_tokens=1)
        torch.cuda.synchronize()
        gemm_bf16.check_errors()
        print(json.dumps({"micro": name, "out": list(y.shape)}))
        return 0
    if name.startswith("gemm_"):
        M, N, K, epi, out = {"gemm_gateup_m8": (8, 2 * I, H, 2, torch.bfloat16),
                             "gemm_down_m8": (8, H, I, 0, torch.bfloat16),
                             "gemm_lmhead_m8": (8, V, H, 0, torch.float32)}[name]
        copies = max(2, min(8, (300 << 20) // (N * K * 2)))
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        ws = [(torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16) for _ in range(copies)]
        for i in range(8):
            y = gemm_bf16.gemm(x, ws[i % copies], None, out, epi=epi)
        torch.cuda.synchronize()
        gemm_bf16.check_errors()
        print(json.dumps({"micro": name, "out": list(y.shape)}))
        return 0
    if name.startswith("attn_decode"):
        B = 1 if "_b1_" in name else 8 if name.endswith("b8") else 64
        ctx = 32768 if name.endswith("ctx32768") else PROMPT + 64
        pages_n = B * (ctx // PAGE + 2)
        pages = torch.randn(2, pages_n, PAGE, nkv, hd, device=dev).to(torch.bfloat16)
        table = torch.randperm(pages_n, device=dev).to(torch.int32).reshape(B, -1).contiguous()
        qkv = torch.randn(B, (nh + 2 * nkv) * hd, device=dev).to(torch.bfloat16)
        cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
        pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
        # few requests with many keys: several clusters a request and a kernel that adds them up
        splits, parts = attention_bf16.decode_partition(B, nh, nkv, ctx)
        for _ in range(6):
            y = attention_bf16.decode(qkv, pages, table, cu, pos, B, nh, nkv, hd,
                                      1 / math.sqrt(hd), 0, PAGE, splits, parts=parts)
        torch.cuda.synchronize()
        print(json.dumps({"micro": name, "splits": splits, "parts": parts, "out": list(y.shape)}))
        return 0
    if name == "prefill_2layers":
        from ginfer_b200.engine import StepEntry
        from ginfer_b200.engine.llm import Engine
        cfg = dict(c)
        cfg["num_hidden_layers"] = 2
        eng = Engine(config=cfg, dtype="bfloat16", max_num_seqs=4, max_seq_len=CONTEXT,
                     num_kvcache_blocks=PREFILL_TOKENS // PAGE + 64, enforce_eager=True)
        prompt = torch.randint(0, V, (PREFILL_TOKENS,)).tolist()
        for _ in range(3):
            eng.runner.step([StepEntry("p", prompt, [PREFILL_TOKENS - 1])])
            eng.runner.end("p")
        torch.cuda.synchronize()
        print(json.dumps({"micro": name, "tokens": PREFILL_TOKENS}))
        return 0
    raise SystemExit(f"unknown workload {name!r}; known: {MICRO}")


# ----------------------------------------------------------------------------- scenarios
SCENARIOS = ("serve64", "chunked", "ref256", "longctx")

# what 11Aln0/ginfer publishes for its own throughput run (README.md:51-53 and the log under
# media/): one A40, a 1.5B Qwen2-architecture model in bf16
REF256_PUBLISHED = {"hardware": "A40", "prefill_tok_s": 31590.0, "decode_tok_s": 5457.0,
                    "total_tok_s": 16138.0}


def run_long_context(shape: str, layers: int | None, context: int = 32768,
                     portion: int | None = None) -> int:
    """One prompt of ``context`` tokens fed in portions of 2,048 (``--portion``: another size; each portion timed on the device
    with CUDA events; the whole prompt three times, the last pass reported: the first two let the
    portions' CUDA graphs be captured), then single tokens decoded
    at that context for one request and for eight: where attention over the cache, not the
    products, decides the time.  Fractions: a portion's flops (products and the attention over
    the keys before and inside it) over the measured tensor peak; a decode step's bytes (weights
    once, the cache of the live requests) over the measured copy bandwidth.  One JSON line."""
    import torch

    from ginfer_b200 import ops
    from ginfer_b200.engine import StepEntry
    from ginfer_b200.engine.llm import Engine
    cfg = dict(SHAPES[shape])
    full_layers = cfg["num_hidden_layers"]
    L = cfg["num_hidden_layers"] = layers or full_layers
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], context + 256)
    V, portion, B = cfg["vocab_size"], int(portion or PREFILL_TOKENS), 8
    eng = Engine(config=cfg, dtype="bfloat16", max_num_seqs=B, max_seq_len=context + 128,
                 max_num_batched_tokens=portion, kvcache_block_size=PAGE,
                 num_kvcache_blocks=B * ((context + 128) // PAGE + 2))
    runner = eng.runner
    peaks, peaks_from = load_peaks()
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, V, (B, context), generator=g).tolist()
    # ---- the prompt in portions
    per_portion = []
    for rep in range(3):
        per_portion = []
        for at in range(0, context, portion):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            last = at + portion >= context
            runner.step([StepEntry("long", prompts[0][at:at + portion], [portion - 1] if last else [])])
            stop.record()
            torch.cuda.synchronize()
            per_portion.append(start.elapsed_time(stop))
        if rep < 2:
            runner.end("long")
    lin = 2.0 * portion * L * linear_params_per_layer(cfg)

    def portion_flops(at):
        keys = portion * at + portion * (portion + 1) / 2
        return lin + L * 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * keys
    total_ms = sum(per_portion)
    flops = sum(portion_flops(at) for at in range(0, context, portion))
    prefill = {"tokens": context, "portion": portion, "ms": round(total_ms, 3),
               "value": round(context / (total_ms * 1e-3), 1),
               "frac": round(flops / (total_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4),
               "first_portion_ms": round(per_portion[0], 3),
               "last_portion_ms": round(per_portion[-1], 3),
               "last_portion_frac": round(portion_flops(context - portion) / (per_portion[-1] * 1e-3) /
                                          (peaks["bf16_tflops"] * 1e12), 4)}
    # ---- decoding at that context: the request above, then eight of them
    decode = {}
    ids = ["long"]
    for batch in (1, B):
        for b in range(len(ids), batch):
            rid = f"long{b}"
            for at in range(0, context, portion):
                runner.step([StepEntry(rid, prompts[b][at:at + portion], [])])
            ids.append(rid)
        feed = torch.randint(0, V, (8 + 32, batch), generator=g).tolist()
        for s_ in range(8):
            ops.argmax(runner.step([StepEntry(ids[b], [feed[s_][b]], [0]) for b in range(batch)]))
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for s_ in range(8, 40):
            ops.argmax(runner.step([StepEntry(ids[b], [feed[s_][b]], [0]) for b in range(batch)]))
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / 32
        nbytes = weight_bytes(cfg, L) + batch * (context + 24) * kv_bytes_per_token(cfg, L)
        decode[f"b{batch}"] = {"tok_s": round(batch / (ms * 1e-3), 1), "ms": round(ms, 4),
                               "frac": round(nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)}
    print(json.dumps({"scenario": "longctx", "model": SHAPE_NAMES[shape], "layers_run": L,
                      "layers_config": full_layers, "context": context, "kv_block": PAGE,
                      "prefill": prefill, "decode": decode, "peaks": peaks_from}))
    return 0


def scenario_plan(name: str, shape: str, layers: int | None):
    """A serving workload without the engine: ``(config, layers of the whole model, prompts,
    sampling parameters, the engine's sizes)``.  Every prompt with its output fits the engine's
    longest sequence and the model's position table (a host test checks that)."""
    import random

    from ginfer_b200.sampling import SamplingParams
    cfg = dict(SHAPES[shape])
    full_layers = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers or full_layers
    rng = random.Random(0)
    V = cfg["vocab_size"]
    if name == "serve64":
        prompts = [[rng.randrange(V) for _ in range(rng.randint(128, 2048))] for _ in range(64)]
        params = [SamplingParams(max_tokens=rng.randint(64, 256), ignore_eos=True)
                  for _ in range(64)]
        kwargs = dict(max_num_seqs=64, max_seq_len=8192, max_num_batched_tokens=2048,
                      num_kvcache_blocks=64 * (2304 // PAGE + 2))
    elif name == "ref256":
        prompts = [[rng.randrange(V) for _ in range(512)] for _ in range(256)]
        params = [SamplingParams(max_tokens=128, ignore_eos=True)] * 256
        kwargs = dict(max_num_seqs=256, max_seq_len=CONTEXT, max_num_batched_tokens=16384,
                      num_kvcache_blocks=256 * (640 // PAGE + 2))
    elif name == "chunked":
        # (prompts of 8,192 tokens: the position table has to reach that far)
        cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], 16384)
        prompts = ([[rng.randrange(V) for _ in range(32)] for _ in range(32)] +
                   [[rng.randrange(V) for _ in range(8192)] for _ in range(8)])
        params = ([SamplingParams(max_tokens=256, ignore_eos=True)] * 32 +
                  [SamplingParams(max_tokens=8, ignore_eos=True)] * 8)
        kwargs = dict(max_num_seqs=40, max_seq_len=16384, max_num_batched_tokens=2048 + 32,
                      num_kvcache_blocks=8 * (8200 // PAGE + 2) + 32 * (288 // PAGE + 2))
    else:
        raise SystemExit(f"unknown scenario {name!r}")
    return cfg, full_layers, prompts, params, kwargs


def run_scenario(name: str, shape: str, layers: int | None) -> int:
    """The serving workloads the baseline names beside the headline, through the Python entry
    point (scheduler, chunked prompts, decode graphs), wall clock, third pass reported (the first
    two capture graphs: of decode steps at first sight, of steps with portions at second).  ``serve64``: continuous batching of 64 requests, prompts of 128..2048
    tokens, 64..256 generated each.  ``chunked``: 8 prompts of 8,192 tokens fed in 2,048-token
    portions beside 32 requests that generate 256 tokens each.  ``ref256``: the reference's own
    throughput run (``ginfer/test/test_engine.cc:57-112``): 256 prompts of 512 random ids, 128
    tokens generated for each, EOS ignored, a budget of 16,384 tokens a step, 256 requests at a
    time, pages of 16; prefill and decode tok/s counted as the reference counts them (a step with
    a prompt portion counts its tokens, another step its requests, each over its own wall time:
    ``ginfer/engine/engine.cc:73-121``) beside the figures it publishes.  One JSON line."""
    import time

    import torch

    from ginfer_b200.engine.llm import Engine
    cfg, full_layers, prompts, params, kwargs = scenario_plan(name, shape, layers)
    eng = Engine(config=cfg, dtype="bfloat16", kvcache_block_size=PAGE, **kwargs)
    result = None
    for _ in range(3):
        torch.cuda.synchronize()
        t0, s0 = time.perf_counter(), eng.runner.steps_run
        st0 = dict(vars(eng.stats))
        outs = eng.generate(prompts, params)
        torch.cuda.synchronize()
        dt, steps = time.perf_counter() - t0, eng.runner.steps_run - s0
        tin, tout = sum(map(len, prompts)), sum(map(len, outs))
        result = {"scenario": name, "model": SHAPE_NAMES[shape], "layers_run": cfg["num_hidden_layers"],
                  "layers_config": full_layers, "requests": len(prompts), "prompt_tokens": tin,
                  "generated_tokens": tout, "seconds": round(dt, 4), "steps": steps,
                  "ms_per_step": round(1e3 * dt / steps, 3),
                  "total_tok_s": round((tin + tout) / dt, 1),
                  "generated_tok_s": round(tout / dt, 1), "preemptions": eng.stats.preemptions}
        reqs = eng.last_requests
        ttft = sorted(1e3 * (r.first_token_time - r.arrival_time) for r in reqs
                      if r.first_token_time is not None)
        tpot = sorted(1e3 * (r.finish_time - r.first_token_time) / (len(r.output) - 1)
                      for r in reqs if r.finish_time and len(r.output) > 1)

        def pct(v, q):
            return round(v[min(len(v) - 1, int(q * len(v)))], 3) if v else None
        # as the reference logs them per sequence (ginfer/engine/engine.cc:54-71): time to the
        # first token from arrival, and the time per token after it
        result["ttft_ms"] = {"p50": pct(ttft, 0.5), "p99": pct(ttft, 0.99)}
        result["tpot_ms"] = {"p50": pct(tpot, 0.5), "p99": pct(tpot, 0.99)}
        if name == "ref256":
            d = {k: getattr(eng.stats, k) - st0[k] for k in
                 ("prefill_tokens", "prefill_seconds", "decode_tokens", "decode_seconds")}
            result["prefill_tok_s"] = round(d["prefill_tokens"] / max(d["prefill_seconds"], 1e-9), 1)
            result["decode_tok_s"] = round(d["decode_tokens"] / max(d["decode_seconds"], 1e-9), 1)
            result["reference_published"] = REF256_PUBLISHED
    print(json.dumps(result))
    return 0


# ----------------------------------------------------------------------------- main
def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None,
                    help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", choices=sorted(SHAPES), default="1.5b",
                    help="layer sizes: the benchmark's own (default) or the larger ones the "
                         "baseline names")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--prefill-reps", type=int, default=5,
                    help="timed repetitions of the 2,048-token prefill (the median is reported)")
    ap.add_argument("--reps", type=int, default=5,
                    help="repetitions of the timed region of K decode steps (the median is "
                         "reported: a region of K steps is tens of milliseconds)")
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--micro", choices=MICRO, default=None,
                    help="run one small kernel workload (for profiling) instead of the benchmark")
    ap.add_argument("--portion", type=int, default=None,
                    help="tokens a step of the long prompt in --scenario longctx (default 2,048)")
    ap.add_argument("--scenario", choices=SCENARIOS, default=None,
                    help="run a serving workload through the entry point instead of the benchmark")
    args = ap.parse_args()
    if args.micro:
        return run_micro(args.micro)
    if args.scenario:
        if args.gpus != 1:
            print(json.dumps({"error": "this engine runs on one GPU", "n_gpus": args.gpus}))
            return 2
        if args.scenario == "longctx":
            return run_long_context(args.shape, args.layers, portion=args.portion)
        return run_scenario(args.scenario, args.shape, args.layers)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "11Aln0/ginfer is a CMake/C++ project without setup.py or pyproject "
                          "(pip: 'not installable'); its CMake downloads nine packages at "
                          "configure time and there is no network"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        print(json.dumps({"error": "this engine runs on one GPU; --gpus N > 1 is not supported",
                          "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch

    from ginfer_b200.engine.llm import Engine
    cfg = dict(SHAPES[args.shape])
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    peaks, peak_src = load_peaks()
    eng = Engine(config=cfg, weights_seed=0, dtype="bfloat16", max_num_batched_tokens=8192,
                 max_num_seqs=64, max_seq_len=CONTEXT, kvcache_block_size=PAGE,
                 num_kvcache_blocks=64 * (PROMPT + 256) // PAGE + PREFILL_TOKENS // PAGE + 64,
                 enforce_eager=args.enforce_eager)
    B = args.batch

    clocks = ClockSampler()
    clocks.start()
    reps = max(1, args.reps)
    ms, launches, all_ms = decode_device_timed(eng, B, args.steps, args.warmup, seed=1, reps=reps)
    clock_info = clocks.stop()
    e2e_ms, h2d, d2h = decode_end_to_end(eng, B, args.steps, args.warmup, seed=2, reps=reps)
    pre_ms = prefill_timed(eng, PREFILL_TOKENS, reps=max(1, args.prefill_reps), warmup=3, seed=3)

    def hbm_fraction(batch: int, step_ms: float, steps: int) -> tuple[float, float]:
        """(GB/s, fraction of the copy bandwidth) of a decode step: every weight once and the
        cache of the live requests at their mean length over the timed steps."""
        mean_ctx = PROMPT + args.warmup + steps / 2
        nbytes = weight_bytes(cfg, layers) + batch * mean_ctx * kv_bytes_per_token(cfg, layers)
        gbs = nbytes / (step_ms * 1e-3) / 1e9
        return gbs, gbs / peaks["hbm_gbs"]

    points, points_frac = {}, {}
    if not args.skip_points:
        for b in (1, 64):
            k = min(args.steps, 64)
            pms, _, _ = decode_device_timed(eng, b, k, args.warmup, seed=10 + b, reps=min(reps, 3))
            points[f"decode_b{b}"] = round(b / (pms * 1e-3), 1)
            points_frac[f"decode_b{b}"] = round(hbm_fraction(b, pms, k)[1], 4)

    achieved, frac = hbm_fraction(B, ms, args.steps)
    flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
    value = B / (ms * 1e-3)
    line = {
        "metric": f"decode tok/s at batch {B} (one B200), {SHAPE_NAMES[args.shape]}",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random token ids, random-init weights N(0, 0.02)",
        "impl": "ours",
        "config": {
            "model": SHAPE_NAMES[args.shape], "layers_run": layers, "layers_config": full_layers,
            "hidden_size": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate_size": cfg["intermediate_size"], "vocab_size": cfg["vocab_size"],
            "global_batch": B, "seq_len": CONTEXT, "prompt_len": PROMPT,
            "kv_block": PAGE, "parallelism": "single GPU",
            "l2": f"inputs larger than L2 ({weight_bytes(cfg, layers) / 1e9:.1f} GB of weights read "
                  "per step)",
            "cuda_graphs": not args.enforce_eager, "peaks": peak_src, "timed_regions": reps,
        },
        "e2e": {"value": round(B / (e2e_ms * 1e-3), 1), "unit": "tok/s",
                "ms_per_step": round(e2e_ms, 4), "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS / (pre_ms * 1e-3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pre_ms, 3),
                    "frac": round(flops / (pre_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1),
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(frac, 4)},
        "points": points,
        "points_roofline_frac": points_frac,
        "ms_per_step_all": [round(t, 4) for t in all_ms],
        "clocks": clock_info,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
