"""Helpers of the replay tests: ways of cutting requests into steps, running the steps through the
engine (in this process or through ``bin/trace_run``), and comparing with the plain
implementation."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys

import numpy as np

import plain_qwen2 as plain

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ----------------------------------------------------------------------------- cutting
def cut_whole(requests: dict[str, list[int]]):
    """Each request alone and whole, one after the other."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "end": [rid], "entries": [
            {"id": rid, "tokens": toks, "want": list(range(len(toks)))}]})
    return steps


def cut_tail_decode(requests, tail: int = 32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": rid, "tokens": toks[:head], "want": list(range(head))}]})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "end": [rid] if i == len(toks) - 1 else [],
                          "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}]})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def cut_portions(requests, sizes=(7, 2, 13, 3, 16, 2, 5, 31, 2, 1, 17)):
    """Portions of changing size, down to two tokens (and one)."""
    steps = []
    k = 0
    for rid, toks in requests.items():
        at = 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            steps.append({"step": len(steps), "end": [rid] if at + n == len(toks) else [],
                          "entries": [{"id": rid, "tokens": toks[at:at + n],
                                       "want": list(range(n))}]})
            at += n
    return steps


# portion sizes that reach the kernels of long prompts: 64 rows and more
LONG_SIZES = (70, 128, 65, 200, 64, 97)


def cut_mixed(requests, max_live: int = 4, seed: int = 0, decode_tail: int = 12,
              singles_first: bool = False, sizes=(2, 3, 5, 8, 13, 21, 34)):
    """Up to ``max_live`` live requests; each step holds portions of some beside single tokens of
    others; a request is sometimes left out of a step.  ``singles_first``: a step's single tokens
    come before its portions (the order in which a scheduler that decodes first sends them).  Returns ``(steps, max_tokens)`` where
    ``max_tokens`` is the most the live requests hold at any time, each rounded up to 64."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, int] = {}          # id -> tokens fed so far
    steps, peak = [], 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, ended = [], []
        for rid in list(live):
            toks = requests[rid]
            at = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # left out of this step
            left = len(toks) - at
            if left > decode_tail:
                n = min(left - decode_tail, rng.choice(list(sizes)))
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[at:at + n], "want": list(range(n))})
            live[rid] = at + n
        held = sum(-(-live[r] // 64) * 64 for r in live)
        peak = max(peak, held)
        for rid in list(live):
            if live[rid] == len(requests[rid]):
                ended.append(rid)
                del live[rid]
        if singles_first:
            entries.sort(key=lambda e: len(e["tokens"]) != 1)
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps, peak


def peak_tokens(steps) -> int:
    live, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            live[e["id"]] = live.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // 64) * 64 for n in live.values()))
        for r in s["end"]:
            live.pop(r, None)
    return peak


# ----------------------------------------------------------------------------- running
def collect(steps, fetch):
    """``fetch(step) -> array [wanted, V]``; returns {(id, position): row}."""
    at: dict[str, int] = {}
    rows = {}
    for s in steps:
        wanted = [(e["id"], at.get(e["id"], 0) + w) for e in s["entries"] for w in e["want"]]
        if wanted:
            arr = fetch(s["step"])
            assert arr.shape[0] == len(wanted), (arr.shape, len(wanted))
            for key, row in zip(wanted, arr):
                assert key not in rows
                rows[key] = row
        for e in s["entries"]:
            at[e["id"]] = at.get(e["id"], 0) + len(e["tokens"])
    return rows


def run_in_process(runner, steps):
    """Drive a :class:`ginfer_b200.engine.ModelRunner` directly."""
    from ginfer_b200.engine import StepEntry
    outs = {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        if entries:
            outs[s["step"]] = runner.step(entries).cpu().numpy()
        for r in s["end"]:
            runner.end(r)
        runner.cache.check()
    return collect(steps, lambda i: outs[i])


def run_trace_program(model_dir, dtype, steps, max_tokens, out_dir, env=None):
    """Drive ``bin/trace_run`` over a pipe, one step after each ``done`` line."""
    os.makedirs(out_dir, exist_ok=True)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir,
           "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens)]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            line = p.stdout.readline().strip()
            assert line == f"done {s['step']}", f"trace_run said {line!r}"
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()
    vocab = json.load(open(os.path.join(model_dir, "config.json")))["vocab_size"]
    return collect(steps, lambda i: np.fromfile(os.path.join(out_dir, f"{i}.f32"),
                                                dtype="<f4").reshape(-1, vocab))


# ----------------------------------------------------------------------------- comparing
_plain_cache: dict = {}


def plain_logits(model_dir, requests, dtype="float32"):
    """{id: float64 logits [T, V]} from the plain implementation.  For ``bfloat16`` the plain
    model stores its activations rounded to bfloat16 where a bfloat16 engine writes them to
    memory (arithmetic stays float64), so that what is left to compare is the engine's own
    arithmetic, not the format's rounding noise, which attention with peaked scores amplifies."""
    out = {}
    cfg = w = None
    for rid, toks in requests.items():
        key = (model_dir, tuple(toks), dtype)
        if key not in _plain_cache:
            if w is None:
                cfg, w = plain.read_model_folder(model_dir)
            if dtype == "bfloat16":
                plain.Stored.bf16()
            try:
                _plain_cache[key] = plain.forward(w, cfg, toks).numpy()
            finally:
                plain.Stored.exact()
        out[rid] = _plain_cache[key]
    return out


def tolerances(dtype: str, ref_scale: float):
    """float32: differences of summation order only.  bfloat16, against the plain model with
    bfloat16-stored activations: a stored value that lands on the other side of a rounding
    boundary differs by one unit in the last place (2^-8 relative); allow four of them at the
    scale of the logits."""
    if dtype == "float32":
        return 2e-5 * max(1.0, ref_scale), 1e-4
    return 2.0 ** -6 * ref_scale, 2.0 ** -6


def compare(rows, expected, dtype, requests):
    scale = max(float(np.abs(v).max()) for v in expected.values())
    atol, rtol = tolerances(dtype, scale)
    assert len(rows) == sum(len(t) for t in requests.values()), "a logits row is missing"
    worst = 0.0
    for (rid, pos), row in sorted(rows.items()):
        ref = expected[rid][pos]
        err = np.abs(row.astype(np.float64) - ref)
        bad = err > atol + rtol * np.abs(ref)
        if bad.any():
            j = int(np.argmax(err))
            raise AssertionError(
                f"first wrong token: request {rid!r} position {pos}: |diff| {err[j]:.3e} at "
                f"vocab {j} (got {row[j]:.6f}, plain {ref[j]:.6f}; atol {atol:.2e}, "
                f"rtol {rtol:.0e}; {int(bad.sum())} of {bad.size} entries off)")
        worst = max(worst, float(err.max()))
    return worst
