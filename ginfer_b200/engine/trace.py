"""Trace replay over the step function (the program behind ``bin/trace_run``)."""
from __future__ import annotations

import argparse
import json
import os
import sys


TRACE_PAGE_SIZE = 16          # divides the 64-token rounding of --max-tokens
TRACE_MAX_LIVE = 4


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--page-size", type=int, default=TRACE_PAGE_SIZE)
    ap.add_argument("--max-live", type=int, default=TRACE_MAX_LIVE)
    ap.add_argument("--enforce-eager", action="store_true",
                    help="launch every kernel of a decode step instead of replaying a CUDA graph")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.max_tokens <= 0:
        print("trace_run: --max-tokens must be positive", file=sys.stderr)
        return 2
    if 64 % args.page_size:
        print("trace_run: --page-size must divide 64", file=sys.stderr)
        return 2
    import torch

    from ..ops import gemm_bf16
    from .loading import load_model
    from .runner import ModelRunner, StepEntry

    os.makedirs(args.out, exist_ok=True)
    model, _cfg = load_model(args.model, args.dtype, args.device)
    budget = -(-args.max_tokens // 64) * 64
    runner = ModelRunner(model, page_size=args.page_size, max_num_seqs=args.max_live,
                         max_seq_len=min(budget, model.plan.max_positions),
                         num_pages=budget // args.page_size,
                         max_num_batched_tokens=budget, enforce_eager=args.enforce_eager)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], list(e["tokens"]), list(e.get("want", [])))
                   for e in rec.get("entries", [])]
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                gemm_bf16.check_errors(args.device)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        for rid in rec.get("end", []):
            runner.end(rid)
        print(f"done {step}", flush=True)
    torch.cuda.synchronize()
    return 0
