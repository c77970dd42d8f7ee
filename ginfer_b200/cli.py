"""Command line: token ids in, generated token ids out.

Options carry the names of the reference's ``engine::Config`` and ``SamplingParams`` fields
(``ginfer/engine/config.h:8-21``, ``ginfer/engine/sampling_params.h:5-8``): ``--model-path``,
``--max-num-batched-tokens``, ``--max-num-seqs``, ``--max-seq-len``,
``--gpu-memory-utilization``, ``--kvcache-block-size``, ``--max-tokens``, ``--ignore-eos``.  The
reference has no command line of its own (its entry points are gtest binaries driven by the
``MODEL_PATH`` environment variable: ``ginfer/test/test_engine.cc:14-55``); ``MODEL_PATH`` is
honoured here as the default of ``--model-path``.

Prompts are token ids: one request per line of ``--prompt-ids`` (a file, ``-`` for standard
input), as space- or comma-separated integers or a JSON list.  Output: one JSON line per request
with its generated ids, then one line of statistics (time to first token, time per output token,
prefill and decode throughput as ``ginfer/engine/engine.cc:54-91`` logs them).

``--random-config CONFIG.json --weights-seed N`` writes a model folder with random weights to
``--model-path`` first (or to a temporary folder) instead of reading one.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="ginfer_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-path", default=os.environ.get("MODEL_PATH"),
                    help="folder with config.json and model.safetensors (default: $MODEL_PATH)")
    ap.add_argument("--random-config", help="config.json to draw random weights for")
    ap.add_argument("--weights-seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--prompt-ids", default="-", help="file of prompts as token ids, '-' = stdin")
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--max-seq-len", type=int, default=4096)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.8)
    ap.add_argument("--kvcache-block-size", type=int, default=16)
    ap.add_argument("--num-kvcache-blocks", type=int, default=None)
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--capture-graphs", action="store_true",
                    help="capture the decode steps' CUDA graphs at start-up, not on first use")
    ap.add_argument("--device", default="cuda:0")
    return ap


def parse_prompt_line(line: str) -> list[int]:
    line = line.strip()
    if line.startswith("["):
        return [int(t) for t in json.loads(line)]
    return [int(t) for t in line.replace(",", " ").split()]


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from .sampling import SamplingParams
    tmp = None
    model_path = args.model_path
    if args.random_config:
        from .weights import write_random_model
        with open(args.random_config, "r", encoding="utf-8") as f:
            cfg = json.load(f)
        if model_path is None:
            tmp = tempfile.TemporaryDirectory()
            model_path = tmp.name
        write_random_model(model_path, cfg, args.weights_seed,
                           storage_dtype="float32" if args.dtype == "float32" else "bfloat16")
    if not model_path:
        print("ginfer_b200: give --model-path (or MODEL_PATH), or --random-config",
              file=sys.stderr)
        return 2
    src = sys.stdin if args.prompt_ids == "-" else open(args.prompt_ids, "r", encoding="utf-8")
    prompts = [parse_prompt_line(ln) for ln in src if ln.strip()]
    if src is not sys.stdin:
        src.close()
    if not prompts:
        print("ginfer_b200: no prompts", file=sys.stderr)
        return 2
    from .engine.llm import Engine
    eng = Engine(model_path=model_path, dtype=args.dtype,
                 max_num_batched_tokens=args.max_num_batched_tokens,
                 max_num_seqs=args.max_num_seqs, max_seq_len=args.max_seq_len,
                 gpu_memory_utilization=args.gpu_memory_utilization,
                 kvcache_block_size=args.kvcache_block_size,
                 num_kvcache_blocks=args.num_kvcache_blocks, enforce_eager=args.enforce_eager,
                 capture_graphs=args.capture_graphs,
                 device=args.device, seed=args.seed)
    sp = SamplingParams(max_tokens=args.max_tokens, ignore_eos=args.ignore_eos,
                        temperature=args.temperature)
    outs = eng.generate(prompts, sp)
    ttft, tpot = [], []
    for i, (req, out) in enumerate(zip(eng.last_requests, outs)):
        print(json.dumps({"request": i, "output_ids": out, "finish_reason": req.finish_reason}))
        if req.first_token_time is not None:
            ttft.append(req.first_token_time - req.arrival_time)
            if len(out) > 1:
                tpot.append((req.finish_time - req.first_token_time) / (len(out) - 1))
    stats = eng.stats.summary()
    stats["avg_ttft_ms"] = 1e3 * sum(ttft) / len(ttft) if ttft else None
    stats["avg_tpot_ms"] = 1e3 * sum(tpot) / len(tpot) if tpot else None
    print(json.dumps({"stats": stats}))
    if tmp is not None:
        tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
