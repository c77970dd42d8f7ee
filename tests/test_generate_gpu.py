"""Generation through the Python entry point and the command line: greedy tokens equal the plain
implementation's, temperature sampling follows the plain inverse-CDF rule, and neither depends on
the batch, the token budget or a preemption."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen2 as plain
from tiny import CONFIGS, make_folder, prompt

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen")
    return {n: make_folder(root, n, seed=4) for n in ("A", "B", "C", "E")}


def _all_pages_free(eng) -> bool:
    cache = eng.runner.cache
    return cache.free_pages() == [p.num_pages for p in cache.pools]


def _engine(d, dtype="float32", **kw):
    from ginfer_b200.engine.llm import Engine
    args = dict(model_path=d, dtype=dtype, max_num_seqs=4, max_num_batched_tokens=32,
                max_seq_len=256, num_kvcache_blocks=40, kvcache_block_size=16)
    args.update(kw)
    return Engine(**args)


# Tiny A (tied head, small weights) answers every prompt with its last token: a test of generated
# tokens on it alone could not fail.  B, C and E generate varied tokens.
@pytest.mark.parametrize("name,lengths,new", [("A", (5, 17, 33), 8), ("B", (1, 40, 90), 12),
                                              ("C", (3, 29, 66), 10), ("E", (2, 70, 45), 10)])
def test_greedy_generation_equals_plain(folders, name, lengths, new):
    from ginfer_b200.sampling import SamplingParams
    d = folders[name]
    cfg, w = plain.read_model_folder(d)
    prompts = [prompt(n, cfg["vocab_size"], seed=n) for n in lengths]
    want = [plain.greedy_generate(w, cfg, p, new) for p in prompts]
    if name != "A":
        assert any(len(set(o)) > 2 for o in want)         # no echo of one token
    sp = SamplingParams(max_tokens=new, ignore_eos=True)
    # a budget of 13 tokens a step: prompts go in portions beside decode tokens
    eng = _engine(d, max_num_batched_tokens=13, kvcache_block_size=8 if name == "B" else 16)
    assert eng.generate(prompts, sp) == want
    assert _all_pages_free(eng)
    # so few pages that requests are preempted and computed again: same tokens
    few = _engine(d, num_kvcache_blocks=9, max_num_batched_tokens=64)
    assert few.generate(prompts, sp) == want
    # without preparing steps ahead: same tokens
    assert _engine(d, pipeline=False, max_num_batched_tokens=13).generate(prompts, sp) == want
    if name == "B":
        assert few.stats.preemptions >= 1


def test_eos_stops_generation(folders):
    from ginfer_b200.sampling import SamplingParams
    d = folders["C"]
    cfg, w = plain.read_model_folder(d)
    p = prompt(9, cfg["vocab_size"], seed=3)
    free = plain.greedy_generate(w, cfg, p, 6)
    assert free[2] not in free[:2]                        # the third token is the first EOS
    cfg2 = dict(cfg)
    cfg2["eos_token_id"] = free[2]
    d2 = d + "_eos"
    os.makedirs(d2, exist_ok=True)
    json.dump(cfg2, open(os.path.join(d2, "config.json"), "w"))
    if not os.path.exists(os.path.join(d2, "model.safetensors")):
        os.link(os.path.join(d, "model.safetensors"), os.path.join(d2, "model.safetensors"))
    for pipeline in (True, False):
        eng = _engine(d2, pipeline=pipeline)
        assert eng.generate([p], SamplingParams(max_tokens=6)) == \
            [free[:free.index(free[2]) + 1]]
        assert eng.last_requests[0].finish_reason == "eos"
        assert _all_pages_free(eng) and not eng.runner.cache.requests
    assert eng.generate([p], SamplingParams(max_tokens=6, ignore_eos=True)) == [free]


def test_temperature_sampling_follows_the_plain_rule_and_ignores_the_batch(folders):
    from ginfer_b200.sampling import SamplingParams, uniform
    d = folders["B"]
    cfg, w = plain.read_model_folder(d)
    prompts = [prompt(n, cfg["vocab_size"], seed=50 + n) for n in (1, 40, 90)]
    sps = [SamplingParams(max_tokens=12, ignore_eos=True, temperature=0.8, seed=1000 + i)
           for i in range(3)]
    eng = _engine(d, kvcache_block_size=8, max_num_batched_tokens=13)
    outs = eng.generate(prompts, sps)
    # replay each request with the plain model: at every step the engine's token must be the
    # plain inverse-CDF choice, unless u falls within rounding distance of a CDF step
    for p, out, sp in zip(prompts, outs, sps):
        ids = list(p)
        for i, tok in enumerate(out):
            logits = plain.forward(w, cfg, ids)[-1]
            u = uniform(sp.seed, i)
            pick = plain.temperature_token(logits, 0.8, u)
            if tok != pick:
                cdf = torch.cumsum(torch.softmax(logits.double() / 0.8, -1), 0)
                lo, hi = sorted((tok, pick))
                assert hi - lo == 1 and abs(float(cdf[lo]) - u) < 1e-5, (i, tok, pick)
            ids.append(tok)
    # alone, and with other seeds beside it: the same tokens
    alone = _engine(d, kvcache_block_size=8)
    assert alone.generate([prompts[1]], sps[1]) == [outs[1]]
    other = [SamplingParams(max_tokens=12, ignore_eos=True, temperature=0.8, seed=5)] * 3
    assert _engine(d, kvcache_block_size=8).generate(prompts, other) != outs


def _plain_row(w, cfg, ids, dtype):
    """The plain implementation's logits for the token after ``ids``; for bfloat16 with its
    activations stored rounded where the engine writes them to memory."""
    if dtype == "bfloat16":
        plain.Stored.bf16()
    try:
        return plain.forward(w, cfg, ids)[-1]
    finally:
        plain.Stored.exact()


def _close_call(row, a: int, b: int, temperature: float, u: float | None, tol: float) -> bool:
    """Whether ``a`` and ``b`` are both defensible choices from the plain logits ``row``: greedy,
    both within ``tol`` (of the logits' scale) of the maximum; sampling, ``u`` within ``tol`` of
    the cumulative probability at the smaller index."""
    if temperature <= 0:
        top = float(row.max())
        scale = float(row.abs().max())
        return min(float(row[a]), float(row[b])) >= top - tol * scale
    cdf = torch.cumsum(torch.softmax(row.double() / temperature, -1), 0)
    return abs(float(cdf[min(a, b)]) - u) < tol


def _agree_up_to_close_calls(w, cfg, prompts, outs_a, outs_b, dtype, temperature=0.0, seeds=None,
                             tol=2.0 ** -6):
    """Token lists of the same requests from two runs: equal, or different first at a place where
    the plain implementation calls it close (what follows a different token differs by right).
    Returns how many requests agree to the end."""
    from ginfer_b200.sampling import uniform
    same = 0
    for i, (p, x, y) in enumerate(zip(prompts, outs_a, outs_b)):
        assert len(x) == len(y)
        if x == y:
            same += 1
            continue
        at = next(j for j in range(len(x)) if x[j] != y[j])
        row = _plain_row(w, cfg, list(p) + list(x[:at]), dtype)
        u = uniform(seeds[i], at) if seeds else None
        assert _close_call(row, x[at], y[at], temperature, u, tol), \
            f"request {i} token {at}: {x[at]} against {y[at]} is no close call"
    return same


@pytest.mark.parametrize("name", ["B", "E"])
@pytest.mark.parametrize("temperature", [0.0, 0.8])
def test_bfloat16_generation_agrees_across_ways_of_batching(tmp_path, name, temperature):
    """bfloat16 through the entry point: the same requests together, under token budgets of 7 and
    13, each alone, with so few pages that requests are preempted, without preparing steps ahead
    and with graphs captured at start-up.  The runs choose the same tokens, greedy and with a
    temperature under fixed seeds; where two runs part, or a run parts from the plain
    implementation (bfloat16-stored), the plain logits call it close (different kernels serve
    different batch shapes and round differently)."""
    from ginfer_b200.sampling import SamplingParams
    d = make_folder(tmp_path, name, seed=4, storage="bfloat16")
    cfg, w = plain.read_model_folder(d)
    prompts = [prompt(n, cfg["vocab_size"], seed=n) for n in (5, 17, 33, 70)]
    seeds = [900 + i for i in range(len(prompts))]
    sps = [SamplingParams(max_tokens=16, ignore_eos=True, temperature=temperature, seed=sd)
           for sd in seeds]
    page = 8 if name == "B" else 16
    kw = dict(kvcache_block_size=page, max_num_batched_tokens=128)
    runs = {
        "together": _engine(d, "bfloat16", **kw).generate(prompts, sps),
        "budget 7": _engine(d, "bfloat16", **dict(kw, max_num_batched_tokens=7)
                            ).generate(prompts, sps),
        "budget 13": _engine(d, "bfloat16", **dict(kw, max_num_batched_tokens=13)
                             ).generate(prompts, sps),
        "few pages": None, "not pipelined": None, "graphs first": None,
    }
    # pages for the first three prompts and one more: when they grow, the youngest gives way
    few = _engine(d, "bfloat16", **dict(kw, num_kvcache_blocks={"B": 12, "E": 7}[name]))
    runs["few pages"] = few.generate(prompts, sps)
    assert few.stats.preemptions >= 1
    runs["not pipelined"] = _engine(d, "bfloat16", pipeline=False, **kw).generate(prompts, sps)
    runs["graphs first"] = _engine(d, "bfloat16", capture_graphs=True, **kw).generate(prompts, sps)
    alone = _engine(d, "bfloat16", **kw)
    runs["alone"] = [alone.generate([p], sp)[0] for p, sp in zip(prompts, sps)]
    base = runs["together"]
    assert any(len(set(o)) > 2 for o in base)
    agree = {k: _agree_up_to_close_calls(w, cfg, prompts, base, v, "bfloat16", temperature, seeds)
             for k, v in runs.items()}
    # the close calls are the exception: most requests agree to the last token in every run
    assert sum(agree.values()) >= 0.7 * len(prompts) * len(runs), agree
    # and against the plain implementation, token by token along the engine's own continuation
    from ginfer_b200.sampling import uniform
    for i, (p, out) in enumerate(zip(prompts, base)):
        ids = list(p)
        for j, tok in enumerate(out):
            row = _plain_row(w, cfg, ids, "bfloat16")
            if temperature <= 0:
                pick = plain.greedy_token(row)
            else:
                pick = plain.temperature_token(row, temperature, uniform(seeds[i], j))
            if tok != pick:
                assert _close_call(row, tok, pick, temperature, uniform(seeds[i], j), 2.0 ** -6), \
                    (i, j, tok, pick)
            ids.append(tok)


def test_command_line(folders, tmp_path):
    d = folders["C"]
    cfg, w = plain.read_model_folder(d)
    prompts = [prompt(n, cfg["vocab_size"], seed=n) for n in (6, 11)]
    f = tmp_path / "prompts.txt"
    f.write_text(" ".join(map(str, prompts[0])) + "\n" + json.dumps(prompts[1]) + "\n")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ginfer_generate"),
                        "--model-path", d, "--dtype", "float32", "--prompt-ids", str(f),
                        "--max-tokens", "5", "--ignore-eos", "--max-num-seqs", "2",
                        "--max-seq-len", "64", "--num-kvcache-blocks", "8"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(x) for x in r.stdout.strip().splitlines()]
    assert [ln["output_ids"] for ln in lines[:2]] == \
        [plain.greedy_generate(w, cfg, p, 5) for p in prompts]
    assert lines[2]["stats"]["decode_tokens"] > 0 and lines[2]["stats"]["avg_ttft_ms"] > 0


def test_no_cpu_path():
    from ginfer_b200 import ops
    with pytest.raises(RuntimeError, match="CUDA device only"):
        ops.embedding(torch.zeros(2, dtype=torch.int32), torch.zeros(4, 8))
    from ginfer_b200.engine.loading import require_cuda
    with pytest.raises(RuntimeError, match="no CPU path"):
        require_cuda("cpu")


@pytest.mark.parametrize("name", ["A", "B"])
def test_graphs_captured_at_start_up_give_the_same_tokens(folders, name):
    """With ``capture_graphs`` the decode steps' CUDA graphs exist before the first request (one
    per batch-size bucket and table width), no further one is captured while generating, and the
    tokens are those of the plain implementation."""
    from ginfer_b200.sampling import SamplingParams
    d = folders[name]
    cfg, w = plain.read_model_folder(d)
    prompts = [prompt(n, cfg["vocab_size"], seed=n) for n in (7, 21, 40, 3, 12, 30, 9, 16, 25, 11)]
    want = [plain.greedy_generate(w, cfg, p, 6) for p in prompts]
    eng = _engine(d, capture_graphs=True, max_num_seqs=12, num_kvcache_blocks=60,
                  max_num_batched_tokens=64)
    before = set(eng.runner._graphs)
    assert {k[0] for k in before} == {1, 2, 3, 4, 5, 6, 7, 8, 16}
    assert eng.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True)) == want
    assert set(eng.runner._graphs) == before and eng.runner.graph_launches > 0
    assert _all_pages_free(eng)


def test_weights_of_an_engine_run_through_the_plain_implementation():
    """``Engine.weights()`` gives the tensors by name, of a folder as stored and of a random model
    as drawn: the plain implementation run on them generates the engine's tokens."""
    from ginfer_b200.sampling import SamplingParams
    from tiny import CONFIGS
    cfg = dict(CONFIGS["B"])
    eng = _engine(None, dtype="float32", config=cfg, weights_seed=9, kvcache_block_size=8)
    w = {k: v.double().cpu() for k, v in eng.weights().items()}
    prompts = [prompt(n, cfg["vocab_size"], seed=n) for n in (6, 19)]
    want = [plain.greedy_generate(w, cfg, p, 5) for p in prompts]
    assert any(len(set(o)) > 2 for o in want)
    assert eng.generate(prompts, SamplingParams(max_tokens=5, ignore_eos=True)) == want


@pytest.mark.parametrize("name,seed", [("C", 0), ("B", 1)])
def test_many_requests_under_pressure_generate_the_plain_tokens(folders, name, seed):
    """Fourteen requests of random lengths, a small token budget and so few pages that requests
    are preempted: portions beside single tokens (which go to the decode kernel), decode batches
    padded to a graph's size, pages used again.  Every request gets the plain implementation's
    tokens."""
    import random

    from ginfer_b200.sampling import SamplingParams
    d = folders[name]
    cfg, w = plain.read_model_folder(d)
    rng = random.Random(seed)
    prompts = [prompt(rng.randint(3, 60), cfg["vocab_size"], seed=100 + i) for i in range(14)]
    news = [rng.randint(1, 10) for _ in prompts]
    want = [plain.greedy_generate(w, cfg, p, n) for p, n in zip(prompts, news)]
    eng = _engine(d, max_num_seqs=12, max_num_batched_tokens=48, num_kvcache_blocks=22,
                  kvcache_block_size=8 if name == "B" else 16)
    got = eng.generate(prompts, [SamplingParams(max_tokens=n, ignore_eos=True) for n in news])
    assert got == want
    assert _all_pages_free(eng)
    assert eng.runner.graph_launches > 0
