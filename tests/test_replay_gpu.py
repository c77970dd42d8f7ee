"""Replay of the same requests under every way of cutting them into steps, in 32-bit and in
bfloat16, against the plain implementation."""
import pytest

import replay
from tiny import CONFIGS, make_folder, prompt

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 70, 130, 49], "B": [1, 40, 90, 200, 66, 133], "C": [3, 64, 97, 35],
           "D": [2, 81, 150, 64, 33], "E": [9, 140, 260, 75, 200]}
PAGE = {"A": 16, "B": 8, "C": 4, "D": 32, "E": 16, "F": 16}
# long requests for the cuts whose portions are 64 tokens and more
LONG_LENGTHS = {"E": [530, 333, 410, 150], "F": [520, 290, 400, 135]}


def _requests(name, lengths=None):
    v = CONFIGS[name]["vocab_size"]
    return {f"r{i}": prompt(n, v, seed=100 * i + n)
            for i, n in enumerate(lengths or LENGTHS[name])}


def _storage(dtype):
    return "bfloat16" if dtype == "bfloat16" else "float32"


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {(n, s): make_folder(root, n, seed=1, storage=s)
            for n in CONFIGS for s in ("float32", "bfloat16")}


def _runner(model_dir, dtype, page, max_tokens, eager=True):
    from ginfer_b200.engine import ModelRunner
    from ginfer_b200.engine.loading import load_model
    model, _ = load_model(model_dir, dtype)
    budget = -(-max_tokens // 64) * 64
    return ModelRunner(model, page_size=page, max_num_seqs=4, max_seq_len=budget,
                       num_pages=budget // page, max_num_batched_tokens=budget,
                       enforce_eager=eager)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cut", [(n, c) for n in "ABC" for c in (
    "whole", "tail", "portions", "mixed", "mixed_singles_first")] + [("D", "tail"), ("D", "mixed")] + [
    ("E", c) for c in ("whole", "tail", "portions", "mixed")])
def test_cuts_agree_with_plain(folders, name, dtype, cut):
    model_dir = folders[(name, _storage(dtype))]
    reqs = _requests(name)
    if cut == "whole":
        steps = replay.cut_whole(reqs)
    elif cut == "tail":
        steps = replay.cut_tail_decode(reqs)
    elif cut == "portions":
        steps = replay.cut_portions(reqs)
    else:
        steps, _ = replay.cut_mixed(reqs, seed=7, singles_first=cut.endswith("first"))
    max_tokens = replay.peak_tokens(steps)          # so few pages that they are used again
    runner = _runner(model_dir, dtype, PAGE[name], max_tokens)
    rows = replay.run_in_process(runner, steps)
    replay.compare(rows, replay.plain_logits(model_dir, reqs, dtype), dtype, reqs)
    assert not runner.cache.requests and all(
        f == p.num_pages for f, p in zip(runner.cache.free_pages(), runner.cache.pools))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["E", "F"])
@pytest.mark.parametrize("cut", ["portions_long", "mixed_long", "mixed_long_singles_first"])
def test_long_portions_agree_with_plain(folders, name, dtype, cut):
    """Portions of 64 to 200 tokens, at head sizes 64 and 128: in bfloat16 the tcgen05 attention
    kernel then runs for portions that do not start their request (positions offset from the
    rows), several requests a launch, and beside single tokens that go to the decode kernel."""
    model_dir = folders[(name, _storage(dtype))]
    reqs = _requests(name, LONG_LENGTHS[name])
    if cut == "portions_long":
        steps = replay.cut_portions(reqs, sizes=replay.LONG_SIZES)
    else:
        steps, _ = replay.cut_mixed(reqs, seed=11, sizes=replay.LONG_SIZES, decode_tail=6,
                                    singles_first=cut.endswith("first"))
    assert any(len(e["tokens"]) >= 64 and len(s["entries"]) > 1
               for s in steps for e in s["entries"]) or cut == "portions_long"
    runner = _runner(model_dir, dtype, PAGE[name], replay.peak_tokens(steps))
    rows = replay.run_in_process(runner, steps)
    replay.compare(rows, replay.plain_logits(model_dir, reqs, dtype), dtype, reqs)
    assert not runner.cache.requests and all(
        f == p.num_pages for f, p in zip(runner.cache.free_pages(), runner.cache.pools))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "E"])
def test_decode_steps_replayed_from_cuda_graphs(folders, name, dtype):
    """Long decoding, one token a step for two requests side by side, with decode steps replayed
    from CUDA graphs (as serving does) and the block table growing past a graph's width."""
    model_dir = folders[(name, _storage(dtype))]
    v = CONFIGS[name]["vocab_size"]
    reqs = {"x": prompt(300, v, seed=1), "y": prompt(180, v, seed=2)}
    steps = [{"step": 0, "end": [], "entries": [
        {"id": "x", "tokens": reqs["x"][:40], "want": list(range(40))},
        {"id": "y", "tokens": reqs["y"][:3], "want": [0, 1, 2]}]}]
    ax, ay = 40, 3
    while ax < 300 or ay < 180:
        ent = []
        if ax < 300:
            ent.append({"id": "x", "tokens": [reqs["x"][ax]], "want": [0]})
            ax += 1
        if ay < 180:
            ent.append({"id": "y", "tokens": [reqs["y"][ay]], "want": [0]})
            ay += 1
        steps.append({"step": len(steps), "entries": ent, "end": []})
    steps[-1]["end"] = ["x", "y"]
    # pages of 4 tokens, of 16 where the decode kernel that loads its tiles by TMA is to run
    runner = _runner(model_dir, dtype, 16 if name == "E" else 4, 512, eager=False)
    rows = replay.run_in_process(runner, steps)
    assert len(runner._graphs) >= 2 and runner.graph_launches > 0
    replay.compare(rows, replay.plain_logits(model_dir, reqs, dtype), dtype, reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "E"])
@pytest.mark.parametrize("eager", [True, False])
def test_first_tokens_one_by_one(folders, name, dtype, eager):
    """A sequence fed one token at a time from its very first token (position 0, the first page,
    the first page edge, the window filling up), two requests side by side that start at
    different steps."""
    model_dir = folders[(name, _storage(dtype))]
    v = CONFIGS[name]["vocab_size"]
    reqs = {"p": prompt(70, v, seed=11), "q": prompt(45, v, seed=12)}
    steps = []
    for i in range(70):
        ent = [{"id": "p", "tokens": [reqs["p"][i]], "want": [0]}]
        if 5 <= i < 50:
            ent.append({"id": "q", "tokens": [reqs["q"][i - 5]], "want": [0]})
        steps.append({"step": i, "entries": ent, "end": ["q"] if i == 49 else []})
    steps[-1]["end"] = ["p"]
    runner = _runner(model_dir, dtype, PAGE[name], 192, eager=eager)
    rows = replay.run_in_process(runner, steps)
    replay.compare(rows, replay.plain_logits(model_dir, reqs, dtype), dtype, reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program_mixed(folders, tmp_path, dtype):
    """The same through ``bin/trace_run`` (page size 16, pool sized by --max-tokens)."""
    model_dir = folders[("B", _storage(dtype))]
    reqs = _requests("B")
    steps, peak = replay.cut_mixed(reqs, seed=3)
    rows = replay.run_trace_program(model_dir, dtype, steps, peak, str(tmp_path / "out"))
    replay.compare(rows, replay.plain_logits(model_dir, reqs, dtype), dtype, reqs)


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("cut", ["tail", "mixed"])
@pytest.mark.parametrize("fold", [16, 64])
def test_cuts_agree_with_plain_when_norms_are_folded_into_products(folders, name, cut, fold,
                                                                    monkeypatch):
    """Short bfloat16 steps can fold the residual additions and the normalisations into the
    neighbouring products (off by default).  With that on, for steps of up to 16 and up to 64
    tokens, the logits are those of the plain implementation too."""
    from ginfer_b200.ops import gemm_bf16
    from ginfer_b200.parts import block
    monkeypatch.setattr(block, "FOLD_MAX_TOKENS", fold)
    monkeypatch.setattr(gemm_bf16, "PLAIN_MAX_TOKENS", fold)
    monkeypatch.setattr(gemm_bf16, "PLAIN_MAX_TOKENS_LONG_K", max(fold, 48))
    monkeypatch.setattr(gemm_bf16, "MAX_TOKENS", fold)
    model_dir = folders[(name, "bfloat16")]
    reqs = _requests(name)
    steps = replay.cut_tail_decode(reqs) if cut == "tail" else replay.cut_mixed(reqs, seed=7)[0]
    runner = _runner(model_dir, "bfloat16", PAGE[name], replay.peak_tokens(steps))
    rows = replay.run_in_process(runner, steps)
    replay.compare(rows, replay.plain_logits(model_dir, reqs, "bfloat16"), "bfloat16", reqs)


@pytest.mark.parametrize("name", ["B", "E"])
def test_prompt_portions_of_a_shape_that_comes_again_are_replayed_from_graphs(folders, name):
    """Steps with prompt portions whose shape (portion lengths, wanted rows, table width) has come
    before are replayed from a CUDA graph, whatever position the portion starts at: three
    requests of 560 tokens, each fed as 260 + 260 + 40.  The 260-token step comes a second time
    at position 260 of the first request (the graph is captured there) and is replayed at
    positions 0 and 260 of the others.  All agree with plain."""
    model_dir = folders[(name, "bfloat16")]
    v = CONFIGS[name]["vocab_size"]
    reqs = {f"q{i}": prompt(560, v, seed=50 + i) for i in range(3)}
    steps = []
    for rid, toks in reqs.items():
        for lo, hi in ((0, 260), (260, 520), (520, 560)):
            steps.append({"step": len(steps), "end": [rid] if hi == 560 else [], "entries": [
                {"id": rid, "tokens": toks[lo:hi], "want": list(range(hi - lo))}]})
    # pages of 16: positions 0 and 260 of a 260-token portion then share a block-table width
    runner = _runner(model_dir, "bfloat16", 16, 576, eager=False)
    from ginfer_b200.engine import StepEntry
    outs, replayed = {}, []
    for s in steps:
        before = runner.graph_launches
        e = s["entries"][0]
        outs[s["step"]] = runner.step([StepEntry(e["id"], e["tokens"], e["want"])]).cpu().numpy()
        replayed.append(runner.graph_launches > before)
        for r in s["end"]:
            runner.end(r)
    # captured in the second step (position 260); replayed at 0 and at 260 afterwards
    assert replayed == [False, True, False, True, True, False, True, True, False], replayed
    rows = replay.collect(steps, lambda i: outs[i])
    replay.compare(rows, replay.plain_logits(model_dir, reqs, "bfloat16"), "bfloat16", reqs)
    assert sum(isinstance(k[0], str) for k in runner._graphs) == 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_decode_batches_are_padded_to_the_batch_size_of_a_graph(folders, name, dtype):
    """Eleven requests decode side by side (the graph is one of 16: five rows of padding that
    write and read the scratch page), then ten and nine as requests end, with so few pages that
    freed ones are taken again by the request that joins late.  All agree with plain."""
    from ginfer_b200.engine import ModelRunner
    from ginfer_b200.engine.loading import load_model
    model_dir = folders[(name, _storage(dtype))]
    v = CONFIGS[name]["vocab_size"]
    lens = [30, 41, 52, 33, 44, 55, 36, 47, 58, 39, 50, 45]
    reqs = {f"p{i}": prompt(n, v, seed=70 + i) for i, n in enumerate(lens)}
    ids = list(reqs)
    first, late = ids[:11], ids[11]
    steps = [{"step": 0, "end": [], "entries": [
        {"id": r, "tokens": reqs[r][:20], "want": list(range(20))} for r in first]}]
    at = {r: 20 for r in first}
    live = list(first)
    while live:
        ent = [{"id": r, "tokens": [reqs[r][at[r]]], "want": [0]} for r in live]
        for r in live:
            at[r] += 1
        done = [r for r in live if at[r] == len(reqs[r])]
        steps.append({"step": len(steps), "entries": ent, "end": done})
        live = [r for r in live if r not in done]
        if done and late not in at and len(live) <= 9:
            at[late] = 0                               # joins with its whole prompt but the last
            n = len(reqs[late]) - 10
            steps.append({"step": len(steps), "end": [], "entries": [
                {"id": late, "tokens": reqs[late][:n], "want": list(range(n))}]})
            at[late] = n
            live.append(late)
    page = PAGE[name]
    model, _ = load_model(model_dir, dtype)
    pages = sum(-(-n // page) for n in lens[:11]) + 1
    runner = ModelRunner(model, page_size=page, max_num_seqs=12, max_seq_len=64,
                         num_pages=pages, max_num_batched_tokens=256, enforce_eager=False)
    assert runner.graph_batch(11) == 16 and runner.graph_batch(8) == 8
    rows = replay.run_in_process(runner, steps)
    assert any(k[0] == 16 for k in runner._graphs) and runner.graph_launches > 0
    replay.compare(rows, replay.plain_logits(model_dir, reqs, dtype), dtype, reqs)
    assert not runner.cache.requests and all(
        f == p.num_pages for f, p in zip(runner.cache.free_pages(), runner.cache.pools))
