"""The persistent kernel that runs every layer of a decode step (off by default): replayed against
the plain implementation, alone and from CUDA graphs, on the tiny configurations."""
import pytest

import replay
from test_replay_gpu import PAGE, _requests, _runner, folders  # noqa: F401  (fixture)
from tiny import CONFIGS, prompt

pytestmark = pytest.mark.gpu


@pytest.fixture()
def fused(monkeypatch):
    monkeypatch.setenv("GINFER_B200_FUSED_DECODE", "1")


def _kernel_of(runner):
    assert runner.model.shortcuts, "the loader did not recognise the stack of layers"
    fd = runner.model.shortcuts[0]
    assert fd.refused is None and fd.kernel is not None, f"the kernel was not used: {fd.refused}"
    return fd.kernel


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("cut", ["tail", "mixed"])
def test_decode_steps_in_one_kernel_agree_with_plain(folders, fused, name, cut):  # noqa: F811
    model_dir = folders[(name, "bfloat16")]
    reqs = _requests(name)
    steps = replay.cut_tail_decode(reqs) if cut == "tail" else replay.cut_mixed(reqs, seed=7)[0]
    runner = _runner(model_dir, "bfloat16", PAGE[name], replay.peak_tokens(steps))
    rows = replay.run_in_process(runner, steps)
    replay.compare(rows, replay.plain_logits(model_dir, reqs, "bfloat16"), "bfloat16", reqs)
    _kernel_of(runner).check_errors()


@pytest.mark.parametrize("name", ["A", "B"])
def test_decode_steps_in_one_kernel_replayed_from_graphs(folders, fused, name):  # noqa: F811
    model_dir = folders[(name, "bfloat16")]
    v = CONFIGS[name]["vocab_size"]
    reqs = {"x": prompt(150, v, seed=1), "y": prompt(90, v, seed=2), "z": prompt(70, v, seed=3)}
    steps = [{"step": 0, "end": [], "entries": [
        {"id": k, "tokens": t[:20], "want": list(range(20))} for k, t in reqs.items()]}]
    at = {k: 20 for k in reqs}
    while any(at[k] < len(reqs[k]) for k in reqs):
        ent = [{"id": k, "tokens": [reqs[k][at[k]]], "want": [0]}
               for k in reqs if at[k] < len(reqs[k])]
        for e in ent:
            at[e["id"]] += 1
        steps.append({"step": len(steps), "end": [], "entries": ent})
    runner = _runner(model_dir, "bfloat16", PAGE[name], replay.peak_tokens(steps), eager=False)
    rows = replay.run_in_process(runner, steps)
    replay.compare(rows, replay.plain_logits(model_dir, reqs, "bfloat16"), "bfloat16", reqs)
    assert runner.graph_launches > 0
    _kernel_of(runner).check_errors()
