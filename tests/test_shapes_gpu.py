"""Layer sizes of larger models than the tiny ones (the Qwen2-1.5B, Qwen2.5-7B and -32B shapes, one
layer, a small vocabulary): the bfloat16 path (tcgen05 products, bf16 attention kernels, CUDA
graphs) against the plain implementation where that is affordable on the CPU, and against the
32-bit path of the same engine (FMA products, fp32-arithmetic attention), which shares no kernel
with it beyond the element-wise ones."""
import numpy as np
import pytest
import torch

import replay
from tiny import make_folder, prompt

pytestmark = pytest.mark.gpu

SHAPES = {
    "7b": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
               intermediate_size=18944),
    "32b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                intermediate_size=27648),
    # sizes that are no multiples of the kernels' tiles: 72 = 64 + 8 channels, 5 heads in 5 groups
    "odd": dict(hidden_size=1192, num_attention_heads=5, num_key_value_heads=5,
                intermediate_size=3000, head_dim=64),
}


# the benchmark's own layer sizes (Qwen2-1.5B)
SHAPES_PLAIN = {
    "1.5b": dict(hidden_size=1536, num_attention_heads=12, num_key_value_heads=2,
                 intermediate_size=8960, head_dim=128),
    "odd": SHAPES["odd"],
}


@pytest.mark.parametrize("name", list(SHAPES_PLAIN))
@pytest.mark.parametrize("cut", ["tail", "mixed_long"])
def test_bfloat16_path_agrees_with_plain_at_real_layer_sizes(tmp_path, name, cut):
    """One layer of the benchmark's sizes (and of sizes that fit no tile), stepped in bfloat16 as
    most of each request at once and its last tokens one by one (decode graphs), and as portions
    of 64 to 200 tokens beside single tokens: every row against the plain implementation."""
    from ginfer_b200.engine import ModelRunner
    from ginfer_b200.engine.loading import load_model
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 1,
           "vocab_size": 643, "rope_theta": 1e6, "rms_norm_eps": 1e-6,
           "max_position_embeddings": 512, "tie_word_embeddings": False,
           "use_sliding_window": False, "torch_dtype": "bfloat16"}
    cfg.update(SHAPES_PLAIN[name])
    d = make_folder(tmp_path, f"shape_{name}", seed=11, storage="bfloat16", sharp=False,
                    config=cfg)
    reqs = {f"r{i}": prompt(n, 643, seed=20 + i) for i, n in enumerate((230, 71, 150))}
    if cut == "tail":
        steps = replay.cut_tail_decode(reqs, tail=6)
    else:
        steps, _ = replay.cut_mixed(reqs, seed=5, sizes=replay.LONG_SIZES, decode_tail=4)
    model, _ = load_model(d, "bfloat16")
    runner = ModelRunner(model, page_size=16, max_num_seqs=4, max_seq_len=256,
                         num_pages=replay.peak_tokens(steps) // 16, max_num_batched_tokens=512,
                         enforce_eager=False)
    rows = replay.run_in_process(runner, steps)
    replay.compare(rows, replay.plain_logits(d, reqs, "bfloat16"), "bfloat16", reqs)


@pytest.mark.parametrize("name", list(SHAPES))
def test_bfloat16_path_agrees_with_the_32_bit_path_at_large_layer_sizes(name):
    from ginfer_b200.engine import ModelRunner, StepEntry
    from ginfer_b200.engine.loading import random_model
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 1,
           "head_dim": 128, "vocab_size": 643, "rope_theta": 1e6, "rms_norm_eps": 1e-6,
           "max_position_embeddings": 512, "tie_word_embeddings": False,
           "use_sliding_window": False, "torch_dtype": "bfloat16"}
    cfg.update(SHAPES[name])
    toks = {"a": prompt(70, 643, 1), "b": prompt(33, 643, 2)}
    late = prompt(92, 643, 3)      # joins while the others decode: portions beside single tokens
    out = {}
    for dtype in ("float32", "bfloat16"):
        model, _ = random_model(cfg, 11, dtype)
        r = ModelRunner(model, page_size=16, max_num_seqs=3, max_seq_len=256, num_pages=32,
                        enforce_eager=(dtype == "float32"))
        rows = [r.step([StepEntry(k, t[:-4], [len(t) - 5]) for k, t in toks.items()]).clone()]
        cuts = {4: late[:80], 3: late[80:90], 2: late[90:91], 1: late[91:]}
        for i in range(4, 0, -1):                       # then token by token (graphs in bf16)
            # (a step's logits are valid until the next step: keep a copy)
            ent = [StepEntry(k, [t[-i]], [0]) for k, t in toks.items()]
            ent.append(StepEntry("late", cuts[i], [len(cuts[i]) - 1]))
            rows.append(r.step(ent).clone())
        out[dtype] = torch.cat(rows).float().cpu()
        del r, model
        torch.cuda.empty_cache()
    a, b = out["float32"], out["bfloat16"]
    scale = a.abs().max().item()
    # random bf16 weights are the same numbers in both runs (drawn in bf16, widened for fp32);
    # what differs is the rounding of activations: a few bf16 ulps of the logits' scale
    worst = (a - b).abs().max().item() / scale
    rms = (a - b).pow(2).mean().sqrt().item() / scale
    print(f"{name}: scale {scale:.3f} worst {worst:.4f} rms {rms:.4f} "
          f"argmax {(a.argmax(-1) == b.argmax(-1)).float().mean().item():.2f}")
    assert rms <= 0.01 and worst <= 0.03, (rms, worst)


@pytest.mark.parametrize("head_dim,heads,kv_heads", [(64, 6, 2), (128, 3, 1)])
def test_a_step_of_many_tokens_agrees_with_portions_plain_and_the_32_bit_path(
        tmp_path, head_dim, heads, kv_heads, monkeypatch):
    """Where it is switched on, from 1,024 tokens on a step's joined q/k/v product rotates q and k
    and writes the cache in its own epilogue (and the gated product joins SiLU*mul).  The same prompt in one step, as a
    short portion followed by one of 1,030 tokens (the epilogue then works at positions and cache
    slots offset from its rows), in two portions below that size (plain products, the rotation
    kernel) and on the 32-bit path must give the same logits, for the prompt's last token and for
    the tokens decoded after it, which read the keys and values the epilogue cached; the
    bfloat16 runs are also held against the plain implementation."""
    from ginfer_b200 import ops
    from ginfer_b200.engine import ModelRunner, StepEntry
    from ginfer_b200.engine.loading import load_model
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 2,
           "hidden_size": 264, "num_attention_heads": heads, "num_key_value_heads": kv_heads,
           "head_dim": head_dim, "intermediate_size": 520, "vocab_size": 643, "rope_theta": 1e4,
           "rms_norm_eps": 1e-6, "max_position_embeddings": 1536, "tie_word_embeddings": False,
           "use_sliding_window": False, "torch_dtype": "bfloat16"}
    d = make_folder(tmp_path, f"many_{head_dim}", seed=3, storage="bfloat16", sharp=False,
                    config=cfg)
    toks = prompt(1100, 643, 5)
    tail = prompt(3, 643, 6)
    from ginfer_b200.ops import gemm_prefill
    monkeypatch.setattr(gemm_prefill, "QKV_EPILOGUE", True)      # (an option: off by default)
    served = []
    inner = ops.qkv_rope_write

    def counted(x, *a, **k):
        y = inner(x, *a, **k)
        served.append((x.shape[0], y is not None))
        return y
    monkeypatch.setattr(ops, "qkv_rope_write", counted)

    def run(dtype, cuts):
        model, _ = load_model(d, dtype)
        r = ModelRunner(model, page_size=16, max_num_seqs=2, max_seq_len=1536, num_pages=80,
                        enforce_eager=True)
        rows, at = [], 0
        for n in cuts:
            y = r.step([StepEntry("a", toks[at:at + n], [n - 1])]).clone()
            at += n
        rows.append(y)
        for t in tail:
            rows.append(r.step([StepEntry("a", [t], [0])]).clone())
        del r, model
        torch.cuda.empty_cache()
        return torch.cat(rows).float().cpu()

    whole = run("bfloat16", [1100])
    assert [m for m, ok in served if ok] == [1100, 1100], served     # both layers, one long step
    served.clear()
    second = run("bfloat16", [70, 1030])
    assert [m for m, ok in served if ok] == [1030, 1030], served
    cut = run("bfloat16", [600, 500])
    full = run("float32", [1100])
    scale = full.abs().max().item()
    for name, other in (("a later portion", second), ("portions", cut), ("32-bit", full)):
        worst = (whole - other).abs().max().item() / scale
        rms = (whole - other).pow(2).mean().sqrt().item() / scale
        print(f"hd {head_dim} against {name}: scale {scale:.3f} worst {worst:.4f} rms {rms:.4f}")
        assert rms <= 0.01 and worst <= 0.03, (name, rms, worst)
    # against the plain implementation: rows 1099 .. 1102 of the whole sequence
    seq = toks + tail
    ref = replay.plain_logits(d, {"a": seq}, "bfloat16")["a"][1099:1103]
    atol, rtol = replay.tolerances("bfloat16", float(np.abs(ref).max()))
    for name, got in (("one step", whole), ("a later portion", second), ("portions", cut)):
        err = np.abs(got.double().numpy() - ref)
        assert (err <= atol + rtol * np.abs(ref)).all(), (name, float(err.max()), atol)


def test_decoding_few_requests_with_thousands_of_keys_agrees_with_plain(tmp_path):
    """A request of 4,600 tokens (and one of 41), their last tokens decoded one by one from CUDA
    graphs: so few requests with so many keys take several thread-block clusters a request and a
    kernel that adds their results up.  Every decoded row against the plain implementation, with a query and
    key sharpened so that a far key carries weight."""
    from ginfer_b200.engine import ModelRunner
    from ginfer_b200.engine.loading import load_model
    from ginfer_b200.ops import attention_bf16
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 1,
           "vocab_size": 300, "rope_theta": 1e6, "rms_norm_eps": 1e-6, "hidden_size": 128,
           "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 64,
           "intermediate_size": 256, "max_position_embeddings": 8192,
           "tie_word_embeddings": False, "use_sliding_window": False, "torch_dtype": "bfloat16"}
    d = make_folder(tmp_path, "long_context", seed=3, storage="bfloat16", config=cfg)
    # (a second, short request beside it: most of the parts hold none of its keys)
    reqs = {"far": prompt(4600, 300, seed=9), "near": prompt(41, 300, seed=10)}
    tail = 5
    steps = [{"step": i, "end": [], "entries": [
        {"id": rid, "tokens": toks[:-tail], "want": list(range(len(toks) - tail))}]}
        for i, (rid, toks) in enumerate(reqs.items())]
    for k in range(tail, 0, -1):                         # then both decode side by side
        steps.append({"step": len(steps), "end": list(reqs) if k == 1 else [], "entries": [
            {"id": rid, "tokens": [toks[-k]], "want": [0]} for rid, toks in reqs.items()]})
    assert attention_bf16.decode_partition(2, 2, 1, 5120)[1] > 1
    model, _ = load_model(d, "bfloat16")
    runner = ModelRunner(model, page_size=16, max_num_seqs=2, max_seq_len=4800, num_pages=320,
                         max_num_batched_tokens=8192, enforce_eager=False)
    rows = replay.run_in_process(runner, steps)
    replay.compare(rows, replay.plain_logits(d, reqs, "bfloat16"), "bfloat16", reqs)
