"""Layer sizes of larger models than the tiny ones (the Qwen2.5-7B and -32B shapes, one layer, a
small vocabulary): the bfloat16 path (tcgen05 products, bf16 attention kernels, CUDA graphs)
against the 32-bit path of the same engine (FMA products, fp32-arithmetic attention), which shares
no kernel with it beyond the element-wise ones."""
import pytest
import torch

from tiny import prompt

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
