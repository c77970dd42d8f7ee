"""Two tiny Qwen2 configurations that differ in every size and option, and helpers that make
model folders for them in a temporary place."""
from __future__ import annotations

import json
import os

import torch

TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "vocab_size": 256,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 512,
    "tie_word_embeddings": True, "use_sliding_window": False, "torch_dtype": "float32",
    "eos_token_id": 255,
}

# every size and option differs from A; sizes are no powers of two
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 224, "vocab_size": 389,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "max_position_embeddings": 640,
    "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 48,
    "max_window_layers": 1, "torch_dtype": "float32", "eos_token_id": [7, 11],
}

# a third one with a head size of 48 (a step of 16 that is no power of two) and 5 heads in 5 groups
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 5,
    "num_key_value_heads": 5, "head_dim": 48, "intermediate_size": 176, "vocab_size": 301,
    "rope_theta": 50000.0, "rms_norm_eps": 3e-6, "max_position_embeddings": 384,
    "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 33,
    "max_window_layers": 0, "torch_dtype": "float32", "eos_token_id": 300,
}

# a fourth one with a head size of 80 (five steps of 16: no multiple of 32), wider heads than the
# model (6 x 80 = 480 channels from a width of 112), one layer: used where a further head size is
# worth a run, not in every test
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 1, "hidden_size": 112, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 80, "intermediate_size": 200, "vocab_size": 277,
    "rope_theta": 200000.0, "rms_norm_eps": 2e-5, "max_position_embeddings": 256,
    "tie_word_embeddings": True, "use_sliding_window": False, "torch_dtype": "float32",
    "eos_token_id": 1,
}

# a fifth one with a head size of 64, which the kernels of the large models serve (prefill
# attention and products on tcgen05, decode attention with tiles by TMA), a window on the second
# layer that is longer than a key tile
TINY_E = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 136, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 312, "vocab_size": 333,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 1024,
    "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 70,
    "max_window_layers": 1, "torch_dtype": "float32", "eos_token_id": 2,
}

# a sixth one with the head size of the large models' checkpoints (128), three heads in one
# group, a window of 150 (more than two key tiles) on its second layer
TINY_F = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 200, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 328, "vocab_size": 311,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 1024,
    "tie_word_embeddings": False, "use_sliding_window": True, "sliding_window": 150,
    "max_window_layers": 1, "torch_dtype": "float32", "eos_token_id": 5,
}

CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F}
# How much a configuration's q and k projections are scaled up (``sharpen``).  Scores grow with
# the head size at a given factor; F (128 channels a head) takes 8 where the others take 12, so
# that its scores spread as far as E's and the 32-bit path's summation order stays below the
# comparison's tolerance.
SHARPNESS = {"F": 8.0}


def sharpen(model_dir: str, q_scale: float = 12.0) -> None:
    """Scale the q and k projections so that attention scores spread over several units: softmax
    becomes peaked and a wrong mask, a missing key or a misplaced page changes the logits
    visibly.  Rewritten with the ``safetensors`` package (not with the framework's writer)."""
    from safetensors import safe_open
    from safetensors.torch import save_file
    path = os.path.join(model_dir, "model.safetensors")
    tensors = {}
    with safe_open(path, framework="pt") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            if k.endswith(("q_proj.weight", "k_proj.weight", "q_proj.bias", "k_proj.bias")):
                t = (t.float() * q_scale).to(t.dtype)
            tensors[k] = t.contiguous()
    save_file(tensors, path)


def make_folder(tmp_path, name: str, seed: int = 0, storage: str = "float32",
                sharp: bool = True, config: dict | None = None) -> str:
    """A model folder of configuration ``name`` (one of ``CONFIGS``, or ``config`` under that
    name).  Folders stored in bfloat16 are sharpened half as much: peaked attention also
    amplifies the flips of bfloat16 rounding, and at a factor of 12 those alone reach 1 % of the
    logits' scale in the three-layer configuration."""
    from ginfer_b200.weights import write_random_model
    d = os.path.join(str(tmp_path), f"tiny_{name}_{storage}_{seed}")
    if not os.path.exists(os.path.join(d, "model.safetensors")):
        write_random_model(d, dict(config or CONFIGS[name]), seed, storage_dtype=storage)
        if sharp:
            factor = SHARPNESS.get(name, 12.0)
            sharpen(d, factor if storage == "float32" else factor / 2)
    return d


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def prompt(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
