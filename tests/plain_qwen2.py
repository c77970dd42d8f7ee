"""A plain, slow Qwen2 for the tests: whole sequences, no cache, no batching, one function per part.

It shares no code with ``ginfer_b200``.  It is written from the reference's formulas (11Aln0/ginfer;
each function cites file:line of that project).  The reference cannot be built or imported on the
test machine (its build downloads nine packages, it has no CPU kernels, and its attention kernels
take head sizes 64 and 128 only), so nothing here was compared with the reference's own output:
this file rests on the formulas.  ``tests/test_plain.py`` holds its parts against hand-made
cases and against the formulas that the reference's own Python tests use as their oracles
(``python/test/test_op.py``).

Arithmetic is float64 on the CPU unless ``dtype`` says otherwise, except where the reference fixes
a 32-bit quantity that changes the result's meaning: the rotary angle is the fp32 product of the
fp32 position and the fp32 inverse frequency.

The sliding window is not in the reference.  Its definition here: layer ``i`` is windowed iff
``use_sliding_window`` and ``i >= max_window_layers``; in a windowed layer the query at position
``p`` sees key ``c`` iff ``c <= p`` and ``p - c < sliding_window``.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np
import torch


# ----------------------------------------------------------------------------- stored precision
class Stored:
    """Which precision activations are *stored* in between parts.  The default stores nothing
    rounded (pure float64).  ``Stored.bf16()`` rounds to bfloat16 wherever the bfloat16 serving
    path of an engine writes an activation to memory: after a norm, a projection, the rotary
    encoding, the attention output and the gated product.  The residual sum stays unrounded (it is
    kept in 32-bit).  Arithmetic stays float64 either way."""
    round = staticmethod(lambda t: t)

    @classmethod
    def bf16(cls):
        cls.round = staticmethod(lambda t: t.to(torch.bfloat16).to(t.dtype))

    @classmethod
    def exact(cls):
        cls.round = staticmethod(lambda t: t)


# ----------------------------------------------------------------------------- reading a folder
def read_model_folder(model_dir: str, dtype=torch.float64):
    """``(config dict, {tensor name: tensor as dtype})`` using the ``safetensors`` package."""
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            weights[k] = f.get_tensor(k).to(dtype)
    return cfg, weights


def head_dim_of(cfg: dict) -> int:
    # ginfer/model/loader/model_loader.cc:45,103-105: head_dim, else hidden_size / num_heads
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


def layer_window(cfg: dict, layer: int) -> int:
    if not cfg.get("use_sliding_window", False):
        return 0
    first = cfg.get("max_window_layers")
    if first is None:
        first = cfg["num_hidden_layers"]
    return int(cfg["sliding_window"]) if layer >= first else 0


# ----------------------------------------------------------------------------- parts
def embed(token_ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    # ginfer/core/op/kernels/cuda/embedding_kernel.cu:16-24: out[t, :] = W[ids[t], :]
    return table[token_ids.long()]


def rms_norm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    # ginfer/core/op/kernels/cuda/rmsnorm_kernel.cu:27-66:
    # ss = sum x^2; rms = sqrt(ss / H + eps); out = x * gamma / rms
    ss = (x * x).sum(dim=-1, keepdim=True)
    rms = torch.sqrt(ss / x.shape[-1] + eps)
    return Stored.round(x * gamma / rms)


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    # ginfer/core/layer/linear.cc:13-35: y = x W^T (+ b), W stored [out, in]
    y = x @ w.t()
    return Stored.round(y if b is None else y + b)


def rotary_cos_sin(positions: torch.Tensor, head_dim: int, theta: float):
    # ginfer/core/op/kernels/cuda/rope_kernel.cu:13-16,61-71:
    # inv_j = 1 / theta^(j / (hd/2)); angle = pos * inv_j (fp32); sin, cos of the angle
    half = head_dim // 2
    inv = 1.0 / np.power(np.float64(theta), np.arange(half, dtype=np.float64) / half)
    inv32 = inv.astype(np.float32)
    pos32 = positions.numpy().astype(np.float32)
    ang = (pos32[:, None] * inv32[None, :]).astype(np.float32).astype(np.float64)
    return torch.from_numpy(np.cos(ang)), torch.from_numpy(np.sin(ang))


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # ginfer/core/op/kernels/cuda/rope_kernel.cu:84-102: pairs (j, j + hd/2):
    # o_j = x_j cos - x_{j+hd/2} sin ; o_{j+hd/2} = x_j sin + x_{j+hd/2} cos
    # x: [T, heads, hd]; cos, sin: [T, hd/2]
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :].to(x.dtype), sin[:, None, :].to(x.dtype)
    return Stored.round(torch.cat([a * c - b * s, a * s + b * c], dim=-1))


def visibility(num_tokens: int, window: int) -> torch.Tensor:
    # ginfer/core/op/kernels/cuda/page_attn_kernel/flash_gqa_varlen_kernel.cu:202,214:
    # key c visible to query row r iff c <= r + (kv_len - q_len); whole sequence: c <= r.
    # Window (not in the reference): and r - c < window.
    r = torch.arange(num_tokens)[:, None]
    c = torch.arange(num_tokens)[None, :]
    ok = c <= r
    if window > 0:
        ok &= (r - c) < window
    return ok


def gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int,
                  scale: float | None = None) -> torch.Tensor:
    # flash_gqa_varlen_kernel.cu:169-172,202-257,439: query head n reads kv head n / (nh/nkv);
    # s = q.k / sqrt(hd); masked to -inf; softmax over keys; o = p v.
    # q [T, nh, hd], k, v [T, nkv, hd] -> [T, nh, hd]
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    ok = visibility(T, window)
    out = torch.empty_like(q)
    for n in range(nh):
        kv = n // group
        s = (q[:, n, :] @ k[:, kv, :].t()) * scale
        s = s.masked_fill(~ok, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, n, :] = p @ v[:, kv, :]
    return Stored.round(out)


def swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor):
    # ginfer/core/layer/transformer/feedforward.cc:22-25 and
    # ginfer/core/op/kernels/cuda/swiglu_kernel.cu:24-27: z = g * 1/(1+exp(-g)) * u; m = z W_d^T
    g, u = linear(x, w_gate), linear(x, w_up)
    z = Stored.round(g * (1.0 / (1.0 + torch.exp(-g))) * u)
    return linear(z, w_down)


def project_qkv(x: torch.Tensor, w: dict, prefix: str, cfg: dict, positions: torch.Tensor):
    # ginfer/core/layer/transformer/attention.cc:61-72: q/k/v projections (bias on q, k, v for
    # Qwen2: ginfer/model/qwen2.cc:15-17), split into heads, rotary on q and k
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    a = prefix + ".self_attn."
    T = x.shape[0]
    q = linear(x, w[a + "q_proj.weight"], w[a + "q_proj.bias"]).reshape(T, nh, hd)
    k = linear(x, w[a + "k_proj.weight"], w[a + "k_proj.bias"]).reshape(T, nkv, hd)
    v = linear(x, w[a + "v_proj.weight"], w[a + "v_proj.bias"]).reshape(T, nkv, hd)
    cos, sin = rotary_cos_sin(positions, hd, float(cfg.get("rope_theta", 10000.0)))
    return apply_rotary(q, cos, sin), apply_rotary(k, cos, sin), v


def decoder_layer(h: torch.Tensor, w: dict, layer: int, cfg: dict, positions: torch.Tensor,
                  shared_kv=None):
    """One pre-norm block; returns ``(h', (k, v))``.  ``shared_kv`` replaces the layer's own keys
    and values (a layer reading another layer's cache)."""
    # ginfer/core/layer/transformer/encoder.cc:33-39
    p = f"model.layers.{layer}"
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    x = rms_norm(h, w[p + ".input_layernorm.weight"], eps)
    q, k, v = project_qkv(x, w, p, cfg, positions)
    if shared_kv is not None:
        k, v = shared_kv
    o = gqa_attention(q, k, v, layer_window(cfg, layer))
    a = linear(o.reshape(h.shape[0], -1), w[p + ".self_attn.o_proj.weight"])   # attention.cc:80-81
    r = h + a
    y = rms_norm(r, w[p + ".post_attention_layernorm.weight"], eps)
    m = swiglu(y, w[p + ".mlp.gate_proj.weight"], w[p + ".mlp.up_proj.weight"],
               w[p + ".mlp.down_proj.weight"])
    return r + m, (k, v)


def forward(w: dict, cfg: dict, token_ids, run=None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one whole sequence.  ``run``: list of ``(layer, cache, write)``;
    default every layer once in order."""
    # ginfer/model/model.cc:152-166 (embed, layers, final norm), lmhead.cc:27, qwen2.cc:42-46 (tied)
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.numel())
    h = embed(ids, w["model.embed_tokens.weight"])
    if run is None:
        run = [(i, i, True) for i in range(cfg["num_hidden_layers"])]
    caches: dict[int, tuple] = {}
    for layer, cache, write in run:
        if write:
            h, caches[cache] = decoder_layer(h, w, layer, cfg, positions)
        else:
            h, _ = decoder_layer(h, w, layer, cfg, positions, shared_kv=caches[cache])
    x = rms_norm(h, w["model.norm.weight"], float(cfg.get("rms_norm_eps", 1e-6)))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else w["lm_head.weight"]
    return x @ head.t()            # logits are not stored in reduced precision


# ----------------------------------------------------------------------------- choosing tokens
def greedy_token(logits_row: torch.Tensor) -> int:
    # ginfer/core/op/kernels/cuda/argmax_kernel.cu:63-98 (values compared as fp32); lowest index
    # among equal maxima
    m = logits_row.max()
    return int(torch.nonzero(logits_row == m)[0, 0])


def temperature_token(logits_row: torch.Tensor, temperature: float, u: float) -> int:
    """First index whose cumulative softmax(logits / temperature) reaches ``u``."""
    p = torch.softmax(logits_row.double() / temperature, dim=-1)
    cdf = torch.cumsum(p, dim=-1)
    idx = int(torch.searchsorted(cdf, torch.tensor(u, dtype=torch.float64)))
    return min(idx, logits_row.numel() - 1)


def greedy_generate(w: dict, cfg: dict, prompt, num_new: int) -> list[int]:
    ids = list(prompt)
    out = []
    for _ in range(num_new):
        t = greedy_token(forward(w, cfg, ids)[-1])
        out.append(t)
        ids.append(t)
    return out
