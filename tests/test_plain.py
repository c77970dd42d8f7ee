"""The plain implementation checked against hand-made cases and its own invariants (no GPU)."""
import math

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from tiny import make_folder, prompt


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    g = torch.tensor([2.0, 0.5], dtype=torch.float64)
    out = plain.rms_norm(x, g, 0.5)
    rms = math.sqrt((9 + 16) / 2 + 0.5)
    assert torch.allclose(out, torch.tensor([[3 * 2 / rms, 4 * 0.5 / rms]], dtype=torch.float64))


def test_rotary_pairs_angles_and_norm():
    hd, theta = 8, 100.0
    pos = torch.tensor([0, 1, 5])
    cos, sin = plain.rotary_cos_sin(pos, hd, theta)
    assert cos.shape == (3, 4)
    assert torch.allclose(cos[0], torch.ones(4, dtype=torch.float64))
    inv = [1.0 / theta ** (j / 4) for j in range(4)]
    assert np.allclose(cos[2].numpy(), np.cos([5 * v for v in inv]), atol=1e-6)
    x = torch.randn(3, 2, hd, dtype=torch.float64)
    y = plain.apply_rotary(x, cos, sin)
    assert torch.allclose(y[0], x[0])                               # position 0: identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))           # a rotation
    j = 1                                                           # pair (j, j + hd/2)
    a, b = x[1, 0, j], x[1, 0, j + 4]
    assert math.isclose(float(y[1, 0, j]), float(a * cos[1, j] - b * sin[1, j]))
    assert math.isclose(float(y[1, 0, j + 4]), float(a * sin[1, j] + b * cos[1, j]))
    # relative: the score of rotated q and k depends on the distance only
    q, k = torch.randn(1, 1, hd, dtype=torch.float64), torch.randn(1, 1, hd, dtype=torch.float64)
    def score(pq, pk):
        cq, sq = plain.rotary_cos_sin(torch.tensor([pq]), hd, theta)
        ck, sk = plain.rotary_cos_sin(torch.tensor([pk]), hd, theta)
        return float((plain.apply_rotary(q, cq, sq) * plain.apply_rotary(k, ck, sk)).sum())
    assert math.isclose(score(9, 4), score(25, 20), rel_tol=1e-5)


def test_visibility_causal_and_window():
    ok = plain.visibility(5, 0)
    assert ok.tolist() == torch.tril(torch.ones(5, 5)).bool().tolist()
    w = plain.visibility(6, 3)
    for r in range(6):
        assert [c for c in range(6) if w[r, c]] == list(range(max(0, r - 2), r + 1))
    assert plain.visibility(4, 9).tolist() == plain.visibility(4, 0).tolist()


def test_gqa_head_mapping_and_softmax():
    T, nh, nkv, hd = 4, 4, 2, 2
    q = torch.zeros(T, nh, hd, dtype=torch.float64)
    k = torch.randn(T, nkv, hd, dtype=torch.float64)
    v = torch.randn(T, nkv, hd, dtype=torch.float64)
    out = plain.gqa_attention(q, k, v, 0)
    for r in range(T):                       # zero queries: the mean of the visible values
        for n in range(nh):
            assert torch.allclose(out[r, n], v[:r + 1, n // 2].mean(dim=0))
    # one key stands out: the output is that key's value
    q = torch.zeros(T, nh, hd, dtype=torch.float64)
    k = torch.zeros(T, nkv, hd, dtype=torch.float64)
    q[3, 1, 0] = 100.0
    k[1, 0, 0] = 100.0
    out = plain.gqa_attention(q, k, v, 0)
    assert torch.allclose(out[3, 1], v[1, 0], atol=1e-9)
    out_w = plain.gqa_attention(q, k, v, 2)  # window 2 hides key 1 from row 3
    assert torch.allclose(out_w[3, 1], v[2:4, 0].mean(dim=0))


def test_swiglu_by_hand():
    x = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    wg = torch.tensor([[0.5, 0.25]], dtype=torch.float64)
    wu = torch.tensor([[2.0, 1.0]], dtype=torch.float64)
    wd = torch.tensor([[3.0], [-1.0]], dtype=torch.float64)
    g, u = 0.5 - 0.5, 2.0 - 2.0
    assert torch.allclose(plain.swiglu(x, wg, wu, wd), torch.zeros(1, 2, dtype=torch.float64))
    x = torch.tensor([[2.0, 0.0]], dtype=torch.float64)
    g, u = 1.0, 4.0
    z = g / (1 + math.exp(-g)) * u
    assert torch.allclose(plain.swiglu(x, wg, wu, wd),
                          torch.tensor([[3 * z, -z]], dtype=torch.float64))


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_forward_is_causal_and_uses_every_option(tmp_path, name):
    d = make_folder(tmp_path, name, seed=2)
    cfg, w = plain.read_model_folder(d)
    toks = prompt(60, cfg["vocab_size"], 9)
    full = plain.forward(w, cfg, toks)
    assert full.shape == (60, cfg["vocab_size"])
    assert torch.allclose(plain.forward(w, cfg, toks[:23]), full[:23], atol=1e-10)
    # each option matters: changing it changes the logits
    def changed(**patch):
        c = dict(cfg)
        c.update(patch)
        return not torch.allclose(plain.forward(w, c, toks), full, atol=1e-6)
    assert changed(rope_theta=cfg["rope_theta"] * 3)
    assert changed(rms_norm_eps=1e-2)
    if cfg.get("use_sliding_window"):
        assert changed(use_sliding_window=False)
        assert changed(sliding_window=cfg["sliding_window"] - 1)
        assert changed(max_window_layers=cfg["num_hidden_layers"])
    w2 = dict(w)
    w2["model.layers.0.self_attn.k_proj.bias"] = w["model.layers.0.self_attn.k_proj.bias"] + 1.0
    assert not torch.allclose(plain.forward(w2, cfg, toks), full, atol=1e-6)
    if cfg.get("tie_word_embeddings"):
        assert "lm_head.weight" not in w
    # a run list: naming a layer twice and reading another layer's cache both change the result
    L = cfg["num_hidden_layers"]
    twice = [(i, i, True) for i in range(L)] + [(0, L, True)]
    assert plain.forward(w, cfg, toks, run=twice).shape == full.shape
    if name == "A":
        shared = [(0, 0, True), (1, 0, False)]
        assert not torch.allclose(plain.forward(w, cfg, toks, run=shared), full, atol=1e-6)


def test_parts_agree_with_the_oracles_of_the_reference_tests():
    """The reference checks its kernels against formulas written out in its own Python tests
    (``python/test/test_op.py``): RMSNorm ``x * gamma / sqrt(mean(x^2) + eps)`` (:30-38), rotary
    encoding with frequencies ``theta^(-2i / head_dim)`` over the pairs ``(i, i + head_dim / 2)``
    (:187-210), ``gate * sigmoid(gate) * up`` (:244-256), and grouped-query attention as
    scaled-dot-product attention over keys repeated per group with a lower-right causal mask
    (:96-120).  The plain implementation's parts, written from the kernels' sources, give the
    same numbers as those formulas restated here (the sliding window has no counterpart there:
    the hand-made cases above define it)."""
    g = torch.Generator().manual_seed(0)
    x = torch.rand(3, 127, 128, generator=g, dtype=torch.float64)
    gamma = torch.rand(128, generator=g, dtype=torch.float64)
    ref = x * gamma / torch.sqrt((x ** 2).mean(-1, keepdim=True) + 1e-5)
    assert torch.allclose(plain.rms_norm(x, gamma, 1e-5), ref, atol=1e-12)
    # rotary: [seq, heads, head_dim], positions 0 .. seq - 1
    for seq, heads, hd, theta in ((128, 32, 128, 10000.0), (64, 12, 64, 10000.0)):
        x = torch.randn(seq, heads, hd, generator=g, dtype=torch.float64)
        half = hd // 2
        freqs = np.array([1.0 / theta ** (2.0 * i / hd) for i in range(half)], dtype=np.float32)
        ang = np.outer(np.arange(seq, dtype=np.float32), freqs)
        sin, cos = torch.from_numpy(np.sin(ang))[:, None, :], torch.from_numpy(np.cos(ang))[:, None, :]
        lo, hi = x[..., :half], x[..., half:]
        ref = torch.cat([lo * cos - hi * sin, lo * sin + hi * cos], dim=-1)
        c, s_ = plain.rotary_cos_sin(torch.arange(seq), hd, theta)
        assert torch.allclose(plain.apply_rotary(x, c, s_), ref, atol=1e-5)
    # gate * sigmoid(gate) * up, as the feed-forward's middle
    gate = torch.randn(4, 256, generator=g, dtype=torch.float64)
    up = torch.randn(4, 256, generator=g, dtype=torch.float64)
    eye = torch.eye(256, dtype=torch.float64)
    ref = gate * torch.sigmoid(gate) * up
    both = torch.cat([gate, up], dim=-1)                  # x = [gate | up]: the products pick them
    w_gate, w_up = torch.cat([eye, 0 * eye], 1), torch.cat([0 * eye, eye], 1)
    assert torch.allclose(plain.swiglu(both, w_gate, w_up, eye), ref, atol=1e-12)
    # attention: q_len == kv_len here (the plain implementation takes whole sequences)
    for heads, kv_heads, hd, T in ((12, 2, 128, 33), (32, 8, 128, 9), (12, 12, 64, 127)):
        q = torch.randn(T, heads, hd, generator=g, dtype=torch.float64)
        k = torch.randn(T, kv_heads, hd, generator=g, dtype=torch.float64)
        v = torch.randn(T, kv_heads, hd, generator=g, dtype=torch.float64)
        rep = heads // kv_heads
        kk = k.permute(1, 0, 2).repeat_interleave(rep, dim=0)
        vv = v.permute(1, 0, 2).repeat_interleave(rep, dim=0)
        mask = torch.ones(T, T, dtype=torch.bool).tril(diagonal=0)
        ref = torch.nn.functional.scaled_dot_product_attention(q.permute(1, 0, 2), kk, vv,
                                                               attn_mask=mask).permute(1, 0, 2)
        assert torch.allclose(plain.gqa_attention(q, k, v, 0), ref, atol=1e-10)


def test_choosing_tokens():
    row = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert plain.greedy_token(row) == 1                         # lowest index among equals
    p = torch.softmax(row.double() / 0.7, dim=-1)
    cdf = torch.cumsum(p, 0)
    assert plain.temperature_token(row, 0.7, float(cdf[0]) / 2) == 0
    assert plain.temperature_token(row, 0.7, float(cdf[0] + cdf[1]) / 2) == 1
    assert plain.temperature_token(row, 0.7, float(cdf[1] + cdf[2]) / 2) == 2
    assert plain.temperature_token(row, 0.7, 0.999999999) == 3


def test_stored_bf16_rounds_activations_only_when_asked(tmp_path):
    d = make_folder(tmp_path, "A", seed=2, storage="bfloat16")
    cfg, w = plain.read_model_folder(d)
    toks = prompt(20, cfg["vocab_size"], 1)
    a = plain.forward(w, cfg, toks)
    plain.Stored.bf16()
    try:
        b = plain.forward(w, cfg, toks)
    finally:
        plain.Stored.exact()
    assert not torch.equal(a, b) and torch.allclose(a, b, atol=0.05 * float(a.abs().max()))
    assert torch.equal(plain.forward(w, cfg, toks), a)
