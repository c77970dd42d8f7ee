"""Safetensors reading/writing, binding by name, the one error for a folder that does not fit, and
the random-weights mode (no GPU)."""
import json
import os
import shutil
import struct

import pytest
import torch

import ginfer_b200  # noqa: F401
from ginfer_b200.config import resolve_architecture
from ginfer_b200.parts import DecoderModel
from ginfer_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_weights,
                                 write_random_model, write_safetensors)
from ginfer_b200.weights.loader import check_and_convert, kept_dtype
from ginfer_b200.weights.safetensors_io import open_model_tensors
from tiny import TINY_A, TINY_B, make_folder


def _model(cfg):
    arch = resolve_architecture(cfg)
    return DecoderModel(arch.build_plan(arch.config_cls.from_dict(cfg)))


def test_round_trip_against_the_safetensors_package(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
               "d": torch.tensor(2.5)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, tensors, metadata={"k": "v"})
    with safe_open(p, framework="pt") as f:                # their reader, our writer
        assert sorted(f.keys()) == ["a", "b", "c", "d"]
        for k, t in tensors.items():
            assert torch.equal(f.get_tensor(k), t)
    p2 = str(tmp_path / "y.safetensors")
    save_file({k: v.contiguous() for k, v in tensors.items()}, p2)
    sf = SafetensorsFile(p2)                               # our reader, their writer
    for k, t in tensors.items():
        got = sf.get(k)
        assert got.dtype == t.dtype and torch.equal(got, t)
    with pytest.raises(SafetensorsError, match="not found"):
        sf.get("zzz")


def test_corrupt_files(tmp_path):
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(str(p))
    p = tmp_path / "hdr.safetensors"
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}}).encode()
    p = tmp_path / "size.safetensors"
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 12)
    with pytest.raises(SafetensorsError, match="12 bytes.*needs 16"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "Q4", "shape": [1], "data_offsets": [0, 1]}}).encode()
    p = tmp_path / "dt.safetensors"
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0")
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(str(p))
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        open_model_tensors(str(tmp_path))


def test_random_model_folder_names_shapes_and_seed(tmp_path):
    d = make_folder(tmp_path, "B", seed=3, storage="bfloat16", sharp=False)
    cfg = json.load(open(os.path.join(d, "config.json")))
    assert cfg["torch_dtype"] == "bfloat16" and cfg["hidden_size"] == 96
    sf = SafetensorsFile(os.path.join(d, "model.safetensors"))
    names = set(sf.names())
    assert "lm_head.weight" in names and "model.norm.weight" in names
    assert "model.layers.2.self_attn.k_proj.bias" in names
    assert len(names) == 1 + 3 * 12 + 1 + 1
    assert sf.get("model.layers.1.mlp.gate_proj.weight").shape == (224, 96)
    assert sf.get("model.layers.0.self_attn.k_proj.weight").shape == (32, 96)
    g = sf.get("model.layers.0.input_layernorm.weight").float()
    assert abs(float(g.mean()) - 1.0) < 0.02
    w = sf.get("model.embed_tokens.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    # same seed: same values; another seed: other values; a tensor does not depend on the rest
    d2 = str(tmp_path / "again")
    write_random_model(d2, dict(TINY_B), 3, storage_dtype="bfloat16")
    sf2 = SafetensorsFile(os.path.join(d2, "model.safetensors"))
    assert torch.equal(sf2.get("lm_head.weight"), sf.get("lm_head.weight"))
    d3 = str(tmp_path / "other")
    write_random_model(d3, dict(TINY_B), 4, storage_dtype="bfloat16")
    assert not torch.equal(SafetensorsFile(os.path.join(d3, "model.safetensors"))
                           .get("lm_head.weight"), sf.get("lm_head.weight"))
    tied = make_folder(tmp_path, "A", sharp=False)
    assert "lm_head.weight" not in SafetensorsFile(os.path.join(tied, "model.safetensors")).names()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file
    d = make_folder(tmp_path, "A", sharp=False)
    path = os.path.join(d, "model.safetensors")
    with safe_open(path, framework="pt") as f:
        t = {k: f.get_tensor(k) for k in f.keys()}
    del t["model.layers.1.self_attn.q_proj.bias"]
    del t["model.norm.weight"]
    t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 100)
    t["model.layers.7.extra.weight"] = torch.zeros(3)
    save_file(t, path)
    with pytest.raises(WeightError) as ei:
        load_weights(_model(TINY_A), d, torch.float32, "cpu")
    e = ei.value
    assert e.missing == ["model.layers.1.self_attn.q_proj.bias", "model.norm.weight"]
    assert e.unexpected == ["model.layers.7.extra.weight"]
    assert [(n, g, w) for n, g, w in e.wrong_shape] == \
        [("model.layers.0.mlp.down_proj.weight", (64, 100), (64, 128))]
    msg = str(e)
    for piece in ("missing (2)", "unexpected (1)", "wrong shape (1)", "file has [64, 100]",
                  "model needs [64, 128]"):
        assert piece in msg


def test_how_tensors_are_kept(tmp_path):
    bf, f32 = torch.bfloat16, torch.float32
    assert kept_dtype("matrix", f32, bf) == bf and kept_dtype("embedding", f32, bf) == bf
    assert kept_dtype("norm", f32, bf) == f32 and kept_dtype("bias", f32, bf) == f32
    assert kept_dtype("norm", bf, bf) == bf and kept_dtype("norm", bf, f32) == f32
    assert kept_dtype("int", torch.int64, bf) == torch.int32
    # a folder stored in 32-bit, served in bf16: matrices become bf16, norm weights and biases stay
    d = make_folder(tmp_path, "A", sharp=False)
    idx = open_model_tensors(d)
    avail = {n: (f.entries[k].shape, f.entries[k].dtype) for n, (f, k) in idx.items()}
    m = _model(TINY_A)
    out = check_and_convert(m.tensor_specs(), avail, lambda n: idx[n][0].get(idx[n][1]), d, bf,
                            "cpu", ignored=m.plan.ignored_tensors)
    assert out["model.layers.0.self_attn.q_proj.weight"].dtype == bf
    assert out["model.embed_tokens.weight"].dtype == bf
    assert out["model.layers.0.input_layernorm.weight"].dtype == f32
    assert out["model.layers.0.self_attn.v_proj.bias"].dtype == f32
    out32 = check_and_convert(m.tensor_specs(), avail, lambda n: idx[n][0].get(idx[n][1]), d,
                              f32, "cpu")
    assert all(t.dtype == f32 for t in out32.values())


def test_a_folder_in_two_shards_loads_like_the_single_file(tmp_path):
    """``model.safetensors.index.json`` with its ``weight_map`` over two shards (how the larger
    checkpoints of this family ship): the same tensors reach the model as from one file."""
    d = make_folder(tmp_path, "B", seed=6, storage="bfloat16", sharp=False)
    single = open_model_tensors(d)
    names = sorted(single)
    half = len(names) // 2
    d2 = str(tmp_path / "sharded")
    os.makedirs(d2)
    shutil.copy(os.path.join(d, "config.json"), d2)
    shards = {"model-00001-of-00002.safetensors": names[:half],
              "model-00002-of-00002.safetensors": names[half:]}
    weight_map = {}
    for fname, part in shards.items():
        write_safetensors(os.path.join(d2, fname),
                          {n: single[n][0].get(single[n][1]).clone() for n in part})
        weight_map.update({n: fname for n in part})
    json.dump({"metadata": {"total_size": 0}, "weight_map": weight_map},
              open(os.path.join(d2, "model.safetensors.index.json"), "w"))
    sharded = open_model_tensors(d2)
    assert sorted(sharded) == names
    assert len({id(f) for f, _ in sharded.values()}) == 2
    m = _model(TINY_B)

    def bound(folder):
        idx = open_model_tensors(folder)
        avail = {n: (f.entries[k].shape, f.entries[k].dtype) for n, (f, k) in idx.items()}
        return check_and_convert(m.tensor_specs(), avail, lambda n: idx[n][0].get(idx[n][1]),
                                 folder, torch.bfloat16, "cpu", ignored=m.plan.ignored_tensors)
    one, two = bound(d), bound(d2)
    assert sorted(one) == sorted(two) == names
    assert all(torch.equal(one[n], two[n]) for n in names)
    # a tensor the index names but no shard holds is reported like any missing tensor
    del weight_map[names[0]]
    json.dump({"weight_map": weight_map},
              open(os.path.join(d2, "model.safetensors.index.json"), "w"))
    with pytest.raises(WeightError) as ei:
        bound(d2)
    assert ei.value.missing == [names[0]]
