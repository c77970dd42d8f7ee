"""Configuration parsing, validation and the architecture registry (no GPU)."""
import json

import pytest

from ginfer_b200.config import (ConfigError, Qwen2Config, load_model_config,
                                registered_architectures, resolve_architecture)
from tiny import TINY_A, TINY_B


def test_required_and_default_keys():
    cfg = Qwen2Config.from_dict({k: v for k, v in TINY_A.items()
                                 if k not in ("head_dim", "rope_theta", "rms_norm_eps",
                                              "eos_token_id", "tie_word_embeddings")})
    assert cfg.head_dim == 64 // 4                   # hidden_size / heads when absent
    assert cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-6
    assert cfg.eos_token_ids == (255,)               # vocab_size - 1 when absent
    assert cfg.tie_word_embeddings is False
    for key in ("hidden_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "intermediate_size", "vocab_size",
                "max_position_embeddings"):
        d = dict(TINY_A)
        del d[key]
        with pytest.raises(ConfigError, match=key):
            Qwen2Config.from_dict(d)


def test_eos_list_and_window_layers():
    cfg = Qwen2Config.from_dict(TINY_B)
    assert cfg.eos_token_ids == (7, 11)
    assert [cfg.layer_window(i) for i in range(3)] == [0, 48, 48]
    a = Qwen2Config.from_dict(TINY_A)
    assert [a.layer_window(i) for i in range(2)] == [0, 0]
    d = dict(TINY_B)
    del d["max_window_layers"]                       # defaults to the layer count: no layer
    assert [Qwen2Config.from_dict(d).layer_window(i) for i in range(3)] == [0, 0, 0]


@pytest.mark.parametrize("patch,match", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"torch_dtype": "int8"}, "torch_dtype"),
    ({"use_sliding_window": True}, "sliding_window"),
    ({"eos_token_id": 4096}, "eos"),
    ({"vocab_size": 0}, "positive"),
    ({"hidden_size": "64"}, "integer"),
    # options of other loaders that would change the result: refused, not ignored
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"use_mrope": True}, "use_mrope"),
    ({"layer_types": ["full_attention"]}, "layer_types must list 2"),
    ({"layer_types": ["full_attention", "sliding_attention"]}, "layer_types\\[1\\]"),
])
def test_validation_errors(patch, match):
    d = dict(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=match):
        Qwen2Config.from_dict(d)


def test_plain_values_of_options_that_are_not_implemented_are_accepted():
    d = dict(TINY_A, rope_scaling=None, hidden_act="silu", use_mrope=False, attention_dropout=0.0,
             layer_types=["full_attention", "full_attention"], use_cache=True)
    assert Qwen2Config.from_dict(d).layer_window(1) == 0
    d["rope_scaling"] = {"rope_type": "default"}
    Qwen2Config.from_dict(d)
    b = dict(TINY_B, layer_types=["full_attention", "sliding_attention", "sliding_attention"])
    cfg = Qwen2Config.from_dict(b)
    assert [cfg.layer_window(i) for i in range(3)] == [0, 48, 48]
    assert Qwen2Config.from_dict(cfg.to_dict()) == cfg


def test_round_trip_and_registry(tmp_path):
    cfg = Qwen2Config.from_dict(TINY_B)
    again = Qwen2Config.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    assert "Qwen2ForCausalLM" in registered_architectures()
    assert resolve_architecture({"architectures": ["Qwen2ForCausalLM"]}).name == "Qwen2ForCausalLM"
    assert resolve_architecture({"model_type": "qwen2"}).name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="registered"):
        resolve_architecture({"architectures": ["NopeForCausalLM"], "model_type": "nope"})
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    arch, c = load_model_config(str(tmp_path))
    assert arch.name == "Qwen2ForCausalLM" and c.hidden_size == 64
    with pytest.raises(ConfigError, match="no config.json"):
        load_model_config(str(tmp_path / "missing"))


def test_plan_has_no_constants_of_its_own():
    """Every size in the plan comes from the configuration."""
    import ginfer_b200  # noqa: F401
    arch = resolve_architecture(TINY_B)
    cfg = arch.config_cls.from_dict(TINY_B)
    plan = arch.build_plan(cfg)
    assert len(plan.layers) == 3 and [e.layer for e in plan.run] == [0, 1, 2]
    m = plan.layers[2].mixer.params
    assert (m["num_heads"], m["num_kv_heads"], m["head_dim"], m["window"]) == (3, 1, 32, 48)
    assert plan.layers[0].mixer.params["window"] == 0
    assert m["position"].params["theta"] == 1e6
    assert plan.layers[1].feed_forward.params["intermediate_size"] == 224
    assert plan.final_norm.params["eps"] == 1e-5
    assert plan.head.params["tied_to"] is None
    a = resolve_architecture(TINY_A)
    plan_a = a.build_plan(a.config_cls.from_dict(TINY_A))
    assert plan_a.head.params["tied_to"] == "model.embed_tokens.weight"
