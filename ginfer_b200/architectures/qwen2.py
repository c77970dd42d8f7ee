"""Qwen2 dense as a plan of parts.

Structure as the reference builds it (``ginfer/model/qwen2.cc:28-54``,
``ginfer/model/model.cc:34-46``): token embedding, ``num_hidden_layers`` pre-norm blocks of GQA
attention (bias on q/k/v, none on o: ``qwen2.cc:15-17``) and SwiGLU, a final RMSNorm with the
same eps (``model.cc:37,43``), an LM head that shares the embedding when
``tie_word_embeddings`` (``qwen2.cc:42-46``).  Tensor names: ``qwen2.cc:34-46`` and
``ginfer/model/loader/model_loader.cc:56-76,109-121``.  Layers at or past ``max_window_layers``
get a sliding window when ``use_sliding_window`` is set (not in the reference).
"""
from __future__ import annotations

from ..config.model_config import Qwen2Config
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, sequential_run


def qwen2_plan(cfg: Qwen2Config) -> ModelPlan:
    rotary = PartSpec("rotary", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta,
                                     max_positions=cfg.max_position_embeddings))
    layers = []
    for i in range(cfg.num_hidden_layers):
        layers.append(LayerSpec(
            prefix=f"model.layers.{i}",
            mixer=PartSpec("attention", dict(
                hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
                num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, position=rotary,
                window=cfg.layer_window(i), qkv_bias=True, out_bias=False, prefix="self_attn")),
            feed_forward=PartSpec("swiglu", dict(
                hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                prefix="mlp")),
            mixer_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps,
                                                weight_name="input_layernorm.weight")),
            feed_forward_norm=PartSpec("rmsnorm", dict(
                size=cfg.hidden_size, eps=cfg.rms_norm_eps,
                weight_name="post_attention_layernorm.weight")),
        ))
    embed_name = "model.embed_tokens.weight"
    return ModelPlan(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                                         name=embed_name)),
        layers=tuple(layers), run=sequential_run(cfg.num_hidden_layers),
        final_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps,
                                            weight_name="model.norm.weight")),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                                     name="lm_head.weight",
                                     tied_to=embed_name if cfg.tie_word_embeddings else None)),
        eos_token_ids=tuple(cfg.eos_token_ids),
        ignored_tensors=(r".*\.rotary_emb\.inv_freq",)
        + ((r"lm_head\.weight",) if cfg.tie_word_embeddings else ()),
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, qwen2_plan, model_types=("qwen2",))
