"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference parses ``config.json`` in two stages: the generic keys in
``ginfer/model/loader/model_loader.cc:17-52`` (``torch_dtype``, ``num_hidden_layers``,
``vocab_size``, ``max_position_embeddings``, ``num_attention_heads``,
``num_key_value_heads``, ``head_dim``, ``eos_token_id``) and the Llama-family keys in
``ginfer/model/loader/model_loader.cc:94-107`` (``hidden_size``, ``intermediate_size``,
``rms_norm_eps`` default 1e-6, ``rope_theta`` default 10000, ``tie_word_embeddings`` default
false, ``head_dim`` defaulting to ``hidden_size / num_attention_heads``).  ``Qwen2Config`` in
the reference adds nothing (``ginfer/model/qwen2.h:21``).  The sliding-window keys are not read
by the reference; they are read here because Qwen2's ``config.json`` carries them.

Every size and constant of the model comes from this object; none is written in code.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Mapping


class ConfigError(ValueError):
    """A ``config.json`` that cannot describe a runnable model."""


_TORCH_DTYPES = ("bfloat16", "float16", "float32")


def _refuse_what_changes_the_arithmetic(d: Mapping[str, Any], layers: int, window_of) -> None:
    """Keys that other loaders of Qwen2 folders honour and that would change the result if they
    were set to anything but their plain value: this engine does not implement them, so a folder
    that sets them is refused instead of being run as if it had not."""
    scaling = d.get("rope_scaling")
    if scaling is not None:
        kind = scaling
        if isinstance(scaling, Mapping):
            kind = scaling.get("rope_type", scaling.get("type"))
        if kind not in (None, "default"):
            raise ConfigError(f"config.json: rope_scaling {scaling!r} is not supported (only plain "
                              "rotary positions at rope_theta)")
    act = d.get("hidden_act")
    if act is not None and act not in ("silu", "swish"):
        raise ConfigError(f"config.json: hidden_act {act!r} is not supported (the feed-forward "
                          "is SiLU(gate) * up)")
    if d.get("use_mrope"):
        raise ConfigError("config.json: use_mrope is not supported")
    kinds = d.get("layer_types")
    if kinds is not None:
        if not isinstance(kinds, (list, tuple)) or len(kinds) != layers:
            raise ConfigError(f"config.json: layer_types must list {layers} layers")
        for i, k in enumerate(kinds):
            want = "sliding_attention" if window_of(i) > 0 else "full_attention"
            if k != want:
                raise ConfigError(
                    f"config.json: layer_types[{i}] is {k!r} but use_sliding_window, "
                    f"sliding_window and max_window_layers make layer {i} {want!r}")


def _require(d: Mapping[str, Any], key: str, typ):
    if key not in d:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json: key '{key}' must be an integer, got {v!r}")
    return v


@dataclass(frozen=True)
class Qwen2Config:
    """Qwen2 dense decoder: pre-norm RMSNorm blocks, GQA attention with q/k/v bias, rotary
    positions, SwiGLU feed-forward, optional tied output head, optional sliding window on the
    layers at or past ``max_window_layers``."""

    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: int | None = None
    max_window_layers: int | None = None
    eos_token_ids: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    architectures: tuple[str, ...] = ("Qwen2ForCausalLM",)
    model_type: str = "qwen2"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen2Config":
        hidden = _require(d, "hidden_size", int)
        layers = _require(d, "num_hidden_layers", int)
        heads = _require(d, "num_attention_heads", int)
        kv_heads = _require(d, "num_key_value_heads", int)
        inter = _require(d, "intermediate_size", int)
        vocab = _require(d, "vocab_size", int)
        max_pos = _require(d, "max_position_embeddings", int)
        head_dim = d.get("head_dim") or 0
        if head_dim == 0:
            if heads <= 0 or hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not divisible by num_attention_heads "
                    f"{heads} and no head_dim is given")
            head_dim = hidden // heads
        eos = d.get("eos_token_id", None)
        if eos is None:
            eos_ids: tuple[int, ...] = (vocab - 1,)
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        use_window = bool(d.get("use_sliding_window", False))
        window = d.get("sliding_window", None)
        max_window_layers = d.get("max_window_layers", None)
        known = {f.name for f in fields(cls)} | {"eos_token_id", "dtype"}
        cfg = cls(
            hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
            num_key_value_heads=kv_heads, head_dim=int(head_dim), intermediate_size=inter,
            vocab_size=vocab, max_position_embeddings=max_pos,
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            use_sliding_window=use_window,
            sliding_window=None if window is None else int(window),
            max_window_layers=None if max_window_layers is None else int(max_window_layers),
            eos_token_ids=eos_ids, torch_dtype=str(dtype),
            architectures=tuple(d.get("architectures", ("Qwen2ForCausalLM",))),
            model_type=str(d.get("model_type", "qwen2")),
            extra={k: v for k, v in d.items() if k not in known},
        )
        cfg.validate()
        _refuse_what_changes_the_arithmetic(d, layers, cfg.layer_window)
        return cfg

    @classmethod
    def from_json_file(cls, path: str) -> "Qwen2Config":
        return cls.from_dict(read_config_json(path))

    def validate(self) -> None:
        pos = {
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
        }
        for k, v in pos.items():
            if v <= 0:
                raise ConfigError(f"config.json: '{k}' must be positive, got {v}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary pairs")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"config.json: rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"config.json: rope_theta must be > 0, got {self.rope_theta}")
        if self.torch_dtype not in _TORCH_DTYPES:
            raise ConfigError(
                f"config.json: torch_dtype '{self.torch_dtype}' is not one of {_TORCH_DTYPES}")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ConfigError(
                    "config.json: use_sliding_window is set but 'sliding_window' is missing or "
                    "not positive")
        for e in self.eos_token_ids:
            if not (0 <= e < self.vocab_size):
                raise ConfigError(f"config.json: eos_token_id {e} is outside the vocabulary")

    # ------------------------------------------------------------------ derived
    def layer_window(self, layer: int) -> int:
        """Sliding window of ``layer`` in tokens, 0 for full attention.  A layer is windowed
        iff ``use_sliding_window`` and ``layer >= max_window_layers`` (``max_window_layers``
        defaults to the number of layers, i.e. no layer)."""
        if not self.use_sliding_window:
            return 0
        first = self.num_hidden_layers if self.max_window_layers is None else self.max_window_layers
        return int(self.sliding_window) if layer >= first else 0

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = dict(self.extra)
        d.update(
            architectures=list(self.architectures), model_type=self.model_type,
            hidden_size=self.hidden_size, num_hidden_layers=self.num_hidden_layers,
            num_attention_heads=self.num_attention_heads,
            num_key_value_heads=self.num_key_value_heads, head_dim=self.head_dim,
            intermediate_size=self.intermediate_size, vocab_size=self.vocab_size,
            max_position_embeddings=self.max_position_embeddings,
            rms_norm_eps=self.rms_norm_eps, rope_theta=self.rope_theta,
            tie_word_embeddings=self.tie_word_embeddings,
            use_sliding_window=self.use_sliding_window, torch_dtype=self.torch_dtype,
            eos_token_id=list(self.eos_token_ids) if len(self.eos_token_ids) != 1
            else self.eos_token_ids[0],
        )
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        if self.max_window_layers is not None:
            d["max_window_layers"] = self.max_window_layers
        return d


def read_config_json(path: str) -> dict[str, Any]:
    """``path`` is a model folder or the ``config.json`` itself."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError as e:
        raise ConfigError(f"no config.json at {path}") from e
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return d
