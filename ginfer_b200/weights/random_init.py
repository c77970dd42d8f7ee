"""Random weights from a configuration and a seed.

The reference has no such mode.  Distributions: matrices, embeddings and biases N(0, 0.02), norm
weights 1 + N(0, 0.02), integer tables uniform.  Every tensor has a generator of its own, seeded
by the seed and the tensor's name, so a tensor's values do not depend on which other tensors the
model has or on the order they are drawn in.
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from ..config.registry import resolve_architecture
from .safetensors_io import write_safetensors

_STORAGE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def draw_tensor(spec, seed: int, std: float = 0.02, device="cpu") -> torch.Tensor:
    """One tensor of a :class:`~ginfer_b200.parts.base.TensorSpec`, fp32 (int32 for tables)."""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    if spec.role == "int":
        return torch.randint(0, spec.int_high, spec.shape, generator=g, dtype=torch.int32,
                             device=device)
    t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device) * std
    if spec.role == "norm":
        t += 1.0
    return t


def random_tensors(model, seed: int, storage: torch.dtype, device="cpu"
                   ) -> dict[str, torch.Tensor]:
    out = {}
    for s in model.tensor_specs():
        t = draw_tensor(s, seed, device=device)
        out[s.name] = t if s.role == "int" else t.to(storage)
    return out


def write_random_model(model_dir: str, config: dict, seed: int,
                       storage_dtype: str | None = None) -> None:
    """Write ``config.json`` and ``model.safetensors`` for the architecture ``config`` names.
    Tensors are stored as ``storage_dtype`` (default: the configuration's ``torch_dtype``)."""
    from ..parts.model import DecoderModel
    arch = resolve_architecture(config)
    cfg = arch.config_cls.from_dict(config)
    model = DecoderModel(arch.build_plan(cfg))
    sd = storage_dtype or getattr(cfg, "torch_dtype", "bfloat16")
    if sd not in _STORAGE:
        raise ValueError(f"storage dtype must be one of {sorted(_STORAGE)}, got {sd!r}")
    os.makedirs(model_dir, exist_ok=True)
    out_cfg = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(config)
    out_cfg["torch_dtype"] = sd
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(out_cfg, f, indent=2)
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      random_tensors(model, seed, _STORAGE[sd]),
                      metadata={"format": "pt", "seed": seed})


def load_random_weights(model, seed: int, dtype: torch.dtype, device) -> None:
    """Fill ``model`` with random weights drawn on ``device`` (no folder is written); for
    measurements at sizes where writing a file would only cost time."""
    from .loader import kept_dtype
    tensors = {}
    for s in model.tensor_specs():
        t = draw_tensor(s, seed, device=device)
        tensors[s.name] = t.to(kept_dtype(s.role, dtype, dtype)).contiguous()
    model.load(tensors, dtype, torch.device(device))
