"""From a model folder (or a configuration and a seed) to a model on the device."""
from __future__ import annotations

import torch

from .. import architectures  # noqa: F401  (registers architectures)
from ..config.registry import load_model_config, resolve_architecture
from ..parts.model import DecoderModel
from ..weights.loader import load_weights
from ..weights.random_init import load_random_weights

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
          "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype must be bfloat16 or float32, not {name}")
        return name
    try:
        return DTYPES[str(name)]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {name!r}") from None


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("ginfer_b200 runs on a CUDA device (B200, sm_100a) only; there is no "
                           "CPU path")
    return device


def load_model(model_path: str, dtype="bfloat16", device="cuda:0"):
    """Read ``config.json``, pick the architecture from the registry, build its plan and load
    ``model.safetensors``.  Returns ``(model, typed config)``."""
    device = require_cuda(device)
    arch, cfg = load_model_config(model_path)
    model = DecoderModel(arch.build_plan(cfg))
    load_weights(model, model_path, parse_dtype(dtype), device)
    return model, cfg


def random_model(config: dict, seed: int, dtype="bfloat16", device="cuda:0"):
    """A model of the architecture ``config`` names with random weights drawn on the device."""
    device = require_cuda(device)
    arch = resolve_architecture(config)
    cfg = arch.config_cls.from_dict(config)
    model = DecoderModel(arch.build_plan(cfg))
    load_random_weights(model, seed, parse_dtype(dtype), device)
    return model, cfg
