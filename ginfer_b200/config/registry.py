"""One registry from an architecture's name to its typed configuration and its model plan.

The reference switches on ``config.json["model_type"]`` (``ginfer/model/model_factory.h:16-27``:
``"qwen2"`` and ``"llama"``).  Here the key is ``architectures[0]`` with ``model_type`` as a
fall-back, and an entry is a pair: the class that parses ``config.json`` and a function that
turns the parsed configuration into a :class:`ginfer_b200.parts.plan.ModelPlan` (which parts make
each layer, in which order the layers run, which cache each layer uses).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .model_config import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Any                      # has from_dict(dict) -> config and to_dict()
    build_plan: Callable[[Any], Any]     # config -> ModelPlan
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_cls, build_plan, model_types=()) -> None:
    """Add (or replace) an architecture.  ``name`` is what ``config.json`` lists under
    ``architectures``; ``model_types`` are accepted ``model_type`` values for folders without
    that list."""
    _ARCHITECTURES[name] = Architecture(name, config_cls, build_plan, tuple(model_types))


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(config_dict: Mapping[str, Any]) -> Architecture:
    archs = config_dict.get("architectures") or []
    for a in archs:
        if a in _ARCHITECTURES:
            return _ARCHITECTURES[a]
    mt = config_dict.get("model_type")
    if mt is not None:
        for arch in _ARCHITECTURES.values():
            if mt in arch.model_types:
                return arch
    raise ConfigError(
        f"config.json names architectures={list(archs)!r}, model_type={mt!r}; "
        f"registered architectures are {registered_architectures()}")


def load_model_config(path: str):
    """Read ``config.json`` from a model folder and return ``(architecture, typed config)``."""
    d = read_config_json(path)
    arch = resolve_architecture(d)
    return arch, arch.config_cls.from_dict(d)
