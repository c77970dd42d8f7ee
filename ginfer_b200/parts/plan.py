"""The description of a model as data: which parts make each layer, in which order the layers
run and which cache each run of a layer reads and writes.

An architecture's ``build_plan(config)`` returns a :class:`ModelPlan`; nothing below this file
knows which architecture it serves.  The reference wires one fixed stack instead
(``ginfer/model/model.cc:34-46``: embedding, ``nlayer`` identical ``EncoderLayer``s, final
RMSNorm, LM head); the plan generalises that stack so that layers may differ and the run order
is a list.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """A part by registered kind, with its sizes and constants as parameters."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (``block``) of a mixer, a feed-forward and their norms.
    ``prefix`` is the tensor-name prefix of the layer (``model.layers.3``)."""
    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    block: PartSpec = PartSpec("prenorm")


@dataclass(frozen=True)
class RunEntry:
    """One run of a layer.  ``layer`` indexes :attr:`ModelPlan.layers` (a layer may be named
    twice).  ``cache`` names the cache this run uses: by default a cache of its own; a run with
    ``write_cache=False`` only reads the cache another run has written earlier in the step."""
    layer: int
    cache: int
    write_cache: bool = True


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    run: tuple[RunEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: tuple[int, ...] = ()
    ignored_tensors: tuple[str, ...] = ()     # regular expressions of tensor names to pass over

    def validate(self) -> None:
        writers: dict[int, int] = {}
        for pos, e in enumerate(self.run):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"run[{pos}] names layer {e.layer}, but there are "
                                 f"{len(self.layers)} layers")
            if e.write_cache:
                if e.cache in writers:
                    raise ValueError(f"run[{pos}] and run[{writers[e.cache]}] both write cache "
                                     f"{e.cache}")
                writers[e.cache] = pos
        for pos, e in enumerate(self.run):
            if not e.write_cache and (e.cache not in writers or writers[e.cache] > pos):
                raise ValueError(f"run[{pos}] reads cache {e.cache} before any run writes it")


def sequential_run(num_layers: int) -> tuple[RunEntry, ...]:
    """Every layer once, in order, each with a cache of its own."""
    return tuple(RunEntry(layer=i, cache=i) for i in range(num_layers))
