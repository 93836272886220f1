"""Data that describes a model: which parts each layer is made of and in which order layers run.

An architecture's ``build_spec(config)`` returns a :class:`ModelSpec`.  The generic decoder
(:mod:`purhie_b200.parts.model`) looks every ``PartSpec.kind`` up in the part registries and builds
the part from ``PartSpec.params``; a part therefore gets every size and constant as a parameter and
never knows which model it belongs to.  Tensor names are parameters too: ``params["names"]`` maps the
part's own role names (``"q_proj"``, ``"weight"`` ...) to the names in the checkpoint.

The reference expresses per-layer variety with a ``LayerKind`` enum and per-layer weight records
(src/inference_internal.h:45-52, 77-90) and runs layers in file order (src/qwen_model.cpp:1196-1279);
here the order is a list of :class:`LayerCall`, which may name a layer twice or let a call read the
cache that an earlier call wrote.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Dict = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a token mixer and a feed-forward, each behind its norm, in a named arrangement."""

    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec
    feed_forward_norm: PartSpec
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers``.  Every call owns a cache entry of its own (so that a layer
    named twice keeps the keys of its two runs apart) unless ``cache_from`` names an earlier call
    (by its index in the schedule): then this call's mixer writes nothing and reads that call's cache.
    """

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec

    def validate(self) -> None:
        n = len(self.layers)
        for i, call in enumerate(self.schedule):
            if not 0 <= call.layer < n:
                raise ValueError(f"schedule[{i}] names layer {call.layer}, the model has {n}")
            if call.cache_from is not None:
                if not 0 <= call.cache_from < i:
                    raise ValueError(f"schedule[{i}].cache_from must name an earlier call, got {call.cache_from}")
                if self.schedule[call.cache_from].cache_from is not None:
                    raise ValueError(f"schedule[{i}].cache_from names a call that itself borrows a cache")
