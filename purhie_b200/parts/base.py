"""The interfaces of the parts a layer is made of, and the registries that map a kind to a class.

A part is built from ``params`` alone (sizes, constants, tensor names), announces the tensors it reads,
is handed them on the device by ``bind`` and then runs inside a step.  Four kinds of part exist:

``Norm``              ``forward(stream, ctx, rows=None) -> normed``: folds the stream's pending addend into
                      the float32 residual and returns the normalised rows in the compute dtype.
``PositionEncoding``  gives the mixer what it needs to place a token: for the rotary family a table of
                      cosines and sines per position and pair, the number of rotated dimensions and the
                      pairing.
``Mixer``             ``cache_need() -> CacheNeed`` tells the cache manager what to keep for it;
                      ``forward(x, ctx, cache) -> Addend`` mixes the tokens of each request.
``FeedForward``       ``forward(x, ctx) -> Addend`` maps [T, E] to [T, E] row by row.
                      (Either may instead add its result into ``ctx.residual`` and return ``Addend(None)``.)

plus the block arrangement that strings them together.  New parts are added with the ``register_*``
functions; the generic decoder looks kinds up at build time, so a model description may name a part that
a test or a user registered.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional

import torch

from ..cache.manager import CacheNeed
from ..weights.loader import TensorSpec


@dataclass
class Addend:
    """A tensor to be added to the residual stream: [T, E], or [splits, T, E] partial sums; None when the part has
    already added its result into ``ctx.residual``."""

    tensor: Optional[torch.Tensor]
    splits: int = 1
    activated: bool = False      # a product whose activation was already applied in the kernel's epilogue


class BuildContext:
    """What parts share while a model is built: the compute dtype and parts that may be shared."""

    def __init__(self, compute_dtype: torch.dtype = torch.float32, options: Optional[dict] = None):
        self.compute_dtype = compute_dtype
        self.options = dict(options or {})
        self._shared: Dict = {}

    def shared(self, key, make: Callable):
        if key not in self._shared:
            self._shared[key] = make()
        return self._shared[key]


class Part:
    """Base of every part.  ``params`` hold every size and constant; ``names`` map roles to tensor names."""

    def __init__(self, params: dict, build: BuildContext):
        self.params = params
        self.names: Dict[str, str] = dict(params.get("names", {}))
        self.compute_dtype = build.compute_dtype

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        """Tensors this part reads, by checkpoint name."""
        return {}

    def ignored_tensors(self):
        """Names that may be present in a checkpoint and are not read."""
        return ()

    def bind(self, tensors: Dict[str, torch.Tensor], device) -> None:
        """Receive the tensors (already on ``device``) and prepare derived buffers."""

    def required_libraries(self):
        """Kernel libraries this part launches from (compiled before the first step)."""
        return ("core",)


class Norm(Part):
    def forward(self, stream, ctx, rows=None, n_rows=None):  # pragma: no cover - interface
        raise NotImplementedError


class PositionEncoding(Part):
    n_rot: int = 0
    interleaved: bool = False

    def rotation_table(self, device) -> Optional[torch.Tensor]:  # pragma: no cover - interface
        """float32 [max_position, n_rot]: per position n_rot/2 cosines then n_rot/2 sines; None: no rotation."""
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> CacheNeed:
        return CacheNeed()

    def forward(self, x, ctx, cache) -> Addend:  # pragma: no cover - interface
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx) -> Addend:  # pragma: no cover - interface
        raise NotImplementedError


NORMS: Dict[str, type] = {}
POSITIONS: Dict[str, type] = {}
MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
ARRANGEMENTS: Dict[str, type] = {}
EMBEDDINGS: Dict[str, type] = {}
HEADS: Dict[str, type] = {}

_TABLES = {"norm": NORMS, "position": POSITIONS, "mixer": MIXERS, "feed_forward": FEED_FORWARDS,
           "arrangement": ARRANGEMENTS, "embedding": EMBEDDINGS, "head": HEADS}


def register_part(family: str, kind: str, cls: type) -> None:
    """Register ``cls`` as the part ``kind`` of ``family`` (norm, position, mixer, feed_forward,
    arrangement, embedding, head)."""
    _TABLES[family][kind] = cls


def unregister_part(family: str, kind: str) -> None:
    _TABLES[family].pop(kind, None)


def make_part(family: str, spec, build: BuildContext):
    table = _TABLES[family]
    if spec.kind not in table:
        raise KeyError(f"no {family} part of kind {spec.kind!r} is registered (have: {', '.join(sorted(table))})")
    return table[spec.kind](spec.params, build)
