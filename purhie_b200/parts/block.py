"""How a layer's parts are strung together.

``pre_norm``: x += mixer(norm1(x)); x += feed_forward(norm2(x)), with each addition folded into the norm
that follows it (the reference fuses them the same way: src/qwen_model.cpp:1175-1187, 1248, 1260).
"""
from __future__ import annotations

from typing import Dict

from ..weights.loader import TensorSpec
from .base import BuildContext, make_part, register_part
from .spec import LayerSpec


class PreNormBlock:
    def __init__(self, layer: LayerSpec, build: BuildContext):
        self.mixer_norm = make_part("norm", layer.mixer_norm, build)
        self.mixer = make_part("mixer", layer.mixer, build)
        self.feed_forward_norm = make_part("norm", layer.feed_forward_norm, build)
        self.feed_forward = make_part("feed_forward", layer.feed_forward, build)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        out: Dict[str, TensorSpec] = {}
        for p in self.parts():
            out.update(p.tensor_specs())
        return out

    def forward(self, stream, ctx, cache) -> None:
        ctx.residual = stream.x
        xn = self.mixer_norm.forward(stream, ctx)
        stream.add(self.mixer.forward(xn, ctx, cache))
        xn = self.feed_forward_norm.forward(stream, ctx)
        stream.add(self.feed_forward.forward(xn, ctx))


register_part("arrangement", "pre_norm", PreNormBlock)
