"""SwiGLU feed-forward: y = Wd (silu(Wg x) * (Wu x)).

Reference: src/qwen_model.cpp:1170-1189 (gate and up as one grouped product, the activation, down),
src/gpu_ops.hip:103-114 (silu(g) * u with g / (1 + exp(-g))).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from ..weights.loader import MATRIX, TensorSpec
from .base import Addend, BuildContext, FeedForward, register_part
from .linear import Linear


class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size, names{gate_proj, up_proj, down_proj}."""

    def __init__(self, params: dict, build: BuildContext):
        super().__init__(params, build)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self._gemm = build.options.get("gemm", "auto")
        self.gate_up_proj = self.down_proj = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n, e, ff = self.names, self.hidden_size, self.intermediate_size
        return {
            n["gate_proj"]: TensorSpec(n["gate_proj"], (ff, e), MATRIX),
            n["up_proj"]: TensorSpec(n["up_proj"], (ff, e), MATRIX),
            n["down_proj"]: TensorSpec(n["down_proj"], (e, ff), MATRIX),
        }

    def bind(self, tensors, device) -> None:
        n = self.names
        parts = [tensors[n["gate_proj"]], tensors[n["up_proj"]]]
        if parts[0].dtype != parts[1].dtype:
            parts = [t.float() for t in parts]
        # gate and up rows interleaved (g0, u0, g1, u1, ...) in one matrix: one product, and matching pairs sit
        # side by side, so the activation can run in the product's epilogue (a layout choice only)
        ff, e = parts[0].shape
        self.gate_up_proj = Linear(torch.stack(parts, dim=1).reshape(2 * ff, e).contiguous(), "gate_up_proj", self._gemm)
        self.down_proj = Linear(tensors[n["down_proj"]], "down_proj", self._gemm)

    def required_libraries(self):
        return tuple(sorted(set(self.gate_up_proj.required_libraries()) | set(self.down_proj.required_libraries())))

    def forward(self, x, ctx) -> Addend:
        T, dt = ctx.T, self.compute_dtype
        gu = self.gate_up_proj(x, ctx, "gate_up", dt, rows=T, allow_split=True, fuse_swiglu=True)
        if gu.activated:
            act = gu.tensor
        else:
            act = ctx.workspace.get("ff_act", (T, self.intermediate_size), dt)
            ops.swiglu(gu.tensor, act, splits=gu.splits)
        return self.down_proj(act, ctx, "ff_out", torch.float32, rows=T, allow_split=True, add_into=ctx.residual)


register_part("feed_forward", "swiglu", SwiGLU)
