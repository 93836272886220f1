"""RMSNorm with the residual add folded in.

y = v * rsqrt(mean(v^2) + eps) * w, v = x + pending addend; the weight multiplies after normalising (plain
w, not 1 + w).  Reference: src/gpu_ops.hip:24-56 (add + norm in one kernel), src/qwen_ops.cpp:8-13.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from ..weights.loader import VECTOR, TensorSpec
from .base import BuildContext, Norm, register_part


class RMSNorm(Norm):
    """params: size, eps, names{weight}."""

    def __init__(self, params: dict, build: BuildContext):
        super().__init__(params, build)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n = self.names["weight"]
        return {n: TensorSpec(n, (self.size,), VECTOR, init="scale")}

    def bind(self, tensors, device) -> None:
        self.weight = tensors[self.names["weight"]]

    def forward(self, stream, ctx, rows=None, n_rows=None):
        n = n_rows if n_rows is not None else (ctx.T if rows is None else rows.numel())
        out = ctx.workspace.get("normed" if rows is None else "normed_rows", (n, self.size), self.compute_dtype)
        pend = stream.pending
        ops.add_rmsnorm(stream.x, pend.tensor if pend else None, self.weight, self.eps, out, rows=rows, n_rows=n,
                        add_splits=pend.splits if pend else 1)
        if rows is None:
            stream.pending = None
        return out


register_part("norm", "rmsnorm", RMSNorm)
