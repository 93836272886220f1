"""y = x W^T for a weight stored [out_features, in_features], and the choice of the kernel that does it.

float32 weights go through the exact-order CUDA-core kernel (the 32-bit path; also a 32-bit tensor met
in a bfloat16 model).  bfloat16 weights go through the tcgen05 tensor-core kernel when it takes the shape,
else through the plain kernel.  The reference picks a kernel by weight type and batch size the same way
(``qmatvec_launch``, src/qmatvec.cpp:274; ``matvec`` / ``matvec_multi``, src/qwen_model.cpp:855-922).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from .base import Addend


class Linear:
    def __init__(self, weight: torch.Tensor, label: str, gemm: str = "auto"):
        if weight.dim() != 2:
            raise ValueError(f"{label}: a linear weight must be a matrix, got {tuple(weight.shape)}")
        self.weight = weight
        self.label = label
        self.out_features, self.in_features = weight.shape
        self.gemm = gemm
        self._fast = None

    def _fast_kernel(self):
        if self._fast is None:
            self._fast = False
            if self.weight.dtype == torch.bfloat16 and self.gemm in ("auto", "tcgen05"):
                from ..csrc import gemm100
                if gemm100.supports(self.weight):
                    self._fast = gemm100
                elif self.gemm == "tcgen05":
                    raise ops.KernelError(f"{self.label}: the tcgen05 kernel does not take a weight of shape "
                                          f"{tuple(self.weight.shape)}")
        return self._fast

    def required_libraries(self):
        return ("core", "gemm100") if self._fast_kernel() else ("core",)

    def __call__(self, x: torch.Tensor, ctx, out_name: str, out_dtype: torch.dtype, rows: Optional[int] = None,
                 allow_split: bool = False, fuse_swiglu: bool = False, add_into: Optional[torch.Tensor] = None) -> Addend:
        """x [rows, in] -> Addend of [rows, out].  ``add_into`` (float32 [rows, out]): where the kernel can add the
        product in its epilogue it does, and the addend comes back empty; otherwise the product is returned as
        usual and the caller's norm adds it."""
        M = rows if rows is not None else x.shape[0]
        ws = ctx.workspace
        if self.weight.dtype == torch.float32 and x.dtype != torch.float32:
            x32 = ws.get("linear_x32", (M, self.in_features), torch.float32)
            ops.cast(x[:M], x32)
            x = x32
        fast = self._fast_kernel()
        if fast and x.dtype == torch.bfloat16:
            return fast.linear(x, self.weight, ctx, out_name, out_dtype, M, allow_split, fuse_swiglu, add_into)
        out = ws.get(out_name, (M, self.out_features), out_dtype)
        ops.gemm_simple(x[:M], self.weight, out)
        return Addend(out, 1)
