"""Token embedding and output head.

x[t] = table[token[t]] without scaling (src/qwen_model.cpp:1234-1244); logits = W_out xn for the rows that
are asked for only (src/qwen_model.cpp:1421-1486).  A tied head shares the embedding table
(src/inference.cpp:1392-1396).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from ..weights.loader import MATRIX, TensorSpec
from .base import BuildContext, Part, register_part
from .linear import Linear


class Embedding(Part):
    """params: vocab_size, hidden_size, names{weight}."""

    def __init__(self, params: dict, build: BuildContext):
        super().__init__(params, build)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.table = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n = self.names["weight"]
        return {n: TensorSpec(n, (self.vocab_size, self.hidden_size), MATRIX)}

    def bind(self, tensors, device) -> None:
        self.table = tensors[self.names["weight"]]

    def forward(self, ctx) -> torch.Tensor:
        x = ctx.workspace.get("residual", (ctx.T, self.hidden_size), torch.float32)
        ops.embed_gather(self.table, ctx.token_ids, x)
        return x


class LMHead(Part):
    """params: hidden_size, vocab_size, and either names{weight} or tied_to (a tensor another part reads)."""

    def __init__(self, params: dict, build: BuildContext):
        super().__init__(params, build)
        self.hidden_size = int(params["hidden_size"])
        self.vocab_size = int(params["vocab_size"])
        self.tied_to = params.get("tied_to")
        self._ignore = tuple(params.get("ignore", ()))
        self._gemm = build.options.get("gemm", "auto")
        self.proj = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        if self.tied_to:
            return {}
        n = self.names["weight"]
        return {n: TensorSpec(n, (self.vocab_size, self.hidden_size), MATRIX)}

    def ignored_tensors(self):
        return self._ignore

    def bind(self, tensors, device) -> None:
        w = tensors[self.tied_to] if self.tied_to else tensors[self.names["weight"]]
        self.proj = Linear(w, "lm_head", self._gemm)

    def required_libraries(self):
        return self.proj.required_libraries() if self.proj else ("core",)

    def forward(self, xn: torch.Tensor, ctx, n_rows: int) -> torch.Tensor:
        """float32 logits [n_rows, vocab]."""
        return self.proj(xn, ctx, "logits", torch.float32, rows=n_rows).tensor


register_part("embedding", "embedding", Embedding)
register_part("head", "lm_head", LMHead)
