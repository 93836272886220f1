"""Grouped-query attention over cache pages, with per-head RMSNorm on q and k and a position encoding.

q = Wq x, k = Wk x, v = Wv x (+ optional biases, added before the norms); each q and k head is
RMS-normalised over head_dim with a weight shared by all heads (same eps as the layer norms), then
rotated; k and v go into the request's pages; query head h attends with kv head h / (HQ / HKV), scale
1 / sqrt(head_dim), causally, optionally only over the last ``window`` positions; then y = Wo o.
Reference: src/qwen_model.cpp:940-975 (full_attention), src/attention.hip:273-313 (prep),
src/attention.cpp:139-288 (host side; scale at :197), src/attention.h:73 (window),
src/inference.cpp:623-646 (tensors and shapes).
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from ..cache.manager import CacheNeed
from ..csrc import ops
from ..weights.loader import MATRIX, VECTOR, TensorSpec
from .base import Addend, BuildContext, Mixer, make_part, register_part
from .linear import Linear


class Attention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm_eps (None: no q/k norm), bias,
    position (PartSpec), window (None: all positions), scale (None: 1/sqrt(head_dim)),
    names{q_proj, k_proj, v_proj, o_proj, q_norm, k_norm, q_bias, k_bias, v_bias}."""

    def __init__(self, params: dict, build: BuildContext):
        super().__init__(params, build)
        p = params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} query heads are not a multiple of {self.num_kv_heads} kv heads")
        self.eps = p.get("qk_norm_eps")
        self.has_bias = bool(p.get("bias", False))
        self.window = p.get("window")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        pos = p.get("position")
        self.position = None
        if pos is not None:
            key = ("position", pos.kind, tuple(sorted((k, v) for k, v in pos.params.items() if k != "names")))
            self.position = build.shared(key, lambda: make_part("position", pos, build))
        self._gemm = build.options.get("gemm", "auto")
        self._attention = build.options.get("attention", "auto")
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.qkv_proj = self.q_only_proj = self.o_proj = None
        self.q_norm = self.k_norm = self.bias = None
        self._table = None

    # ---- weights ---------------------------------------------------------------------------------
    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n, e = self.names, self.hidden_size
        specs = {
            n["q_proj"]: TensorSpec(n["q_proj"], (self.q_width, e), MATRIX),
            n["k_proj"]: TensorSpec(n["k_proj"], (self.kv_width, e), MATRIX),
            n["v_proj"]: TensorSpec(n["v_proj"], (self.kv_width, e), MATRIX),
            n["o_proj"]: TensorSpec(n["o_proj"], (e, self.q_width), MATRIX),
        }
        if self.eps is not None:
            specs[n["q_norm"]] = TensorSpec(n["q_norm"], (self.head_dim,), VECTOR, init="scale")
            specs[n["k_norm"]] = TensorSpec(n["k_norm"], (self.head_dim,), VECTOR, init="scale")
        if self.has_bias:
            specs[n["q_bias"]] = TensorSpec(n["q_bias"], (self.q_width,), VECTOR)
            specs[n["k_bias"]] = TensorSpec(n["k_bias"], (self.kv_width,), VECTOR)
            specs[n["v_bias"]] = TensorSpec(n["v_bias"], (self.kv_width,), VECTOR)
        return specs

    def bind(self, tensors, device) -> None:
        n = self.names
        parts = [tensors[n["q_proj"]], tensors[n["k_proj"]], tensors[n["v_proj"]]]
        if len({t.dtype for t in parts}) > 1:
            parts = [t.float() for t in parts]
        # one matrix [q | k | v] so that the three projections are one product (a layout choice only)
        qkv = torch.cat(parts, dim=0).contiguous()
        self.qkv_proj = Linear(qkv, "qkv_proj", self._gemm)
        self.q_only_proj = Linear(qkv[:self.q_width], "q_proj", self._gemm)
        self.o_proj = Linear(tensors[n["o_proj"]], "o_proj", self._gemm)
        if self.eps is not None:
            self.q_norm, self.k_norm = tensors[n["q_norm"]], tensors[n["k_norm"]]
        if self.has_bias:
            self.bias = torch.cat([tensors[n["q_bias"]], tensors[n["k_bias"]], tensors[n["v_bias"]]]).contiguous()
        if self.position is not None:
            self._table = self.position.rotation_table(device)

    def required_libraries(self):
        libs = set(self.qkv_proj.required_libraries()) | set(self.o_proj.required_libraries())
        if self._use_flash():
            libs.add("flash")
        return tuple(sorted(libs))

    def _use_flash(self) -> bool:
        if self.compute_dtype != torch.bfloat16 or self._attention == "generic":
            return False
        from ..csrc import flash
        ok = flash.supports(self.head_dim, self.num_heads // self.num_kv_heads)
        if not ok and self._attention == "flash":
            raise ops.KernelError(f"the flash attention kernels do not take head_dim {self.head_dim} with "
                                  f"{self.num_heads // self.num_kv_heads} query heads per kv head")
        return ok

    # ---- cache -----------------------------------------------------------------------------------
    def cache_need(self) -> CacheNeed:
        return CacheNeed.pages(self.num_kv_heads, self.head_dim, self.window)

    # ---- step ------------------------------------------------------------------------------------
    def forward(self, x, ctx, cache) -> Addend:
        T, ws, dt = ctx.T, ctx.workspace, self.compute_dtype
        g = ctx.groups[cache.group]
        if cache.writable:
            qkv = self.qkv_proj(x, ctx, "qkv", dt, rows=T, allow_split=True)
            kv_heads = self.num_kv_heads
        else:
            qkv = self.q_only_proj(x, ctx, "qkv", dt, rows=T, allow_split=True)
            kv_heads = 0
        q = ws.get("q", (T, self.num_heads, self.head_dim), dt)
        bias = self.bias if (self.bias is None or cache.writable) else self.bias[:self.q_width]
        ops.qk_norm_rope_kv_write(
            qkv.tensor, q, ctx.positions, num_heads=self.num_heads, num_kv_heads=kv_heads, head_dim=self.head_dim,
            eps=self.eps if self.eps is not None else 0.0, q_norm=self.q_norm, k_norm=self.k_norm, bias=bias,
            cos_sin=self._table, n_rot=self.position.n_rot if self.position is not None else 0,
            slot_mapping=g.slot_mapping if cache.writable else None, k_base=cache.k_base, v_base=cache.v_base,
            page_stride=cache.page_stride, page_size=cache.page_size, splits=qkv.splits,
            interleaved=bool(self.position.interleaved) if self.position is not None else False)
        out = ws.get("attn_out", (T, self.q_width), dt)
        if self._use_flash():
            from ..csrc import flash
            flash.attention(q, cache, g, ctx, out, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                            head_dim=self.head_dim, window=self.window, scale=self.scale)
        else:
            ops.attention_generic(q, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, g.block_table,
                                  ctx.row_seg, ctx.positions, out, num_heads=self.num_heads,
                                  num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, window=self.window,
                                  scale=self.scale)
        return self.o_proj(out, ctx, "o_out", torch.float32, rows=T, allow_split=True, add_into=ctx.residual)


register_part("mixer", "attention", Attention)
