"""Python face of the tcgen05 matrix product (gemm_tcgen05.cu), for the kernel's own tests and measurements.

Few tokens (decoding, short portions): the weight fills the 128-row side of the tensor-core instruction
and the tokens the other side ("swapped"), K is split over CTAs so that all SMs stream weights, and the
float32 partial results are summed by the kernel that consumes the product.  Many tokens: 128-token by
256-feature tiles, and 256 by 256 on pairs of CTAs (cta_group::2) once those fill the device.  The engine
chooses among these in parts/linear.cpp.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p
from typing import Optional, Tuple

import torch

from . import ops
from .ops import KernelError, call, register_signatures

register_signatures("gemm100", {
    "ph_gemm_bf16_tcgen05": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p],
    "ph_gemm_bf16_tcgen05_pair": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
})

BLOCK_K = 64
_flags = {}
_sm_count = {}

ERRORS = {101: "the TMA producer waited too long for a free stage", 102: "the MMA warp waited too long",
          103: "the epilogue waited too long for an accumulator"}


def supports(weight: torch.Tensor) -> bool:
    return (weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[1] % 8 == 0
            and weight.data_ptr() % 16 == 0 and weight.is_contiguous())


def error_flag(device) -> torch.Tensor:
    flag = _flags.get(device)
    if flag is None:
        key = torch.device(device)
        if key not in _flags:
            _flags[key] = torch.zeros(1, dtype=torch.int32, device=key)
        flag = _flags[device] = _flags[key]
    return flag


def check_errors(device) -> None:
    """Raise if a kernel gave up on a wait since the last check (synchronises the device)."""
    key = torch.device(device)
    if key in _flags:
        code = int(_flags[key].item())
        if code:
            _flags[key].zero_()
            raise KernelError(f"gemm_tcgen05: {ERRORS.get(code, 'error')} (status {code})")


def sm_count(device) -> int:
    key = torch.device(device)
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _sm_count[key]


def gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, swapped: bool, block_n: int, splits: int = 1,
         max_ctas: int = 0, swiglu: bool = False, accumulate: bool = False, row_sumsq: Optional[torch.Tensor] = None,
         row_width: int = 0, row_eps: float = 0.0, norm_ahead: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None
         ) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T (out [splits, M, N] float32 partial sums when splits > 1).  With
    ``swiglu`` the rows of w are (gate, up) pairs and out is [M, N / 2] = silu(gate) * up.  ``accumulate``
    (plain orientation, float32, one split): out += the product.  ``row_sumsq`` [M, chunks] (swapped with bfloat16
    out, or plain with block_n 256): the rows of x lack the factor rsqrt(sum(row_sumsq[m]) / row_width + row_eps);
    the epilogue applies it.  ``norm_ahead`` (weight float32 [N], rows bfloat16 [M, N], sumsq float32 [M, 2 * ceil(N / 256)];
    plain, block_n 256, accumulate): rows = (the new out) * weight, sumsq[m, j] = the sum of squares of the new out
    over columns 128 j .. 128 j + 127."""
    for name, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise KernelError(f"gemm_tcgen05: {name} must be a contiguous bfloat16 CUDA tensor")
    N, K = w.shape
    M = x.numel() // K
    if x.shape[-1] != K or out.numel() != splits * M * (N // 2 if swiglu else N) or not out.is_contiguous():
        raise KernelError(f"gemm_tcgen05: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    call("gemm100", "ph_gemm_bf16_tcgen05", x.data_ptr(), w.data_ptr(), out.data_ptr(), ops._code(out.dtype), M, N, K,
         1 if swapped else 0, block_n, splits, max_ctas, 1 if swiglu else 0, 1 if accumulate else 0,
         None if row_sumsq is None else row_sumsq.data_ptr(), 0 if row_sumsq is None else row_sumsq.shape[-1], row_width,
         float(row_eps), *_norm_ahead_pointers(norm_ahead, M, N), error_flag(x.device).data_ptr(), ops._stream())
    return out


def _norm_ahead_pointers(norm_ahead, M: int, N: int):
    if norm_ahead is None:
        return None, None, None
    weight, rows, sumsq = norm_ahead
    tiles = 2 * ((N + 255) // 256)
    if (weight.dtype != torch.float32 or weight.numel() != N or rows.dtype != torch.bfloat16 or rows.numel() != M * N
            or sumsq.dtype != torch.float32 or sumsq.numel() != M * tiles
            or not (weight.is_contiguous() and rows.is_contiguous() and sumsq.is_contiguous())):
        raise KernelError(f"gemm_tcgen05: norm_ahead wants weight float32 [{N}], rows bfloat16 [{M}, {N}], sumsq float32 [{M}, {tiles}]")
    return weight.data_ptr(), rows.data_ptr(), sumsq.data_ptr()


def gemm_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, splits: int = 1, max_clusters: int = 0,
              swiglu: bool = False, accumulate: bool = False, row_sumsq: Optional[torch.Tensor] = None,
              row_width: int = 0, row_eps: float = 0.0,
              norm_ahead: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T on pairs of CTAs (cta_group::2), tiles of 256 x 256; float32 partial sums
    [splits, M, N] when splits > 1; ``swiglu``, ``row_sumsq`` and ``norm_ahead`` as in gemm."""
    for name, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise KernelError(f"gemm_tcgen05_pair: {name} must be a contiguous bfloat16 CUDA tensor")
    N, K = w.shape
    M = x.numel() // K
    if x.shape[-1] != K or out.numel() != splits * M * (N // 2 if swiglu else N) or not out.is_contiguous():
        raise KernelError(f"gemm_tcgen05_pair: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    call("gemm100", "ph_gemm_bf16_tcgen05_pair", x.data_ptr(), w.data_ptr(), out.data_ptr(), ops._code(out.dtype), M, N, K,
         splits, max_clusters, 1 if swiglu else 0, 1 if accumulate else 0,
         None if row_sumsq is None else row_sumsq.data_ptr(), 0 if row_sumsq is None else row_sumsq.shape[-1], row_width,
         float(row_eps), *_norm_ahead_pointers(norm_ahead, M, N), error_flag(x.device).data_ptr(), ops._stream())
    return out
