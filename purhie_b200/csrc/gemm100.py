"""Python face of the tcgen05 matrix product (gemm_tcgen05.cu) and the choice of its shape.

Few tokens (decoding, short portions): the weight fills the 128-row side of the tensor-core instruction
and the tokens the other side ("swapped"), K is split over CTAs so that all SMs stream weights, and the
float32 partial results are summed by the kernel that consumes the product.  Many tokens: 128-token by
256-feature tiles, and 256 by 256 on pairs of CTAs (cta_group::2) once those fill the device.
"""
from __future__ import annotations

import functools
from ctypes import c_int, c_void_p
from typing import Optional

import torch

from . import ops
from .ops import KernelError, call, register_signatures

register_signatures("gemm100", {
    "ph_gemm_bf16_tcgen05": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_void_p, c_void_p],
    "ph_gemm_bf16_tcgen05_pair": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_int, c_void_p, c_void_p],
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
         max_ctas: int = 0, swiglu: bool = False, accumulate: bool = False) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T (out [splits, M, N] float32 partial sums when splits > 1).  With
    ``swiglu`` the rows of w are (gate, up) pairs and out is [M, N / 2] = silu(gate) * up.  ``accumulate``
    (plain orientation, float32, one split): out += the product."""
    for name, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise KernelError(f"gemm_tcgen05: {name} must be a contiguous bfloat16 CUDA tensor")
    N, K = w.shape
    M = x.numel() // K
    if x.shape[-1] != K or out.numel() != splits * M * (N // 2 if swiglu else N) or not out.is_contiguous():
        raise KernelError(f"gemm_tcgen05: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    call("gemm100", "ph_gemm_bf16_tcgen05", x.data_ptr(), w.data_ptr(), out.data_ptr(), ops._code(out.dtype), M, N, K,
         1 if swapped else 0, block_n, splits, max_ctas, 1 if swiglu else 0, 1 if accumulate else 0,
         error_flag(x.device).data_ptr(), ops._stream())
    return out


def gemm_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, splits: int = 1, max_clusters: int = 0,
              swiglu: bool = False, accumulate: bool = False) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T on pairs of CTAs (cta_group::2), tiles of 256 x 256; float32 partial sums
    [splits, M, N] when splits > 1; ``swiglu`` as in gemm."""
    for name, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise KernelError(f"gemm_tcgen05_pair: {name} must be a contiguous bfloat16 CUDA tensor")
    N, K = w.shape
    M = x.numel() // K
    if x.shape[-1] != K or out.numel() != splits * M * (N // 2 if swiglu else N) or not out.is_contiguous():
        raise KernelError(f"gemm_tcgen05_pair: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    call("gemm100", "ph_gemm_bf16_tcgen05_pair", x.data_ptr(), w.data_ptr(), out.data_ptr(), ops._code(out.dtype), M, N, K,
         splits, max_clusters, 1 if swiglu else 0, 1 if accumulate else 0, error_flag(x.device).data_ptr(), ops._stream())
    return out


@functools.lru_cache(maxsize=4096)
def plan(M: int, N: int, K: int, sms: int, allow_split: bool):
    """(swapped, block_n, splits) for a product of M tokens with an [N, K] weight.

    With few tokens the product is weight streaming: the work items (128-feature tile, split of K) should fill
    whole waves of the SMs, so the number of splits is the one with the best wave efficiency (items / (waves *
    SMs)), the fewest splits winning among near-equals, each split keeping at least four blocks of K."""
    kblocks = -(-K // BLOCK_K)
    if M >= 128:
        return False, (256 if N > 128 else 128 if N > 64 else 64), 1
    block_n = 16
    while block_n < M:
        block_n *= 2
    splits = 1
    if allow_split:
        a_tiles = -(-N // 128)
        best = -1.0
        slots = sms * (2 if block_n <= 64 else 1)          # the kernel runs two CTAs per SM for small tiles
        for s in range(1, min(16, max(1, kblocks // 4)) + 1):
            items = a_tiles * s
            eff = items / (-(-items // slots) * slots)
            if eff > best + 0.03:
                best, splits = eff, s
    return True, block_n, splits


@functools.lru_cache(maxsize=4096)
def plan_many(M: int, N: int, K: int, sms: int, allow_split: bool, fused_epilogue: bool = False):
    """(pair, splits) for a product of M >= 128 tokens in the plain orientation: the one-CTA kernel (tiles of 128
    tokens x 256 features) or the pair kernel (256 x 256 on two SMs), and into how many parts K is cut.

    Estimated cost in units of one block of K on one SM's tile: rounds of the CTAs (or pairs) times the item's
    blocks (the pair spends 0.87 of a block's time per block: half the shared-memory traffic per flop) plus six for
    an item's start and epilogue, plus the float32 partial results' way to memory and back when K is split.  A
    fused epilogue (the activation) needs the whole sum in one place: no split."""
    kblocks = -(-K // BLOCK_K)
    best, choice = None, (False, 1)
    split_options = (1, 2, 3, 4, 6, 8) if allow_split and not fused_epilogue else (1,)
    for pair in (False, True):
        if pair and (M <= 128 or N <= 128):
            continue
        tiles = (-(-M // 256) if pair else -(-M // 128)) * -(-N // 256)
        slots = sms // 2 if pair else sms
        for s in split_options:
            if s > 1 and kblocks // s < 8:
                continue
            rounds = -(-(tiles * s) // slots)
            cost = rounds * ((0.87 if pair else 1.0) * kblocks / s + 6.0)
            if s > 1:
                cost += 2.0 * s * M * N * 4 / 4.0e12 / 0.33e-6
            if best is None or cost < best - 1e-9:
                best, choice = cost, (pair, s)
    return choice


def linear(x: torch.Tensor, w: torch.Tensor, ctx, out_name: str, out_dtype: torch.dtype, M: int, allow_split: bool,
           fuse_swiglu: bool = False, add_into: Optional[torch.Tensor] = None):
    """The product through the tcgen05 kernel.  ``fuse_swiglu`` (w holds (gate, up) row pairs): when the plain
    orientation runs, the activation is applied in the epilogue and the result [M, N / 2] is marked activated."""
    from ..parts.base import Addend
    N, K = w.shape
    sms = sm_count(x.device)
    swapped, block_n, splits = plan(M, N, K, sms, allow_split)
    pair = False
    if not swapped and block_n == 256:
        fused = fuse_swiglu and N % 2 == 0
        pair, splits = plan_many(M, N, K, sms, allow_split, fused_epilogue=fused)
        if fused:
            out = ctx.workspace.get(out_name + "_act", (M, N // 2), out_dtype)
            if pair:
                gemm_pair(x[:M], w, out, swiglu=True)
            else:
                gemm(x[:M], w, out, swapped=False, block_n=block_n, swiglu=True)
            return Addend(out, 1, activated=True)
    elif fuse_swiglu and N % 2 == 0 and (splits == 1 or swapped):
        # few tokens: K stays whole, so that the epilogue holds whole sums and can apply the activation; the
        # weight tiles alone (N / 128 of them) keep the SMs streaming
        out = ctx.workspace.get(out_name + "_act", (M, N // 2), out_dtype)
        gemm(x[:M], w, out, swapped=swapped, block_n=block_n, swiglu=True)
        return Addend(out, 1, activated=True)
    if (add_into is not None and not swapped and splits == 1 and add_into.dtype == torch.float32 and add_into.is_contiguous()
            and add_into.shape[-1] == N and add_into.numel() >= M * N):
        # many tokens, K whole: the residual sum happens in the epilogue and the product never goes to memory
        target = add_into.view(-1, N)[:M]
        if pair:
            gemm_pair(x[:M], w, target, accumulate=True)
        else:
            gemm(x[:M], w, target, swapped=False, block_n=block_n, accumulate=True)
        return Addend(None, 0)
    if splits > 1:
        out = ctx.workspace.get(out_name + "_partial", (splits, M, N), torch.float32)
    else:
        out = ctx.workspace.get(out_name, (M, N), out_dtype)
    if pair:
        gemm_pair(x[:M], w, out, splits=splits)
    else:
        gemm(x[:M], w, out, swapped=swapped, block_n=block_n, splits=splits)
    return Addend(out, splits)
