"""Python face of the tensor-core attention kernels, for the kernels' own tests and measurements.

A step's rows go two ways: segments of one token (decoding) through a split-key kernel, every other
segment (a portion of a prompt) through a tiled kernel.  Both read keys and values from the pages.  The
engine chooses among them, and the number of splits, in parts/attention.cpp.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import ops
from .ops import KernelError, call, register_signatures

register_signatures("flash", {
    "ph_attention_prefill": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_int, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "ph_attention_decode_bulk": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                 c_float, c_int, c_void_p, c_void_p],
    "ph_attention_prefill_tc5": [c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float,
                                 c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "ph_attention_decode": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
                            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                            c_void_p],
})

BLOCK_KEYS = 64
MAX_SPLITS = 32
_sm_count = {}


def supports(head_dim: int, group_size: int) -> bool:
    return head_dim in (64, 128) and 1 <= group_size <= 16


def _sms(device) -> int:
    key = torch.device(device)
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _sm_count[key]


CTAS_PER_SM = 3            # decode CTAs that fit one SM (68 KB of shared memory each at head_dim 128)
CTA_FIXED_COST = 4.0       # a CTA's start and end (query load, first block's latency, merge), in units of one block's time


def decode_splits(n_rows: int, num_kv_heads: int, max_ctx: int, sms: int, window: Optional[int] = None) -> int:
    """Splits of the key range.  CTAs run in waves of CTAS_PER_SM per SM; the number of splits is the one
    that minimises waves x (fixed cost + blocks per split), so that neither a nearly empty last wave nor the
    per-CTA overhead dominates."""
    span = min(max_ctx, window) if window else max_ctx
    blocks = max(1, -(-span // BLOCK_KEYS))
    pairs = max(1, n_rows * num_kv_heads)
    slots = CTAS_PER_SM * sms
    best, best_cost = 1, None
    for s in range(1, min(blocks, MAX_SPLITS) + 1):
        per = -(-blocks // s)
        if s > 1 and -(-blocks // per) != s:
            continue                       # the same blocks per split as a smaller s: only empty CTAs more
        waves = -(-(pairs * s) // slots)
        cost = waves * (CTA_FIXED_COST + per)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def prefill(q, k_base, v_base, page_stride, page_size, block_table, seg_start, seg_ctx_len, tile_seg, tile_first,
            n_tiles, out, *, num_heads, num_kv_heads, head_dim, window, scale) -> None:
    call("flash", "ph_attention_prefill", q.data_ptr(), k_base.data_ptr(), v_base.data_ptr(), page_stride, page_size,
         block_table.data_ptr(), block_table.shape[-1], seg_start.data_ptr(), seg_ctx_len.data_ptr(), tile_seg.data_ptr(),
         tile_first.data_ptr(), n_tiles, out.data_ptr(), num_heads, num_kv_heads, head_dim, int(window or 0), float(scale),
         ops._stream())


def tc5_supports(head_dim: int, page_size: int) -> bool:
    return head_dim == 128 and page_size in (8, 16, 32, 64)


def tc5_splits(n_tiles: int, num_heads: int, max_ctx: int, sms: int, window: Optional[int] = None) -> int:
    """CTAs per tile of the tcgen05 prefill kernel.  The time is about (rounds of the CTAs over two slots per SM) x
    (blocks of 64 keys per CTA + a few for its start) plus, when tiles are shared, what writing and merging the
    partial results costs; the count with the least wins.  Many tiles, or tiles that look back over few keys, stay
    whole; a short portion late in a long context is cut so that its CTAs fill the device once."""
    span = min(max_ctx, window + 128) if window else max_ctx
    blocks = max(1, -(-span // 64))
    ctas = max(1, n_tiles * num_heads)
    best, best_cost = 1, None
    for s in range(1, min(16, blocks) + 1):
        cost = -(-(ctas * s) // (2 * sms)) * (-(-blocks // s) + 4)
        if s > 1:
            # the second kernel's launch, and every row's partial results (512 bytes per head and CTA) written and
            # read back, in units of a block's time
            cost += 8 + 0.5 * s + 0.024 * ctas * s
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def prefill_tc5(q, n_rows, k_base, v_base, page_stride, page_size, num_pages, block_table, seg_start, seg_ctx_len, tile_seg,
                tile_first, n_tiles, out, *, num_heads, num_kv_heads, head_dim, window, scale, splits: int = 1,
                workspace=None) -> None:
    """The tcgen05 prefill kernel (attention_prefill_tc5.cu); tiles of 128 rows, each shared by ``splits`` CTAs."""
    part_o = part_ml = None
    if splits > 1:
        part_o = workspace.get("attn_tile_part_o", (n_rows, num_heads, splits, head_dim), torch.float32)
        part_ml = workspace.get("attn_tile_part_ml", (n_rows, num_heads, splits, 2), torch.float32)
    call("flash", "ph_attention_prefill_tc5", q.data_ptr(), n_rows, k_base.data_ptr(), v_base.data_ptr(), page_stride,
         page_size, num_pages, block_table.data_ptr(), block_table.shape[-1], seg_start.data_ptr(), seg_ctx_len.data_ptr(),
         tile_seg.data_ptr(), tile_first.data_ptr(), n_tiles, out.data_ptr(), num_heads, num_kv_heads, head_dim,
         int(window or 0), float(scale), splits, None if part_o is None else part_o.data_ptr(),
         None if part_ml is None else part_ml.data_ptr(), error_flag(q.device).data_ptr(), ops._stream())


def decode(q, k_base, v_base, page_stride, page_size, block_table, row_list, n_rows, row_seg, positions, out, workspace, *,
           num_heads, num_kv_heads, head_dim, window, scale, splits) -> None:
    part_o = part_ml = None
    if splits > 1:
        part_o = workspace.get("attn_part_o", (n_rows, num_heads, splits, head_dim), torch.float32)
        part_ml = workspace.get("attn_part_ml", (n_rows, num_heads, splits, 2), torch.float32)
    call("flash", "ph_attention_decode", q.data_ptr(), k_base.data_ptr(), v_base.data_ptr(), page_stride, page_size,
         block_table.data_ptr(), block_table.shape[-1], None if row_list is None else row_list.data_ptr(), n_rows,
         row_seg.data_ptr(), positions.data_ptr(), None if part_o is None else part_o.data_ptr(),
         None if part_ml is None else part_ml.data_ptr(), out.data_ptr(), num_heads, num_kv_heads, head_dim, splits,
         int(window or 0), float(scale), ops._stream())


_flags = {}
BULK_ERRORS = {111: "the attention producer waited too long for a free stage",
               112: "an attention consumer waited too long for keys",
               121: "the prefill attention producer waited too long", 122: "the prefill attention tensor-core warp waited too long",
               123: "a prefill attention softmax warp waited too long"}


def error_flag(device) -> torch.Tensor:
    key = torch.device(device)
    if key not in _flags:
        _flags[key] = torch.zeros(1, dtype=torch.int32, device=key)
    return _flags[key]


def check_errors(device) -> None:
    """Raise if the persistent decode kernel gave up on a wait since the last check (synchronises)."""
    key = torch.device(device)
    if key in _flags:
        code = int(_flags[key].item())
        if code:
            _flags[key].zero_()
            raise KernelError(f"attention kernel: {BULK_ERRORS.get(code, 'error')} (status {code})")


def bulk_splits(n_rows: int, num_kv_heads: int, max_ctx: int, sms: int, window: Optional[int] = None) -> int:
    """Splits for the persistent kernel: two CTAs per SM take items in turn, so the time is (items per CTA, rounded
    up) x (blocks of 64 keys per item + what an item costs beside its blocks), plus the merge kernel when the keys
    are split; pick the split count that minimises it.  A split item costs about a block and a half more (its
    partial result goes to memory), a whole one next to nothing, and the merge grows with the number of parts it
    reads: measured at 1 to 128 rows of 1,024 to 8,192 keys."""
    span = min(max_ctx, window) if window else max_ctx
    blocks = max(1, -(-span // BLOCK_KEYS))
    pairs = max(1, n_rows * num_kv_heads)
    best, best_cost = 1, None
    for s in range(1, min(blocks, MAX_SPLITS) + 1):
        per = -(-blocks // s)
        if s > 1 and -(-blocks // per) != s:
            continue
        cost = -(-(pairs * s) // (2 * sms)) * (per + (1.5 if s > 1 else 0.25)) + (2.0 + 0.15 * s if s > 1 else 0.0)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def bulk_supports(page_size: int) -> bool:
    return page_size % 8 == 0 and BLOCK_KEYS % page_size == 0


def decode_bulk(q, k_base, v_base, page_stride, page_size, num_pages, block_table, row_list, n_rows, row_seg, positions, out,
                workspace, *, num_heads, num_kv_heads, head_dim, window, scale, splits, max_ctas: int = 0) -> None:
    """The persistent decode kernel fed by TMA copies of whole pages (attention_decode_bulk.cu)."""
    part_o = part_ml = None
    if splits > 1:
        part_o = workspace.get("attn_part_o", (n_rows, num_heads, splits, head_dim), torch.float32)
        part_ml = workspace.get("attn_part_ml", (n_rows, num_heads, splits, 2), torch.float32)
    call("flash", "ph_attention_decode_bulk", q.data_ptr(), k_base.data_ptr(), v_base.data_ptr(), page_stride, page_size,
         num_pages, block_table.data_ptr(), block_table.shape[-1], None if row_list is None else row_list.data_ptr(), n_rows,
         row_seg.data_ptr(), positions.data_ptr(), None if part_o is None else part_o.data_ptr(),
         None if part_ml is None else part_ml.data_ptr(), out.data_ptr(), num_heads, num_kv_heads, head_dim, splits,
         int(window or 0), float(scale), max_ctas, error_flag(q.device).data_ptr(), ops._stream())
