"""What a step hands to the parts: the batch's metadata, the cache views and scratch memory.

A step is a flat batch of T token rows that belong to S segments; a segment is the next tokens of one
request (a portion of its prompt, or one decoded token).  Every part sees the same metadata; none of it
says which model is running.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .base import Addend


Q_TILE = 64        # rows of a query tile of the mma.sync prefill attention kernel
Q_TILE_LARGE = 128 # rows of a query tile of the tcgen05 prefill attention kernel


class Workspace:
    """Scratch tensors by name, reused from step to step and grown on demand.

    A tensor of a given name keeps its address as long as requests do not outgrow it, which is what a
    captured CUDA graph needs; ``frozen`` turns growth into an error.
    """

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self.frozen = False

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < n:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow while frozen")
            buf = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[key] = buf
        return buf[:n].view(*shape)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._bufs.values())


@dataclass
class GroupStep:
    """One page group's view of the step."""

    block_table: torch.Tensor            # int32 [S, table_width]: page of each logical block, -1 = given back
    slot_mapping: torch.Tensor           # int32 [T]: page * page_size + offset where each row's k and v go
    page_size: int


@dataclass
class CacheView:
    """The cache of one run-order entry, as its mixer sees it."""

    kind: str = "none"                   # "none" | "pages" | "state"
    group: int = -1
    k_base: Optional[torch.Tensor] = None   # K of this entry in page 0 (a view of the pool); pages are
    v_base: Optional[torch.Tensor] = None   # page_stride elements apart
    page_stride: int = 0
    page_size: int = 0
    num_pages: int = 0                      # pages of the pool the views belong to
    writable: bool = True                # False: another entry writes this cache, this one only reads
    state: Optional[torch.Tensor] = None    # [max_requests, *state_shape]


@dataclass
class StepContext:
    T: int
    S: int
    token_ids: torch.Tensor              # int32 [T]
    positions: torch.Tensor              # int32 [T] absolute position of each row in its request
    row_seg: torch.Tensor                # int32 [T] segment of each row
    seg_start: torch.Tensor              # int32 [S + 1] first row of each segment
    seg_ctx_len: torch.Tensor            # int32 [S] tokens of the request once this step is done
    seg_slot: torch.Tensor               # int32 [S] state slot of each segment's request
    q_lens: List[int]                    # host copies, for launch decisions
    ctx_lens: List[int]
    groups: List[GroupStep]
    workspace: Workspace
    compute_dtype: torch.dtype
    decode_only: bool = False
    # rows of single-token segments (None when every row is one: the list is then 0 .. T-1)
    decode_rows: Optional[torch.Tensor] = None
    n_decode_rows: int = 0
    decode_max_ctx: int = 0              # how far back the decode rows look, as the power of two that holds it
    prefill_max_ctx: int = 0             # the same for the prompt portions
    # The float32 residual [T, E] that the addend a mixer or feed-forward returns will be added to.  A part may add
    # its result into it itself (in the epilogue of its last product, say) and return Addend(None).
    residual: Optional[torch.Tensor] = None
    # the other segments cut into tiles of Q_TILE rows: segment and first row (within the portion) of each tile
    q_tile_seg: Optional[torch.Tensor] = None
    q_tile_first: Optional[torch.Tensor] = None
    n_q_tiles: int = 0
    # the same segments cut into tiles of Q_TILE_LARGE rows (the tcgen05 prefill kernel)
    q_tile_large_seg: Optional[torch.Tensor] = None
    q_tile_large_first: Optional[torch.Tensor] = None
    n_q_tiles_large: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens) if self.q_lens else 0

    @property
    def max_ctx_len(self) -> int:
        return max(self.ctx_lens) if self.ctx_lens else 0


class ResidualStream:
    """The float32 residual [T, E] plus an addend that the next norm folds in (x += addend, then norm),
    so that the sum and the normalisation are one pass over the row."""

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.pending: Optional[Addend] = None

    def add(self, addend: Addend) -> None:
        if self.pending is not None:
            raise RuntimeError("the residual stream already has a pending addend")
        self.pending = None if addend.tensor is None else addend          # None: the part added into x itself
