"""The engine: a model, its cache and the one step function.

``Engine.step(entries)`` takes a batch of (request, its next tokens, the places whose logits are wanted):
portions of prompts beside single decoded tokens, cut anywhere.  It runs only the tokens it is given, as
one batch, against the cache that earlier steps left, and returns float32 logits at the wanted places.
The scheduler, the Python entry point and the trace replay tool all drive this function; there is no
other forward pass.  The reference has three entry points instead (one decode row, consecutive rows of
one sequence, one decode row of each of n sequences: src/qwen_model.h:36-42, 150-161) and never mixes
prompt portions with decode rows in one pass (src/inference.cpp:3071-3143).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages, OutOfSlots
from ..config.base import ModelConfig, load_config, lookup_architecture
from ..parts.context import Q_TILE, Q_TILE_LARGE, GroupStep, StepContext, Workspace
from ..parts.model import DecoderModel

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class StepError(ValueError):
    """A batch that cannot be run: an unknown token id, a position past the model's limit, a request in
    the batch twice."""


@dataclass
class StepEntry:
    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()             # places among ``tokens`` whose logits are returned


@dataclass
class StepStats:
    tokens: int = 0
    prompt_rows: int = 0
    decode_rows: int = 0
    wanted: int = 0
    pages_free: List[int] = field(default_factory=list)


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype} is not supported (bfloat16 or float32)")
        return dtype
    try:
        return _DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype {dtype!r} is not supported (bfloat16 or float32)") from None


@dataclass
class _Layout:
    flat: List[int]
    sizes: List[int]
    T: int
    S: int
    widths: List[int]
    q_lens: List[int]
    ctx_lens: List[int]
    n_want: int
    n_decode: int
    n_tiles: int
    decode_max_ctx: int
    n_tiles_large: int = 0
    prefill_max_ctx: int = 0


@dataclass
class _DecodeGraph:
    workspace: Workspace
    meta: torch.Tensor
    graph: Optional[torch.cuda.CUDAGraph] = None
    logits: Optional[torch.Tensor] = None
    rows: Optional[torch.Tensor] = None
    launches: int = 0


def _bucket(n: int) -> int:
    """0, or the power of two (at least 256) that n fits."""
    if n <= 0:
        return 0
    b = 256
    while b < n:
        b *= 2
    return b


class PendingTokens:
    """Tokens being sampled on the device: ``ids`` (int32 on the device, valid in stream order at once) and their
    copy to pinned host memory, complete when ``event`` is."""

    def __init__(self, capacity: int):
        self.capacity = capacity
        self.host = torch.empty(capacity, dtype=torch.int32).pin_memory()
        self.params = torch.empty(24 * capacity, dtype=torch.uint8).pin_memory()
        self.event = torch.cuda.Event()
        self.ids: Optional[torch.Tensor] = None
        self.rows = 0

    def result(self) -> List[int]:
        self.event.synchronize()
        return self.host[:self.rows].tolist()


class Engine:
    def __init__(self, model: DecoderModel, config: Optional[ModelConfig], *, page_size: int = 16,
                 max_tokens: int = 4096, max_requests: int = 4, num_pages=None, device="cuda:0",
                 poison_cache: bool = False, cuda_graphs: bool = True, max_graph_batch: int = 256,
                 max_graphs: int = 24):
        """``model`` is bound to its weights already.  The cache holds ``max_tokens`` tokens per page group
        (each request's count rounded up to whole pages) for up to ``max_requests`` live requests;
        ``num_pages`` overrides the page count (one number or one per group).  With ``cuda_graphs`` a batch
        of single tokens replays a captured graph of the model's launches."""
        if not torch.cuda.is_available():
            raise RuntimeError("purhie_b200 runs on a CUDA device only; no GPU is visible and there is no host path")
        self.model = model
        self.config = config
        self.device = torch.device(device)
        self.dtype = model.compute_dtype
        self.page_size = page_size
        self.max_requests = max_requests
        if num_pages is None:
            num_pages = -(-max_tokens // page_size)
        self.cache = CacheManager(model.cache_needs(), page_size, num_pages, max_requests)
        self.cache.materialize(self.device, self.dtype, poison=poison_cache)
        self.views = model.cache_views(self.cache)
        self.workspace = Workspace(self.device)
        self.vocab_size = model.spec.vocab_size
        self.max_position = model.spec.max_position
        self.last_stats = StepStats()
        # rows per tile of the products for many tokens (the tcgen05 pair kernel): a scheduler may end a step there
        self.row_tile = 256 if self.dtype == torch.bfloat16 else None
        self._meta_host = [(None, None), (None, None)]
        self._pending_ring: List[Optional[PendingTokens]] = [None] * 4
        self._pending_turn = 0
        self._meta_turn = 0
        self.cuda_graphs = cuda_graphs
        self.max_graph_batch = max_graph_batch
        self.max_graphs = max_graphs
        self._graphs: Dict[tuple, _DecodeGraph] = {}
        self.graph_prompts = True                       # batches with prompt portions are captured when they recur ...
        self.graph_prompt_tokens = 1024                 # ... and are small enough for the host's launches to be what they wait for
        self.max_prompt_graphs = 8
        self._step_graphs: Dict[tuple, _DecodeGraph] = {}
        self._step_seen: Dict[tuple, int] = {}
        self.last_upload_bytes = 0
        from ..csrc.build import load_library
        for lib in model.required_libraries():          # compile what this model needs, now
            load_library(lib)

    # ---- construction ----------------------------------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", device="cuda:0", options: Optional[dict] = None,
                    **kw) -> "Engine":
        arch, config = load_config(model_dir)
        model = DecoderModel(arch.build_spec(config), parse_dtype(dtype), options)
        model.load(model_dir, device)
        return cls(model, config, device=device, **kw)

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int, dtype="bfloat16", device="cuda:0", std: float = 0.02,
                    scale_low: float = 1.0, scale_high: float = 1.0, options: Optional[dict] = None,
                    **kw) -> "Engine":
        """Random weights made directly on the device (no folder is written).  Values differ from those of
        :func:`purhie_b200.weights.write_random_model`, which draws on the host."""
        from ..api import load_model_random
        model = load_model_random(config, seed, dtype, device, std, scale_low, scale_high, options)._decoder
        return cls(model, config, device=device, **kw)

    # ---- requests --------------------------------------------------------------------------------
    def add_request(self, request_id) -> None:
        self.cache.add_request(request_id)

    def has_request(self, request_id) -> bool:
        return self.cache.has_request(request_id)

    def release(self, request_id) -> None:
        self.cache.release(request_id)

    def length(self, request_id) -> int:
        return self.cache.length(request_id)

    # ---- the step --------------------------------------------------------------------------------
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} is in the batch twice")
            seen.add(e.request_id)
            if not self.cache.has_request(e.request_id):
                raise StepError(f"request {e.request_id!r} is not live (add_request first)")
            n = len(e.tokens)
            if n < 1:
                raise StepError(f"request {e.request_id!r} brings no tokens")
            if n > 16:
                lo, hi = min(e.tokens), max(e.tokens)            # one pass in C instead of a check per token
                bad = lo if not 0 <= int(lo) else hi if not int(hi) < self.vocab_size else None
            else:
                bad = next((t for t in e.tokens if not 0 <= int(t) < self.vocab_size), None)
            if bad is not None:
                raise StepError(f"request {e.request_id!r}: token id {bad} is outside the vocabulary of "
                                f"{self.vocab_size}")
            if self.cache.length(e.request_id) + n > self.max_position:
                raise StepError(f"request {e.request_id!r} would reach position "
                                f"{self.cache.length(e.request_id) + n}, the model's limit is {self.max_position}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"request {e.request_id!r}: wanted place {w} is outside its {n} tokens")

    def _layout(self, entries: Sequence[StepEntry], table_width: Optional[int] = None) -> "_Layout":
        """Reserve pages for the batch and lay its metadata out as one int32 buffer."""
        cache = self.cache
        reserved = []
        try:
            for e in entries:
                cache.reserve(e.request_id, len(e.tokens))
                reserved.append(e)
        except OutOfPages:
            # give back what this step took, so that a refused step changes nothing
            for e in reserved:
                cache.unreserve(e.request_id)
            raise
        tokens, positions, row_seg, seg_start, ctx_lens, q_lens, slots, want = [], [], [], [0], [], [], [], []
        for s, e in enumerate(entries):
            start = cache.length(e.request_id)
            n = len(e.tokens)
            base = len(tokens)
            tokens.extend(e.tokens if type(e.tokens) is list else (int(t) for t in e.tokens))
            positions.extend(range(start, start + n))
            row_seg.extend([s] * n)
            seg_start.append(base + n)
            ctx_lens.append(start + n)
            q_lens.append(n)
            slots.append(cache.slot_of(e.request_id))
            want.extend(base + int(w) for w in e.want)
        T, S = len(tokens), len(entries)
        decode_rows, tile_seg, tile_first, decode_max_ctx, big_seg, big_first = [], [], [], 0, [], []
        for s, n in enumerate(q_lens):
            if n == 1:
                decode_rows.append(seg_start[s])
                decode_max_ctx = max(decode_max_ctx, ctx_lens[s])
            else:
                for first in range(0, n, Q_TILE):
                    tile_seg.append(s)
                    tile_first.append(first)
                for first in range(0, n, Q_TILE_LARGE):
                    big_seg.append(s)
                    big_first.append(first)
        # the tiles that look furthest back come first: the attention grid starts them first, and the short ones
        # fill the tail
        for segs, firsts, rows in ((tile_seg, tile_first, Q_TILE), (big_seg, big_first, Q_TILE_LARGE)):
            order = sorted(range(len(segs)), key=lambda i: -(ctx_lens[segs[i]] - q_lens[segs[i]] + min(firsts[i] + rows, q_lens[segs[i]])))
            segs[:], firsts[:] = [segs[i] for i in order], [firsts[i] for i in order]
        widths = []
        for g in cache.groups:
            w = max(len(cache.block_table(e.request_id, g.index)) for e in entries)
            widths.append(max(table_width or 0, -(-w // 8) * 8))
        sizes = [T, T, T, S + 1, S, S, max(len(want), 1)] + [S * w for w in widths] + [T] * len(cache.groups) + \
                [max(len(decode_rows), 1), max(len(tile_seg), 1), max(len(tile_seg), 1), max(len(big_seg), 1),
                 max(len(big_seg), 1)]
        flat: List[int] = []
        flat += tokens + positions + row_seg + seg_start + ctx_lens + slots + (want if want else [0])
        for g, w in zip(cache.groups, widths):
            for e in entries:
                table = cache.block_table(e.request_id, g.index)
                flat += table + [-1] * (w - len(table))
        for g in cache.groups:
            for e in entries:
                flat += cache.token_slots(e.request_id, g.index, cache.length(e.request_id), len(e.tokens))
        flat += (decode_rows or [0]) + (tile_seg or [0]) + (tile_first or [0]) + (big_seg or [0]) + (big_first or [0])
        return _Layout(flat, sizes, T, S, widths, q_lens, ctx_lens, len(want), len(decode_rows), len(tile_seg),
                       decode_max_ctx, len(big_seg), max([c for c, n in zip(ctx_lens, q_lens) if n > 1], default=0))

    def _upload(self, flat: List[int], dev: torch.Tensor) -> None:
        """One copy of the metadata to the device, through two pinned buffers used in turn: a buffer is
        rewritten only after the copy that last read it is done."""
        total = len(flat)
        self.last_upload_bytes = 4 * total
        self._meta_turn ^= 1
        buf, event = self._meta_host[self._meta_turn]
        if buf is None or buf.numel() < total:
            buf = torch.empty(max(2 * total, 4096), dtype=torch.int32).pin_memory()
            event = torch.cuda.Event()
        else:
            event.synchronize()
        self._meta_host[self._meta_turn] = (buf, event)
        buf.numpy()[:total] = flat                     # straight into the pinned memory
        dev.copy_(buf[:total], non_blocking=True)
        event.record()

    def _context(self, lay: "_Layout", dev: torch.Tensor, workspace: Workspace):
        """The step context over the metadata in ``dev``.  Returns (ctx, want_rows)."""
        G, S = len(self.cache.groups), lay.S
        parts, off = [], 0
        for n in lay.sizes:
            parts.append(dev[off:off + n])
            off += n
        groups = [GroupStep(parts[7 + i].view(S, lay.widths[i]), parts[7 + G + i], self.page_size) for i in range(G)]
        ctx = StepContext(T=lay.T, S=S, token_ids=parts[0], positions=parts[1], row_seg=parts[2], seg_start=parts[3],
                          seg_ctx_len=parts[4], seg_slot=parts[5], q_lens=lay.q_lens, ctx_lens=lay.ctx_lens,
                          groups=groups, workspace=workspace, compute_dtype=self.dtype, decode_only=lay.n_tiles == 0,
                          decode_rows=None if lay.n_tiles == 0 else parts[7 + 2 * G], n_decode_rows=lay.n_decode,
                          decode_max_ctx=_bucket(lay.decode_max_ctx), prefill_max_ctx=_bucket(lay.prefill_max_ctx),
                          q_tile_seg=parts[8 + 2 * G],
                          q_tile_first=parts[9 + 2 * G], n_q_tiles=lay.n_tiles, q_tile_large_seg=parts[10 + 2 * G],
                          q_tile_large_first=parts[11 + 2 * G], n_q_tiles_large=lay.n_tiles_large)
        return ctx, parts[6]

    def build_context(self, entries: Sequence[StepEntry]):
        """Reserve pages and upload the batch's metadata.  Returns (ctx, want_rows, n_want)."""
        lay = self._layout(entries)
        dev = self.workspace.get("step_meta", (len(lay.flat),), torch.int32)
        self._upload(lay.flat, dev)
        ctx, want_rows = self._context(lay, dev, self.workspace)
        return ctx, want_rows, lay.n_want

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one batch.  Returns float32 logits [wanted places, vocab] on the device in the order of the
        entries and of each entry's ``want`` (None when nothing is wanted); they live in scratch memory that
        the next step reuses.  Raises :class:`OutOfPages`, leaving everything as it was, when the cache
        cannot hold the batch.

        ``device_tokens`` (int32 on the device, one per entry): a batch of single tokens takes its token ids from
        there instead of from the entries, whose ids are then placeholders.  That lets a caller launch a step
        with the tokens the step before sampled without waiting for them (:meth:`sample_async`)."""
        entries = list(entries)
        if not entries:
            return None
        self._validate(entries)
        if self.decodes_as_graph(entries):
            logits, T, n_want = self._decode_with_graph(entries, device_tokens)
            q_lens = [1] * T
        elif device_tokens is not None:
            raise StepError("token ids from the device need a batch of single tokens that runs as a graph")
        else:
            logits, T, q_lens, n_want = self._step_any(entries)
        for e in entries:
            self.cache.advance(e.request_id, len(e.tokens))
        self.last_stats = StepStats(tokens=T, prompt_rows=sum(q for q in q_lens if q > 1),
                                    decode_rows=sum(1 for q in q_lens if q == 1), wanted=n_want,
                                    pages_free=self.cache.free_pages())
        return logits

    # ---- batches with prompt portions -----------------------------------------------------------------
    def _step_any(self, entries: Sequence[StepEntry]):
        """A batch with prompt portions.  Its launches depend on the lengths of the portions, the number of wanted
        rows, the width of the block tables and (in powers of two) how far back the portions and the decode rows
        look, not on the tokens: a combination of at most graph_prompt_tokens tokens that comes a third time (the
        chunks of a long prompt, a scheduler's steady mix) is captured as a graph with scratch memory of its own and
        replayed from then on, which takes the few hundred launcher calls of a step off the host; larger batches keep
        the device busy longer than the host needs to launch them.  Returns (logits, T, q_lens, wanted)."""
        ps = self.page_size
        need = max(-(-(self.cache.length(e.request_id) + len(e.tokens)) // ps) for e in entries) if self.cache.groups else 1
        width = 8
        while width < need:
            width *= 2
        lay = self._layout(entries, table_width=width)
        key = (tuple(lay.q_lens), tuple(len(e.want) for e in entries), tuple(lay.widths), _bucket(lay.decode_max_ctx),
               _bucket(lay.prefill_max_ctx))
        g = self._step_graphs.get(key) if self.cuda_graphs and self.graph_prompts else None
        if g is None and self.cuda_graphs and self.graph_prompts:
            seen = self._step_seen.get(key, 0)
            if len(self._step_seen) > 4096:
                self._step_seen.clear()
            self._step_seen[key] = seen + 1
            if seen >= 2 and lay.T <= self.graph_prompt_tokens:
                while len(self._step_graphs) >= self.max_prompt_graphs:
                    self._step_graphs.pop(next(iter(self._step_graphs)))
                g = _DecodeGraph(Workspace(self.device), torch.empty(len(lay.flat), dtype=torch.int32, device=self.device))
                self._step_graphs[key] = g
        if g is None:
            dev = self.workspace.get("step_meta", (len(lay.flat),), torch.int32)
            self._upload(lay.flat, dev)
            ctx, want_rows = self._context(lay, dev, self.workspace)
            return self._forward(ctx, want_rows, lay.n_want), lay.T, lay.q_lens, lay.n_want
        self._step_graphs[key] = self._step_graphs.pop(key)               # most recently used last
        self._upload(lay.flat, g.meta)
        from ..csrc import ops
        if g.graph is None:
            ctx, want_rows = self._context(lay, g.meta, g.workspace)
            g.logits = self._forward(ctx, want_rows, lay.n_want)           # this step's result, and every first-use set-up
            g.workspace.frozen = True
            graph = torch.cuda.CUDAGraph()
            before = ops.launches
            with torch.cuda.graph(graph):
                self._forward(ctx, want_rows, lay.n_want)
            g.launches = ops.launches - before
            ops.launches = before
            g.graph = graph
        else:
            g.graph.replay()
            ops.launches += g.launches
        return g.logits, lay.T, lay.q_lens, lay.n_want

    def _forward(self, ctx, want_rows, n_want):
        from ..csrc import ops
        with ops.on_current_stream():
            return self.model.forward(ctx, self.views, want_rows, n_want)

    # ---- decoding through CUDA graphs --------------------------------------------------------------
    def decodes_as_graph(self, entries: Sequence[StepEntry]) -> bool:
        return self.cuda_graphs and len(entries) <= self.max_graph_batch and all(len(e.tokens) == 1 for e in entries)

    def _decode_with_graph(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None):
        """A batch of single tokens: the launches of the whole model are captured once per (batch size, block
        table width, attention splits) and replayed.  Each graph owns its scratch memory and metadata buffer,
        so nothing it points at ever moves."""
        S = len(entries)
        need = max(len(self.cache.block_table(e.request_id, g.index)) + 1 for e in entries for g in self.cache.groups) \
            if self.cache.groups else 1
        width = 8
        while width < need:
            width *= 2
        # the graph computes every row's logits, so the layout (and its size) does not depend on what is wanted
        lay = self._layout([StepEntry(e.request_id, e.tokens, [0]) for e in entries], table_width=width)
        want = [i for i, e in enumerate(entries) if len(e.want)]
        ctx_bucket = 256
        while ctx_bucket < lay.decode_max_ctx:
            ctx_bucket *= 2
        key = (S, tuple(lay.widths), ctx_bucket)
        g = self._graphs.get(key)
        if g is None:
            if len(self._graphs) >= self.max_graphs:
                self._graphs.pop(next(iter(self._graphs)))
            g = _DecodeGraph(Workspace(self.device), torch.empty(len(lay.flat), dtype=torch.int32, device=self.device))
            self._graphs[key] = g
        self._upload(lay.flat, g.meta)
        if device_tokens is not None:
            g.meta[:S].copy_(device_tokens[:S], non_blocking=True)        # the token ids lead the metadata
        # every row's logits are computed; the wanted ones are picked afterwards
        all_rows = torch.arange(S, dtype=torch.int32, device=self.device) if g.rows is None else g.rows
        g.rows = all_rows
        if g.graph is None:
            ctx, want_rows = self._context(lay, g.meta, g.workspace)
            ctx.decode_max_ctx = ctx_bucket      # the number of attention splits must not change between replays
            # the first time: run the launches directly (this is the step's result, and whatever a kernel
            # sets up on first use is set up), then capture the same launches for the next time
            g.logits = self._forward(ctx, all_rows, S)
            g.workspace.frozen = True
            from ..csrc import ops
            graph = torch.cuda.CUDAGraph()
            before = ops.launches
            with torch.cuda.graph(graph):
                self._forward(ctx, all_rows, S)
            g.launches = ops.launches - before
            ops.launches = before
            g.graph = graph
        else:
            from ..csrc import ops
            g.graph.replay()
            ops.launches += g.launches
        if len(want) == S:
            return g.logits, S, S
        if not want:
            return None, S, 0
        idx = torch.tensor(want, dtype=torch.long, device=self.device)
        return g.logits.index_select(0, idx), S, len(want)

    # ---- sampling --------------------------------------------------------------------------------
    def sample_async(self, logits: torch.Tensor, samplers) -> Optional["PendingTokens"]:
        """Start sampling one token per row on the device and their copy to the host without waiting for either.
        Returns None when the rows' samplers do not all run the same device kernel (see :meth:`sample`).  Each
        sampler draws its uniform number now."""
        from ..csrc import ops
        R = len(samplers)
        if logits is None or logits.shape[0] != R:
            raise StepError(f"{R} samplers for {0 if logits is None else logits.shape[0]} rows of logits")
        modes = {s.device_mode() for s in samplers}
        if len(modes) != 1 or None in modes:
            return None
        mode = modes.pop()
        self._pending_turn = (self._pending_turn + 1) % len(self._pending_ring)
        slot = self._pending_ring[self._pending_turn]
        if slot is None or slot.capacity < R:
            slot = PendingTokens(max(R, 64))
            self._pending_ring[self._pending_turn] = slot
        else:
            slot.event.synchronize()                  # its last copies are done: the pinned buffers may be rewritten
        ids = torch.empty(R, dtype=torch.int32, device=self.device)
        if mode == "greedy":
            ops.argmax(logits, ids)
        else:
            rec = slot.params.numpy()[:24 * R].view(ops.CHAIN_ROW)
            if mode == "chain":
                for j, s in enumerate(samplers):
                    rec[j] = s.chain_record()
                rows = self.workspace.get("sample_rows", (R, 24), torch.uint8)
                rows.view(-1).copy_(slot.params[:24 * R], non_blocking=True)
                ops.sample_chain(logits, rows, ids)
            else:
                for j, s in enumerate(samplers):
                    rec[j] = (s.uniform(), 1.0, 0.0, s.params.temperature, 0)
                rows = self.workspace.get("sample_rows", (R, 24), torch.uint8)
                rows.view(-1).copy_(slot.params[:24 * R], non_blocking=True)
                packed = rows.view(-1)
                temps = self.workspace.get("sample_temps", (R,), torch.float32)
                unis = self.workspace.get("sample_unis", (R,), torch.float64)
                unis.copy_(packed.view(torch.float64).view(R, 3)[:, 0])
                temps.copy_(packed.view(torch.float32).view(R, 6)[:, 4])
                ops.sample_temperature(logits, temps, unis, ids)
        slot.host[:R].copy_(ids, non_blocking=True)
        slot.event.record()
        slot.ids, slot.rows = ids, R
        return slot

    def sample(self, logits: torch.Tensor, samplers) -> List[int]:
        """One token per row of ``logits`` with the row's sampler.  Greedy, plain temperature sampling and the
        chain with top-k on run in the device kernels (the uniform number still comes from the sampler's
        generator, one per token); penalties, and top-p or min-p without top-k, run on the host over a copy of
        the row."""
        from ..csrc import ops
        R = len(samplers)
        if logits is None or logits.shape[0] != R:
            raise StepError(f"{R} samplers for {0 if logits is None else logits.shape[0]} rows of logits")
        modes = [s.device_mode() for s in samplers]
        out: List[Optional[int]] = [None] * R
        if "greedy" in modes:
            ids = self.workspace.get("sample_greedy", (R,), torch.int32)
            ops.argmax(logits, ids)
            host = ids.cpu().tolist()
            for i, m in enumerate(modes):
                if m == "greedy":
                    out[i] = host[i]
        if "temperature" in modes:
            temps = torch.tensor([s.params.temperature if m == "temperature" else 1.0
                                  for s, m in zip(samplers, modes)], dtype=torch.float32)
            unis = torch.tensor([s.uniform() if m == "temperature" else 0.0 for s, m in zip(samplers, modes)],
                                dtype=torch.float64)
            ids = self.workspace.get("sample_temp", (R,), torch.int32)
            ops.sample_temperature(logits, temps.to(self.device), unis.to(self.device), ids)
            host = ids.cpu().tolist()
            for i, m in enumerate(modes):
                if m == "temperature":
                    out[i] = host[i]
        if "chain" in modes:
            import numpy as np
            which = [i for i, m in enumerate(modes) if m == "chain"]
            rec = np.zeros(len(which), dtype=ops.CHAIN_ROW)
            for j, i in enumerate(which):
                rec[j] = samplers[i].chain_record()
            rows = torch.from_numpy(rec.view(np.uint8).reshape(len(which), 24)).to(self.device)
            picked = logits if len(which) == R else logits.index_select(0, torch.tensor(which, device=self.device))
            ids = self.workspace.get("sample_chain", (len(which),), torch.int32)
            ops.sample_chain(picked, rows, ids)
            for i, tok in zip(which, ids.cpu().tolist()):
                out[i] = tok
        for i, m in enumerate(modes):
            if m is None:
                out[i] = samplers[i].sample(logits[i].float().cpu().numpy())
        return out
