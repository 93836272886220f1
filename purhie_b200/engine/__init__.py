"""The engine as Python sees it: a model with its cache, and the one step function.

``Engine.step(entries)`` hands a batch of (request, its next tokens, the places whose logits are wanted) to the host
library's ``engine_step`` and returns float32 logits ``[wanted places, vocab]`` as a NumPy array.  Request ids may
be any hashable Python value; the library knows them by number.  Everything else (validation, pages, metadata,
launches, CUDA graphs) happens in ``engine/engine.cpp``.
"""
from __future__ import annotations

import ctypes
import json
from ctypes import POINTER, c_float, c_int32
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from .. import native
from ..native import KernelError, OutOfPages, OutOfSlots, StepError


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
    replayed_graph: bool = False


class Engine:
    """A loaded model and its cache.  Build one with :meth:`from_folder` or :meth:`from_random`."""

    def __init__(self, handle, *, page_size: int = 16, max_tokens: int = 4096, max_requests: int = 4, num_pages=None,
                 poison_cache: bool = False, cuda_graphs: bool = True, step_options: Optional[dict] = None,
                 n_ctx: int = 0, engine_options: Optional[dict] = None, attach: bool = False):
        L = native.lib()
        self._handle = handle
        self._owns = not attach
        self._ids: Dict[object, int] = {}
        self._next_id = 1 << 20                       # clear of the sequence numbers of the C API
        self.last_stats = StepStats()
        if attach:                                    # a model whose cache somebody else made (purhie_b200.api.Model)
            self.vocab_size = L.inference_vocab_size(handle)
            self.hidden_size = L.inference_hidden_size(handle)
            self.page_size, self.max_requests = page_size, L.inference_batch_size(handle)
            return
        native.ensure_libraries_for(handle)
        opts = dict(engine_options or {})
        opts.update({"poison_cache": poison_cache, "cuda_graphs": cuda_graphs})
        if num_pages is not None:
            opts["num_pages"] = num_pages
        if step_options:
            opts["step"] = step_options
        try:
            native.check(L.inference_kv_cache_init_ex(handle, n_ctx, max_requests, page_size, max_tokens,
                                                      json.dumps(opts).encode()))
        except Exception:
            L.inference_free_model(handle)
            self._handle = None
            raise
        self.vocab_size = L.inference_vocab_size(handle)
        self.hidden_size = L.inference_hidden_size(handle)
        self.page_size = page_size
        self.max_requests = max_requests
        self.last_stats = StepStats()

    # ---- construction ----------------------------------------------------------------------------------
    @staticmethod
    def load_handle(model_dir: str, dtype: str = "bfloat16", options: Optional[dict] = None):
        L = native.lib()
        h = L.inference_load_model_ex(str(model_dir).encode(), dtype.encode(), json.dumps(options or {}).encode())
        if not h:
            raise native.last_error()
        return h

    @staticmethod
    def random_handle(config, seed: int, dtype: str = "bfloat16", std: float = 0.02, scale_low: float = 1.0,
                      scale_high: float = 1.0, options: Optional[dict] = None):
        from ..weights import _config_json
        L = native.lib()
        h = L.inference_load_model_random_ex(_config_json(config), int(seed), dtype.encode(), float(std), float(scale_low),
                                             float(scale_high), json.dumps(options or {}).encode())
        if not h:
            raise native.last_error()
        return h

    @classmethod
    def from_folder(cls, model_dir: str, dtype: str = "bfloat16", options: Optional[dict] = None, **kw) -> "Engine":
        """``options``: kernel choices of the parts ({"gemm": ..., "attention": ...}); the rest as ``__init__``."""
        return cls(cls.load_handle(model_dir, dtype, options), **kw)

    @classmethod
    def from_random(cls, config, seed: int, dtype: str = "bfloat16", std: float = 0.02, scale_low: float = 1.0,
                    scale_high: float = 1.0, options: Optional[dict] = None, **kw) -> "Engine":
        """Random weights made on the device: the values :func:`purhie_b200.weights.write_random_model` stores for
        the same seed."""
        return cls(cls.random_handle(config, seed, dtype, std, scale_low, scale_high, options), **kw)

    @classmethod
    def attach(cls, model) -> "Engine":
        """The step function of a :class:`purhie_b200.api.Model` whose cache is made already: the same engine its
        generation uses, with requests of its own beside the model's sequences."""
        return cls(model.handle, attach=True)

    def close(self) -> None:
        if self._handle and self._owns:
            native.lib().inference_free_model(self._handle)
        self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._handle

    # ---- requests ----------------------------------------------------------------------------------------
    def _id(self, request_id) -> int:
        try:
            return self._ids[request_id]
        except KeyError:
            raise StepError(f"request {request_id!r} is not live (add_request first)") from None

    def add_request(self, request_id) -> None:
        if request_id in self._ids:
            raise ValueError(f"request {request_id!r} is already live")
        n = self._next_id
        native.check(native.lib().engine_request_add(self._handle, n))
        self._next_id += 1
        self._ids[request_id] = n

    def has_request(self, request_id) -> bool:
        return request_id in self._ids

    def release(self, request_id) -> None:
        native.check(native.lib().engine_request_release(self._handle, self._ids.pop(request_id)))

    def length(self, request_id) -> int:
        return native.lib().engine_request_length(self._handle, self._id(request_id))

    # ---- the step ------------------------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> Optional[np.ndarray]:
        """Run one batch.  Returns float32 logits [wanted places, vocab] in the order of the entries and of each
        entry's ``want`` (None when nothing is wanted).  Raises :class:`OutOfPages`, leaving everything as it was,
        when the cache cannot hold the batch, and :class:`StepError` for a batch that cannot be run."""
        entries = list(entries)
        if not entries:
            return None
        batch, keep, wanted = self._batch(entries)
        out = native.StepOutputC()
        logits = np.empty((max(wanted, 1), self.vocab_size), dtype=np.float32)
        out.logits = logits.ctypes.data_as(POINTER(c_float))
        out.logits_capacity = logits.size
        native.check(native.lib().engine_step(self._handle, ctypes.byref(batch), ctypes.byref(out)))
        self.last_stats = StepStats(out.tokens, out.prompt_rows, out.decode_rows, out.n_rows, bool(out.replayed_graph))
        return logits[:out.n_rows] if out.n_rows else None

    def _batch(self, entries):
        """The C batch for ``entries`` (and the arrays it points into, which the caller keeps alive)."""
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} is in the batch twice")
            seen.add(e.request_id)
        arr = (native.StepEntryC * len(entries))()
        keep = [arr]
        wanted = 0
        for i, e in enumerate(entries):
            toks = np.ascontiguousarray(np.asarray(e.tokens, dtype=np.int64))
            if toks.size and (toks.min() < -2**31 or toks.max() >= 2**31):
                raise StepError(f"request {e.request_id!r}: a token id does not fit 32 bits")
            toks = toks.astype(np.int32)
            want = np.ascontiguousarray(np.asarray(list(e.want), dtype=np.int32))
            keep.append((toks, want))
            arr[i].request = self._id(e.request_id)
            arr[i].tokens = toks.ctypes.data_as(POINTER(c_int32))
            arr[i].n_tokens = int(toks.size)
            arr[i].want = want.ctypes.data_as(POINTER(c_int32))
            arr[i].n_want = int(want.size)
            wanted += int(want.size)
        return native.StepBatchC(arr, len(entries)), keep, wanted

    # ---- timing on the device (the benchmark's) ------------------------------------------------------------------
    def time_step(self, entries: Sequence[StepEntry]) -> float:
        """Run one batch between two CUDA events on the engine's stream; returns its milliseconds.  The logits stay
        on the device."""
        batch, keep, _ = self._batch(list(entries))
        ms = ctypes.c_double(0.0)
        native.check(native.lib().qe_time_step(self._handle, ctypes.byref(batch), ctypes.byref(ms)))
        return ms.value

    def time_decode_steps(self, request_ids: Sequence, tokens, warmup: int, steps: int, sample: bool = True):
        """``warmup + steps`` decode steps of the given live requests: ``tokens[i][k]`` is what request i is fed in
        step k (host ids in every step); with ``sample`` every step's logits go through the greedy sampling kernel and
        the ids are copied to the host.  Returns (milliseconds per step over the last ``steps``, launcher calls)."""
        n = len(request_ids)
        ids = (ctypes.c_longlong * n)(*[self._id(r) for r in request_ids])
        toks = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32).reshape(n, warmup + steps))
        ms, launches = ctypes.c_double(0.0), ctypes.c_longlong(0)
        native.check(native.lib().qe_time_decode_steps(self._handle, ids, n, toks.ctypes.data_as(POINTER(c_int32)), warmup, steps,
                                                       int(sample), ctypes.byref(ms), ctypes.byref(launches)))
        return ms.value, launches.value

    # ---- a look inside ----------------------------------------------------------------------------------------
    def info(self) -> dict:
        """Free and total pages per group, the groups' entries, cache needs per run-order entry, views, graphs."""
        return native.answer(native.lib().qe_engine_info(self._handle))

    def free_pages(self) -> List[int]:
        return self.info()["free_pages"]

    def total_pages(self) -> List[int]:
        return self.info()["total_pages"]

    def check_cache(self) -> None:
        """Raise unless no page is lost, held twice or free while held."""
        native.check(native.lib().qe_engine_cache_check(self._handle))

    def set_layer_dump(self, fn) -> None:
        """``fn(entry, residual [rows, width] float32)`` after every run-order entry of the following steps
        (None: off).  Graphs are not replayed while it is set."""
        if fn is None:
            self._dump_cb = None
            native.check(native.lib().qe_engine_set_layer_dump(self._handle, native.LAYER_DUMP_CB(), None))
            return

        def trampoline(user, entry, ptr, rows, width):
            fn(entry, np.ctypeslib.as_array(ptr, shape=(rows, width)).copy())

        self._dump_cb = native.LAYER_DUMP_CB(trampoline)
        native.check(native.lib().qe_engine_set_layer_dump(self._handle, self._dump_cb, None))


__all__ = ["Engine", "StepEntry", "StepStats", "StepError", "OutOfPages", "OutOfSlots", "KernelError"]
