"""The Python entry point: a thin layer over the C library (``api/inference.h``), one method per C function.

Names and meanings follow the C functions with the ``inference_`` prefix dropped, which in turn follow the
reference's C API (src/inference.h there): ``load_model`` (:40), ``kv_cache_init`` (:115), ``set_seed`` (:120),
``reset`` / ``n_past`` (:177-178), ``prefill`` (:183), ``prefill_logits`` (:197), ``decode_token`` (:203),
``generate_ex`` (:223), ``GenOptions`` and ``gen_default_options`` (:244-264), ``generate_stream`` (:275),
``seq_new / seq_select / seq_current / seq_free`` (:284-287), ``stream_begin / stream_step / stream_step_batch``
(:297-317), ``get_logits`` (:459), ``n_ctx / vocab_size / hidden_size / model_name`` (:462-466); error codes
(:18-30) come as :class:`InferenceError`, stop reasons (:229-236) as strings.  There is no tokenizer: prompts and
results are token ids.  Beyond the reference: ``generate`` runs many prompts at once through the request queue
(prompt portions and decode rows share batches), and ``stream_run`` takes many steps with one call.
"""
from __future__ import annotations

import ctypes
import json
from ctypes import POINTER, byref, c_float, c_int, c_int32
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import numpy as np

from . import native
from .native import InferenceError
from .sampling import SamplerParams

OK, ERR_INVALID_ARG, ERR_OUT_OF_MEMORY, ERR_MODEL_LOAD, ERR_KV_CACHE = 0, -1, -2, -3, -4
ERR_KERNEL_LAUNCH, ERR_INVALID_STATE, ERR_NOT_IMPLEMENTED, ERR_CONTEXT_FULL, ERR_CANCELLED = -6, -7, -8, -9, -10

STOP_REASONS = ("none", "eog", "max_tokens", "stop_string", "callback", "context_full", "cancelled")
STOP_NONE, STOP_EOG, STOP_MAX_TOKENS, STOP_STRING, STOP_CALLBACK, STOP_CONTEXT_FULL, STOP_CANCELLED = STOP_REASONS


def strerror(code: int) -> str:
    return native.lib().inference_strerror(code).decode()


@dataclass
class GenOptions:
    """``inference_gen_options``."""
    sampler: SamplerParams = field(default_factory=SamplerParams)
    max_new_tokens: int = 256
    ignore_eog: bool = False
    reuse_prefix: bool = False
    on_token: Optional[Callable] = None      # (user, token, text, text_len) -> nonzero to stop
    user: object = None
    prefill_chunk: int = 0

    def to_c(self, keep: list) -> native.GenOptionsC:
        c = native.lib().inference_gen_default_options()
        c.sampler = self.sampler.to_c()
        c.max_new_tokens = self.max_new_tokens
        c.ignore_eog = int(self.ignore_eog)
        c.reuse_prefix = int(self.reuse_prefix)
        c.prefill_chunk = self.prefill_chunk
        if self.on_token is not None:
            fn, user = self.on_token, self.user

            def trampoline(_user, token, _text, _len):
                return int(bool(fn(user, token, "", 0)))

            cb = native.TOKEN_CB(trampoline)
            keep.append(cb)
            c.on_token = cb
        return c


def gen_default_options() -> GenOptions:
    return GenOptions(sampler=SamplerParams.defaults())


class Stream:
    """Step-wise generation on one sequence (``inference_stream_t``)."""

    def __init__(self, model: "Model", handle, keep):
        self.model, self._h, self._keep = model, handle, keep
        self.emitted: List[int] = []
        self.reason = STOP_NONE
        self.done = False

    @property
    def seq(self) -> int:
        return native.lib().inference_stream_seq(self._h)

    def free(self) -> None:
        if self._h:
            native.lib().inference_stream_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Model:
    def __init__(self, handle, model_dir: Optional[str] = None):
        self._h = handle
        self.model_dir = model_dir

    def free(self) -> None:
        if self._h:
            native.lib().inference_free_model(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    # ---- set-up ------------------------------------------------------------------------------------
    def kv_cache_init(self, n_ctx: int, max_sequences: int = 4, page_size: int = 16, kv_tokens: Optional[int] = None,
                      **engine_options) -> int:
        """A cache for sequences of up to ``n_ctx`` tokens.  The pool holds ``kv_tokens`` tokens in all (default:
        ``max_sequences`` full contexts).  ``engine_options``: poison_cache, cuda_graphs, num_pages,
        max_batch_tokens, prefill_chunk, run_ahead, step (kernel choices)."""
        if n_ctx < 1:
            raise InferenceError("n_ctx must be positive", ERR_INVALID_ARG)
        native.ensure_libraries_for(self._h)
        native.check(native.lib().inference_kv_cache_init_ex(self._h, n_ctx, max_sequences, page_size, kv_tokens or 0,
                                                             json.dumps(engine_options).encode()))
        return OK

    def kv_cache_free(self) -> None:
        native.lib().inference_kv_cache_free(self._h)

    def synchronize(self) -> None:
        """Wait until everything launched so far is done (raises if a kernel reported giving up on a wait)."""
        native.check(native.lib().inference_synchronize(self._h))

    def set_eog_tokens(self, ids: Sequence[int]) -> None:
        """The end-of-generation token ids (by default those of the model's configuration)."""
        native.check(native.lib().inference_set_eog_tokens(self._h, native.int32_array(list(ids)), len(ids)))

    def sequence_length_in_cache(self, seq: int) -> int:
        """Tokens of sequence ``seq`` whose keys are in the cache (the last generated token is fed by the next call)."""
        return native.lib().engine_request_length(self._h, seq)

    def set_seed(self, seed: int) -> None:
        native.lib().inference_set_seed(self._h, int(seed))

    def set_prefill_batch(self, n: int) -> None:
        native.lib().inference_set_prefill_batch(self._h, int(n))

    # ---- facts -------------------------------------------------------------------------------------
    def n_ctx(self) -> int:
        return native.lib().inference_n_ctx(self._h)

    def vocab_size(self) -> int:
        return native.lib().inference_vocab_size(self._h)

    def hidden_size(self) -> int:
        return native.lib().inference_hidden_size(self._h)

    def max_position(self) -> int:
        return native.lib().inference_max_position(self._h)

    def model_name(self) -> str:
        return native.lib().inference_model_name(self._h).decode()

    def batch_size(self) -> int:
        return native.lib().inference_batch_size(self._h)

    def engine_info(self) -> dict:
        return native.answer(native.lib().qe_engine_info(self._h))

    # ---- sequences ---------------------------------------------------------------------------------
    def seq_new(self) -> int:
        return native.lib().inference_seq_new(self._h)

    def seq_select(self, seq: int) -> int:
        return native.check(native.lib().inference_seq_select(self._h, seq))

    def seq_current(self) -> int:
        return native.lib().inference_seq_current(self._h)

    def seq_free(self, seq: int) -> int:
        return native.check(native.lib().inference_seq_free(self._h, seq))

    def reset(self) -> None:
        """Start the current sequence anew (position 0)."""
        native.lib().inference_reset(self._h)

    def n_past(self) -> int:
        return native.lib().inference_n_past(self._h)

    # ---- forward passes ----------------------------------------------------------------------------
    def prefill(self, tokens: Sequence[int]) -> int:
        arr = native.int32_array(list(tokens))
        return native.check(native.lib().inference_prefill(self._h, arr, len(tokens)))

    def prefill_logits(self, tokens: Sequence[int]) -> np.ndarray:
        """Like :meth:`prefill`, and returns the logits after every one of the tokens, float32 [n, vocab]."""
        arr = native.int32_array(list(tokens))
        out = np.empty((len(tokens), self.vocab_size()), dtype=np.float32)
        native.check(native.lib().inference_prefill_logits(self._h, arr, len(tokens), out.ctypes.data_as(POINTER(c_float))))
        return out

    def decode_token(self, token_id: int) -> int:
        """One token at position n_past; returns the greedy next token."""
        nxt = c_int(0)
        native.check(native.lib().inference_decode_token(self._h, int(token_id), byref(nxt)))
        return nxt.value

    def get_logits(self) -> np.ndarray:
        """Logits of the last token of the current sequence (float32 [vocab])."""
        out = np.empty(self.vocab_size(), dtype=np.float32)
        native.check(native.lib().inference_get_logits(self._h, None, out.ctypes.data_as(POINTER(c_float))))
        return out

    # ---- generation --------------------------------------------------------------------------------
    def generate_ex(self, prompt_ids: Sequence[int], max_new_tokens: int, params: Optional[SamplerParams] = None) -> List[int]:
        """New sequence, prefill, then sample up to ``max_new_tokens`` (stops early at EOS, which is not returned, or
        when the context is full)."""
        arr = native.int32_array(list(prompt_ids))
        out = (c_int32 * max(max_new_tokens, 1))()
        n = c_int(0)
        c = params.to_c() if params is not None else None
        native.check(native.lib().inference_generate_ex(self._h, arr, len(prompt_ids), max_new_tokens,
                                                        byref(c) if c is not None else None, out, byref(n)))
        return list(out[:n.value])

    def generate_stream(self, prompt_ids: Sequence[int], options: Optional[GenOptions] = None):
        """Continue the current sequence with ``prompt_ids`` and generate.  Returns (tokens, stop reason)."""
        opts = options or gen_default_options()
        keep: list = []
        c = opts.to_c(keep)
        arr = native.int32_array(list(prompt_ids))
        cap = max(opts.max_new_tokens, 1)
        out = (c_int32 * cap)()
        n, reason = c_int(0), c_int(0)
        native.check(native.lib().inference_generate_stream(self._h, arr, len(prompt_ids), byref(c), out, cap, byref(n),
                                                            byref(reason)))
        return list(out[:min(n.value, cap)]), STOP_REASONS[reason.value]

    def last_prompt_stats(self):
        a, b = c_int(0), c_int(0)
        native.lib().inference_last_prompt_stats(self._h, byref(a), byref(b))
        return a.value, b.value

    def stream_begin(self, prompt_ids: Sequence[int], options: Optional[GenOptions] = None) -> Stream:
        opts = options or gen_default_options()
        keep: list = []
        c = opts.to_c(keep)
        arr = native.int32_array(list(prompt_ids))
        h = native.lib().inference_stream_begin(self._h, arr, len(prompt_ids), byref(c))
        if not h:
            raise native.last_error()
        return Stream(self, h, keep)

    def stream_step(self, stream: Stream):
        """One step of one stream: (going, token); token is None for a step that only prefilled."""
        return self.stream_step_batch([stream])[0]

    @staticmethod
    def _settle(streams, results, n, step):
        row = []
        for i, st in enumerate(streams):
            r = results[step * n + i]
            tok = r.token if r.token >= 0 else None
            if tok is not None:
                st.emitted.append(tok)
            if r.rc == 0 and not st.done:
                st.done, st.reason = True, STOP_REASONS[r.reason]
            row.append((r.rc == 1, tok))
        return row

    def stream_step_batch(self, streams: Sequence[Stream]):
        """One step of each stream with ONE pass for all: prompt portions and decode rows share the batch.  Returns
        [(going, token)] in the order of ``streams``."""
        n = len(streams)
        handles = (ctypes.c_void_p * n)(*[s._h for s in streams])
        results = (native.StepResultC * n)()
        native.check(native.lib().inference_stream_step_batch(handles, n, results))
        return self._settle(streams, results, n, 0)

    def stream_run(self, streams: Sequence[Stream], n_steps: int):
        """Up to ``n_steps`` steps of every stream: the list of what :meth:`stream_step_batch` would return step by
        step (shorter when every stream ends earlier).  While all live streams are decoding with device samplers a
        step is launched with the token ids the step before left on the device, before the host has read them."""
        n = len(streams)
        n_steps = min(n_steps, 1 << 16)
        handles = (ctypes.c_void_p * n)(*[s._h for s in streams])
        results = (native.StepResultC * (n * n_steps))()
        taken = native.check(native.lib().inference_stream_run(handles, n, n_steps, results))
        return [self._settle(streams, results, n, k) for k in range(taken)]

    # ---- many prompts at once ------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16, temperature: float = 0.0, seed: int = 0,
                 params: Optional[SamplerParams] = None, ignore_eos: bool = True) -> List[List[int]]:
        """Generate for all ``prompts`` through the request queue (the scheduler admits them, cuts their prompts into
        portions under the token budget and preempts when pages run out); returns the new tokens of each prompt.
        Prompt i samples with seed ``seed + i``."""
        L = native.lib()
        ids = []
        for i, p in enumerate(prompts):
            sp = params or (SamplerParams.greedy() if temperature <= 0 else SamplerParams.pure_temperature(temperature))
            sp = SamplerParams(**{**sp.__dict__, "seed": seed + i})
            opts = native.RequestOptionsC(sp.to_c(), max_new_tokens, int(ignore_eos))
            arr = native.int32_array(list(p))
            ids.append(native.check(L.inference_request_add(self._h, arr, len(p), byref(opts))))
        while native.check(L.inference_step(self._h)) > 0:
            pass
        out, self.last_stop_reasons = [], []
        for rid in ids:
            buf = (c_int32 * max(max_new_tokens, 1))()
            n, fin, reason = c_int(0), c_int(0), c_int(0)
            native.check(L.inference_request_poll(self._h, rid, buf, max_new_tokens, byref(n), byref(fin), byref(reason)))
            out.append(list(buf[:min(n.value, max_new_tokens)]))
            self.last_stop_reasons.append(STOP_REASONS[reason.value])
            native.check(L.inference_request_free(self._h, rid))
        return out


def load_model(path: str, dtype: str = "bfloat16", options: Optional[dict] = None) -> Model:
    """``inference_load_model``: read config.json and the safetensors of ``path`` onto the device."""
    h = native.lib().inference_load_model_ex(str(path).encode(), dtype.encode(), json.dumps(options or {}).encode())
    if not h:
        raise native.last_error()
    return Model(h, str(path))


def load_model_random(config, seed: int, dtype: str = "bfloat16", std: float = 0.02, scale_low: float = 1.0,
                      scale_high: float = 1.0, options: Optional[dict] = None) -> Model:
    """A model of ``config`` (a typed configuration, a dict or config.json text) with seeded random weights made on
    the device: the values :func:`purhie_b200.weights.write_random_model` stores for the same seed."""
    from .weights import _config_json
    h = native.lib().inference_load_model_random_ex(_config_json(config), int(seed), dtype.encode(), float(std),
                                                    float(scale_low), float(scale_high), json.dumps(options or {}).encode())
    if not h:
        raise native.last_error()
    return Model(h)
