"""The host library (libqengine.so) as Python sees it: loaded with ctypes, one signature per C function.

Everything that computes or keeps books lives in the C++ library (configuration, weights, parts, cache manager,
step function, scheduler, samplers, the C API of ``api/inference.h``); the Python packages beside this module are
thin faces over it.  An error code from the library becomes the Python exception of the same kind, with the
library's text.  The library and the kernel libraries it opens are compiled on first use (``csrc/build.py``).
"""
from __future__ import annotations

import ctypes
import json
from ctypes import (POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_longlong, c_uint, c_uint64, c_void_p)

from .csrc.build import build_dir, build_library, load_library


class InferenceError(RuntimeError):
    """An error from the library; ``code`` is the C API's error code."""

    code = -7

    def __init__(self, message: str = "", code: int = None):
        if code is not None:
            self.code = code
        super().__init__(message)


class ConfigError(InferenceError, ValueError):
    """A ``config.json`` that cannot be used: a missing key, a wrong type, an unsupported option."""
    code = -3


class SafetensorsError(InferenceError, ValueError):
    """A file that is not a well-formed safetensors file."""
    code = -3


class WeightError(InferenceError, ValueError):
    """The tensors of a model folder do not fit the model.  Lists everything that is wrong."""
    code = -3

    def __init__(self, message="", code=None, details=None):
        super().__init__(message, code)
        d = details or {}
        self.missing = list(d.get("missing", []))
        self.unexpected = list(d.get("unexpected", []))
        self.wrong_shape = list(d.get("wrong_shape", []))
        self.wrong_type = list(d.get("wrong_type", []))


class StepError(InferenceError, ValueError):
    """A batch that cannot be run: an unknown token id, a position past the model's limit, a request twice."""
    code = -1


class OutOfPages(InferenceError):
    """The pool has fewer free pages than were asked for.  Nothing was taken."""
    code = -9


class OutOfSlots(InferenceError):
    """Every per-request state slot is in use."""
    code = -4


class KernelError(InferenceError):
    """A kernel launcher refused its arguments, a launch failed, or a kernel gave up on a wait."""
    code = -6


class CheckError(InferenceError, AssertionError):
    """The bookkeeping found itself inconsistent."""
    code = -7


_KINDS = {c.__name__: c for c in (ConfigError, SafetensorsError, WeightError, StepError, OutOfPages, OutOfSlots,
                                  KernelError, CheckError)}


class SamplerParamsC(ctypes.Structure):
    _fields_ = [("temperature", c_float), ("top_k", c_int), ("top_p", c_float), ("min_p", c_float),
                ("repeat_penalty", c_float), ("repeat_last_n", c_int), ("seed", c_uint64), ("presence_penalty", c_float)]


TOKEN_CB = ctypes.CFUNCTYPE(c_int, c_void_p, c_int32, c_char_p, c_int)
LAYER_DUMP_CB = ctypes.CFUNCTYPE(None, c_void_p, c_int, POINTER(c_float), c_int, c_int)


class GenOptionsC(ctypes.Structure):
    _fields_ = [("sampler", SamplerParamsC), ("max_new_tokens", c_int), ("stop_strings", c_void_p), ("n_stop_strings", c_int),
                ("ignore_eog", c_int), ("reuse_prefix", c_int), ("checkpoint_tail", c_int), ("on_token", TOKEN_CB),
                ("user", c_void_p), ("prefill_chunk", c_int)]


class StepResultC(ctypes.Structure):
    _fields_ = [("token", c_int32), ("text", c_char_p), ("text_len", c_int), ("reason", c_int), ("rc", c_int)]


class RequestOptionsC(ctypes.Structure):
    _fields_ = [("sampler", SamplerParamsC), ("max_new_tokens", c_int), ("ignore_eog", c_int)]


class StepEntryC(ctypes.Structure):
    _fields_ = [("request", c_longlong), ("tokens", POINTER(c_int32)), ("n_tokens", c_int), ("want", POINTER(c_int32)),
                ("n_want", c_int)]


class StepBatchC(ctypes.Structure):
    _fields_ = [("entries", POINTER(StepEntryC)), ("n_entries", c_int)]


class StepOutputC(ctypes.Structure):
    _fields_ = [("logits", POINTER(c_float)), ("logits_capacity", c_longlong), ("n_rows", c_int), ("vocab_size", c_int),
                ("tokens", c_int), ("prompt_rows", c_int), ("decode_rows", c_int), ("replayed_graph", c_int)]


_P = c_void_p
_SIGNATURES = {
    # name: (restype, argtypes)
    "inference_strerror": (c_char_p, [c_int]),
    "inference_get_last_error": (c_char_p, []),
    "qe_last_error_kind": (c_char_p, []),
    "sampler_default_params": (SamplerParamsC, []),
    "sampler_create": (_P, [POINTER(SamplerParamsC)]),
    "sampler_free": (None, [_P]),
    "sampler_sample": (c_int, [_P, POINTER(c_float), c_int]),
    "sampler_accept": (None, [_P, c_int]),
    "sampler_reset": (None, [_P]),
    "inference_load_model": (_P, [c_char_p]),
    "inference_load_model_ex": (_P, [c_char_p, c_char_p, c_char_p]),
    "inference_load_model_random": (_P, [c_char_p, c_uint64, c_char_p]),
    "inference_load_model_random_ex": (_P, [c_char_p, c_uint64, c_char_p, c_double, c_double, c_double, c_char_p]),
    "inference_write_random_model": (c_int, [c_char_p, c_char_p, c_uint64, c_double, c_double, c_double, c_char_p]),
    "inference_free_model": (None, [_P]),
    "inference_kv_cache_init": (c_int, [_P, c_int]),
    "inference_kv_cache_init_ex": (c_int, [_P, c_int, c_int, c_int, c_longlong, c_char_p]),
    "inference_kv_cache_free": (None, [_P]),
    "inference_synchronize": (c_int, [_P]),
    "inference_set_eog_tokens": (c_int, [_P, POINTER(c_int32), c_int]),
    "inference_set_seed": (None, [_P, c_uint]),
    "inference_set_prefill_batch": (None, [_P, c_int]),
    "inference_reset": (None, [_P]),
    "inference_n_past": (c_int, [_P]),
    "inference_prefill": (c_int, [_P, POINTER(c_int32), c_int]),
    "inference_prefill_logits": (c_int, [_P, POINTER(c_int32), c_int, POINTER(c_float)]),
    "inference_decode_token": (c_int, [_P, c_int, POINTER(c_int)]),
    "inference_get_logits": (c_int, [_P, POINTER(c_int), POINTER(c_float)]),
    "inference_generate_ex": (c_int, [_P, POINTER(c_int32), c_int, c_int, POINTER(SamplerParamsC), POINTER(c_int32),
                                      POINTER(c_int)]),
    "inference_gen_default_options": (GenOptionsC, []),
    "inference_generate_stream": (c_int, [_P, POINTER(c_int32), c_int, POINTER(GenOptionsC), POINTER(c_int32), c_int,
                                          POINTER(c_int), POINTER(c_int)]),
    "inference_last_prompt_stats": (c_int, [_P, POINTER(c_int), POINTER(c_int)]),
    "inference_seq_new": (c_int, [_P]),
    "inference_seq_select": (c_int, [_P, c_int]),
    "inference_seq_current": (c_int, [_P]),
    "inference_seq_free": (c_int, [_P, c_int]),
    "inference_stream_begin": (_P, [_P, POINTER(c_int32), c_int, POINTER(GenOptionsC)]),
    "inference_stream_step": (c_int, [_P, POINTER(c_int32), POINTER(c_char_p), POINTER(c_int), POINTER(c_int)]),
    "inference_stream_tokens": (c_int, [_P]),
    "inference_stream_seq": (c_int, [_P]),
    "inference_stream_free": (None, [_P]),
    "inference_stream_step_batch": (c_int, [POINTER(_P), c_int, POINTER(StepResultC)]),
    "inference_stream_run": (c_int, [POINTER(_P), c_int, c_int, POINTER(StepResultC)]),
    "inference_request_add": (c_longlong, [_P, POINTER(c_int32), c_int, POINTER(RequestOptionsC)]),
    "inference_step": (c_int, [_P]),
    "inference_request_poll": (c_int, [_P, c_longlong, POINTER(c_int32), c_int, POINTER(c_int), POINTER(c_int),
                                       POINTER(c_int)]),
    "inference_request_cancel": (c_int, [_P, c_longlong]),
    "inference_request_free": (c_int, [_P, c_longlong]),
    "engine_request_add": (c_int, [_P, c_longlong]),
    "engine_request_release": (c_int, [_P, c_longlong]),
    "engine_request_length": (c_int, [_P, c_longlong]),
    "engine_step": (c_int, [_P, POINTER(StepBatchC), POINTER(StepOutputC)]),
    "inference_n_ctx": (c_int, [_P]),
    "inference_batch_size": (c_int, [_P]),
    "inference_model_name": (c_char_p, [_P]),
    "inference_vocab_size": (c_int, [_P]),
    "inference_hidden_size": (c_int, [_P]),
    "inference_max_position": (c_int, [_P]),
    # for tests and tools
    "qe_config_read": (c_char_p, [c_char_p]),
    "qe_config_load": (c_char_p, [c_char_p]),
    "qe_registered_architectures": (c_char_p, []),
    "qe_registered_parts": (c_char_p, [c_char_p]),
    "qe_model_spec": (c_char_p, [c_char_p]),
    "qe_expected_tensors": (c_char_p, [c_char_p]),
    "qe_check_model_folder": (c_int, [c_char_p]),
    "qe_weight_error_details": (c_char_p, []),
    "qe_safetensors_list": (c_char_p, [c_char_p]),
    "qe_safetensors_read": (c_longlong, [c_char_p, c_char_p, c_void_p, c_longlong]),
    "qe_device_dtype": (c_char_p, [c_char_p, c_char_p, c_char_p]),
    "qe_random_tensor": (c_int, [c_char_p, c_char_p, c_longlong, c_uint64, c_double, c_double, c_double, POINTER(c_float)]),
    "qe_sampler_device_mode": (c_char_p, [_P]),
    "qe_sampler_chain_max_k": (c_int, []),
    "qe_sampler_uniform": (c_double, [_P]),
    "qe_sampler_chain_record": (None, [_P, c_void_p]),
    "qe_plan_gemm": (c_char_p, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "qe_sampler_histogram": (c_int, [_P, POINTER(c_float), c_int, c_longlong, POINTER(c_longlong)]),
    "qe_model_required_libraries": (c_char_p, [_P]),
    "qe_engine_info": (c_char_p, [_P]),
    "qe_engine_cache_check": (c_int, [_P]),
    "qe_engine_set_error_word": (c_int, [_P, c_int, c_int]),
    "qe_engine_set_layer_dump": (c_int, [_P, LAYER_DUMP_CB, c_void_p]),
    "qe_time_step": (c_int, [_P, POINTER(StepBatchC), POINTER(c_double)]),
    "qe_time_decode_steps": (c_int, [_P, POINTER(c_longlong), c_int, POINTER(c_int32), c_int, c_int, c_int, POINTER(c_double),
                                     POINTER(c_longlong)]),
    "qe_profile_enable": (None, [c_int]),
    "qe_profile_enabled": (c_int, []),
    "qe_profile_leave_out": (None, [c_char_p]),
    "qe_profile_report": (c_char_p, [c_int]),
    "qe_launches": (c_longlong, []),
    "qe_set_library_dir": (None, [c_char_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded host library, compiled first if need be (with the plain kernels it cannot do without)."""
    global _lib
    if _lib is None:
        build_library("core")
        handle = load_library("qengine")
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                continue                      # an optional group of hooks registers its own signatures
            fn.restype = restype
            fn.argtypes = argtypes
        handle.qe_set_library_dir(build_dir().encode())
        _lib = handle
    return _lib


def declare(name: str, restype, argtypes) -> None:
    """Give a further exported function its signature (the test hooks of other modules)."""
    fn = getattr(lib(), name)
    fn.restype = restype
    fn.argtypes = argtypes


def last_error() -> InferenceError:
    """The library's last error on this thread as the exception of its kind."""
    L = lib()
    text = (L.inference_get_last_error() or b"").decode("utf-8", "replace")
    kind = (L.qe_last_error_kind() or b"").decode()
    cls = _KINDS.get(kind, InferenceError)
    if cls is WeightError:
        try:
            details = json.loads(L.qe_weight_error_details().decode())
        except (ValueError, AttributeError):
            details = {}
        return WeightError(text, details=details)
    return cls(text)


def check(rc: int) -> int:
    """Raise the library's error when ``rc`` is negative; else return it."""
    if rc is not None and rc < 0:
        err = last_error()
        err.code = rc
        raise err
    return rc


def text(ptr) -> str:
    """A JSON or text answer from a hook; None means the call failed."""
    if ptr is None:
        raise last_error()
    return ptr.decode("utf-8")


def answer(ptr):
    return json.loads(text(ptr))


def ensure_libraries_for(model_handle) -> None:
    """Compile the kernel libraries the loaded model launches from (they are opened by the host library itself)."""
    for name in answer(lib().qe_model_required_libraries(model_handle)):
        build_library(name)


def profile_enabled() -> bool:
    return bool(lib().qe_profile_enabled())


def profile_report(reset: bool = True) -> dict:
    """Time per kernel class since the last reset: {launcher: {"calls", "ms", "bytes", "flops"}} (empty unless
    PURHIE_PROFILE=1 is in the environment or ``lib().qe_profile_enable(1)`` was called)."""
    return answer(lib().qe_profile_report(int(reset)))


def format_profile(report: dict, title: str = "forward") -> str:
    """The report as lines: per launcher its calls, milliseconds, share of the total, and GB/s and TFLOP/s where the
    launches' bytes and flops are known."""
    total = sum(v["ms"] for v in report.values()) or 1e-12
    lines = [f"[profile] {title}: {sum(v['calls'] for v in report.values())} launches, {total:.3f} ms on the device"]
    for name, v in sorted(report.items(), key=lambda kv: -kv[1]["ms"]):
        line = f"[profile]   {name:<24} {v['calls']:>7} calls {v['ms']:>10.3f} ms {100 * v['ms'] / total:>5.1f}%"
        if v["bytes"] > 0 and v["ms"] > 0:
            line += f"  {v['bytes'] / v['ms'] / 1e6:>8.1f} GB/s  {v['flops'] / v['ms'] / 1e9:>8.1f} TFLOP/s"
        lines.append(line)
    return "\n".join(lines)


def int32_array(values):
    n = len(values)
    arr = (c_int32 * max(n, 1))()
    if n:
        arr[:n] = values
    return arr
