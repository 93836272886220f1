"""Layers put together from parts: mixer, feed-forward, norm, position encoding, block arrangement.

The parts, their interfaces and the registries are C++ (``parts/parts.h`` is the whole contract; the parts this
library brings are the ``.cpp`` files beside it).  A part defined elsewhere derives from one of the families in
that header and registers a factory: :func:`build_plugin` compiles such a source file against the library and
:func:`load_plugin` opens it, which runs its ``qe_plugin_init``.  :class:`PartProbe` builds ONE part from
``{kind, params}`` and runs it alone on the device, for tests of a part beside its plain reference.
"""
from __future__ import annotations

import ctypes
import json
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_longlong, c_uint64, c_void_p
from typing import Dict, List, Optional, Sequence

import numpy as np

from .. import native
from ..config import registered_parts
from ..csrc.build import build_plugin

_plugins = {}
_DECLARED = False


def load_plugin(path: str) -> None:
    """Open a shared object of parts (made by :func:`build_plugin`) and run its ``qe_plugin_init``, which registers
    the parts, arrangements and architectures it brings."""
    native.lib()                                    # the host library first: the plugin is linked against it
    handle = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    init = getattr(handle, "qe_plugin_init", None)
    if init is not None:
        init.restype = ctypes.c_int
        if init() != 0:
            raise native.InferenceError(f"{path}: qe_plugin_init failed")
    _plugins[path] = handle


def unload_plugin(path: str) -> None:
    """Run the plugin's ``qe_plugin_exit`` (which takes its registrations back); the object stays mapped."""
    handle = _plugins.pop(path, None)
    if handle is not None and getattr(handle, "qe_plugin_exit", None) is not None:
        handle.qe_plugin_exit()


def _lib():
    global _DECLARED
    L = native.lib()
    if not _DECLARED:
        P, F = c_void_p, POINTER(c_float)
        for name, res, args in [
            ("qe_part_create", P, [c_char_p, c_char_p, c_char_p, c_char_p]), ("qe_part_free", None, [P]),
            ("qe_part_tensor_specs", c_char_p, [P]), ("qe_part_bind_folder", c_int, [P, c_char_p]),
            ("qe_part_bind_random", c_int, [P, c_uint64, c_double, c_double, c_double]), ("qe_part_cache_need", c_char_p, [P]),
            ("qe_part_norm", c_int, [P, F, F, c_int, c_int, F, F]), ("qe_part_position_info", c_char_p, [P]),
            ("qe_part_position_table", c_int, [P, F, c_longlong]), ("qe_part_embedding", c_int, [P, POINTER(c_int32), c_int, c_int, F]),
            ("qe_part_head", c_int, [P, F, c_int, c_int, F]), ("qe_part_feed_forward", c_int, [P, F, c_int, c_int, F]),
            ("qe_part_mixer_cache", c_int, [P, c_int, c_int, c_int, c_int]), ("qe_part_mixer_add_request", c_int, [P, c_longlong]),
            ("qe_part_mixer_release", c_int, [P, c_longlong]),
            ("qe_part_mixer_step", c_int, [P, POINTER(c_longlong), POINTER(c_int), c_int, F, c_int, F]),
        ]:
            native.declare(name, res, args)
        _DECLARED = True
    return L


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(POINTER(c_float))


class PartProbe:
    """One part, built through the registries and run alone.  ``family``: norm, position, mixer, feed_forward,
    embedding, head.  Inputs and results are float32 NumPy arrays on the host (inputs are rounded to the compute
    dtype where the part takes that dtype; split partial sums are added up)."""

    def __init__(self, family: str, kind: str, params: dict, dtype: str = "float32", options: Optional[dict] = None):
        native.build_library("core")
        if dtype == "bfloat16":
            native.build_library("flash")
            native.build_library("gemm100")
        spec = json.dumps({"kind": kind, "params": params}).encode()
        self._h = _lib().qe_part_create(family.encode(), spec, dtype.encode(), json.dumps(options or {}).encode())
        if not self._h:
            raise native.last_error()
        self.family, self.dtype = family, dtype

    def __del__(self):
        try:
            _lib().qe_part_free(self._h)
        except Exception:
            pass

    def tensor_specs(self) -> List[Dict]:
        return native.answer(_lib().qe_part_tensor_specs(self._h))

    def bind_folder(self, folder: str) -> None:
        """Bind to the tensors of ``folder/model.safetensors`` (tensors the part does not read are ignored)."""
        native.check(_lib().qe_part_bind_folder(self._h, str(folder).encode()))

    def bind_random(self, seed: int, std: float = 0.02, scale_low: float = 1.0, scale_high: float = 1.0) -> None:
        native.check(_lib().qe_part_bind_random(self._h, seed, std, scale_low, scale_high))

    def cache_need(self) -> Dict:
        return native.answer(_lib().qe_part_cache_need(self._h))

    # ---- families
    def norm(self, x, add=None):
        """(the stream afterwards = x + add, the normed rows)."""
        x = _f32(x)
        add = None if add is None else _f32(add)
        T, E = x.shape
        out_x, out_y = np.empty_like(x), np.empty_like(x)
        native.check(_lib().qe_part_norm(self._h, _ptr(x), _ptr(add), T, E, _ptr(out_x), _ptr(out_y)))
        return out_x, out_y

    def position_info(self) -> Dict:
        return native.answer(_lib().qe_part_position_info(self._h))

    def position_table(self) -> np.ndarray:
        info = self.position_info()
        out = np.empty((info["rows"], info["width"]), dtype=np.float32)
        native.check(_lib().qe_part_position_table(self._h, _ptr(out), out.size))
        return out

    def embedding(self, ids: Sequence[int], width: int) -> np.ndarray:
        arr = native.int32_array(list(ids))
        out = np.empty((len(ids), width), dtype=np.float32)
        native.check(_lib().qe_part_embedding(self._h, arr, len(ids), width, _ptr(out)))
        return out

    def head(self, xn, vocab: int) -> np.ndarray:
        xn = _f32(xn)
        out = np.empty((xn.shape[0], vocab), dtype=np.float32)
        native.check(_lib().qe_part_head(self._h, _ptr(xn), xn.shape[0], xn.shape[1], _ptr(out)))
        return out

    def feed_forward(self, x) -> np.ndarray:
        x = _f32(x)
        out = np.empty_like(x)
        native.check(_lib().qe_part_feed_forward(self._h, _ptr(x), x.shape[0], x.shape[1], _ptr(out)))
        return out

    # ---- a mixer and its cache
    def mixer_cache(self, page_size: int, num_pages: int, max_requests: int = 4, poison: bool = True) -> None:
        native.check(_lib().qe_part_mixer_cache(self._h, page_size, num_pages, max_requests, int(poison)))

    def add_request(self, request: int) -> None:
        native.check(_lib().qe_part_mixer_add_request(self._h, request))

    def release(self, request: int) -> None:
        native.check(_lib().qe_part_mixer_release(self._h, request))

    def mixer_step(self, segments, x) -> np.ndarray:
        """One step: ``segments`` = [(request, new rows)], ``x`` all rows [T, E] in segment order; the mixer's output
        rows [T, E]."""
        x = _f32(x)
        n = len(segments)
        reqs = (c_longlong * n)(*[s[0] for s in segments])
        rows = (c_int * n)(*[s[1] for s in segments])
        out = np.empty_like(x)
        native.check(_lib().qe_part_mixer_step(self._h, reqs, rows, n, _ptr(x), x.shape[1], _ptr(out)))
        return out


__all__ = ["PartProbe", "build_plugin", "load_plugin", "unload_plugin", "registered_parts"]
