"""Layers put together from parts: mixer, feed-forward, norm, position encoding, block arrangement.

The parts, their interfaces and the registries are C++ (``parts/parts.h`` is the whole contract; the parts this
library brings are the ``.cpp`` files beside it).  A part defined elsewhere derives from one of the families in
that header and registers a factory; :func:`load_plugin` opens a shared object that does so when it is loaded.
"""
from __future__ import annotations

import ctypes

from .. import native
from ..config import registered_parts

_plugins = []


def load_plugin(path: str) -> None:
    """Open a shared object whose static initialisers (or ``qe_plugin_init``) register parts or architectures."""
    native.lib()                                    # the host library first: the plugin links against its symbols
    handle = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    init = getattr(handle, "qe_plugin_init", None)
    if init is not None:
        init.restype = ctypes.c_int
        if init() != 0:
            raise native.InferenceError(f"{path}: qe_plugin_init failed")
    _plugins.append(handle)


__all__ = ["load_plugin", "registered_parts"]
