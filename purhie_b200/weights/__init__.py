"""Weights as Python sees them: random model folders, the tensor list of a configuration, the folder check.

The safetensors reader and writer, the one-error check, the dtype policy and the seeded generator are the host
library's (``weights/*.cpp``, ``weights/random.h``).
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass
from typing import Dict, List, Tuple, Union

from .. import native
from ..config import ModelConfig
from ..native import SafetensorsError, WeightError

MATRIX, VECTOR, TABLE = "matrix", "vector", "table"


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    role: str = MATRIX
    init: str = "normal"          # how random weights fill it: "normal" (mean 0) or "scale" (around 1)


def _config_json(config: Union[ModelConfig, Dict, str]) -> bytes:
    if isinstance(config, ModelConfig):
        return config.to_json().encode()
    if isinstance(config, dict):
        return json.dumps(config).encode()
    return str(config).encode()


def expected_tensors(config) -> Dict[str, TensorSpec]:
    """The tensors a model of this configuration reads, from its parts (no device needed)."""
    items = native.answer(native.lib().qe_expected_tensors(_config_json(config)))
    return {t["name"]: TensorSpec(t["name"], tuple(t["shape"]), t["role"], t["init"]) for t in items}


def write_random_model(model_dir: str, config, seed: int, std: float = 0.02, scale_low: float = 1.0,
                       scale_high: float = 1.0, dtype: str = "bfloat16") -> str:
    """Write ``config.json`` and ``model.safetensors`` into ``model_dir``: matrices N(0, std) stored as ``dtype``
    (bfloat16 or float32), norm weights U(scale_low, scale_high) stored as float32; every value a function of
    (seed, tensor name, index) alone.  Returns the folder."""
    native.check(native.lib().inference_write_random_model(str(model_dir).encode(), _config_json(config), int(seed),
                                                           float(std), float(scale_low), float(scale_high), dtype.encode()))
    return str(model_dir)


def check_model_folder(model_dir: str) -> None:
    """Check a folder's tensors against its own config.json; raises ONE :class:`WeightError` that lists missing and
    unexpected tensors, wrong shapes and wrong types (or :class:`SafetensorsError` / ``ConfigError``)."""
    native.check(native.lib().qe_check_model_folder(str(model_dir).encode()))


def list_tensors(model_dir: str) -> List[Dict]:
    """[{"name", "dtype", "shape", "bytes"}] of a folder, whatever shard a tensor is in."""
    return native.answer(native.lib().qe_safetensors_list(str(model_dir).encode()))


def read_tensor_bytes(model_dir: str, name: str) -> bytes:
    """One tensor's bytes as stored."""
    size = next((t["bytes"] for t in list_tensors(model_dir) if t["name"] == name), None)
    if size is None:
        raise SafetensorsError(f"{model_dir}: no tensor {name!r}")
    buf = ctypes.create_string_buffer(max(size, 1))
    native.check(native.lib().qe_safetensors_read(str(model_dir).encode(), name.encode(), buf, size))
    return buf.raw[:size]


def random_values(name: str, n: int, seed: int, init: str = "normal", std: float = 0.02, scale_low: float = 1.0,
                  scale_high: float = 1.0):
    """The first ``n`` float32 values of the tensor ``name`` under ``seed`` (a list)."""
    out = (ctypes.c_float * n)()
    native.check(native.lib().qe_random_tensor(name.encode(), init.encode(), n, seed, std, scale_low, scale_high, out))
    return list(out)


def device_dtype(stored: str, role: str, compute: str) -> str:
    """The dtype a tensor has on the device, given how it is stored and what it is for."""
    return native.text(native.lib().qe_device_dtype(stored.encode(), role.encode(), compute.encode()))


__all__ = ["MATRIX", "VECTOR", "TABLE", "TensorSpec", "WeightError", "SafetensorsError", "expected_tensors",
           "write_random_model", "check_model_folder", "list_tensors", "read_tensor_bytes", "random_values", "device_dtype"]
