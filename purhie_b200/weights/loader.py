"""Loading a model's tensors by name, with one error for everything that does not fit.

Every part of a model announces the tensors it needs as :class:`TensorSpec` (name, shape, role).  The
loader checks the whole folder against the whole list before it copies anything and raises one
:class:`WeightError` that lists missing tensors, unexpected tensors and wrong shapes together.  The
reference binds tensors one at a time and stops at the first problem (``bind_weight``
src/inference.cpp:362-389, ``bind_norm`` :392-407, ``check_shape`` :426-430, "missing tensor" :365).

Storage on the device:
  * role ``matrix``: the compute dtype.  With compute dtype bfloat16 a tensor stored as BF16 stays
    BF16, F16 is converted to BF16, and a tensor stored in 32-bit stays in 32-bit (the linear part then
    multiplies it with the 32-bit kernel).  With compute dtype float32 everything is widened to float32.
  * role ``vector`` (norm weights, biases): float32 always; widening BF16 is exact.
  * role ``table`` (integer tables): int32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, Tuple

import torch

from .safetensors_io import SafetensorsFolder

MATRIX, VECTOR, TABLE = "matrix", "vector", "table"


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    role: str = MATRIX
    init: str = "normal"          # how random weights fill it: "normal" (mean 0) or "scale" (around 1)


class WeightError(ValueError):
    """The tensors of a model folder do not fit the model.  Lists everything that is wrong."""

    def __init__(self, model_dir: str, missing, unexpected, wrong_shape, wrong_type=()):
        self.model_dir = model_dir
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)          # (name, got, expected)
        self.wrong_type = list(wrong_type)            # (name, got dtype name, role)
        lines = [f"{model_dir}: the tensors do not fit the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, got, role in self.wrong_type:
            lines.append(f"  wrong type: {name} is stored as {got}, which a {role} cannot be")
        super().__init__("\n".join(lines))


_FLOATS = (torch.float64, torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def device_dtype(stored: torch.dtype, role: str, compute_dtype: torch.dtype) -> torch.dtype:
    """The dtype a tensor has on the device, given how it is stored and what it is for."""
    if role == TABLE:
        return torch.int32
    if role == VECTOR or compute_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_folder(folder: SafetensorsFolder, expected: Dict[str, TensorSpec], ignore: Iterable[str] = ()) -> None:
    ignore = set(ignore)
    present = set(folder.names())
    missing = [n for n in expected if n not in present]
    unexpected = sorted(n for n in present if n not in expected and n not in ignore)
    wrong_shape, wrong_type = [], []
    for name, spec in expected.items():
        if name not in present:
            continue
        e = folder.entries[name]
        if tuple(e.shape) != tuple(spec.shape):
            wrong_shape.append((name, e.shape, spec.shape))
        ok = e.dtype in _INTS if spec.role == TABLE else e.dtype in _FLOATS
        if not ok:
            wrong_type.append((name, e.dtype_name, spec.role))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(folder.model_dir, missing, unexpected, wrong_shape, wrong_type)


def load_tensors(model_dir: str, expected: Dict[str, TensorSpec], compute_dtype: torch.dtype, device,
                 ignore: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Check ``model_dir`` against ``expected`` and return the tensors on ``device``."""
    folder = SafetensorsFolder(model_dir)
    try:
        check_folder(folder, expected, ignore)
        out: Dict[str, torch.Tensor] = {}
        for name, spec in expected.items():
            src = folder.tensor(name)
            dt = device_dtype(src.dtype, spec.role, compute_dtype)
            t = src.to(device=device).to(dtype=dt).contiguous()
            if t.data_ptr() == src.data_ptr():
                t = t.clone()                       # never hand out a view of the file mapping
            out[name] = t
        return out
    finally:
        folder.close()
