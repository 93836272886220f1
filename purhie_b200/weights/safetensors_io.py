"""Reading and writing safetensors files through a memory mapping.

File layout: an 8-byte little-endian header length, a JSON header that maps tensor names to
``{"dtype", "shape", "data_offsets"}`` with offsets relative to the end of the header, then the data.
A model folder holds either ``model.safetensors`` or ``model.safetensors.index.json`` whose
``weight_map`` names the shard of every tensor.  The reference's reader does the same over an mmap
(src/safetensors_mmap.cpp:213-256 for a shard: header longer than the file :225, bad dtype / shape
entries :236-239, tensor outside the file :246, duplicate across shards :250, ``__metadata__`` skipped
:233; :260-287 for a folder, shards in order of first appearance :269-279).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors file."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    dtype_name: str
    shape: Tuple[int, ...]
    file: "SafetensorsFile"
    begin: int
    end: int


class SafetensorsFile:
    """One mapped ``.safetensors`` file.  Tensors are views of the mapping (no copy until used)."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a header length ({size} bytes)")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if 8 + hlen > size:
            raise SafetensorsError(f"{path}: header of {hlen} bytes is longer than the file ({size} bytes)")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.data_start = 8 + hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dname, shape, (b, e) = info["dtype"], info["shape"], info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: tensor {name!r} has a malformed entry") from None
            if dname not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dname!r}")
            if not isinstance(shape, list) or any(isinstance(s, bool) or not isinstance(s, int) or s < 0 for s in shape):
                raise SafetensorsError(f"{path}: tensor {name!r} has a malformed shape {shape!r}")
            dtype, width = _DTYPES[dname]
            n = 1
            for s in shape:
                n *= s
            if not (isinstance(b, int) and isinstance(e, int)) or b < 0 or e < b or e - b != n * width:
                raise SafetensorsError(f"{path}: tensor {name!r}: offsets [{b}, {e}) do not match shape {shape} "
                                       f"of {dname}")
            if self.data_start + e > size:
                raise SafetensorsError(f"{path}: tensor {name!r} ends at byte {self.data_start + e}, the file has "
                                       f"{size}")
            self.entries[name] = TensorEntry(name, dtype, dname, tuple(shape), self, b, e)

    def tensor(self, entry: TensorEntry) -> torch.Tensor:
        n = 1
        for s in entry.shape:
            n *= s
        if n == 0:
            return torch.empty(entry.shape, dtype=entry.dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")       # the mapping is read-only; the views are only ever read
            t = torch.frombuffer(self._map, dtype=entry.dtype, count=n, offset=self.data_start + entry.begin)
        return t.view(entry.shape)

    def close(self) -> None:
        # The mapping itself is left to the garbage collector: tensors made by tensor() point into it.
        self._f.close()


class SafetensorsFolder:
    """All tensors of a model folder, by name."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.files: List[SafetensorsFile] = []
        self.entries: Dict[str, TensorEntry] = {}
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        if os.path.exists(index):
            try:
                with open(index, "r", encoding="utf-8") as f:
                    weight_map = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError) as e:
                raise SafetensorsError(f"{index}: no usable 'weight_map' ({e})") from None
            shards: List[str] = []
            for shard in weight_map.values():
                if shard not in shards:
                    shards.append(shard)
            for shard in shards:
                self._add(os.path.join(model_dir, shard))
            for name, shard in weight_map.items():
                if name not in self.entries:
                    raise SafetensorsError(f"{index}: tensor {name!r} is not in {shard}")
        elif os.path.exists(single):
            self._add(single)
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")

    def _add(self, path: str) -> None:
        f = SafetensorsFile(path)
        for name, entry in f.entries.items():
            if name in self.entries:
                raise SafetensorsError(f"tensor {name!r} is in both {self.entries[name].file.path} and {path}")
            self.entries[name] = entry
        self.files.append(f)

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        return e.file.tensor(e)

    def close(self) -> None:
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: Dict[str, str] = None,
                      sizes: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]] = None) -> None:
    """Write tensors to ``path``.

    ``tensors`` is an iterable of (name, CPU tensor).  When ``sizes`` gives every tensor's dtype and shape
    in the order of the iterable, tensors are produced one at a time while the file is written, so that a
    model larger than the host's memory can be generated; otherwise the iterable is collected first.
    """
    if sizes is None:
        tensors = list(tensors)
        sizes = {n: (t.dtype, tuple(t.shape)) for n, t in tensors}
    header = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    for name, (dtype, shape) in sizes.items():
        if dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {dtype} cannot be stored")
        n = 1
        for s in shape:
            n *= s
        nbytes = n * _DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-(8 + len(blob)) % 64)          # data starts on a 64-byte boundary
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        written = set()
        order = list(sizes)
        for name, t in tensors:
            if len(written) >= len(order) or name != order[len(written)]:
                raise SafetensorsError(f"tensor {name!r} arrived out of the announced order")
            dtype, shape = sizes[name]
            if t.dtype != dtype or tuple(t.shape) != tuple(shape):
                raise SafetensorsError(f"tensor {name!r}: got {t.dtype} {tuple(t.shape)}, announced {dtype} {shape}")
            t = t.detach().contiguous().cpu()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().data)
            written.add(name)
        if written != set(sizes):
            raise SafetensorsError(f"tensors announced but not written: {sorted(set(sizes) - written)}")
    os.replace(tmp, path)
