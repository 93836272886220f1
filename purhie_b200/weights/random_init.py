"""Seeded random weights: a model folder (config.json, model.safetensors) from a configuration.

The reference has no such mode in the engine; it makes tiny checkpoints offline
(tools/gen_tiny_ckpt.py:53-61: seed 1234, norm weights around 1 "so a wrong mapping shows").  Here every
tensor is drawn from a generator keyed by (seed, tensor name), so a tensor's values depend neither on
the order in which tensors are made nor on which other tensors exist.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Tuple

import torch

from ..config.base import ModelConfig, lookup_architecture
from .loader import MATRIX, TABLE, VECTOR, TensorSpec
from .safetensors_io import write_safetensors


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(spec: TensorSpec, seed: int, std: float, scale_low: float, scale_high: float,
                  device="cpu") -> torch.Tensor:
    """Float32 values of one tensor: N(0, std) for ``init == "normal"``, U(low, high) for ``"scale"``."""
    if spec.role == TABLE:
        raise ValueError(f"{spec.name}: integer tables have no random fill")
    g = torch.Generator(device=device)
    g.manual_seed(tensor_seed(seed, spec.name))
    if spec.init == "scale":
        if scale_low == scale_high:
            return torch.full(spec.shape, float(scale_low), dtype=torch.float32, device=device)
        t = torch.rand(spec.shape, generator=g, dtype=torch.float32, device=device)
        return t * (scale_high - scale_low) + scale_low
    return torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device) * std


def expected_tensors(config: ModelConfig) -> Dict[str, TensorSpec]:
    """The tensors a model of this configuration reads, from its parts (built without a device)."""
    from ..parts.model import DecoderModel
    arch = lookup_architecture(config.architecture)
    return DecoderModel(arch.build_spec(config)).tensor_specs()


def random_tensors(config: ModelConfig, seed: int, std: float = 0.02, scale_low: float = 1.0,
                   scale_high: float = 1.0, matrix_dtype: torch.dtype = torch.bfloat16,
                   vector_dtype: torch.dtype = torch.float32, device="cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    for name, spec in expected_tensors(config).items():
        t = random_tensor(spec, seed, std, scale_low, scale_high, device)
        yield name, t.to(matrix_dtype if spec.role == MATRIX else vector_dtype)


def write_random_model(model_dir: str, config: ModelConfig, seed: int, std: float = 0.02, scale_low: float = 1.0,
                       scale_high: float = 1.0, dtype: str = "bfloat16", vector_dtype: str = "float32") -> str:
    """Write ``config.json`` and ``model.safetensors`` into ``model_dir`` and return the folder."""
    names = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}
    mdt, vdt = names[dtype], names[vector_dtype]
    os.makedirs(model_dir, exist_ok=True)
    d = config.to_dict()
    d["torch_dtype"] = dtype
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=1)
    specs = expected_tensors(config)
    sizes = {n: (mdt if s.role == MATRIX else vdt, tuple(s.shape)) for n, s in specs.items()}
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      random_tensors(config, seed, std, scale_low, scale_high, mdt, vdt),
                      metadata={"format": "pt", "seed": str(seed)}, sizes=sizes)
    return model_dir
