"""Typed model configurations and the architecture registry.

A configuration is read from the keys of the architecture's own ``config.json``; no size or constant
that ``config.json`` gives is written in code anywhere else in the package.  The registry maps the
name in ``architectures[0]`` to a configuration class and to a function that turns a configuration
into a :class:`purhie_b200.parts.spec.ModelSpec` (the description from which the generic decoder is
assembled).  The reference keeps the same mapping as a whitelist of architecture names
(src/inference.cpp:1237-1239, error for an unknown one at :1267-1268) and, on the converter side, as
a name -> package registry (perl/ROCm-Inference/lib/ROCm/Inference/Convert.pm:34, 1475-1479).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, Tuple, Type


class ConfigError(ValueError):
    """A ``config.json`` that cannot be used: a missing key, a wrong type or an unsupported option."""


@dataclass(frozen=True)
class ModelConfig:
    """Base class of every architecture's configuration."""

    architecture: str

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":  # pragma: no cover - abstract
        raise NotImplementedError

    def to_dict(self) -> dict:  # pragma: no cover - abstract
        raise NotImplementedError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Type[ModelConfig]
    build_spec: Callable  # (config) -> ModelSpec


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig], build_spec: Callable) -> None:
    """Make ``architectures: [name]`` loadable.  Registering a name twice replaces the entry."""
    _REGISTRY[name] = Architecture(name, config_cls, build_spec)


def unregister_architecture(name: str) -> None:
    _REGISTRY.pop(name, None)


def registered_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_REGISTRY))


def lookup_architecture(name: str) -> Architecture:
    try:
        return _REGISTRY[name]
    except KeyError:
        raise ConfigError(
            f"unsupported architecture {name!r}; registered: {', '.join(registered_architectures()) or '(none)'}"
        ) from None


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no config.json in the model folder") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return d


def architecture_name(d: dict) -> str:
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return archs[0]


def load_config(model_dir: str) -> Tuple[Architecture, ModelConfig]:
    """Read ``model_dir/config.json`` and return (architecture entry, typed configuration)."""
    d = read_config_json(model_dir)
    arch = lookup_architecture(architecture_name(d))
    return arch, arch.config_cls.from_dict(d)


# ---- helpers for typed reading -------------------------------------------------------------------

_MISSING = object()


def take_int(d: dict, key: str, default=_MISSING, *, minimum: int = 1):
    v = d.get(key)
    if v is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: missing key {key!r}")
        return default
    if isinstance(v, float) and v == int(v):
        v = int(v)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: {key!r} must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: {key!r} must be >= {minimum}, got {v}")
    return v


def take_float(d: dict, key: str, default=_MISSING) -> float:
    v = d.get(key)
    if v is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: missing key {key!r}")
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {key!r} must be a number, got {v!r}")
    return float(v)


def take_bool(d: dict, key: str, default: bool) -> bool:
    v = d.get(key, default)
    if v is None:
        return default
    if not isinstance(v, bool):
        raise ConfigError(f"config.json: {key!r} must be true or false, got {v!r}")
    return v
