"""Typed model configurations and the architecture registry, as Python sees them.

The reading, the defaults, the checks and the registry are the host library's (``config/config.cpp``); a
:class:`ModelConfig` here holds what the library read back, every default filled in, as attributes.
"""
from __future__ import annotations

import json
from typing import Dict, List

from .. import native
from ..native import ConfigError


class ModelConfig:
    """A configuration the library accepted.  ``to_dict()`` is the config.json it stands for; every key is also
    an attribute."""

    def __init__(self, values: Dict):
        self._values = dict(values)

    @classmethod
    def from_dict(cls, d: Dict) -> "ModelConfig":
        """Read a ``config.json`` dictionary through the architecture registry (raises :class:`ConfigError`)."""
        return cls(native.answer(native.lib().qe_config_read(json.dumps(d).encode())))

    def __getattr__(self, name):
        try:
            return self.__dict__["_values"][name]
        except KeyError:
            raise AttributeError(name) from None

    def __eq__(self, other):
        return isinstance(other, ModelConfig) and self._values == other._values

    def __repr__(self):
        return f"{type(self).__name__}({self._values})"

    @property
    def architecture(self) -> str:
        return self._values["architectures"][0]

    def to_dict(self) -> Dict:
        d = dict(self._values)
        d.pop("parameter_count", None)
        if d.get("sliding_window") is None:
            d.pop("sliding_window", None)
            d.pop("layer_types", None)
        return d

    def to_json(self) -> str:
        return json.dumps(self.to_dict())

    def model_spec(self) -> Dict:
        """The description the generic decoder is assembled from: embedding, layers (arrangement and named
        sub-parts, each {kind, params}), the run order, final norm and head."""
        return native.answer(native.lib().qe_model_spec(self.to_json().encode()))


class Qwen3Config(ModelConfig):
    """``Qwen3ForCausalLM``: see ``config/config.h`` for the keys and their defaults."""

    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def parameter_count(self) -> int:
        return self._values["parameter_count"]


def load_config(model_dir: str) -> ModelConfig:
    """Read ``model_dir/config.json`` (raises :class:`ConfigError`: missing, not JSON, unknown architecture)."""
    d = native.answer(native.lib().qe_config_load(str(model_dir).encode()))
    return ModelConfig.from_dict(d) if d["architectures"][0] != "Qwen3ForCausalLM" else Qwen3Config.from_dict(d)


def registered_architectures() -> List[str]:
    return native.answer(native.lib().qe_registered_architectures())


def registered_parts(family: str) -> List[str]:
    """Kinds registered for a family: norm, position, mixer, feed_forward, embedding, head, arrangement."""
    return native.answer(native.lib().qe_registered_parts(family.encode()))


__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "load_config", "registered_architectures", "registered_parts"]
