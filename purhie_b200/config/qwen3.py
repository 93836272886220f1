"""Configuration of the Qwen3 dense decoder (``Qwen3ForCausalLM``) and its model description.

Keys and their meaning follow the reference: the converter reads ``num_hidden_layers``,
``hidden_size``, ``intermediate_size``, ``num_attention_heads``, ``num_key_value_heads``, ``head_dim``,
``max_position_embeddings``, ``rope_theta`` (plain or inside ``rope_parameters``) and ``rms_norm_eps``
(perl/ROCm-Inference/lib/ROCm/Inference/Convert.pm:72-80, 555-615); the loader's defaults are head_dim
= hidden/heads (src/inference.cpp:1326), context 4096 (:1338-1339), rope base 10000 (:1359) and eps 1e-6
(:1360); a missing ``lm_head.weight`` means a tied head (:1392-1396) and optional q/k/v biases are
bound when present (:631-633).  The window keys (``use_sliding_window``, ``sliding_window``,
``max_window_layers``, ``layer_types``) choose, layer by layer, between attention over all earlier
positions and attention over the last ``sliding_window`` of them (the meaning of ``window`` in
src/attention.h:73: a token at p sees positions > p - window).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import (ConfigError, ModelConfig, register_architecture, take_bool, take_float, take_int)
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

FULL = "full_attention"
SLIDING = "sliding_attention"


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    num_hidden_layers: int
    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    attention_bias: bool
    layer_types: Tuple[str, ...]
    sliding_window: Optional[int]
    hidden_act: str = "silu"

    # ---- reading ---------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "Qwen3Config":
        archs = d.get("architectures") or ["Qwen3ForCausalLM"]
        n_layers = take_int(d, "num_hidden_layers")
        hidden = take_int(d, "hidden_size")
        heads = take_int(d, "num_attention_heads")
        kv_heads = take_int(d, "num_key_value_heads", heads)
        head_dim = take_int(d, "head_dim", None)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"config.json: no 'head_dim' and hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads}")
            head_dim = hidden // heads
        rope_params = d.get("rope_parameters")
        theta = d.get("rope_theta")
        if theta is None and isinstance(rope_params, dict):
            theta = rope_params.get("rope_theta")
        if theta is None:
            theta = 10000.0
        if isinstance(theta, bool) or not isinstance(theta, (int, float)) or theta <= 0:
            raise ConfigError(f"config.json: 'rope_theta' must be a positive number, got {theta!r}")
        scaling = d.get("rope_scaling")
        if scaling is None and isinstance(rope_params, dict):
            rt = rope_params.get("rope_type", "default")
            if rt not in (None, "default"):
                scaling = {"rope_type": rt}
        if scaling is not None:
            rt = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
            if rt not in (None, "default"):
                raise ConfigError(f"config.json: rope scaling {rt!r} is not supported (only plain rotary position "
                                  f"encoding)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (silu only)")

        window = take_int(d, "sliding_window", None)
        use_window = take_bool(d, "use_sliding_window", False)
        layer_types = d.get("layer_types")
        if layer_types is not None:
            if (not isinstance(layer_types, list) or len(layer_types) != n_layers
                    or any(t not in (FULL, SLIDING) for t in layer_types)):
                raise ConfigError(f"config.json: 'layer_types' must list {n_layers} entries of {FULL!r} / {SLIDING!r}")
            layer_types = tuple(layer_types)
        elif use_window:
            first = take_int(d, "max_window_layers", n_layers, minimum=0)
            layer_types = tuple(SLIDING if i >= first else FULL for i in range(n_layers))
        else:
            layer_types = (FULL,) * n_layers
        if SLIDING in layer_types and window is None:
            raise ConfigError("config.json: a layer uses sliding attention but 'sliding_window' is not given")
        if SLIDING not in layer_types:
            window = None

        cfg = cls(
            architecture=archs[0],
            num_hidden_layers=n_layers,
            hidden_size=hidden,
            intermediate_size=take_int(d, "intermediate_size"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=take_int(d, "vocab_size"),
            max_position_embeddings=take_int(d, "max_position_embeddings", 4096),
            rope_theta=float(theta),
            rms_norm_eps=take_float(d, "rms_norm_eps", 1e-6),
            tie_word_embeddings=take_bool(d, "tie_word_embeddings", False),
            attention_bias=take_bool(d, "attention_bias", False),
            layer_types=layer_types,
            sliding_window=window,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even (rotary pairs)")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be > 0, got {self.rms_norm_eps}")

    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "hidden_act": self.hidden_act,
        }
        if self.sliding_window is not None:
            d["use_sliding_window"] = True
            d["sliding_window"] = self.sliding_window
            d["layer_types"] = list(self.layer_types)
        else:
            d["use_sliding_window"] = False
        return d

    # ---- sizes that follow from the keys ---------------------------------------------------------
    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def parameter_count(self) -> int:
        e, ff, v = self.hidden_size, self.intermediate_size, self.vocab_size
        per_layer = (self.q_width + 2 * self.kv_width) * e + e * self.q_width + 3 * e * ff + 2 * e + 2 * self.head_dim
        if self.attention_bias:
            per_layer += self.q_width + 2 * self.kv_width
        total = self.num_hidden_layers * per_layer + v * e + e
        if not self.tie_word_embeddings:
            total += v * e
        return total


def qwen3_model_spec(cfg: Qwen3Config) -> ModelSpec:
    """Qwen3 dense as parts: per layer RMSNorm -> grouped-query attention (per-head RMSNorm on q and k,
    rotate-half rotary) -> residual, RMSNorm -> SwiGLU -> residual; then a final RMSNorm and the output
    matrix, shared with the embedding when ``tie_word_embeddings`` (the order of
    src/qwen_model.cpp:1196-1279 with full_attention :940-975 and ffn :1170-1189)."""
    position = PartSpec("rope_neox", {"theta": cfg.rope_theta, "n_rot": cfg.head_dim,
                                      "max_position": cfg.max_position_embeddings})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        names = {"q_proj": p + "self_attn.q_proj.weight", "k_proj": p + "self_attn.k_proj.weight",
                 "v_proj": p + "self_attn.v_proj.weight", "o_proj": p + "self_attn.o_proj.weight",
                 "q_norm": p + "self_attn.q_norm.weight", "k_norm": p + "self_attn.k_norm.weight"}
        if cfg.attention_bias:
            names.update({"q_bias": p + "self_attn.q_proj.bias", "k_bias": p + "self_attn.k_proj.bias",
                          "v_bias": p + "self_attn.v_proj.bias"})
        mixer = PartSpec("attention", {
            "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "qk_norm_eps": cfg.rms_norm_eps, "bias": cfg.attention_bias, "position": position,
            "window": cfg.sliding_window if cfg.layer_types[i] == SLIDING else None,
            "names": names})
        ff = PartSpec("swiglu", {
            "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
            "names": {"gate_proj": p + "mlp.gate_proj.weight", "up_proj": p + "mlp.up_proj.weight",
                      "down_proj": p + "mlp.down_proj.weight"}})
        layers.append(LayerSpec(
            mixer=mixer,
            mixer_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                            "names": {"weight": p + "input_layernorm.weight"}}),
            feed_forward=ff,
            feed_forward_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                                   "names": {"weight": p + "post_attention_layernorm.weight"}}),
            arrangement="pre_norm"))
    embed_name = "model.embed_tokens.weight"
    head_params = {"hidden_size": cfg.hidden_size, "vocab_size": cfg.vocab_size}
    if cfg.tie_word_embeddings:
        head_params["tied_to"] = embed_name
        head_params["ignore"] = ("lm_head.weight",)
    else:
        head_params["names"] = {"weight": "lm_head.weight"}
    spec = ModelSpec(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, max_position=cfg.max_position_embeddings,
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                         "names": {"weight": embed_name}}),
        layers=tuple(layers),
        schedule=tuple(LayerCall(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                        "names": {"weight": "model.norm.weight"}}),
        head=PartSpec("lm_head", head_params))
    spec.validate()
    return spec


register_architecture("Qwen3ForCausalLM", Qwen3Config, qwen3_model_spec)
