"""Configuration and registry (no GPU)."""
import json
import math

import pytest

from purhie_b200.config import (ConfigError, Qwen3Config, load_config, registered_architectures, registered_parts)
from helpers import TINY_A, TINY_B, TINY_B0, TINY_C


def test_reads_every_key_of_both_tiny_configs():
    a, b = Qwen3Config.from_dict(TINY_A), Qwen3Config.from_dict(TINY_B)
    for key in ("num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads", "head_dim",
                "vocab_size", "max_position_embeddings", "rope_theta", "rms_norm_eps", "tie_word_embeddings",
                "attention_bias"):
        assert getattr(a, key) == TINY_A[key] and getattr(b, key) == TINY_B[key]
        assert getattr(a, key) != getattr(b, key), key          # the two differ in every size and option
    assert a.layer_types == ["full_attention"] * 2 and a.sliding_window is None
    assert b.layer_types == ["full_attention", "sliding_attention", "sliding_attention"] and b.sliding_window == 24
    c = Qwen3Config.from_dict(TINY_C)
    assert c.layer_types == ["full_attention", "sliding_attention"]
    b0 = Qwen3Config.from_dict(TINY_B0)
    assert b0.attention_bias is False and b0.sliding_window is None and b0.head_dim == 32 and b0.q_width != b0.hidden_size


def test_defaults_follow_the_reference():
    d = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "rope_theta", "rms_norm_eps",
                                                       "max_position_embeddings", "tie_word_embeddings")}
    c = Qwen3Config.from_dict(d)
    assert c.head_dim == 64 // 4 and c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6
    assert c.max_position_embeddings == 4096 and c.tie_word_embeddings is False


def test_rope_theta_inside_rope_parameters():
    d = dict(TINY_A)
    del d["rope_theta"]
    d["rope_parameters"] = {"rope_theta": 5e5, "rope_type": "default"}
    assert Qwen3Config.from_dict(d).rope_theta == 5e5


@pytest.mark.parametrize("patch,word", [
    ({"num_hidden_layers": None}, "num_hidden_layers"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "yarn"),
    ({"rope_parameters": {"rope_type": "linear", "rope_theta": 1e4}}, "linear"),
    ({"hidden_act": "gelu"}, "gelu"),
    ({"use_sliding_window": True, "max_window_layers": 0}, "sliding_window"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
])
def test_bad_configs_are_refused_with_the_key_named(patch, word):
    d = dict(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(d)
    assert word in str(e.value)


def test_round_trip_through_json(tmp_path):
    for cfg in (TINY_A, TINY_B, TINY_B0, TINY_C):
        c = Qwen3Config.from_dict(cfg)
        (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
        c2 = load_config(str(tmp_path))
        assert c2.architecture == "Qwen3ForCausalLM" and c2 == c


def test_registry_names_unknown_architecture(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["LlamaForCausalLM"]}))
    with pytest.raises(ConfigError) as e:
        load_config(str(tmp_path))
    assert "LlamaForCausalLM" in str(e.value) and "Qwen3ForCausalLM" in str(e.value)
    assert "Qwen3ForCausalLM" in registered_architectures()
    (tmp_path / "config.json").write_text(json.dumps({"architectures": []}))
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_missing_or_broken_config_json(tmp_path):
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("[1, 2]")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_model_spec_takes_every_number_from_the_config():
    from purhie_b200.weights import expected_tensors
    b = Qwen3Config.from_dict(TINY_B)
    spec = b.model_spec()
    assert len(spec["layers"]) == 3 and [c["layer"] for c in spec["schedule"]] == [0, 1, 2]
    assert all(c["cache_from"] is None for c in spec["schedule"])
    parts = spec["layers"][1]["parts"]
    assert spec["layers"][1]["arrangement"] == "pre_norm" and sorted(parts) == ["feed_forward", "feed_forward_norm", "mixer", "mixer_norm"]
    m = parts["mixer"]["params"]
    assert (m["num_heads"], m["num_kv_heads"], m["head_dim"], m["window"], m["qk_norm_eps"], m["bias"]) == \
        (8, 2, 32, 24, 1e-5, True)
    assert spec["layers"][0]["parts"]["mixer"]["params"]["window"] is None
    assert m["position"] == {"kind": "rope_neox", "params": {"theta": 1e6, "n_rot": 32, "max_position": 256}}
    assert parts["feed_forward"]["kind"] == "swiglu" and parts["feed_forward"]["params"]["intermediate_size"] == 224
    assert parts["mixer_norm"]["params"] == {"size": 96, "eps": 1e-5, "names": {"weight": "model.layers.1.input_layernorm.weight"}}
    assert spec["head"]["params"].get("tied_to") is None
    a = Qwen3Config.from_dict(TINY_A).model_spec()
    assert a["head"]["params"]["tied_to"] == "model.embed_tokens.weight"
    assert b.parameter_count() == sum(math.prod(s.shape) for s in expected_tensors(b).values())


def test_the_parts_this_library_brings_are_registered():
    assert "rmsnorm" in registered_parts("norm") and "rope_neox" in registered_parts("position")
    assert "attention" in registered_parts("mixer") and "swiglu" in registered_parts("feed_forward")
    assert "embedding" in registered_parts("embedding") and "lm_head" in registered_parts("head")
    assert "pre_norm" in registered_parts("arrangement")
