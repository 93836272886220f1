"""Weights: safetensors by name, one error for every misfit, random models (no GPU)."""
import json
import os
import struct

import pytest
import torch

from purhie_b200.config import Qwen3Config
from purhie_b200.weights import (SafetensorsError, SafetensorsFolder, TensorSpec, WeightError, check_folder,
                                 device_dtype, expected_tensors, load_tensors, random_tensors, write_random_model,
                                 write_safetensors)
from helpers import TINY_A, TINY_A_INIT, TINY_B, TINY_B_INIT, make_model


def test_random_model_is_read_back_by_an_independent_reader(tmp_path):
    from safetensors import safe_open
    cfg = make_model(tmp_path, TINY_B, TINY_B_INIT, "bfloat16")
    specs = expected_tensors(cfg)
    with safe_open(str(tmp_path / "model.safetensors"), framework="pt") as f:
        assert set(f.keys()) == set(specs)
        for name, spec in specs.items():
            t = f.get_tensor(name)
            assert tuple(t.shape) == tuple(spec.shape)
            assert t.dtype == (torch.bfloat16 if spec.role == "matrix" else torch.float32)
        w = f.get_tensor("model.layers.1.input_layernorm.weight")
        assert 0.8 <= w.min() and w.max() <= 1.2 and w.std() > 0.01
        m = f.get_tensor("model.layers.2.mlp.down_proj.weight").float()
        assert abs(m.std().item() - 0.03) < 0.003 and abs(m.mean().item()) < 0.003
    assert "lm_head.weight" in specs and "model.layers.0.self_attn.q_proj.bias" in specs
    assert json.load(open(tmp_path / "config.json"))["num_hidden_layers"] == 3


def test_random_values_depend_on_seed_and_name_only():
    cfg = Qwen3Config.from_dict(TINY_A)
    a = dict(random_tensors(cfg, 0, 0.02, 0.9, 1.1))
    b = dict(random_tensors(cfg, 0, 0.02, 0.9, 1.1))
    c = dict(random_tensors(cfg, 1, 0.02, 0.9, 1.1))
    name = "model.layers.1.self_attn.k_proj.weight"
    assert torch.equal(a[name], b[name]) and not torch.equal(a[name], c[name])
    assert "lm_head.weight" not in a                          # tied head: the embedding serves
    # the same tensor name in a deeper model has the same values
    deeper = Qwen3Config.from_dict(dict(TINY_A, num_hidden_layers=3))
    assert torch.equal(dict(random_tensors(deeper, 0, 0.02, 0.9, 1.1))[name], a[name])


def test_loader_keeps_dtypes_as_stated(tmp_path):
    make_model(tmp_path, TINY_A, TINY_A_INIT, "bfloat16")
    cfg = Qwen3Config.from_dict(TINY_A)
    specs = expected_tensors(cfg)
    t = load_tensors(str(tmp_path), specs, torch.bfloat16, "cpu")
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert t["model.norm.weight"].dtype == torch.float32
    t32 = load_tensors(str(tmp_path), specs, torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in t32.values())
    assert torch.equal(t32["model.embed_tokens.weight"], t["model.embed_tokens.weight"].float())
    # a tensor stored in 32-bit stays so; integer tables become int32
    assert device_dtype(torch.float32, "matrix", torch.bfloat16) == torch.float32
    assert device_dtype(torch.float16, "matrix", torch.bfloat16) == torch.bfloat16
    assert device_dtype(torch.int64, "table", torch.bfloat16) == torch.int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_A)
    tensors = dict(random_tensors(cfg, 0))
    del tensors["model.layers.0.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.extra.weight"] = torch.zeros(3)
    tensors["model.layers.1.self_attn.q_norm.weight"] = torch.zeros(8)
    tensors["model.layers.1.self_attn.o_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    tensors["model.layers.1.self_attn.k_norm.weight"] = torch.zeros(16, dtype=torch.int32)
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors.items())
    with pytest.raises(WeightError) as e:
        load_tensors(str(tmp_path), expected_tensors(cfg), torch.float32, "cpu")
    err = e.value
    assert sorted(err.missing) == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert sorted(n for n, _, _ in err.wrong_shape) == ["model.layers.1.self_attn.o_proj.weight",
                                                        "model.layers.1.self_attn.q_norm.weight"]
    assert [n for n, _, _ in err.wrong_type] == ["model.layers.1.self_attn.k_norm.weight"]
    msg = str(err)
    for word in ("missing (2)", "unexpected (1)", "model.layers.0.mlp.extra.weight", "[64, 32]", "[64, 64]", "I32"):
        assert word in msg


def test_tied_head_ignores_a_stray_lm_head(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_A)
    tensors = dict(random_tensors(cfg, 0))
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors.items())
    from purhie_b200.parts import DecoderModel
    from purhie_b200.config import qwen3_model_spec
    model = DecoderModel(qwen3_model_spec(cfg))
    folder = SafetensorsFolder(str(tmp_path))
    check_folder(folder, model.tensor_specs(), model.ignored_tensors())     # no error
    with pytest.raises(WeightError):
        check_folder(folder, model.tensor_specs())


def test_sharded_folder_and_duplicates(tmp_path):
    a = {"x": torch.arange(6, dtype=torch.float32).view(2, 3)}
    b = {"y": torch.ones(4, dtype=torch.bfloat16)}
    write_safetensors(str(tmp_path / "s1.safetensors"), a.items())
    write_safetensors(str(tmp_path / "s2.safetensors"), b.items())
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    f = SafetensorsFolder(str(tmp_path))
    assert torch.equal(f.tensor("x"), a["x"]) and torch.equal(f.tensor("y"), b["y"])
    write_safetensors(str(tmp_path / "s2.safetensors"), {**b, **a}.items())
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFolder(str(tmp_path))
    assert "both" in str(e.value)


def test_malformed_files_are_refused(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x00\x01")
    with pytest.raises(SafetensorsError):
        SafetensorsFolder(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFolder(str(tmp_path))
    assert "longer than the file" in str(e.value)
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\x00" * 8)
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFolder(str(tmp_path))
    assert "ends at byte" in str(e.value)
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\x00" * 16)
    with pytest.raises(SafetensorsError):
        SafetensorsFolder(str(tmp_path))
    os.unlink(p)
    with pytest.raises(SafetensorsError):
        SafetensorsFolder(str(tmp_path))
