"""Weights: safetensors by tensor name, one error for every misfit, random models (no GPU).

Folders with faults are written with the ``safetensors`` package, which shares no code with the library's reader."""
import json
import os
import struct

import numpy as np
import pytest
import torch
from safetensors import safe_open
from safetensors.torch import save_file

from purhie_b200.config import Qwen3Config
from purhie_b200.weights import (SafetensorsError, WeightError, check_model_folder, device_dtype, expected_tensors,
                                 list_tensors, random_values, read_tensor_bytes, write_random_model)
from helpers import TINY_A, TINY_A_INIT, TINY_B, TINY_B_INIT, make_model


def read_all(folder):
    with safe_open(os.path.join(str(folder), "model.safetensors"), framework="pt") as f:
        return {k: f.get_tensor(k) for k in f.keys()}


def test_random_model_is_read_back_by_an_independent_reader(tmp_path):
    cfg = make_model(tmp_path, TINY_B, TINY_B_INIT, "bfloat16")
    specs = expected_tensors(cfg)
    got = read_all(tmp_path)
    assert set(got) == set(specs)
    for name, spec in specs.items():
        assert tuple(got[name].shape) == tuple(spec.shape)
        assert got[name].dtype == (torch.bfloat16 if spec.role == "matrix" else torch.float32)
    w = got["model.layers.1.input_layernorm.weight"]
    assert 0.8 <= w.min() and w.max() <= 1.2 and w.std() > 0.01
    m = got["model.layers.2.mlp.down_proj.weight"].float()
    assert abs(m.std().item() - 0.03) < 0.003 and abs(m.mean().item()) < 0.003
    # the draws look normal: about 68.3 % within one sigma, 95.4 % within two, tails on both sides
    big = got["lm_head.weight"].float().flatten() / 0.03
    assert abs((big.abs() < 1).float().mean().item() - 0.6827) < 0.01 and abs((big.abs() < 2).float().mean().item() - 0.9545) < 0.006
    assert big.min() < -3.5 and big.max() > 3.5 and abs((big > 0).float().mean().item() - 0.5) < 0.01
    assert "lm_head.weight" in specs and "model.layers.0.self_attn.q_proj.bias" in specs
    assert json.load(open(tmp_path / "config.json"))["num_hidden_layers"] == 3
    check_model_folder(str(tmp_path))
    assert {t["name"] for t in list_tensors(str(tmp_path))} == set(specs)
    raw = read_tensor_bytes(str(tmp_path), "model.norm.weight")
    assert np.array_equal(np.frombuffer(raw, dtype="<f4"), got["model.norm.weight"].numpy())


def test_random_values_depend_on_seed_and_name_only(tmp_path):
    a, b, c, deeper = tmp_path / "a", tmp_path / "b", tmp_path / "c", tmp_path / "d"
    make_model(a, TINY_A, TINY_A_INIT, "float32")
    make_model(b, TINY_A, TINY_A_INIT, "float32")
    make_model(c, TINY_A, dict(TINY_A_INIT, seed=1), "float32")
    make_model(deeper, dict(TINY_A, num_hidden_layers=3), TINY_A_INIT, "float32")
    ta, tb, tc, td = read_all(a), read_all(b), read_all(c), read_all(deeper)
    name = "model.layers.1.self_attn.k_proj.weight"
    assert torch.equal(ta[name], tb[name]) and not torch.equal(ta[name], tc[name])
    assert "lm_head.weight" not in ta                          # tied head: the embedding serves
    assert torch.equal(td[name], ta[name])                     # the same tensor name in a deeper model has the same values
    # element i is a function of (seed, name, i): a prefix of the stream is the prefix of the tensor
    first = random_values(name, 10, TINY_A_INIT["seed"], "normal", TINY_A_INIT["std"])
    assert np.array_equal(np.array(first, dtype=np.float32), ta[name].flatten()[:10].numpy())
    # bfloat16 storage is the float32 values rounded to nearest even
    e = tmp_path / "e"
    make_model(e, TINY_A, TINY_A_INIT, "bfloat16")
    assert torch.equal(read_all(e)[name], ta[name].to(torch.bfloat16))


def test_dtype_policy():
    # a matrix follows the compute dtype, except that a tensor stored in 32-bit stays so; vectors are float32; tables int32
    assert device_dtype("bfloat16", "matrix", "bfloat16") == "bfloat16"
    assert device_dtype("float16", "matrix", "bfloat16") == "bfloat16"
    assert device_dtype("float32", "matrix", "bfloat16") == "float32"
    assert device_dtype("bfloat16", "matrix", "float32") == "float32"
    assert device_dtype("bfloat16", "vector", "bfloat16") == "float32"
    assert device_dtype("int64", "table", "bfloat16") == "int32"


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = make_model(tmp_path, TINY_A, TINY_A_INIT, "bfloat16")
    tensors = read_all(tmp_path)
    del tensors["model.layers.0.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.extra.weight"] = torch.zeros(3)
    tensors["model.layers.1.self_attn.q_norm.weight"] = torch.zeros(8)
    tensors["model.layers.1.self_attn.o_proj.weight"] = torch.zeros(64, 32, dtype=torch.bfloat16)
    tensors["model.layers.1.self_attn.k_norm.weight"] = torch.zeros(16, dtype=torch.int32)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        check_model_folder(str(tmp_path))
    err = e.value
    assert sorted(err.missing) == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.mlp.extra.weight"]
    assert sorted(w.split(" ")[0] for w in err.wrong_shape) == ["model.layers.1.self_attn.o_proj.weight",
                                                                "model.layers.1.self_attn.q_norm.weight"]
    assert [w.split(" ")[0] for w in err.wrong_type] == ["model.layers.1.self_attn.k_norm.weight"]
    msg = str(err)
    for word in ("missing (2)", "unexpected (1)", "model.layers.0.mlp.extra.weight", "[64, 32]", "[64, 64]", "I32"):
        assert word in msg


def test_tied_head_ignores_a_stray_lm_head(tmp_path):
    make_model(tmp_path, TINY_A, TINY_A_INIT, "bfloat16")
    tensors = read_all(tmp_path)
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    check_model_folder(str(tmp_path))                                  # no error: a tied head may find one and does not read it
    tensors["lm_head.bias"] = torch.zeros(256)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        check_model_folder(str(tmp_path))
    assert e.value.unexpected == ["lm_head.bias"]


def test_sharded_folder_and_duplicates(tmp_path):
    make_model(tmp_path, TINY_A, TINY_A_INIT, "float32")
    tensors = read_all(tmp_path)
    os.unlink(tmp_path / "model.safetensors")
    names = sorted(tensors)
    first, second = names[: len(names) // 2], names[len(names) // 2:]
    save_file({n: tensors[n] for n in first}, str(tmp_path / "s1.safetensors"))
    save_file({n: tensors[n] for n in second}, str(tmp_path / "s2.safetensors"))
    index = {"weight_map": {**{n: "s2.safetensors" for n in second}, **{n: "s1.safetensors" for n in first}}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    check_model_folder(str(tmp_path))
    listed = list_tensors(str(tmp_path))
    assert [t["name"] for t in listed][:len(second)] == sorted(second)         # shards in order of first appearance
    raw = read_tensor_bytes(str(tmp_path), first[0])
    assert raw == tensors[first[0]].numpy().tobytes()
    save_file({n: tensors[n] for n in second + first[:1]}, str(tmp_path / "s2.safetensors"))
    with pytest.raises(SafetensorsError) as e:
        check_model_folder(str(tmp_path))
    assert "both" in str(e.value)
    index["weight_map"]["ghost"] = "s1.safetensors"
    save_file({n: tensors[n] for n in second}, str(tmp_path / "s2.safetensors"))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(SafetensorsError) as e:
        check_model_folder(str(tmp_path))
    assert "ghost" in str(e.value)


def test_malformed_files_are_refused(tmp_path):
    make_model(tmp_path, TINY_A, TINY_A_INIT, "float32")
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x00\x01")
    with pytest.raises(SafetensorsError):
        check_model_folder(str(tmp_path))
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError) as e:
        check_model_folder(str(tmp_path))
    assert "longer than the file" in str(e.value)
    p.write_bytes(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError) as e:
        check_model_folder(str(tmp_path))
    assert "JSON" in str(e.value)
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\x00" * 8)
    with pytest.raises(SafetensorsError) as e:
        check_model_folder(str(tmp_path))
    assert "ends at byte" in str(e.value)
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\x00" * 16)
    with pytest.raises(SafetensorsError) as e:
        check_model_folder(str(tmp_path))
    assert "do not match" in str(e.value)
    hdr = json.dumps({"x": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\x00" * 4)
    with pytest.raises(SafetensorsError) as e:
        check_model_folder(str(tmp_path))
    assert "unsupported dtype" in str(e.value)
    os.unlink(p)
    with pytest.raises(SafetensorsError):
        check_model_folder(str(tmp_path))
