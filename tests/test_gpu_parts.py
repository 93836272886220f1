"""Each part of a layer alone against the plain functions, and parts that the framework does not have: a toy mixer
with state and step metadata of its own, a toy position encoding, a toy feed-forward with routing, an arrangement
with a third norm, a run order that names a layer twice and lets a call read another call's cache (GPU).  The toys
are C++ in tests/toy_parts/toy_parts.cu, compiled by this test and registered through the public registries when the
shared object is loaded; no file of the framework changes."""
import json
import math
import os

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

from plain import qwen3_plain as P
from helpers import ROOT, random_tokens, rel_err

pytestmark = pytest.mark.gpu


def folder_with(tmp_path, tensors, name="w"):
    d = tmp_path / name
    d.mkdir(exist_ok=True)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(d / "model.safetensors"))
    return str(d)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part_folds_the_pending_addend(dtype, tmp_path):
    from purhie_b200.parts import PartProbe
    n = PartProbe("norm", "rmsnorm", {"size": 100, "eps": 1e-4, "names": {"weight": "w"}}, dtype)
    assert n.tensor_specs() == [{"name": "w", "shape": [100], "role": "vector", "init": "scale"}]
    w = torch.rand(100) + 0.5
    n.bind_folder(folder_with(tmp_path, {"w": w}))
    x, add = torch.randn(7, 100), torch.randn(7, 100)
    out_x, y = n.norm(x.numpy(), add.numpy())
    v = (x + add).double()
    assert rel_err(torch.from_numpy(out_x), v) < 1e-6
    assert rel_err(torch.from_numpy(y), P.rmsnorm(v, w.double(), 1e-4)) < (1e-5 if dtype == "float32" else 6e-3)
    out_x, y = n.norm(x.numpy())                                     # nothing pending: the stream stays
    assert np.array_equal(out_x, x.numpy())


def test_rotary_table_is_made_in_double_precision():
    from purhie_b200.parts import PartProbe
    r = PartProbe("position", "rope_neox", {"theta": 1e6, "n_rot": 32, "max_position": 300})
    r.bind_random(0)
    assert r.position_info() == {"n_rot": 32, "interleaved": False, "position_column": 0, "rows": 300, "width": 32}
    t = torch.from_numpy(r.position_table())
    v = torch.randn(1, 1, 32, dtype=torch.float64)
    for pos in (0, 1, 255, 299):
        c, s = t[pos, :16].double(), t[pos, 16:].double()
        mine = torch.cat([v[0, 0, :16] * c - v[0, 0, 16:] * s, v[0, 0, :16] * s + v[0, 0, 16:] * c])
        assert (mine - P.rope_rotate_half(v, [pos], 1e6, 32).view(-1)).abs().max() < 1e-6
    # per-pair frequency factors divide the frequencies; the pairing is a parameter
    f = PartProbe("position", "rope_neox", {"theta": 1e4, "n_rot": 8, "max_position": 50, "pairing": "interleaved",
                                            "freq_factors": [1.0, 2.0, 4.0, 8.0]})
    f.bind_random(0)
    assert f.position_info()["interleaved"] is True
    t = f.position_table()
    for i, factor in enumerate((1.0, 2.0, 4.0, 8.0)):
        assert abs(t[37, i] - math.cos(37 * 1e4 ** (-2 * i / 8) / factor)) < 1e-6


@pytest.mark.parametrize("dtype,window,HQ,HKV,D", [("float32", None, 6, 3, 24), ("float32", 9, 4, 1, 16),
                                                   ("bfloat16", None, 8, 2, 64), ("bfloat16", 20, 4, 4, 128)])
def test_attention_part_alone(dtype, window, HQ, HKV, D, tmp_path):
    """One attention mixer, its own weights: a prompt portion in one step, then the rest in a second step that reads
    the first step's pages, then two more rows one at a time beside another request, against the plain attention
    block over the whole sequence."""
    from purhie_b200.parts import PartProbe
    E, ps, n1, n2 = 80, 8, 37, 30
    names = {k: k for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm", "q_bias", "k_bias", "v_bias")}
    pos_spec = {"kind": "rope_neox", "params": {"theta": 5e4, "n_rot": D, "max_position": 128}}
    att = PartProbe("mixer", "attention", {"hidden_size": E, "num_heads": HQ, "num_kv_heads": HKV, "head_dim": D, "qk_norm_eps": 1e-5,
                                           "bias": True, "position": pos_spec, "window": window, "names": names}, dtype)
    specs = {s["name"]: s for s in att.tensor_specs()}
    assert specs["q_proj"]["shape"] == [HQ * D, E] and specs["k_bias"]["role"] == "vector" and len(specs) == 9
    g = torch.Generator().manual_seed(0)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    w = {n: (torch.randn(s["shape"], generator=g) * (0.2 if s["role"] == "matrix" else 0.3) + (1.0 if s["init"] == "scale" else 0.0))
         for n, s in specs.items()}
    stored = {n: (t.to(tdt) if specs[n]["role"] == "matrix" else t) for n, t in w.items()}
    att.bind_folder(folder_with(tmp_path, stored))
    need = att.cache_need()
    assert (need["kind"], need["kv_heads"], need["head_dim"], need["window"]) == ("pages", HKV, D, window)
    att.mixer_cache(ps, 24, max_requests=2, poison=True)
    att.add_request(1); att.add_request(2)
    x = torch.randn(n1 + n2 + 2, E, generator=g)
    other = torch.randn(5, E, generator=g)
    xr = x.to(tdt).float()
    outs = [att.mixer_step([(1, n1)], xr[:n1].numpy()), att.mixer_step([(2, 3), (1, n2)], torch.cat([other[:3], xr[n1:n1 + n2]]).numpy())[3:]]
    for k in range(2):
        outs.append(att.mixer_step([(1, 1), (2, 1)], torch.cat([xr[n1 + n2 + k:n1 + n2 + k + 1], other[3 + k:4 + k]]).numpy())[:1])
    got = torch.from_numpy(np.concatenate(outs))
    wd = {("self_attn." + k.replace("_bias", "_proj.bias") if k.endswith("_bias") else "self_attn." + k + ".weight"): stored[k].double()
          for k in w}
    cfg = {"num_attention_heads": HQ, "num_key_value_heads": HKV, "head_dim": D, "hidden_size": E, "rms_norm_eps": 1e-5,
           "attention_bias": True, "rope_theta": 5e4}
    ref = P.attention_block(xr.double(), wd, "", cfg, list(range(n1 + n2 + 2)), window)
    assert rel_err(got, ref) < (2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_swiglu_part_alone(dtype, tmp_path):
    from purhie_b200.parts import PartProbe
    E, FF, T = 72, 200, 19
    ff = PartProbe("feed_forward", "swiglu", {"hidden_size": E, "intermediate_size": FF,
                                              "names": {"gate_proj": "g", "up_proj": "u", "down_proj": "d"}}, dtype)
    g = torch.Generator().manual_seed(1)
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    w = {s["name"]: (torch.randn(s["shape"], generator=g) * 0.2).to(tdt) for s in ff.tensor_specs()}
    ff.bind_folder(folder_with(tmp_path, w))
    x = torch.randn(T, E, generator=g).to(tdt).float()
    got = torch.from_numpy(ff.feed_forward(x.numpy()))
    wd = {"mlp.gate_proj.weight": w["g"].double(), "mlp.up_proj.weight": w["u"].double(), "mlp.down_proj.weight": w["d"].double()}
    assert rel_err(got, P.swiglu_mlp(x.double(), wd, "")) < (1e-5 if dtype == "float32" else 2e-2)


def test_embedding_and_tied_head_parts(tmp_path):
    from purhie_b200.parts import PartProbe
    emb = PartProbe("embedding", "embedding", {"vocab_size": 300, "hidden_size": 40, "names": {"weight": "e"}})
    head = PartProbe("head", "lm_head", {"hidden_size": 40, "vocab_size": 300, "tied_to": "e"})
    assert head.tensor_specs() == []
    table = torch.randn(300, 40)
    folder = folder_with(tmp_path, {"e": table})
    emb.bind_folder(folder)
    ids = [3, 299, 0, 3, 17]
    x = emb.embedding(ids, 40)
    assert np.array_equal(x, table[ids].numpy())
    # a tied head announces no tensor of its own and reads the embedding's
    from purhie_b200.native import InferenceError
    with pytest.raises(InferenceError):
        head.bind_folder(folder)                                      # alone it has not announced "e": the model does that for it
    own = PartProbe("head", "lm_head", {"hidden_size": 40, "vocab_size": 300, "names": {"weight": "e"}})
    own.bind_folder(folder)
    logits = own.head(x, 300)
    assert rel_err(torch.from_numpy(logits), torch.from_numpy(x).double() @ table.double().T) < 1e-5


# ---- toys: parts that are not in the framework ----------------------------------------------------------

@pytest.fixture(scope="module")
def toys(tmp_path_factory):
    from purhie_b200.parts import build_plugin, load_plugin, unload_plugin
    path = build_plugin(os.path.join(ROOT, "tests", "toy_parts", "toy_parts.cu"), str(tmp_path_factory.mktemp("plugin")))
    load_plugin(path)
    yield path
    unload_plugin(path)


def test_toy_parts_alone_against_torch(toys, tmp_path):
    from purhie_b200.config import registered_architectures, registered_parts
    from purhie_b200.parts import PartProbe
    assert "toy_running_mean" in registered_parts("mixer") and "toy_top1" in registered_parts("feed_forward")
    assert "toy_scaled_rope" in registered_parts("position") and "toy_sandwich" in registered_parts("arrangement")
    assert "ToyForCausalLM" in registered_architectures()
    E = 24
    g = torch.Generator().manual_seed(2)
    # the stateful mixer: the mean carries over from step to step and from request to request not at all
    w = torch.randn(E, E, generator=g) * 0.3
    m = PartProbe("mixer", "toy_running_mean", {"hidden_size": E, "names": {"weight": "w"}})
    m.bind_folder(folder_with(tmp_path, {"w": w}))
    assert m.cache_need() == {"kind": "state", "kv_heads": 0, "head_dim": 0, "window": None, "state_shape": [E + 1]}
    m.mixer_cache(8, 4, max_requests=2)
    m.add_request(1); m.add_request(2)
    xa, xb = torch.randn(11, E, generator=g), torch.randn(6, E, generator=g)
    ref = lambda x: (torch.cumsum(x.double(), 0) / torch.arange(1, len(x) + 1)[:, None]) @ w.double().T
    outs_a = [m.mixer_step([(1, 4)], xa[:4].numpy()), m.mixer_step([(2, 6), (1, 5)], torch.cat([xb, xa[4:9]]).numpy())]
    outs_a.append(m.mixer_step([(1, 2)], xa[9:].numpy()))
    got_a = torch.from_numpy(np.concatenate([outs_a[0], outs_a[1][6:], outs_a[2]]))
    assert rel_err(got_a, ref(xa)) < 1e-5 and rel_err(torch.from_numpy(outs_a[1][:6]), ref(xb)) < 1e-5
    m.release(1); m.add_request(3)                                    # a new request in a used slot starts from zero
    assert rel_err(torch.from_numpy(m.mixer_step([(3, 11)], xa.numpy())), ref(xa)) < 1e-5
    # the routed feed-forward: the router's argmax picks the matrix
    f = PartProbe("feed_forward", "toy_top1", {"hidden_size": E, "experts": 3})
    tensors = {"toy.router": torch.randn(3, E, generator=g)}
    tensors.update({f"toy.expert{e}": torch.randn(E, E, generator=g) * 0.3 for e in range(3)})
    f.bind_folder(folder_with(tmp_path, tensors, "ff"))
    x = torch.randn(17, E, generator=g)
    choice = (x.double() @ tensors["toy.router"].double().T).argmax(-1)
    want = torch.stack([tensors[f"toy.expert{int(c)}"].double() @ x[t].double() for t, c in enumerate(choice)])
    assert len(set(choice.tolist())) == 3 and rel_err(torch.from_numpy(f.feed_forward(x.numpy())), want) < 1e-5
    # the scaled rotary table
    r = PartProbe("position", "toy_scaled_rope", {"theta": 1e4, "n_rot": 16, "factor": 4.0, "max_position": 128})
    r.bind_random(0)
    t = r.position_table()
    assert t.shape == (128, 16) and abs(t[100, 3] - math.cos(100 * 1e4 ** (-6 / 16) / 4.0)) < 1e-6


def test_toy_mixer_keeps_values_narrower_than_its_keys_in_pages(toys, tmp_path):
    """A mixer from the plugin that states keys of 12 and values of 5 elements: the cache manager gives it pages of
    that shape, and stepping it in portions and one token at a time, two requests side by side over pages that are
    handed out in turn, gives what causal attention over the whole sequences gives."""
    from purhie_b200.parts import PartProbe
    E, DK, DV = 20, 12, 5
    g = torch.Generator().manual_seed(4)
    w = {n: torch.randn(*shape, generator=g) * 0.4 for n, shape in (("wq", (DK, E)), ("wk", (DK, E)), ("wv", (DV, E)), ("wo", (E, DV)))}
    m = PartProbe("mixer", "toy_narrow_value_attention", {"hidden_size": E, "key_dim": DK, "value_dim": DV,
                                                           "names": {n: n for n in w}})
    m.bind_folder(folder_with(tmp_path, w, "narrow"))
    assert m.cache_need() == {"kind": "pages", "kv_heads": 1, "head_dim": DK, "value_dim": DV, "window": None, "state_shape": []}
    m.mixer_cache(4, 12, max_requests=2)                             # pages of 4 tokens

    def ref(x):
        x = x.double()
        q, k, v = x @ w["wq"].double().T, x @ w["wk"].double().T, x @ w["wv"].double().T
        s = (q @ k.T) / math.sqrt(DK)
        s = s.masked_fill(torch.triu(torch.ones(len(x), len(x), dtype=torch.bool), 1), float("-inf"))
        return torch.softmax(s, -1) @ v @ w["wo"].double().T

    xa, xb = torch.randn(14, E, generator=g), torch.randn(9, E, generator=g)
    m.add_request(1); m.add_request(2)
    a0 = m.mixer_step([(1, 6)], xa[:6].numpy())
    ba = m.mixer_step([(2, 9), (1, 3)], torch.cat([xb, xa[6:9]]).numpy())
    a2 = [m.mixer_step([(1, 1)], xa[i:i + 1].numpy()) for i in range(9, 14)]
    got_a = torch.from_numpy(np.concatenate([a0, ba[9:]] + a2))
    assert rel_err(got_a, ref(xa)) < 1e-5 and rel_err(torch.from_numpy(ba[:9]), ref(xb)) < 1e-5
    m.release(1); m.add_request(3)                                    # request 3 gets the pages request 1 gave back
    assert rel_err(torch.from_numpy(m.mixer_step([(3, 14)], xa.numpy())), ref(xa)) < 1e-5


def test_toy_architecture_is_registered_built_and_stepped(toys, tmp_path):
    from purhie_b200.config import load_config
    from purhie_b200.engine import Engine, StepEntry
    from purhie_b200.weights import expected_tensors, write_random_model
    cfg = {"architectures": ["ToyForCausalLM"], "hidden_size": 32, "vocab_size": 64}
    specs = expected_tensors(cfg)
    assert "l1.mean" in specs and "toy.expert2" in specs and "l1.post" in specs and specs["toy.router"].role == "vector"
    write_random_model(str(tmp_path), cfg, 3, std=0.3, scale_low=0.8, scale_high=1.2, dtype="float32")
    assert load_config(str(tmp_path)).architecture == "ToyForCausalLM"
    toks = random_tokens(50, 64, 9)
    eng = Engine.from_folder(str(tmp_path), dtype="float32", page_size=8, max_tokens=256, max_requests=3)
    info = eng.info()
    # the cache manager gave the stateful mixer a slot and the two owning attention calls one group
    assert info["needs"] == ["pages", "state", "pages", "none"]
    assert len(info["groups"]) == 1 and info["groups"][0]["entries"] == [0, 2] and info["state_entries"] == [1]
    eng.add_request("whole")
    whole = eng.step([StepEntry("whole", toks, list(range(50)))])
    assert np.isfinite(whole).all() and whole.std() > 0
    # cut into portions and mixed with another request: the same logits (the state carries over exactly)
    eng.add_request("cut"); eng.add_request("other")
    parts, i = [], 0
    for n in (7, 2, 1, 13, 1, 26):
        lg = eng.step([StepEntry("other", random_tokens(3, 64, i), []), StepEntry("cut", toks[i:i + n], list(range(n)))])
        parts.append(lg); i += n
    cut = np.concatenate(parts)
    assert rel_err(torch.from_numpy(cut), torch.from_numpy(whole)) < 1e-5
    # a new request in a reused slot starts from a zeroed state; single tokens replay a graph with the toy's kernels in it
    eng.release("whole"); eng.add_request("again")
    head = eng.step([StepEntry("again", toks[:40], list(range(40)))])
    tail = np.concatenate([eng.step([StepEntry("again", toks[40 + k:41 + k], [0])]) for k in range(10)])
    assert rel_err(torch.from_numpy(np.concatenate([head, tail])), torch.from_numpy(whole)) < 1e-5
    assert eng.info()["graph_replays"] > 0
    # the fourth call really reads the first call's cache: it owns no pages
    views = eng.info()["views"]
    assert views[3]["writable"] is False and views[3]["k_base"] == views[0]["k_base"] and views[2]["k_base"] != views[0]["k_base"]
    eng.close()


def test_the_run_order_is_data(toys):
    """The toy architecture's description comes back from the library as data: a layer named twice, a call that reads
    another call's cache, an arrangement with sub-parts of its own naming."""
    from purhie_b200.config import ModelConfig
    spec = ModelConfig.from_dict({"architectures": ["ToyForCausalLM"], "hidden_size": 32, "vocab_size": 64}).model_spec()
    assert [(c["layer"], c["cache_from"]) for c in spec["schedule"]] == [(0, None), (1, None), (0, None), (0, 0)]
    assert spec["layers"][1]["arrangement"] == "toy_sandwich" and "mixer_post_norm" in spec["layers"][1]["parts"]
    assert spec["layers"][0]["parts"]["mixer"]["params"]["position"]["kind"] == "toy_scaled_rope"
