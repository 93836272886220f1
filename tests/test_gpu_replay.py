"""The engine against the plain implementation under every way of cutting the work (GPU).

For each tiny configuration and for float32 and bfloat16: each request alone and whole; most of it in one step and
the last 32 tokens one by one; portions of changing size down to two tokens; and up to four live requests mixed in
one batch with so few pages that they are used again.  float32 must agree with the plain implementation to 1e-4 of
the largest logit with the same argmax everywhere; bfloat16 to 3e-2, a different argmax only where the tolerance can
explain it.  Nothing is widened to pass.
"""
import pytest
import torch

from plain import qwen3_plain as P
from helpers import (TINY, TraceRun, engine_runner, make_model, random_tokens, rel_err, run_schedule,
                     same_top1_or_near_tie, schedule_mixed, schedule_portions, schedule_tail, schedule_whole)

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [1, 5, 17, 33, 64, 97, 120], "B": [2, 40, 97, 16, 130, 9, 250], "B0": [2, 40, 97, 16, 130, 9, 250],
           "C": [3, 70, 200, 31, 129, 48]}
TOL = {"float32": 1e-4, "bfloat16": 3e-2}
_cache = {}


def setup(name, dtype, tmp_path_factory):
    """(model folder, requests, plain logits) for a configuration; weights stored in the run's dtype."""
    key = (name, dtype)
    if key not in _cache:
        cfg_dict, init = TINY[name]
        folder = tmp_path_factory.mktemp(f"model_{name}_{dtype}")
        cfg = make_model(folder, cfg_dict, init, dtype)
        reqs = {f"r{i}": random_tokens(n, cfg.vocab_size, 100 + i) for i, n in enumerate(LENGTHS[name])}
        pc, pw = P.read_model(str(folder))
        ref = {rid: P.forward(pc, pw, toks) for rid, toks in reqs.items()}
        _cache[key] = (str(folder), reqs, ref, init["page_size"])
    return _cache[key]


def check(got, ref, dtype, what):
    for rid in ref:
        assert got[rid].shape == ref[rid].shape, (what, rid)
        err = rel_err(got[rid], ref[rid])
        assert err < TOL[dtype], f"{what} {rid}: relative error {err:.3e}"
        if dtype == "float32":
            assert torch.equal(got[rid].argmax(-1), ref[rid].argmax(-1)), f"{what} {rid}: argmax"
        else:
            assert not same_top1_or_near_tie(got[rid], ref[rid], TOL[dtype]), f"{what} {rid}: argmax differs away from a tie"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "B0", "C"])
def test_every_way_of_cutting_agrees_with_the_plain_implementation(name, dtype, tmp_path_factory):
    from purhie_b200.engine import Engine
    folder, reqs, ref, page = setup(name, dtype, tmp_path_factory)
    longest = max(len(t) for t in reqs.values())
    results = {}
    for mode, steps, max_tokens in (
            ("whole", schedule_whole(reqs), 256),
            ("tail32", schedule_tail(reqs), 256),
            ("portions", schedule_portions(reqs), 256),
            # four live requests in a pool that cannot hold all requests at once: pages are used again
            ("mixed", schedule_mixed(reqs, seed=3), 4 * (-(-longest // 64) * 64))):
        eng = Engine.from_folder(folder, dtype=dtype, page_size=page, max_tokens=max_tokens, max_requests=4,
                                 poison_cache=True)
        step, release = engine_runner(eng)
        results[mode] = run_schedule(step, release, steps)
        check(results[mode], ref, dtype, f"{name}/{dtype}/{mode}")
        eng.check_cache()
        assert eng.free_pages() == eng.total_pages()
        eng.close()
    if dtype == "float32":
        # the 32-bit path fixes the order of every sum: cutting changes nothing at all
        for mode in ("tail32", "portions", "mixed"):
            for rid in ref:
                assert torch.equal(results[mode][rid], results["whole"][rid]), f"{name}/{mode}/{rid} not bit-equal"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, tmp_path_factory, tmp_path):
    """bin/trace_run as a user drives it: a subprocess, JSON lines in, .f32 files and ``done`` lines out."""
    folder, reqs, ref, page = setup("B", dtype, tmp_path_factory)
    tr = TraceRun(folder, dtype, tmp_path / "out", max_tokens=4 * 256, extra=["--page-size", str(page)])
    try:
        got = run_schedule(lambda k, entries, end: tr.step(k, entries, end), None, schedule_mixed(reqs, seed=11))
    finally:
        tr.close()
    check(got, ref, dtype, f"trace_run/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_dumps_find_the_first_wrong_layer_by_bisection(dtype, tmp_path):
    """``trace_run --dump-layers`` writes the residual stream after every entry of the run order.  A folder whose
    layers 3 and 4 have changed places is replayed, a prompt whole and then its last tokens one by one; halving the
    range of layers against the plain implementation's per-layer outputs lands on layer 3, in the prompt step and in
    a decode step, and on no layer for the folder as it was written."""
    import json
    import os
    import numpy as np
    from safetensors import safe_open
    from safetensors.torch import save_file
    cfg_dict = dict(TINY["A"][0], num_hidden_layers=6)
    good, swapped = tmp_path / "good", tmp_path / "swapped"
    cfg = make_model(good, cfg_dict, TINY["A"][1], dtype)
    os.makedirs(swapped)
    tensors = {}
    with safe_open(str(good / "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            other = name.replace("layers.3.", "layers.#.").replace("layers.4.", "layers.3.").replace("layers.#.", "layers.4.")
            tensors[other] = f.get_tensor(name).contiguous()
    save_file(tensors, str(swapped / "model.safetensors"))
    (swapped / "config.json").write_text((good / "config.json").read_text())
    toks = random_tokens(45, cfg.vocab_size, 5)
    pc, pw = P.read_model(str(good))
    layers = []
    P.forward(pc, pw, toks, layer_outputs=layers)
    L, E = cfg.num_hidden_layers, cfg.hidden_size
    tol = 1e-4 if dtype == "float32" else 3e-2

    def first_wrong(folder):
        out = tmp_path / f"out_{folder.name}"
        tr = TraceRun(folder, dtype, out, max_tokens=128, extra=["--dump-layers"])
        try:
            tr.step(0, [("a", toks[:40], [])])
            for k in range(40, 45):
                tr.step(k, [("a", toks[k:k + 1], [0])])
        finally:
            tr.close()

        def wrong(step, rows, layer):
            got = torch.from_numpy(np.fromfile(out / f"{step}.layer{layer}.f32", dtype="<f4").reshape(-1, E).copy())
            return rel_err(got, layers[layer][rows]) > tol

        found = []
        for step, rows in ((0, slice(0, 40)), (44, slice(44, 45))):
            if not wrong(step, rows, L - 1):
                found.append(None)
                continue
            lo, hi = 0, L - 1                     # the first wrong layer lies in [lo, hi]
            while lo < hi:
                mid = (lo + hi) // 2
                if wrong(step, rows, mid):
                    hi = mid
                else:
                    lo = mid + 1
            found.append(lo)
        return found

    assert first_wrong(good) == [None, None]
    assert first_wrong(swapped) == [3, 3]


def test_first_tokens_and_long_decoding(tmp_path_factory):
    """The first tokens of a sequence (positions 0, 1, 2 one by one) and 250 decoded tokens in a row."""
    from purhie_b200.engine import Engine
    for dtype in ("float32", "bfloat16"):
        folder, reqs, ref, page = setup("B", dtype, tmp_path_factory)
        toks = reqs["r6"]
        eng = Engine.from_folder(folder, dtype=dtype, page_size=page, max_tokens=256, max_requests=2)
        step, release = engine_runner(eng)
        steps = [([("r6", toks[i:i + 1], [0])], []) for i in range(len(toks))]
        got = run_schedule(step, release, steps)
        check(got, {"r6": ref["r6"]}, dtype, f"token by token/{dtype}")
        info = eng.info()
        assert info["graphs"] >= 1 and info["graph_replays"] > 200
        eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_batches_replayed_as_graphs_give_the_logits_of_single_launches(dtype, tmp_path_factory):
    """Three requests decoding side by side, some rows wanted and some not: with CUDA graphs the steps replay a graph
    per (batch size, table width, context bucket), without them every kernel is launched by the host; the logits are
    equal (the same bits in float32) and agree with the plain implementation."""
    from purhie_b200.engine import Engine, StepEntry
    folder, reqs, ref, page = setup("B", dtype, tmp_path_factory)
    names = ["r2", "r4", "r6"]                                     # 97, 130 and 250 tokens
    heads = {"r2": 20, "r4": 3, "r6": 200}

    def run(graphs):
        eng = Engine.from_folder(folder, dtype=dtype, page_size=page, max_tokens=1024, max_requests=4, cuda_graphs=graphs)
        for rid in names:
            eng.add_request(rid)
            eng.step([StepEntry(rid, reqs[rid][:heads[rid]], [])])
        rows = {rid: [] for rid in names}
        for k in range(40):
            live = [rid for rid in names if not (rid == "r4" and k % 3 == 2)]      # one request sits a step out now and then
            pos = {rid: eng.length(rid) for rid in live}
            want = {rid: ([0] if (k + len(rid)) % 4 else []) for rid in live}
            if not any(want.values()):
                want[live[0]] = [0]
            lg = eng.step([StepEntry(rid, [reqs[rid][pos[rid]]], want[rid]) for rid in live])
            i = 0
            for rid in live:
                if want[rid]:
                    rows[rid].append((pos[rid], torch.from_numpy(lg[i].copy())))
                    i += 1
        n_graphs = eng.info()["graphs"]
        eng.close()
        return rows, n_graphs

    plain_rows, g0 = run(False)
    graph_rows, g1 = run(True)
    assert g0 == 0 and g1 >= 2                                    # two batch sizes at least
    for rid in names:
        assert [p for p, _ in plain_rows[rid]] == [p for p, _ in graph_rows[rid]]
        a = torch.stack([r for _, r in plain_rows[rid]])
        b = torch.stack([r for _, r in graph_rows[rid]])
        want = torch.stack([ref[rid][p] for p, _ in graph_rows[rid]])
        if dtype == "float32":
            assert torch.equal(a, b)
        check({rid: b}, {rid: want}, dtype, f"graph replay/{dtype}")
        check({rid: a}, {rid: want}, dtype, f"launch by launch/{dtype}")


def test_step_refuses_bad_batches_and_leaves_the_cache_alone(tmp_path_factory):
    from purhie_b200.engine import Engine, OutOfPages, StepEntry, StepError
    folder, reqs, ref, page = setup("A", "float32", tmp_path_factory)
    eng = Engine.from_folder(folder, dtype="float32", page_size=16, max_tokens=64, max_requests=2)
    eng.add_request("a"); eng.add_request("b")
    with pytest.raises(StepError):
        eng.step([StepEntry("a", [1, 2, 999], [0])])                # token outside the vocabulary
    with pytest.raises(StepError):
        eng.step([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])])
    with pytest.raises(StepError):
        eng.step([StepEntry("zz", [1], [0])])
    with pytest.raises(StepError):
        eng.step([StepEntry("a", [1, 2], [2])])
    with pytest.raises(StepError):
        eng.step([StepEntry("a", list(range(129)), [])])             # past max_position_embeddings
    eng.step([StepEntry("a", list(range(40)), [])])
    free = eng.free_pages()
    with pytest.raises(OutOfPages):
        eng.step([StepEntry("b", list(range(10)), []), StepEntry("a", list(range(30)), [])])
    assert eng.free_pages() == free and eng.length("a") == 40 and eng.length("b") == 0
    eng.check_cache()


def test_a_kernel_that_gave_up_on_a_wait_is_reported_not_passed_on(tmp_path_factory):
    """The tensor-core kernels bound their waits and report giving up through an error word on the device.  The
    engine reads the words with every result it hands out; a non-zero word raises instead of returning logits."""
    from purhie_b200 import native
    from purhie_b200.engine import Engine, KernelError, StepEntry
    folder, reqs, ref, page = setup("B", "bfloat16", tmp_path_factory)
    eng = Engine.from_folder(folder, dtype="bfloat16", page_size=page, max_tokens=256, max_requests=2)
    eng.add_request("a")
    assert eng.step([StepEntry("a", reqs["r1"][:8], [7])]) is not None
    native.check(native.lib().qe_engine_set_error_word(eng.handle, 1, 112))
    with pytest.raises(KernelError) as e:
        eng.step([StepEntry("a", reqs["r1"][8:9], [0])])
    assert "waited too long" in str(e.value)
    assert eng.step([StepEntry("a", reqs["r1"][9:10], [0])]) is not None       # the word was cleared: the engine goes on


@pytest.mark.parametrize("seed", [3, 5, 8, 13, 21, 35])
def test_drawn_configurations_and_schedules(seed, tmp_path):
    """Configurations drawn at random (head sizes 16 to 128 in steps of 16, one to four groups of one to eight heads,
    widths and vocabularies that are no power of two, windows on some layers, pages of 8 to 32 tokens) under drawn
    schedules, in both precisions.  In float32 a different argmax is accepted only where the plain implementation's
    two best logits are within 2e-4 of the largest."""
    import random
    from purhie_b200.engine import Engine
    rng = random.Random(seed)
    D = rng.choice([16, 32, 64, 64, 128, 128, 48, 80])
    HKV = rng.choice([1, 2, 3, 4])
    L = rng.randint(1, 3)
    cfg_dict = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=L, hidden_size=8 * rng.randint(4, 40),
                    intermediate_size=8 * rng.randint(6, 80), num_attention_heads=HKV * rng.choice([1, 2, 3, 4, 5, 8]),
                    num_key_value_heads=HKV, head_dim=D, vocab_size=rng.randint(100, 3000), max_position_embeddings=512,
                    rope_theta=rng.choice([1e4, 1e6]), rms_norm_eps=rng.choice([1e-6, 1e-5]),
                    tie_word_embeddings=rng.random() < 0.5, attention_bias=rng.random() < 0.3)
    if rng.random() < 0.5:
        cfg_dict.update(layer_types=[rng.choice(["full_attention", "sliding_attention"]) for _ in range(L)],
                        sliding_window=rng.choice([8, 24, 40, 100, 200]))
    init = dict(seed=seed, std=rng.choice([0.02, 0.05]), scale_low=0.8, scale_high=1.2, page_size=rng.choice([8, 16, 32]))
    lengths = [rng.choice([1, 2, 3, 17, 33, 64, 65, 127, 128, 129, 200, 255, 256, 257, 300, 400, 511])
               for _ in range(rng.randint(3, 5))]
    sizes = [rng.choice([1, 2, 3, 5, 8, 13, 16, 17, 31, 64, 100, 130]) for _ in range(11)]
    for dtype in ("float32", "bfloat16"):
        folder = tmp_path / dtype
        cfg = make_model(folder, cfg_dict, init, dtype)
        reqs = {f"r{i}": random_tokens(n, cfg.vocab_size, 1000 * seed + i) for i, n in enumerate(lengths)}
        pc, pw = P.read_model(str(folder))
        ref = {rid: P.forward(pc, pw, toks) for rid, toks in reqs.items()}
        for mode, steps, max_tokens in (("tail32", schedule_tail(reqs), 512),
                                        ("portions", schedule_portions(reqs, sizes=sizes), 512),
                                        ("mixed", schedule_mixed(reqs, seed=seed), 4 * (-(-max(lengths) // 64) * 64))):
            eng = Engine.from_folder(str(folder), dtype=dtype, page_size=init["page_size"], max_tokens=max_tokens,
                                     max_requests=4, poison_cache=True)
            step, release = engine_runner(eng)
            got = run_schedule(step, release, steps)
            for rid in ref:
                what = f"seed {seed} {cfg_dict} {dtype}/{mode}/{rid}"
                assert rel_err(got[rid], ref[rid]) < TOL[dtype], what
                assert not same_top1_or_near_tie(got[rid], ref[rid], TOL[dtype]), what
            eng.check_cache()
            eng.close()
