"""Generation through the Python entry point (a thin layer over the C API), the request queue and the command line (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from plain import qwen3_plain as P
from helpers import ROOT, TINY, make_model, random_tokens

pytestmark = pytest.mark.gpu


def plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(P.forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in ("A", "B", "B0", "C"):
        folder = tmp_path_factory.mktemp(f"gen_{name}")
        cfg = make_model(folder, *TINY[name], "float32")
        out[name] = (str(folder), cfg) + P.read_model(str(folder))
    return out


@pytest.mark.parametrize("name,lengths,n_new", [("A", [1, 5, 17, 33], 8), ("B0", [2, 40, 97], 12), ("B", [2, 40, 97], 12)])
def test_greedy_generation_matches_the_plain_implementation(models, name, lengths, n_new):
    from purhie_b200.api import load_model
    from purhie_b200.sampling import SamplerParams
    folder, cfg, pc, pw = models[name]
    model = load_model(folder, dtype="float32")
    # prompts cut into chunks of 13 under a budget of 24 tokens when they go through the queue
    model.kv_cache_init(cfg.max_position_embeddings, max_sequences=4, page_size=TINY[name][1]["page_size"],
                        max_batch_tokens=24, prefill_chunk=13)
    prompts = [random_tokens(n, cfg.vocab_size, 50 + i) for i, n in enumerate(lengths)]
    expected = [plain_greedy(pc, pw, p, n_new) for p in prompts]
    # one at a time
    for p, exp in zip(prompts, expected):
        assert model.generate_ex(p, n_new, SamplerParams.greedy()) == exp
    # all at once through the scheduler
    before = model.engine_info()["scheduler_steps"]
    got = model.generate(prompts, max_new_tokens=n_new)
    assert got == expected
    assert model.engine_info()["scheduler_steps"] - before > n_new            # prompts really were cut
    assert model.last_stop_reasons == ["max_tokens"] * len(prompts)


def test_streams_join_mid_decode_and_sequences_do_not_disturb_each_other(models):
    from purhie_b200.api import GenOptions, load_model
    from purhie_b200.sampling import SamplerParams
    folder, cfg, pc, pw = models["B"]
    model = load_model(folder, dtype="float32")
    model.kv_cache_init(256, max_sequences=3, page_size=8)
    prompts = [random_tokens(n, cfg.vocab_size, 70 + i) for i, n in enumerate((2, 40, 97))]
    expected = [plain_greedy(pc, pw, p, 12) for p in prompts]
    opts = lambda: GenOptions(sampler=SamplerParams.greedy(), max_new_tokens=12, ignore_eog=True, prefill_chunk=13)
    streams = [model.stream_begin(prompts[0], opts())]
    silent = 0
    for step in range(40):
        if step == 3:                                      # the others join while the first decodes
            for p in prompts[1:]:
                model.seq_select(model.seq_new())
                streams.append(model.stream_begin(p, opts()))
        res = model.stream_step_batch(streams)
        silent += sum(1 for going, tok in res if going and tok is None)
        if all(s.done for s in streams):
            break
    assert [s.emitted for s in streams] == expected
    assert silent >= 97 // 13                              # steps that only prefilled a chunk emit nothing
    assert all(s.reason == "max_tokens" for s in streams)
    # a sequence continues where it stopped, and its logits are those after its last token
    model.seq_select(0)
    assert model.n_past() == 2 + 12
    ref = P.forward(pc, pw, prompts[0] + expected[0])[-1]
    lg = model.get_logits()
    assert np.abs(lg - ref.numpy()).max() < 1e-4 * float(ref.abs().max())
    more, reason = model.generate_stream([], GenOptions(sampler=SamplerParams.greedy(), max_new_tokens=3, ignore_eog=True))
    assert expected[0] + more == plain_greedy(pc, pw, prompts[0], 15)
    # a stream that is dropped half way gives the sequence back as far as it got
    model.seq_select(1)
    st = model.stream_begin(random_tokens(5, cfg.vocab_size, 1), opts())
    model.stream_step(st)
    st.free()
    assert model.n_past() == 40 + 12 + 5 + len(st.emitted)


def test_temperature_sampling_is_seeded_and_follows_the_host_chain(models):
    from purhie_b200.api import GenOptions, load_model
    from purhie_b200.sampling import Sampler, SamplerParams
    folder, cfg, pc, pw = models["B"]
    model = load_model(folder, dtype="float32")
    model.kv_cache_init(256, max_sequences=2, page_size=8)
    prompt = random_tokens(40, cfg.vocab_size, 81)
    sp = SamplerParams.pure_temperature(0.7, seed=1)
    a = model.generate_ex(prompt, 12, sp)
    b = model.generate_ex(prompt, 12, sp)
    c = model.generate_ex(prompt, 12, SamplerParams.pure_temperature(0.7, seed=2))
    assert a == b and a != c
    # the same tokens from the plain implementation's logits and the host sampler with the same seed
    s, toks = Sampler(sp), list(prompt)
    for _ in range(12):
        toks.append(s.sample(P.forward(pc, pw, toks)[-1].float().numpy()))
    assert toks[len(prompt):] == a
    # the full chain (top-k, top-p, min-p, penalty) runs on the host over the engine's logits
    full = SamplerParams(temperature=0.9, top_k=20, top_p=0.9, min_p=0.02, repeat_penalty=1.2, seed=3)
    d = model.generate_ex(prompt, 10, full)
    s, toks = Sampler(full), list(prompt)
    for t in prompt:
        s.accept(t)
    for _ in range(10):
        t = s.sample(P.forward(pc, pw, toks)[-1].float().numpy())
        s.accept(t); toks.append(t)
    assert toks[len(prompt):] == d
    # the chain with top-k on and no penalty runs in the device kernel and picks what the host chain picks
    dev = SamplerParams(temperature=0.9, top_k=20, top_p=0.9, min_p=0.02, seed=4)
    e = model.generate_ex(prompt, 10, dev)
    s, toks = Sampler(dev), list(prompt)
    for _ in range(10):
        toks.append(s.sample(P.forward(pc, pw, toks)[-1].float().numpy()))
    assert toks[len(prompt):] == e
    # a callback stops generation after the token it saw
    seen = []
    out, reason = model.generate_stream(prompt, GenOptions(sampler=SamplerParams.greedy(), max_new_tokens=30, ignore_eog=True,
                                                           on_token=lambda user, tok, text, n: (seen.append(tok), len(seen) >= 4)[1]))
    assert reason == "callback" and out == seen and len(out) == 4


@pytest.mark.parametrize("sampler", ["greedy", "chain", "temperature"])
def test_running_ahead_gives_the_tokens_and_the_stops_of_single_steps(models, sampler):
    """stream_run launches a step with the token ids the step before left on the device.  Compared with the same
    streams stepped one call at a time: equal tokens step by step, equal stop reasons, equal sequences and cache
    lengths; streams end by their budget at different steps and by an end-of-generation token (found out one step
    late: the token is taken back out of the cache)."""
    from purhie_b200.api import GenOptions, load_model
    from purhie_b200.sampling import SamplerParams
    folder, cfg, pc, pw = models["A"]
    prompts = [random_tokens(n, cfg.vocab_size, 90 + i) for i, n in enumerate((3, 21, 9, 30))]
    budgets = [7, 30, 30, 12]

    def params(i):
        if sampler == "greedy":
            return SamplerParams.greedy()
        if sampler == "temperature":
            return SamplerParams.pure_temperature(0.9, seed=i + 1)
        return SamplerParams(temperature=0.9, top_k=5, top_p=0.9, min_p=0.02, seed=i + 1)

    def run(ahead, eos):
        model = load_model(folder, dtype="float32")
        model.kv_cache_init(cfg.max_position_embeddings, max_sequences=4, page_size=TINY["A"][1]["page_size"])
        model.set_eog_tokens(eos)
        streams = []
        for i, (p, b) in enumerate(zip(prompts, budgets)):
            opts = GenOptions(sampler=params(i), max_new_tokens=b, ignore_eog=(i == 1))
            model.seq_select(model.seq_new() if i else 0)
            streams.append(model.stream_begin(p, opts))
        if ahead:
            steps = model.stream_run(streams, 40)
        else:
            steps = []
            while not all(st.done for st in streams):
                steps.append(model.stream_step_batch(streams))
        n_past, cached = [], []
        for st in streams:
            model.seq_select(st.seq)
            n_past.append(model.n_past())
            cached.append(model.sequence_length_in_cache(st.seq))
        graphs = model.engine_info()["graph_replays"]
        return steps, [st.emitted for st in streams], [st.reason for st in streams], n_past, cached, graphs

    # no end-of-generation ids first, then one that the longest stream is known to produce on the way
    base = run(False, [])
    eos = [base[1][2][5]]
    for eos_ids in ([], eos):
        a, b = run(False, eos_ids), run(True, eos_ids)
        assert a[0] == b[0] and a[1] == b[1] and a[2] == b[2]
        assert a[3] == b[3]
        # a sequence whose stream ended while a step was in flight has its last token in the cache already; the
        # end-of-generation token is in neither
        assert all(x <= y <= n for x, y, n in zip(a[4], b[4], b[3]))
        assert b[5] > 0
    assert len(set(base[2])) == 1 and "eog" in run(True, eos)[2]


def test_queue_running_ahead_changes_no_token(models):
    """The queue's decode phase launches steps with the ids the step before left on the device; requests of different
    lengths, a seeded chain sampler, an end-of-generation id on the way: the same outputs and stop reasons as with
    every step read before the next is launched."""
    from purhie_b200.api import load_model
    from purhie_b200.sampling import SamplerParams
    folder, cfg, pc, pw = models["B"]
    prompts = [random_tokens(n, cfg.vocab_size, 120 + i) for i, n in enumerate((5, 33, 18, 2))]

    def run(ahead, eos):
        model = load_model(folder, dtype="float32")
        model.kv_cache_init(256, max_sequences=4, page_size=8, max_batch_tokens=64, prefill_chunk=16, run_ahead=ahead)
        model.set_eog_tokens(eos)
        sp = SamplerParams(temperature=0.8, top_k=6, top_p=0.9, min_p=0.01)
        out = model.generate(prompts, max_new_tokens=25, params=sp, seed=40, ignore_eos=False)
        return out, model.last_stop_reasons, model.engine_info()["scheduler_steps"]

    base = run(False, [])
    for eos in ([], [base[0][1][9]]):
        a, b = run(False, eos), run(True, eos)
        assert a[0] == b[0] and a[1] == b[1]
        assert b[2] <= a[2] + 2                              # at most the step in flight when a request ended is extra
    assert "eog" in b[1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_run_out_on_the_device_and_every_request_still_gets_its_tokens(models, dtype, tmp_path):
    """Five greedy requests in a pool that holds about two of them: the scheduler preempts the newest, which starts
    over later on pages that others have used meanwhile (NaN-poisoned on the way), and every output is what the
    request gives alone."""
    from purhie_b200.api import load_model
    folder, cfg, pc, pw = models["B"]
    if dtype == "bfloat16":                                   # weights stored as bfloat16, so that the tensor-core products run
        folder = str(tmp_path)
        make_model(folder, *TINY["B"], "bfloat16")
        pc, pw = P.read_model(folder)
    prompts = [random_tokens(n, cfg.vocab_size, 300 + i) for i, n in enumerate((40, 23, 57, 9, 31))]
    n_new = 24
    model = load_model(folder, dtype=dtype)
    model.kv_cache_init(256, max_sequences=4, page_size=8, kv_tokens=160, max_batch_tokens=48, prefill_chunk=16, poison_cache=True)
    got = model.generate(prompts, max_new_tokens=n_new)
    info = model.engine_info()
    assert info["preemptions"] > 0 and info["free_pages"] == info["total_pages"]
    if dtype == "float32":
        assert got == [plain_greedy(pc, pw, p, n_new) for p in prompts]
    else:
        # bfloat16: teacher-forced through the plain implementation, every token is its best or within what the
        # tolerance of bfloat16 (3e-2 of the largest logit, on both logits) can swap
        for p, out in zip(prompts, got):
            assert len(out) == n_new
            logits = P.forward(pc, pw, p + out)
            for i, tok in enumerate(out):
                row = logits[len(p) - 1 + i]
                assert (row.max() - row[tok]).item() <= 2 * 3e-2 * row.abs().max().item(), (i, tok)


def test_prefix_reuse_context_full_and_errors(models):
    from purhie_b200.api import ERR_CONTEXT_FULL, ERR_INVALID_STATE, GenOptions, InferenceError, load_model
    from purhie_b200.sampling import SamplerParams
    folder, cfg, pc, pw = models["A"]
    model = load_model(folder, dtype="float32")
    with pytest.raises(InferenceError) as e:
        model.prefill([1, 2])
    assert e.value.code == ERR_INVALID_STATE
    model.kv_cache_init(64, max_sequences=2)
    p1 = random_tokens(30, 256, 5)
    greedy = SamplerParams.greedy()
    out1, _ = model.generate_stream(p1, GenOptions(sampler=greedy, max_new_tokens=4, ignore_eog=True))
    # a re-rendered prompt that shares 20 tokens: only the rest is prefilled
    p2 = p1[:20] + random_tokens(9, 256, 6)
    out2, _ = model.generate_stream(p2, GenOptions(sampler=greedy, max_new_tokens=4, ignore_eog=True, reuse_prefix=True))
    assert model.last_prompt_stats() == (20, 9) and out2 == plain_greedy(pc, pw, p2, 4)
    # the context fills: a stop reason, not an error
    model.reset()
    out3, reason = model.generate_stream(random_tokens(60, 256, 7), GenOptions(sampler=greedy, max_new_tokens=50, ignore_eog=True))
    assert reason == "context_full" and len(out3) == 4 and model.n_past() == 64
    with pytest.raises(InferenceError) as e:
        model.prefill([1])
    assert e.value.code == ERR_CONTEXT_FULL
    # all-row logits and the greedy decode_token loop agree
    model.reset()
    lg = model.prefill_logits(p1)
    assert lg.shape == (30, 256)
    nxt = int(lg[-1].argmax())
    assert model.decode_token(nxt) == plain_greedy(pc, pw, p1, 2)[1]
    assert model.vocab_size() == 256 and model.hidden_size() == 64 and model.n_ctx() == 64 and model.max_position() == 128
    # a prefill that cannot be fed leaves the sequence where the cache is
    small = load_model(folder, dtype="float32")
    small.kv_cache_init(128, max_sequences=1, page_size=16, kv_tokens=32)
    small.set_prefill_batch(16)
    with pytest.raises(InferenceError) as e:
        small.prefill(random_tokens(50, 256, 8))
    assert e.value.code == ERR_CONTEXT_FULL
    assert small.n_past() == small.sequence_length_in_cache(0) == 32


def test_qwen_demo_command_line(models, tmp_path):
    folder, cfg, pc, pw = models["C"]
    demo = [sys.executable, os.path.join(ROOT, "bin", "qwen_demo")]
    prompt = random_tokens(20, cfg.vocab_size, 33)
    exp = plain_greedy(pc, pw, prompt, 5)
    (tmp_path / "p.txt").write_text(" ".join(map(str, prompt)))
    for arg in (",".join(map(str, prompt)), "@" + str(tmp_path / "p.txt")):
        r = subprocess.run(demo + [folder, arg, "5", "--dtype", "float32", "--ctx", "128"], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr
        lines = r.stdout.strip().splitlines()
        assert lines[0].startswith("Sampling: temp 0 ")
        assert [int(x) for x in lines[2:7]] == exp
        assert lines[-1].startswith("Timing: prefill 20 tokens")
    r = subprocess.run(demo + [folder, "1,2", "--kv-q8"], capture_output=True, text=True)
    assert r.returncode == 1 and "--kv-q8" in r.stderr
    # with PURHIE_PROFILE=1 the same tokens, and the device time per kernel class at the end
    r = subprocess.run(demo + [folder, ",".join(map(str, prompt)), "5", "--dtype", "float32", "--ctx", "128"], capture_output=True,
                       text=True, timeout=300, env=dict(os.environ, PURHIE_PROFILE="1"))
    assert r.returncode == 0, r.stderr
    assert [int(x) for x in r.stdout.strip().splitlines()[2:7]] == exp
    prof = [l for l in r.stderr.splitlines() if l.startswith("[profile]")]
    names = {l.split()[1] for l in prof[1:]}
    assert {"gemm_simple", "add_rmsnorm", "qk_norm_rope_kv_write", "attention_generic", "embed_gather", "argmax"} <= names
    gemm = next(l for l in prof if " gemm_simple " in l)
    assert "GB/s" in gemm and "TFLOP/s" in gemm               # the products note their bytes and flops
    # several prompts, one a line, through the request queue with a small budget and a small page
    other = random_tokens(45, cfg.vocab_size, 34)
    (tmp_path / "many.txt").write_text(" ".join(map(str, prompt)) + "\n" + ",".join(map(str, other)) + "\n")
    r = subprocess.run(demo + [folder, "--tokens-file", str(tmp_path / "many.txt"), "5", "--dtype", "float32", "--ctx", "128",
                               "--block-size", "8", "--max-batch-tokens", "32", "--chunk", "16", "--ignore-eos"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    rows = [l for l in r.stdout.splitlines() if l.startswith("Request ")]
    assert [int(x) for x in rows[0].split("):")[1].split()] == exp
    assert [int(x) for x in rows[1].split("):")[1].split()] == plain_greedy(pc, pw, other, 5)
    assert "Timing: 2 requests, 65 prompt tokens and 10 generated tokens" in r.stdout
    # random weights from a configuration file: the tokens of the folder written with the same seed
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TINY["C"][0]))
    init = TINY["C"][1]
    make_model(tmp_path / "same", dict(TINY["C"][0]), dict(init, scale_low=1.0, scale_high=1.0, std=0.02), "float32")
    pc2, pw2 = P.read_model(str(tmp_path / "same"))
    r = subprocess.run(demo + ["--random", str(cfg_path), "--weights-seed", str(init["seed"]), "--tokens", ",".join(map(str, prompt)),
                               "5", "--dtype", "float32", "--ctx", "128"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [int(x) for x in r.stdout.strip().splitlines()[2:7]] == plain_greedy(pc2, pw2, prompt, 5)
