"""Generation through the Python entry point, the scheduler and the command line (GPU)."""
import os
import subprocess
import sys

import pytest
import torch

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
    for name in ("A", "B", "C"):
        folder = tmp_path_factory.mktemp(f"gen_{name}")
        cfg = make_model(folder, *TINY[name], "float32")
        out[name] = (str(folder), cfg) + P.read_model(str(folder))
    return out


@pytest.mark.parametrize("name,lengths,n_new", [("A", [1, 5, 17, 33], 8), ("B", [2, 40, 97], 12)])
def test_greedy_generation_matches_the_plain_implementation(models, name, lengths, n_new):
    from purhie_b200.api import load_model
    from purhie_b200.sampling import SamplerParams
    folder, cfg, pc, pw = models[name]
    model = load_model(folder, dtype="float32")
    model.kv_cache_init(cfg.max_position_embeddings, max_sequences=4, page_size=TINY[name][1]["page_size"])
    prompts = [random_tokens(n, cfg.vocab_size, 50 + i) for i, n in enumerate(lengths)]
    expected = [plain_greedy(pc, pw, p, n_new) for p in prompts]
    # one at a time
    for p, exp in zip(prompts, expected):
        assert model.generate_ex(p, n_new, SamplerParams.greedy()) == exp
    # all at once through the scheduler, prompts cut into chunks of 13 under a budget of 24 tokens
    got = model.generate(prompts, max_new_tokens=n_new, max_batch_tokens=24, prefill_chunk=13)
    assert got == expected
    assert model.last_scheduler.steps > n_new            # prompts really were cut


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
    # logits of the last token are kept per sequence, and a sequence continues where it stopped
    model.seq_select(0)
    assert model.n_past() == 2 + 12
    more, reason = model.generate_stream([], GenOptions(sampler=SamplerParams.greedy(), max_new_tokens=3, ignore_eog=True))
    assert expected[0] + more == plain_greedy(pc, pw, prompts[0], 15)


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


@pytest.mark.parametrize("sampler", ["greedy", "chain", "temperature"])
def test_running_ahead_gives_the_tokens_the_stops_and_the_draws_of_single_steps(models, sampler):
    """stream_run launches a step with the token ids the step before left on the device.  Compared with the
    same streams stepped one call at a time: equal tokens step by step, equal stop reasons, equal sequences, and
    samplers that go on with equal draws; streams end by their budget at different steps, by an end-of-generation
    token (found out one step late: the token is taken back out of the cache) and by a callback."""
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
        model.eos_ids = eos
        streams = []
        for i, (p, b) in enumerate(zip(prompts, budgets)):
            stop_at = (lambda user, tok, text, n, seen=[]: (seen.append(tok), len(seen) >= 9)[1]) if i == 2 else None
            opts = GenOptions(sampler=params(i), max_new_tokens=b, ignore_eog=(i == 1), on_token=stop_at)
            model.seq_select(model.seq_new() if i else 0)
            streams.append(model.stream_begin(p, opts))
        if ahead:
            steps = model.stream_run(streams, 40)
        else:
            steps = []
            while not all(st.done for st in streams):
                steps.append(model.stream_step_batch(streams))
        tail = [st.sampler.uniform() for st in streams]
        seqs = [list(model._seqs[st.seq].tokens) for st in streams]
        lengths = [model.engine.length(("seq", st.seq)) for st in streams]
        logits = [model._seqs[st.seq].logits.clone() for st in streams]
        return steps, [st.emitted for st in streams], [st.reason for st in streams], tail, seqs, lengths, logits

    # no end-of-generation ids first, then one that the longest stream is known to produce on the way
    base = run(False, [])
    eos = [base[1][3][5]]
    for eos_ids in ([], eos):
        a, b = run(False, eos_ids), run(True, eos_ids)
        assert a[0] == b[0] and a[1] == b[1] and a[2] == b[2]
        assert a[3] == b[3]                                  # the generators stand where they would
        assert a[4] == b[4] and a[5] == b[5]
        for x, y in zip(a[6], b[6]):
            assert torch.equal(x, y)
    assert any(len(set(r)) > 1 for r in [base[2]])           # the streams did end for different reasons


def test_scheduler_running_ahead_changes_no_token(models):
    """The scheduler's decode phase launches steps with the ids the step before left on the device; requests of
    different budgets, a seeded chain sampler, an end-of-generation id on the way: the same outputs and stop reasons
    as with every step read before the next is launched."""
    from purhie_b200.api import load_model
    from purhie_b200.engine.scheduler import Request, Scheduler
    from purhie_b200.sampling import SamplerParams
    folder, cfg, pc, pw = models["B"]
    prompts = [random_tokens(n, cfg.vocab_size, 120 + i) for i, n in enumerate((5, 33, 18, 2))]
    budgets = [6, 25, 14, 25]

    def run(ahead, eos):
        model = load_model(folder, dtype="float32")
        model.kv_cache_init(256, max_sequences=4, page_size=8)
        eng = model.engine
        eng.release(("seq", 0))
        sched = Scheduler(eng, max_batch_tokens=64, prefill_chunk=16, n_ctx=256)
        sched.run_ahead = ahead
        for i, (p, b) in enumerate(zip(prompts, budgets)):
            sp = SamplerParams(temperature=0.8, top_k=6, top_p=0.9, min_p=0.01, seed=40 + i)
            sched.add(Request(("r", i), list(p), sp, b, eos, False))
        done = sched.run()
        return [(done[("r", i)].output, done[("r", i)].stop_reason) for i in range(4)], sched.steps

    base, _ = run(False, [])
    for eos in ([], [base[1][0][9]]):
        a, steps_a = run(False, eos)
        b, steps_b = run(True, eos)
        assert a == b
        assert steps_b <= steps_a + 2                        # at most the step in flight when a request ended is extra


def test_pages_run_out_on_the_device_and_every_request_still_gets_its_tokens(models):
    """Five greedy requests in a pool that holds about two of them: the scheduler preempts the newest, which starts
    over later on pages that others have used meanwhile, and every output is what the request gives alone."""
    from purhie_b200.api import load_model
    from purhie_b200.engine.scheduler import Request, Scheduler
    from purhie_b200.sampling import SamplerParams
    folder, cfg, pc, pw = models["B"]
    prompts = [random_tokens(n, cfg.vocab_size, 300 + i) for i, n in enumerate((40, 23, 57, 9, 31))]
    n_new = 24
    expected = [plain_greedy(pc, pw, p, n_new) for p in prompts]
    model = load_model(folder, dtype="float32")
    model.kv_cache_init(256, max_sequences=4, page_size=8, kv_tokens=160)
    eng = model.engine
    eng.release(("seq", 0))
    sched = Scheduler(eng, max_batch_tokens=48, prefill_chunk=16, n_ctx=256)
    for i, p in enumerate(prompts):
        sched.add(Request(("r", i), list(p), SamplerParams.greedy(), n_new, [], True))
    done = sched.run()
    assert [done[("r", i)].output for i in range(5)] == expected
    assert sched.preemptions > 0
    eng.cache.check()
    assert eng.cache.free_pages() == [g.allocator.num_pages for g in eng.cache.groups]


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
    assert model.last_prompt_stats == (20, 9) and out2 == plain_greedy(pc, pw, p2, 4)
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
    assert model.vocab_size() == 256 and model.hidden_size() == 64 and model.n_ctx() == 64


def test_qwen_demo_command_line(models, tmp_path):
    folder, cfg, pc, pw = models["C"]
    prompt = random_tokens(20, cfg.vocab_size, 33)
    exp = plain_greedy(pc, pw, prompt, 5)
    (tmp_path / "p.txt").write_text(" ".join(map(str, prompt)))
    for arg in (",".join(map(str, prompt)), "@" + str(tmp_path / "p.txt")):
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen_demo"), folder, arg, "5", "--dtype", "float32",
                            "--ctx", "128"], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr
        lines = r.stdout.strip().splitlines()
        assert lines[0].startswith("Sampling: temp 0 ")
        assert [int(x) for x in lines[2:7]] == exp
        assert lines[-1].startswith("Timing: prefill 20 tokens")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen_demo"), folder, "1,2", "--kv-q8"], capture_output=True, text=True)
    assert r.returncode == 1 and "--kv-q8" in r.stderr
