"""The engine at real layer sizes (GPU): float32 against the plain implementation, bfloat16 against float32.

The tiny configurations of the other tests leave paths untouched that only real sizes reach: a decode row whose
context is cut into more splits than it has blocks to fill, products on pairs of CTAs, K in parts, attention tiles
shared by several CTAs, sums over 12,288 terms.  Two layers of an 8B-class shape (hidden 4096, 32 query heads over 8
kv heads of 128, feed-forward 12288), of a 0.6B-class shape (hidden 1024 under a query width of 2048, tied
embeddings) and of a 32B-class shape (hidden 5120, groups of eight query heads, feed-forward 25600) with random
weights and the vocabulary cut to 32,000.
"""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPE = dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_hidden_layers=2, num_attention_heads=32,
             num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=32000, rms_norm_eps=1e-6,
             rope_theta=1000000.0, max_position_embeddings=8192, tie_word_embeddings=False, attention_bias=False)
SHAPES = {"8b": SHAPE,
          "0.6b": dict(SHAPE, hidden_size=1024, num_attention_heads=16, intermediate_size=3072, tie_word_embeddings=True),
          "32b": dict(SHAPE, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)}


def rel(a, b):
    a, b = torch.as_tensor(a).double(), torch.as_tensor(b).double()
    return float((a - b).norm() / b.norm())


def ids(n, seed, vocab=32000):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_every_way_of_feeding_is_as_close_to_float32_as_a_whole_prompt(shape):
    from purhie_b200.engine import Engine, StepEntry
    toks = ids(2700, 11)
    others = [ids(n + 24, 20 + i) for i, n in enumerate((17, 300, 1000, 2047, 64, 129, 700))]
    out = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_random(SHAPES[shape], 7, dtype=dtype, page_size=16, max_tokens=16384, max_requests=8)
        res = {}
        eng.add_request("w")
        res["whole"] = eng.step([StepEntry("w", toks[:2524], list(range(2499, 2524)))])      # from the prompt's last place on
        eng.release("w")
        # one request decoding alone at 2,500 tokens: its context is cut into more splits than it has blocks for
        eng.add_request("d")
        eng.step([StepEntry("d", toks[:2500], [])])
        res["decode"] = np.concatenate([eng.step([StepEntry("d", [toks[2500 + k]], [0])]) for k in range(24)])
        # ... then beside seven others of other lengths, and beside a prompt that comes in chunks
        for i, o in enumerate(others):
            eng.add_request(i)
            eng.step([StepEntry(i, o[:len(o) - 24], [])])
        rows = []
        for k in range(24):
            ent = [StepEntry("d", [toks[2524 + k]], [0])] + [StepEntry(i, [o[len(o) - 24 + k]], []) for i, o in enumerate(others)]
            rows.append(eng.step(ent))
        res["batch"] = np.concatenate(rows)
        for i in range(len(others)):
            eng.release(i)
        # a short portion late in the context: one attention tile that looks back over 2,600 keys, shared by several CTAs
        res["late"] = eng.step([StepEntry("d", toks[2548:2600], [0, 25, 51])])
        eng.add_request("c")
        for s in range(0, 2500, 500):
            lg = eng.step([StepEntry("c", toks[s:s + 500], [499] if s + 500 >= 2500 else [])])
        res["chunks"] = lg
        out[dtype] = res
        eng.close()
    f32, b16 = out["float32"], out["bfloat16"]
    assert np.array_equal(f32["whole"][1:], f32["decode"])               # float32: the same bits however it is fed
    assert np.array_equal(f32["whole"][:1], f32["chunks"])
    whole = rel(b16["whole"], f32["whole"])
    assert whole < 3e-2
    for name, want in (("decode", f32["whole"][1:]), ("chunks", f32["whole"][:1])):
        err = rel(b16[name], want)
        assert err < 1.5 * whole + 2e-3, f"{name}: {err:.3e} against {whole:.3e} for a whole prompt"
    # the batch continues the same request for 24 more tokens, the late portion for 52 more: compare with the float32
    # engine's own
    for name in ("batch", "late"):
        err = rel(b16[name], f32[name])
        assert err < 1.5 * whole + 2e-3, f"{name}: {err:.3e} against {whole:.3e}"
        assert not np.isnan(b16[name]).any()


@pytest.mark.parametrize("n_decode,portion", [(8, 512), (32, 512), (32, 480)])
def test_a_prompt_portion_beside_decode_rows_at_real_layer_sizes(n_decode, portion):
    """One step with decode rows beside a prompt portion at the 8B-class layer shape: 520 or 544 rows through the
    products on CTA pairs, the portion through the tcgen05 attention and the decode rows through the split-key
    attention, all in one pass.  float32 gives the bits of the same tokens fed in steps of their own; bfloat16 stays
    as close to float32 as it is for a whole prompt."""
    from purhie_b200.engine import Engine, StepEntry
    prompt = ids(1024 + portion, 5)
    decoders = [ids(40 + 37 * i, 100 + i) for i in range(n_decode)]
    got = {}
    for dtype in ("float32", "bfloat16"):
        for mode in ("mixed", "apart"):
            eng = Engine.from_random(SHAPES["8b"], 7, dtype=dtype, page_size=16, max_tokens=65536, max_requests=n_decode + 1)
            eng.add_request("p")
            eng.step([StepEntry("p", prompt[:1024], [])])
            for i, d in enumerate(decoders):
                eng.add_request(i)
                eng.step([StepEntry(i, d[:-1], [])])
            dec = [StepEntry(i, d[-1:], [0]) for i, d in enumerate(decoders)]
            por = StepEntry("p", prompt[1024:], [0, portion // 2, portion - 1])
            if mode == "mixed":
                got[dtype, mode] = eng.step(dec + [por])
            else:
                got[dtype, mode] = np.concatenate([eng.step(dec), eng.step([por])])
            eng.close()
    assert np.array_equal(got["float32", "mixed"], got["float32", "apart"])
    base = rel(got["bfloat16", "apart"], got["float32", "apart"])
    assert base < 3e-2
    err = rel(got["bfloat16", "mixed"], got["float32", "mixed"])
    assert err < 1.5 * base + 2e-3 and not np.isnan(got["bfloat16", "mixed"]).any()


def test_float32_at_the_8b_layer_shape_agrees_with_the_plain_implementation(tmp_path):
    """Two layers at hidden 4096, 32 query heads over 8 kv heads of 128 and feed-forward 12288: the float32 engine
    against the plain implementation (float64, whole sequences) to 1e-4 of the largest logit with the same argmax,
    for a whole prompt, decoding and a chunked feed; the bfloat16 engine against the same plain logits to 3e-2."""
    from helpers import same_top1_or_near_tie
    from plain import qwen3_plain as P
    from purhie_b200.engine import Engine, StepEntry
    from purhie_b200.weights import write_random_model
    toks = ids(104, 3)
    folders = {}
    for dtype in ("float32", "bfloat16"):
        folders[dtype] = str(tmp_path / dtype)
        write_random_model(folders[dtype], SHAPES["8b"], 2, 0.02, 1.0, 1.0, dtype)
    for dtype, tol in (("float32", 1e-4), ("bfloat16", 3e-2)):
        pc, pw = P.read_model(folders[dtype])
        ref = P.forward(pc, pw, toks)
        eng = Engine.from_folder(folders[dtype], dtype=dtype, page_size=16, max_tokens=1024, max_requests=3)
        eng.add_request("whole"); eng.add_request("decode"); eng.add_request("chunks")
        whole = eng.step([StepEntry("whole", toks, list(range(len(toks))))])
        head = eng.step([StepEntry("decode", toks[:96], list(range(96)))])
        tail = [eng.step([StepEntry("decode", toks[96 + k:97 + k], [0])]) for k in range(8)]
        chunks = [eng.step([StepEntry("chunks", toks[s:s + 40], list(range(len(toks[s:s + 40]))))]) for s in range(0, 104, 40)]
        eng.close()
        for name, got in (("whole", whole), ("decode", np.concatenate([head] + tail)), ("chunks", np.concatenate(chunks))):
            got = torch.from_numpy(got.copy())
            err = float((got.double() - ref).abs().max() / ref.abs().max())
            assert err < tol, f"{dtype}/{name}: {err:.3e}"
            if dtype == "float32":
                assert torch.equal(got.argmax(-1), ref.argmax(-1)), f"{dtype}/{name}: argmax"
                assert np.array_equal(got.numpy(), whole), f"{name}: float32 is not bit-equal across the cuts"
            else:
                assert not same_top1_or_near_tie(got, ref, tol), f"{dtype}/{name}: argmax differs away from a tie"


@pytest.mark.skipif(os.environ.get("PURHIE_FULL_SIZE") == "0", reason="whole models (33 and 131 GB in float32) are switched off")
@pytest.mark.parametrize("shape,needs_gb", [("8b", 40), ("32b", 145)])
def test_whole_models_in_float32_and_bfloat16(shape, needs_gb):
    """All 36 layers of the Qwen3-8B shape and all 64 of the Qwen3-32B shape (131 GB in float32), four 256-token
    prompts: whole in one step, and in chunks of 100 / 100 / 48 with the last 8 tokens decoded as a batch of four.
    float32 gives the same bits either way.  bfloat16 is compared with float32: its error grows with the depth (1e-2 of
    the largest logit at 2 layers, 5.6e-2 at 36 and at 64), and its argmax differs only where float32 itself holds the
    two tokens closer together than that error.  Measured: 2 of 32 rows at the 8B shape, 4 to 6 at the 32B shape."""
    import bench
    from helpers import same_top1_or_near_tie
    from purhie_b200.engine import Engine, StepEntry
    torch.cuda.empty_cache()
    free_gb = torch.cuda.mem_get_info()[0] / 1e9
    if free_gb < needs_gb:
        pytest.skip(f"{free_gb:.0f} GB free on the device, the float32 model needs {needs_gb}")
    _, config, seed, std, _ = bench.SHAPES[shape]
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, config["vocab_size"], 256).tolist() for _ in range(4)]
    out = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_random(config, seed, dtype=dtype, std=std, page_size=16, max_tokens=16 * 512, max_requests=8)
        for i in range(4):
            eng.add_request(("w", i)); eng.add_request(("c", i))
        whole = eng.step([StepEntry(("w", i), p, list(range(248, 256))) for i, p in enumerate(prompts)])
        for lo, hi in ((0, 100), (100, 200), (200, 248)):
            eng.step([StepEntry(("c", i), p[lo:hi], []) for i, p in enumerate(prompts)])
        rows = [eng.step([StepEntry(("c", i), p[248 + k:249 + k], [0]) for i, p in enumerate(prompts)]) for k in range(8)]
        out[dtype] = (whole, np.stack(rows, 1).reshape(32, -1))
        eng.close()
    assert np.array_equal(out["float32"][0], out["float32"][1])
    ref = torch.from_numpy(out["float32"][0].copy())
    for got in out["bfloat16"]:
        got = torch.from_numpy(got.copy())
        assert rel(got, ref) < 1e-1 and not torch.isnan(got).any()
        assert not same_top1_or_near_tie(got, ref, 1e-1)


def test_the_norm_factor_applied_by_the_consumer_gives_what_the_norm_kernel_gives():
    """Few-token steps leave the norm's factor per row to the consumer of the normed rows (the gate/up product's
    epilogue, the per-head norm behind the qkv product); the step option "row_factor": "norm" keeps it in the norm's
    kernel.  Both in bfloat16 at the 8B-class layer shape, a short prompt, eight requests decoding side by side and a
    chunk of 100 tokens: the two differ by bfloat16 roundings only, and both stay as close to float32."""
    from purhie_b200.engine import Engine, StepEntry
    reqs = [ids(40 + 11 * i, 400 + i) for i in range(8)]
    got = {}
    for name, dtype, opts in (("f32", "float32", None), ("consumer", "bfloat16", None), ("norm", "bfloat16", {"row_factor": "norm"})):
        eng = Engine.from_random(SHAPES["8b"], 7, dtype=dtype, page_size=16, max_tokens=4096, max_requests=9, step_options=opts)
        rows = []
        for i, r in enumerate(reqs):
            eng.add_request(i)
            rows.append(eng.step([StepEntry(i, r[:-4], [len(r) - 5])]))
        for k in range(4):
            rows.append(eng.step([StepEntry(i, [r[len(r) - 4 + k]], [0]) for i, r in enumerate(reqs)]))
        eng.add_request("chunk")
        rows.append(eng.step([StepEntry("chunk", ids(100, 77), [0, 50, 99])]))
        got[name] = np.concatenate(rows)
        eng.close()
    base = rel(got["norm"], got["f32"])
    assert base < 3e-2
    assert rel(got["consumer"], got["f32"]) < 1.5 * base + 2e-3
    assert rel(got["consumer"], got["norm"]) < 2e-2 and not np.isnan(got["consumer"]).any()


def test_the_norm_done_in_the_epilogue_of_the_product_in_front_gives_what_its_own_kernel_gives():
    """With many rows the o and down products add into the residual in their epilogue and do the pass of the norm
    behind them there as well (weighted rows and sums of squares per tile; the consumer applies the factor).  Step
    options switch that off ("norm_ahead": "off": the norm is a kernel again, the factor stays with the consumer) or
    switch both off ("row_factor": "norm").  Portions of 300, 700 and 130 tokens of one request beside decode rows of
    others, and a portion whose length is no multiple of anything: all three forms agree to bfloat16 roundings and
    stay as close to float32."""
    from purhie_b200.engine import Engine, StepEntry
    from purhie_b200 import native
    long = ids(1130 + 4, 901)
    others = [ids(60 + 7 * i, 910 + i) for i in range(3)]
    got, norm_kernels = {}, {}
    for name, dtype, opts in (("f32", "float32", None), ("ahead", "bfloat16", None), ("kernel", "bfloat16", {"norm_ahead": "off"}),
                              ("norm", "bfloat16", {"row_factor": "norm"})):
        eng = Engine.from_random(SHAPES["8b"], 7, dtype=dtype, page_size=16, max_tokens=4096, max_requests=5, step_options=opts)
        rows = []
        for i, r in enumerate(others):
            eng.add_request(i)
            eng.step([StepEntry(i, r[:-3], [])])
        eng.add_request("long")
        rows.append(eng.step([StepEntry("long", long[:300], [0, 127, 128, 255, 256, 299])]))
        native.lib().qe_profile_enable(1)
        native.profile_report(True)
        rows.append(eng.step([StepEntry("long", long[300:1000], [0, 699])] + [StepEntry(i, [r[-3]], [0]) for i, r in enumerate(others)]))
        report = native.profile_report(True)
        native.lib().qe_profile_enable(0)
        norm_kernels[name] = sum(report.get(k, {"calls": 0})["calls"] for k in ("add_rmsnorm", "add_weight_sumsq"))
        rows.append(eng.step([StepEntry(i, [r[-2]], [0]) for i, r in enumerate(others)] + [StepEntry("long", long[1000:1130], [129])]))
        for k in range(4):
            rows.append(eng.step([StepEntry("long", [long[1130 + k]], [0])]))
        got[name] = np.concatenate(rows)
        eng.close()
    base = rel(got["norm"], got["f32"])
    assert base < 3e-2
    for name in ("ahead", "kernel"):
        assert not np.isnan(got[name]).any()
        assert rel(got[name], got["f32"]) < 1.5 * base + 2e-3, name
        assert rel(got[name], got["norm"]) < 2e-2, name
    assert rel(got["ahead"], got["kernel"]) < 1e-2
    # two layers: the first layer's first norm and the norm before the head stay kernels; the other three norms do not
    assert norm_kernels["kernel"] == 5 and norm_kernels["norm"] == 5 and norm_kernels["ahead"] == 2, norm_kernels


def test_a_sliding_window_layer_at_real_layer_sizes():
    """Two 8B-class layers, the second with a window of 1,000 keys: a 3,000-token prompt whole and in portions of 700,
    each followed by 20 decoded tokens.  float32 gives the same bits either way (places at the window's edge among the
    wanted ones); bfloat16 stays as close to float32 as without a window; the window group gives back the pages the
    window has passed."""
    from purhie_b200.engine import Engine, StepEntry
    shape = dict(SHAPES["8b"], use_sliding_window=True, sliding_window=1000, max_window_layers=1,
                 layer_types=["full_attention", "sliding_attention"])
    toks = ids(3020, 31)
    wanted = (999, 1000, 1001, 2999)
    out = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_random(shape, 7, dtype=dtype, page_size=16, max_tokens=3 * 3200, max_requests=3)
        res = {}
        eng.add_request("w")
        res["whole"] = eng.step([StepEntry("w", toks[:3000], list(wanted))])
        res["decode"] = np.concatenate([eng.step([StepEntry("w", [toks[3000 + k]], [0])]) for k in range(20)])
        eng.add_request("c")
        rows = []
        for s in range(0, 3000, 700):
            part = toks[s:min(s + 700, 3000)]
            want = [i - s for i in wanted if s <= i < s + len(part)]
            r = eng.step([StepEntry("c", part, want)])
            if want:
                rows.append(r)
        res["chunks"] = np.concatenate(rows)
        res["decode_after_chunks"] = np.concatenate([eng.step([StepEntry("c", [toks[3000 + k]], [0])]) for k in range(20)])
        free = eng.info()["free_pages"]
        assert free[1] > free[0] + 200                     # two requests of 3,020 tokens: the window group holds 1,000 of each
        out[dtype] = res
        eng.close()
    f32, b16 = out["float32"], out["bfloat16"]
    assert np.array_equal(f32["whole"], f32["chunks"]) and np.array_equal(f32["decode"], f32["decode_after_chunks"])
    for name in f32:
        assert not np.isnan(b16[name]).any()
        assert rel(b16[name], f32[name]) < 3e-2, name


def test_greedy_generation_through_the_queue_does_not_depend_on_who_else_decodes():
    """Five prompts of 30 to 2,000 tokens through the request queue in float32 at the 8B-class layer shape: their
    prompts come in portions, so the number of rows the greedy kernel picks for changes from step to step (it shares
    one scratch between those calls).  Every request gets the tokens it gets when it runs alone."""
    from purhie_b200.api import load_model_random
    from purhie_b200.config import Qwen3Config
    cfg = Qwen3Config.from_dict(SHAPES["8b"])
    model = load_model_random(cfg, 7, "float32")
    model.kv_cache_init(4096, max_sequences=6, page_size=16, kv_tokens=6 * 2200)
    prompts = [ids(n, 950 + i) for i, n in enumerate((30, 700, 1300, 90, 2000))]
    together = model.generate(prompts, max_new_tokens=12)
    alone = [model.generate([p], max_new_tokens=12)[0] for p in prompts]
    assert together == alone
    assert all(len(t) == 12 and all(0 <= x < 32000 for x in t) for t in together)
    model.free()


@pytest.mark.parametrize("seed", [0, 1])
def test_drawn_schedules_at_real_layer_sizes(seed):
    """Forty drawn steps at the 8B-class layer shape: up to four live requests, portions of 1 to 900 tokens beside
    decode rows, requests that sit a step out, pages poisoned when freed and few enough to be used again.  Every
    wanted row of the bfloat16 engine lies within 3e-2 of the float32 engine's (by the row's largest logit)."""
    from purhie_b200.engine import Engine, StepEntry
    rng = np.random.default_rng(seed)
    reqs, steps, next_id = {}, [], 0
    for _ in range(40):
        entries, end = [], []
        live = [r for r in reqs if reqs[r]["fed"] < len(reqs[r]["toks"])]
        while len(live) < 4 and rng.random() < 0.6:
            n = int(rng.choice([5, 40, 300, 900, 1700]))
            reqs[next_id] = {"toks": rng.integers(0, 32000, n + int(rng.integers(1, 12))).tolist(), "fed": 0, "prompt": n}
            live.append(next_id)
            next_id += 1
        for r in live:
            if rng.random() < 0.25:
                continue
            q = reqs[r]
            left = q["prompt"] - q["fed"]
            n = int(min(left, rng.choice([1, 2, 7, 64, 128, 129, 300, 513, 900]))) if left > 0 else 1
            want = sorted(set(int(x) for x in rng.integers(0, n, min(n, 3)))) if rng.random() < 0.8 else []
            entries.append((r, q["toks"][q["fed"]:q["fed"] + n], want))
            q["fed"] += n
            if q["fed"] >= len(q["toks"]):
                end.append(r)
        if entries:
            steps.append((entries, end))
    out = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_random(SHAPES["8b"], 7, dtype=dtype, page_size=16, max_tokens=4 * 1800, max_requests=4, poison_cache=True)
        known, res = set(), []
        for entries, end in steps:
            for r, _, _ in entries:
                if r not in known:
                    eng.add_request(r)
                    known.add(r)
            lg = eng.step([StepEntry(r, t, w) for r, t, w in entries])
            res.append(None if lg is None or len(lg) == 0 else np.asarray(lg))
            for r in end:
                eng.release(r)
        out[dtype] = res
        eng.close()
    rows = 0
    for i, (a, b) in enumerate(zip(out["bfloat16"], out["float32"])):
        if b is None:
            continue
        assert not np.isnan(b).any() and not np.isnan(a).any(), i
        err = np.abs(a - b).max(axis=1) / np.abs(b).max(axis=1)
        assert err.max() < 3e-2, (i, float(err.max()))
        rows += len(err)
    assert rows > 80


def test_batch_64_decoding_as_graphs_at_real_layer_sizes():
    """64 requests of 30 to 1,500 tokens decode six steps side by side (graph replays from the second step on) at the
    8B-class layer shape: bfloat16 stays as close to the float32 engine as it is for single requests."""
    from purhie_b200.engine import Engine, StepEntry
    reqs = [ids(30 + (i * 211) % 1471 + 6, 300 + i) for i in range(64)]
    got = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_random(SHAPES["8b"], 7, dtype=dtype, page_size=16, max_tokens=65 * 1536, max_requests=64)
        for i, r in enumerate(reqs):
            eng.add_request(i)
            eng.step([StepEntry(i, r[:-6], [])])
        rows = [eng.step([StepEntry(i, [r[len(r) - 6 + k]], [0]) for i, r in enumerate(reqs)]) for k in range(6)]
        assert eng.info()["graph_replays"] >= 4
        got[dtype] = np.stack(rows)
        eng.close()
    err = rel(got["bfloat16"], got["float32"])
    assert err < 3e-2 and not np.isnan(got["bfloat16"]).any()
    per_request = [rel(got["bfloat16"][:, i], got["float32"][:, i]) for i in range(64)]
    assert max(per_request) < 6e-2, (int(np.argmax(per_request)), max(per_request))


def test_twenty_thousand_tokens_through_one_layer():
    """One 8B-class layer over 20,000 tokens: whole, in portions of 4,096, decoding after it and a late short portion.
    float32 gives the same bits however it is cut; bfloat16 stays within a percent of it."""
    from purhie_b200.engine import Engine, StepEntry
    shape = dict(SHAPES["8b"], num_hidden_layers=1, max_position_embeddings=32768, vocab_size=8000)
    toks = ids(20040, 17, vocab=8000)
    N = 20000
    got = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_random(shape, 9, dtype=dtype, page_size=16, max_tokens=3 * 20480, max_requests=3)
        eng.add_request("whole"); eng.add_request("cut")
        res = {"whole": eng.step([StepEntry("whole", toks[:N], [N - 1])])}
        for s in range(0, N, 4096):
            part = toks[s:min(s + 4096, N)]
            lg = eng.step([StepEntry("cut", part, [len(part) - 1] if s + 4096 >= N else [])])
        res["cut"] = lg
        res["decode"] = np.concatenate([eng.step([StepEntry("cut", toks[N + k:N + k + 1], [0])]) for k in range(8)])
        res["late"] = eng.step([StepEntry("whole", toks[N:N + 40], [7, 39])])
        got[dtype] = res
        eng.close()
    f32, b16 = got["float32"], got["bfloat16"]
    assert np.array_equal(f32["whole"], f32["cut"])
    assert np.array_equal(f32["late"][0], f32["decode"][7])                 # position 20,007 either way
    for name in ("whole", "cut", "decode", "late"):
        assert rel(b16[name], f32[name]) < 1e-2, name
