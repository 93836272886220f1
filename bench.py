#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Qwen3-8B shape with random weights, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--shape 8b|0.6b|32b] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 from 2,048-token prefixes, timed on the
device (CUDA events on the engine's stream) over exactly K decode steps after W warm-up steps, each step fed its
token ids from the host and ending in the greedy sampling kernel; ``e2e`` is the same through the Python entry point
(purhie_b200.api: streams, host token ids in and sampled tokens out every step) by the wall clock; ``prefill`` is
one 2,048-token prompt from submit to logits; ``roofline`` is the decode step's bytes (every weight once plus the
live requests' cache) over its time; ``points`` holds decode at batch 1 and 64 and a mixed step (32 decoded tokens
beside a 512-token prompt chunk).  Token ids are uniform random (synthetic).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the headline benchmark configuration: the Qwen3-8B shape
QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096, intermediate_size=12288,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936,
                max_position_embeddings=4096, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False)
# the two other benchmark shapes (Qwen3-0.6B and Qwen3-32B); the default run stays the 8B shape
QWEN3_06B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, intermediate_size=3072, num_attention_heads=16,
                 num_key_value_heads=8, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, intermediate_size=25600, num_attention_heads=64,
                 num_key_value_heads=8)
SHAPES = {"8b": ("Qwen3-8B", QWEN3_8B, 2, 0.02, (1, 64)), "0.6b": ("Qwen3-0.6B", QWEN3_06B, 3, 0.02, (1, 64)),
          "32b": ("Qwen3-32B", QWEN3_32B, 4, 0.015, (1, 32))}
CONTEXT, PREFIX, PREFILL_TOKENS = 4096, 2048, 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    """The roofline denominators: the measured copy bandwidth, and the cuBLAS bf16 rate as a burst (a kernel timed
    alone, which is how the prefill is timed here) and sustained under the power cap."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained") or d["bf16_tflops"]), "source": "measured"}
        except (ValueError, KeyError, OSError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                clocks.append(float(f[0])); mx = float(f[1])
            except ValueError:
                continue
            for name, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks)}


def reference_arm():
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a HIP engine for AMD gfx1151 (Makefile + hipcc, GGUF models); it has no Python "
                      "package to install (pip finds neither setup.py nor pyproject.toml) and no CUDA path"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: the headline 8B shape or another")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has (named in config); layer sizes stay")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64 and the mixed step")
    ap.add_argument("--phase", default="all", choices=["all", "decode", "prefill"],
                    help="run one phase only, with few launches around it (for profiling under ncu)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (the benchmark's configuration has 16)")
    ap.add_argument("--step-options", default="", metavar="JSON",
                    help="kernel choices of the step, for comparing two forms of it on one box, e.g. '{\"norm_ahead\": \"off\"}'")
    ap.add_argument("--leave-out", default="", metavar="NAMES",
                    help="with --phase decode: launchers (comma separated, e.g. add_rmsnorm,decode_bulk) that the timed steps "
                         "skip; the difference to a run without shows what they cost inside the graph (no benchmark value)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import numpy as np
    from purhie_b200.api import GenOptions, load_model_random
    from purhie_b200.config import Qwen3Config
    from purhie_b200.engine import Engine, StepEntry
    from purhie_b200.sampling import SamplerParams

    shape_name, shape, SEED, STD, point_batches = SHAPES[args.shape]
    if args.layers is None:
        args.layers = shape["num_hidden_layers"]
    cfg = Qwen3Config.from_dict(dict(shape, num_hidden_layers=args.layers))
    pk = peaks()
    model = load_model_random(cfg, SEED, "bfloat16", std=STD)
    max_batch = args.batch if args.phase != "all" else max(max(point_batches), args.batch)
    if args.phase != "all":
        args.no_points = True
    kv_tokens = max_batch * (PREFIX + 2 * (args.steps + args.warmup) + 256) + PREFILL_TOKENS + 64
    step_options = {"step": json.loads(args.step_options)} if args.step_options else {}
    model.kv_cache_init(CONTEXT, max_sequences=max_batch + 2, page_size=args.page_size, kv_tokens=kv_tokens, **step_options)
    eng = Engine.attach(model)
    rng = np.random.default_rng(SEED)
    ids = lambda n: rng.integers(0, cfg.vocab_size, size=n).tolist()
    median = lambda xs: sorted(xs)[len(xs) // 2]

    # ---- prefill of one 2,048-token prompt ----------------------------------------------------------
    prompt = ids(PREFILL_TOKENS)

    def prefill_once():
        eng.add_request("prefill")
        ms = eng.time_step([StepEntry("prefill", prompt, [PREFILL_TOKENS - 1])])
        eng.release("prefill")
        return ms

    if args.phase == "decode":
        prefill_ms = float("nan")
    else:
        for _ in range(3 if args.phase == "all" else 1):
            prefill_once()
        from purhie_b200 import native as _native
        if _native.profile_enabled():
            _native.profile_report(True)             # the warm-up runs do not count
        prefill_ms = median([prefill_once() for _ in range(5 if args.phase == "all" else 1)])
    if args.phase == "prefill":
        from purhie_b200 import native
        if native.profile_enabled():
            sys.stderr.write(native.format_profile(native.profile_report(), f"prefill of {PREFILL_TOKENS} tokens, {args.layers} layers") + "\n")
        print(json.dumps({"phase": "prefill", "ms": prefill_ms, "layers": args.layers}))
        return 0
    T, E, FF, V = PREFILL_TOKENS, cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    qw, kvw, D = cfg.q_width, cfg.kv_width, cfg.head_dim
    layer_mm = E * (qw + 2 * kvw) + qw * E + 3 * E * FF
    prefill_flops = cfg.num_hidden_layers * (2.0 * T * layer_mm + 4.0 * cfg.num_attention_heads * D * T * (T + 1) / 2) + 2.0 * V * E
    tflops = prefill_flops / (prefill_ms * 1e-3) / 1e12
    prefill = {"value": round(T / prefill_ms * 1e3, 1), "tokens": T, "ms": round(prefill_ms, 3),
               "frac": round(tflops / pk["bf16_tflops"], 4), "frac_of_sustained": round(tflops / pk["bf16_tflops_sustained"], 4),
               "tflops": round(tflops, 1), "peak": pk["source"]}

    # ---- prefixes of 2,048 tokens for every request ---------------------------------------------------
    for i in range(max_batch):
        eng.add_request(i)
        eng.step([StepEntry(i, ids(PREFIX), [])])

    weight_bytes = 2.0 * (cfg.num_hidden_layers * layer_mm + V * E)       # the embedding table is gathered, not streamed
    kv_bytes_per_token = 2.0 * 2 * cfg.num_hidden_layers * kvw

    def decode_run(batch, steps, warmup):
        ctx0 = eng.length(0) + warmup
        toks = [ids(steps + warmup) for _ in range(batch)]
        ms, launches = eng.time_decode_steps(list(range(batch)), toks, warmup, steps, sample=True)
        bytes_step = weight_bytes + batch * (ctx0 + steps / 2.0) * kv_bytes_per_token
        return ms, launches, bytes_step

    if args.leave_out:
        if args.phase != "decode":
            print("bench.py: --leave-out goes with --phase decode")
            return 2
        from purhie_b200 import native
        native.lib().qe_profile_leave_out(args.leave_out.encode())     # the graphs are captured after this
    from purhie_b200 import native as _native
    if _native.profile_enabled():
        _native.profile_report(True)                 # what came before the timed steps does not count
    sampler = ClockSampler()
    sampler.start()
    ms_step, launches, bytes_step = decode_run(args.batch, args.steps, args.warmup)
    clocks = sampler.stop()
    points = {}
    if not args.no_points:
        for b in point_batches:
            ms_b, _, by = decode_run(b, min(args.steps, 32), 3)
            points[f"decode_b{b}"] = round(b / ms_b * 1e3, 1)
            points[f"decode_b{b}_hbm_frac"] = round(by / (ms_b * 1e-3) / (pk["hbm_gbs"] * 1e9), 4)
        # a step of 32 decoded tokens beside one 512-token prompt chunk (the small shape's benchmark workload),
        # launched kernel by kernel every time
        n_dec, chunk = min(32, max_batch), 512
        chunk_ids = ids(chunk)

        def mixed_once():
            eng.add_request("chunk")
            ms = eng.time_step([StepEntry(i, [chunk_ids[i]], [0]) for i in range(n_dec)] + [StepEntry("chunk", chunk_ids, [chunk - 1])])
            eng.release("chunk")
            return ms

        for _ in range(3):
            mixed_once()
        points[f"mixed_b{n_dec}_chunk{chunk}_ms"] = round(median([mixed_once() for _ in range(5)]), 3)
    if args.phase == "decode":
        from purhie_b200 import native
        if native.profile_enabled():             # PURHIE_PROFILE=1: every launch between events, graphs off
            sys.stderr.write(native.format_profile(native.profile_report(), f"decode, batch {args.batch}, {args.layers} layers") + "\n")
        print(json.dumps({"phase": "decode", "batch": args.batch, "ms_per_step": ms_step, "layers": args.layers,
                          "left_out": args.leave_out or None}))
        return 0

    # ---- end to end through the Python entry point ------------------------------------------------------
    for i in range(max_batch):
        eng.release(i)
    streams = []
    opts = GenOptions(sampler=SamplerParams.greedy(), max_new_tokens=args.steps + args.warmup + 8, ignore_eog=True)
    for i in range(args.batch):
        seq = model.seq_new()
        model.seq_select(seq)
        streams.append(model.stream_begin(ids(PREFIX), opts))
    model.stream_run(streams, args.warmup)
    model.synchronize()
    t0 = time.perf_counter()
    done = model.stream_run(streams, args.steps)          # host token ids in, every step's sampled ids out
    model.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    assert len(done) == args.steps and all(tok is not None for step in done for _, tok in step)
    h2d = model.engine_info()["upload_bytes"]                   # the step's packed int32 metadata (ids, positions, tables)
    e2e = {"value": round(args.batch / e2e_ms * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch + 8}

    # ---- the small shape is bound by launches: the same decode with every kernel launched by the host -----------
    if args.shape == "0.6b" and not args.no_points:
        for st in streams:
            st.free()
        model.kv_cache_init(CONTEXT, max_sequences=3, page_size=args.page_size, kv_tokens=2 * (PREFIX + 256), cuda_graphs=False)
        eng2 = Engine.attach(model)
        eng2.add_request(0)
        eng2.step([StepEntry(0, ids(PREFIX), [])])
        ms_off, launches_off = eng2.time_decode_steps([0], [ids(35)], 3, 32, sample=True)
        points["decode_b1_graphs_off"] = round(1 / ms_off * 1e3, 1)
        points["decode_b1_launches_per_step"] = launches_off // 32

    value = args.batch / ms_step * 1e3
    achieved = bytes_step / (ms_step * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {args.batch} from 2,048-token prefixes ({shape_name} shape)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": f"{shape_name} shape, random weights seed {SEED}", "global_batch": args.batch, "seq_len": PREFIX,
                   "context": CONTEXT, "parallelism": "single GPU", "layers": args.layers,
                   "layers_of_config": shape["num_hidden_layers"], "hidden": E, "q_heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": D, "intermediate": FF, "vocab": V,
                   "kv_page_tokens": args.page_size, "kv_dtype": "bf16", "l2": f"weights ({weight_bytes / 1e9:.1f} GB) exceed L2 every step",
                   "cuda_graphs": True, "prefill_tokens": PREFILL_TOKENS, "sampling": "greedy, inside the timed step"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"]},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
