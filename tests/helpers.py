"""Shared by the tests: the two tiny configurations, model folders in temporary places, comparisons."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny configurations that differ in every size and option.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64, intermediate_size=128,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256, max_position_embeddings=128,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, attention_bias=False)
TINY_A_INIT = dict(seed=0, std=0.02, scale_low=0.9, scale_high=1.1, page_size=16)

TINY_B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96, intermediate_size=224,
              num_attention_heads=8, num_key_value_heads=2, head_dim=32, vocab_size=512, max_position_embeddings=256,
              rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False, attention_bias=True,
              use_sliding_window=True, sliding_window=24, max_window_layers=1)
TINY_B_INIT = dict(seed=1, std=0.03, scale_low=0.8, scale_high=1.2, page_size=8)
# The second configuration as the benchmark description writes it: no attention bias, attention over all keys.
TINY_B0 = {k: v for k, v in TINY_B.items() if k not in ("use_sliding_window", "sliding_window", "max_window_layers")}
TINY_B0["attention_bias"] = False

# A third shape for the fast kernels: head size 64 and 128 are what they take.
TINY_C = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=160, intermediate_size=352,
              num_attention_heads=6, num_key_value_heads=2, head_dim=64, vocab_size=1000, max_position_embeddings=512,
              rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False, attention_bias=False,
              layer_types=["full_attention", "sliding_attention"], sliding_window=40)
TINY_C_INIT = dict(seed=7, std=0.05, scale_low=0.7, scale_high=1.3, page_size=16)

TINY = {"A": (TINY_A, TINY_A_INIT), "B": (TINY_B, TINY_B_INIT), "B0": (TINY_B0, TINY_B_INIT), "C": (TINY_C, TINY_C_INIT)}


def make_model(folder, cfg_dict, init, dtype="float32"):
    """Write a random model folder (matrices stored in ``dtype``); returns the typed configuration."""
    from purhie_b200.config import Qwen3Config
    from purhie_b200.weights import write_random_model
    cfg = Qwen3Config.from_dict(cfg_dict)
    write_random_model(str(folder), cfg, init["seed"], init["std"], init["scale_low"], init["scale_high"], dtype)
    return cfg


def random_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    return ((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30)).item()


def same_top1_or_near_tie(got, ref, tol):
    """Rows whose argmax differs must be near-ties in the reference (the reference's rule for reduced precision,
    tests/seq_verify.cpp:64-99 there, accepts a first difference only at a small gap).  The gap allowed here is what
    the granted tolerance can explain and no more: the error bound is ``tol`` of the largest logit of the request, so
    two logits can swap only if they were within twice that."""
    got, ref = got.double().cpu(), ref.double().cpu()
    bad = []
    allowed = 2.0 * tol * ref.abs().max().item()
    for i in range(ref.shape[0]):
        a, b = int(got[i].argmax()), int(ref[i].argmax())
        if a != b and (ref[i, b] - ref[i, a]).item() > allowed:
            bad.append(i)
    return bad


class TraceRun:
    """Drives bin/trace_run as a user does: a subprocess, steps on standard input, ``done`` lines back."""

    def __init__(self, model_dir, dtype, out_dir, max_tokens, extra=()):
        self.out_dir = str(out_dir)
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype,
               "--out", self.out_dir, "--max-tokens", str(max_tokens)] + list(extra)
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        self.vocab = json.load(open(os.path.join(str(model_dir), "config.json")))["vocab_size"]

    def step(self, step, entries, end=()):
        rec = {"step": step, "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries],
               "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {step}", f"trace_run answered {line!r}"
        path = os.path.join(self.out_dir, f"{step}.f32")
        if any(len(w) for _, _, w in entries):
            import numpy as np
            return torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(-1, self.vocab).copy())
        assert not os.path.exists(path)
        return None

    def close(self):
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=60)
        assert rc == 0, f"trace_run exited with {rc}"


# ---- replay schedules --------------------------------------------------------------------------------

def schedule_whole(requests):
    """Each request alone and whole: one step each."""
    steps = []
    for rid, toks in requests.items():
        steps.append(([(rid, toks, list(range(len(toks))))], [rid]))
    return steps


def schedule_tail(requests, tail=32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(len(toks) - tail, 0)
        if head:
            steps.append(([(rid, toks[:head], list(range(head)))], []))
        for i in range(head, len(toks)):
            steps.append(([(rid, toks[i:i + 1], [0])], [rid] if i == len(toks) - 1 else []))
    return steps


def schedule_portions(requests, sizes=(13, 2, 8, 3, 2, 5, 1, 21, 2, 2, 34, 1, 7)):
    """Portions of changing size, down to two tokens (and single ones)."""
    steps = []
    for rid, toks in requests.items():
        i, k = 0, 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            steps.append(([(rid, toks[i:i + n], list(range(n)))], [rid] if i + n == len(toks) else []))
            i += n
    return steps


def schedule_mixed(requests, max_live=4, seed=0, prompt_frac=0.6):
    """Up to ``max_live`` live requests: portions of the prompts of some beside single tokens of others;
    some requests sit a step out; a finished request ends and the next one joins."""
    import random
    rng = random.Random(seed)
    order = list(requests)
    pos = {rid: 0 for rid in order}
    prompt_len = {rid: max(1, int(len(requests[rid]) * prompt_frac)) for rid in order}
    live, nxt, steps = [], 0, []
    while nxt < len(order) or live:
        while len(live) < max_live and nxt < len(order):
            live.append(order[nxt]); nxt += 1
        entries, end = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                    # left out of this step
            toks, p = requests[rid], pos[rid]
            if p < prompt_len[rid]:
                n = min(rng.choice([2, 3, 5, 8, 13, 16, 17, 31]), prompt_len[rid] - p)
            else:
                n = 1
            n = min(n, len(toks) - p)
            entries.append((rid, toks[p:p + n], list(range(n))))
            pos[rid] = p + n
            if pos[rid] == len(toks):
                end.append(rid); live.remove(rid)
        if entries:
            steps.append((entries, end))
    return steps


def run_schedule(step_fn, release_fn, steps):
    """Run ``steps`` and gather, per request, the logits of every position in order."""
    out = {}
    for k, (entries, end) in enumerate(steps):
        logits = step_fn(k, entries, end)
        row = 0
        for rid, toks, want in entries:
            n = len(want)
            if n:
                out.setdefault(rid, []).append(logits[row:row + n].clone())
                row += n
        if release_fn:
            for rid in end:
                release_fn(rid)
    return {rid: torch.cat(parts) for rid, parts in out.items()}


def engine_runner(engine):
    from purhie_b200.engine import StepEntry

    def step(k, entries, end):
        for rid, _, _ in entries:
            if not engine.has_request(rid):
                engine.add_request(rid)
        lg = engine.step([StepEntry(rid, toks, want) for rid, toks, want in entries])
        return None if lg is None else torch.from_numpy(lg.copy())

    return step, engine.release
