"""Command line in the manner of the reference's ``qwen_demo`` (src/demo_qwen.cpp:1-12, 59-77, 182-223).

    qwen_demo <model_dir | --random CONFIG.json> "<token ids>" | @prompt_file [n_gen] [--temp T] [--top-k K]
              [--top-p P] [--min-p P] [--repeat-penalty R] [--seed S] [--ctx N (default 4096)] [--batch N]
              [--dtype bfloat16|float32] [--tokens "ids"] [--tokens-file F] [--random-prompt LEN]
              [--weights-seed S] [--block-size B] [--max-batch-tokens N] [--chunk N] [--ignore-eos]

Options the reference has keep its names and meanings: greedy unless ``--temp`` is given; ``--batch`` is the number
of tokens per prefill pass (default 1024); ``--seed`` seeds the sampler.  There is no tokenizer, so a prompt is a
list of token ids separated by commas or blanks (``@file`` reads them from a file; ``--random-prompt LEN`` draws LEN
uniform ids with ``--seed``).  ``--random CONFIG.json`` takes the place of the model folder: the weights are drawn
from ``--weights-seed`` and nothing is written.  ``--tokens-file F`` holds one prompt a line; with more than one
prompt they all run at once through the request queue (``--max-batch-tokens``: the token budget of a step,
``--chunk``: the longest prompt portion in a step) and each request's tokens are printed on a line.
``--block-size`` is the number of tokens per cache page.  Generation stops at an end-of-generation token of the
model's configuration unless ``--ignore-eos``.  The options of the reference that belong to parts that are not built
(``--lm-head-q8``, ``--draft``, ``--drafts``, ``--kv-q8``, ``--kv-q4``, ``--stage``) are refused by name.
With ``PURHIE_PROFILE=1`` in the environment the device time per kernel class is printed at the end (the reference
prints its breakdown under ``QWEN_PROFILE=1``).
"""
from __future__ import annotations

import json
import re
import sys
import time

USAGE = ("Usage: qwen_demo <model_dir | --random CONFIG.json> \"<token ids>\" | @prompt_file [n_gen] [--temp T] [--top-k K] "
         "[--top-p P] [--min-p P]\n       [--repeat-penalty R] [--seed S] [--ctx N] [--batch N] [--dtype bfloat16|float32] "
         "[--tokens \"ids\"] [--tokens-file F]\n       [--random-prompt LEN] [--weights-seed S] [--block-size B] "
         "[--max-batch-tokens N] [--chunk N] [--ignore-eos]\n")
_NOT_BUILT = {"--lm-head-q8": 0, "--draft": 1, "--drafts": 1, "--kv-q8": 0, "--kv-q4": 0, "--stage": 1}


def parse_ids(text: str):
    return [int(t) for t in re.split(r"[\s,]+", text.strip()) if t]


def uniform_ids(n: int, vocab: int, seed: int):
    """n token ids uniform in [0, vocab), a function of the seed alone."""
    import numpy as np
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) < 2:
        sys.stdout.write(USAGE)
        return 1
    from .api import GenOptions, InferenceError, load_model, load_model_random
    from .sampling import SamplerParams
    sp = SamplerParams.defaults()
    sp.temperature = 0.0                      # greedy unless asked
    o = dict(n_gen=16, ctx=4096, batch=0, dtype="bfloat16", random_prompt=0, random=None, weights_seed=0, block=16,
             budget=2048, chunk=512, ignore_eos=False, tokens=None, tokens_file=None)
    positional = []
    i = 0
    while i < len(argv):
        a = argv[i]
        v = argv[i + 1] if i + 1 < len(argv) else "0"
        if a == "--temp": sp.temperature = float(v); i += 1
        elif a == "--top-k": sp.top_k = int(v); i += 1
        elif a == "--top-p": sp.top_p = float(v); i += 1
        elif a == "--min-p": sp.min_p = float(v); i += 1
        elif a == "--repeat-penalty": sp.repeat_penalty = float(v); i += 1
        elif a == "--seed": sp.seed = int(v); i += 1
        elif a == "--ctx": o["ctx"] = int(v); i += 1
        elif a == "--batch": o["batch"] = int(v); i += 1
        elif a == "--dtype": o["dtype"] = {"bf16": "bfloat16", "fp32": "float32"}.get(v, v); i += 1
        elif a == "--random-prompt": o["random_prompt"] = int(v); i += 1
        elif a == "--random": o["random"] = v; i += 1
        elif a == "--weights-seed": o["weights_seed"] = int(v); i += 1
        elif a == "--block-size": o["block"] = int(v); i += 1
        elif a == "--max-batch-tokens": o["budget"] = int(v); i += 1
        elif a == "--chunk": o["chunk"] = int(v); i += 1
        elif a == "--ignore-eos": o["ignore_eos"] = True
        elif a == "--tokens": o["tokens"] = v; i += 1
        elif a == "--tokens-file": o["tokens_file"] = v; i += 1
        elif a in _NOT_BUILT:
            sys.stderr.write(f"qwen_demo: option {a} belongs to a part of the reference that this engine does not have\n")
            return 1
        elif a.startswith("--"):
            sys.stderr.write(f"qwen_demo: unknown option {a}\n{USAGE}")
            return 1
        else:
            positional.append(a)
        i += 1
    model_path = None if o["random"] else (positional.pop(0) if positional else None)
    prompt_arg = None
    if not (o["tokens"] or o["tokens_file"] or o["random_prompt"]) and positional:
        prompt_arg = positional.pop(0)
    if positional:
        try:
            o["n_gen"] = int(positional[0])
        except ValueError:
            sys.stderr.write(f"qwen_demo: {positional[0]!r} is not a number of tokens to generate\n{USAGE}")
            return 1
    if not model_path and not o["random"]:
        sys.stdout.write(USAGE)
        return 1
    print(f"Sampling: temp {sp.temperature:g} top_k {sp.top_k} top_p {sp.top_p:g} min_p {sp.min_p:g} "
          f"repeat_penalty {sp.repeat_penalty:g} seed {sp.seed}")
    try:
        if o["random"]:
            with open(o["random"], "r", encoding="utf-8") as f:
                config = json.load(f)
            model = load_model_random(config, o["weights_seed"], dtype=o["dtype"])
        else:
            model = load_model(model_path, dtype=o["dtype"])
        # the prompts
        if o["random_prompt"] > 0:
            prompts = [uniform_ids(o["random_prompt"], model.vocab_size(), sp.seed)]
        elif o["tokens_file"]:
            with open(o["tokens_file"]) as f:
                prompts = [parse_ids(line) for line in f if line.strip()]
        elif o["tokens"]:
            prompts = [parse_ids(o["tokens"])]
        elif prompt_arg and prompt_arg.startswith("@") and len(prompt_arg) > 1:
            try:
                with open(prompt_arg[1:]) as f:
                    prompts = [parse_ids(f.read())]
            except OSError:
                sys.stderr.write(f"cannot read prompt file {prompt_arg[1:]}\n")
                return 1
        elif prompt_arg:
            prompts = [parse_ids(prompt_arg)]
        else:
            prompts = []
        if not prompts or any(not p for p in prompts):
            sys.stderr.write("qwen_demo: a prompt holds no token ids\n")
            return 1
        n_seq = min(len(prompts), 64)
        n_ctx = min(o["ctx"] if o["ctx"] > 0 else 4096, model.max_position())
        model.kv_cache_init(n_ctx, max_sequences=n_seq, page_size=o["block"],
                            max_batch_tokens=o["budget"], prefill_chunk=o["chunk"])
        if o["batch"] > 0:
            model.set_prefill_batch(o["batch"])
        if len(prompts) == 1:
            prompt = prompts[0]
            print(f"Prompt tokens ({len(prompt)}):", " ".join(str(t) for t in prompt[:32]) + (" ..." if len(prompt) > 32 else ""))
            model.synchronize()
            t0 = time.perf_counter()
            model.prefill(prompt)
            model.synchronize()
            t1 = time.perf_counter()
            out, reason = model.generate_stream([], GenOptions(sampler=sp, max_new_tokens=o["n_gen"], ignore_eog=o["ignore_eos"],
                                                               on_token=lambda u, tok, text, n: print(tok, flush=True) or 0))
            model.synchronize()
            t2 = time.perf_counter()
            n_prompt, n_out = len(prompt), len(out)
        else:
            # several prompts: all at once through the request queue
            model.synchronize()
            t0 = time.perf_counter()
            outs = model.generate(prompts, max_new_tokens=o["n_gen"], params=sp, seed=sp.seed, ignore_eos=o["ignore_eos"])
            model.synchronize()
            t2 = t1 = time.perf_counter()
            for k, (p, out, why) in enumerate(zip(prompts, outs, model.last_stop_reasons)):
                print(f"Request {k} ({len(p)} prompt tokens, stop: {why}):", " ".join(str(t) for t in out))
            n_prompt, n_out, reason = sum(len(p) for p in prompts), sum(len(x) for x in outs), "all"
            pre_ms = gen_ms = (t2 - t0) * 1e3
            print(f"Timing: {len(prompts)} requests, {n_prompt} prompt tokens and {n_out} generated tokens in {gen_ms:.1f} ms "
                  f"({n_out / max(gen_ms, 1e-9) * 1e3:.1f} generated tok/s)")
            return 0
    except (InferenceError, OSError, ValueError) as e:
        sys.stderr.write(f"qwen_demo: {e}\n")
        return 1
    from . import native
    if native.profile_enabled():             # PURHIE_PROFILE=1: where the device time went, per kernel class
        sys.stderr.write(native.format_profile(native.profile_report(), "prefill and generation") + "\n")
    pre_ms, gen_ms = (t1 - t0) * 1e3, (t2 - t1) * 1e3
    print(f"Timing: prefill {n_prompt} tokens {pre_ms:.1f} ms ({n_prompt / max(pre_ms, 1e-9) * 1e3:.1f} tok/s), "
          f"generation {n_out} tokens {gen_ms:.1f} ms ({n_out / max(gen_ms, 1e-9) * 1e3:.1f} tok/s), stop: {reason}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
