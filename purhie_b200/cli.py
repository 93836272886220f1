"""Command line in the manner of the reference's ``qwen_demo`` (src/demo_qwen.cpp:1-12, 59-77, 182-223).

    qwen_demo <model_dir> "<token ids>" | @prompt_file [n_gen] [--temp T] [--top-k K] [--top-p P]
              [--min-p P] [--repeat-penalty R] [--seed S] [--ctx N (default 4096)] [--batch N]
              [--dtype bfloat16|float32] [--random-prompt LEN]

Options have the reference's names and meanings; greedy unless ``--temp`` is given; ``--batch`` is the
number of tokens per prefill batch (default 1024).  There is no tokenizer, so the prompt is a list of token
ids separated by commas or blanks (``@file`` reads them from a file; ``--random-prompt LEN`` draws LEN
uniform ids with ``--seed``).  The options of the reference that belong to parts that are not built
(``--lm-head-q8``, ``--draft``, ``--drafts``, ``--kv-q8``, ``--kv-q4``, ``--stage``) are refused by name.
"""
from __future__ import annotations

import re
import sys
import time

USAGE = ("Usage: qwen_demo <model_dir> \"<token ids>\" | @prompt_file [n_gen] [--temp T] [--top-k K] [--top-p P] "
         "[--min-p P]\n       [--repeat-penalty R] [--seed S] [--ctx N] [--batch N] [--dtype bfloat16|float32] "
         "[--random-prompt LEN]\n")
_NOT_BUILT = {"--lm-head-q8": 0, "--draft": 1, "--drafts": 1, "--kv-q8": 0, "--kv-q4": 0, "--stage": 1}


def parse_ids(text: str):
    return [int(t) for t in re.split(r"[\s,]+", text.strip()) if t]


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) < 2:
        sys.stdout.write(USAGE)
        return 1
    from .api import GenOptions, InferenceError, load_model
    from .sampling.sampler import SamplerParams
    model_path, prompt_arg = argv[0], argv[1]
    sp = SamplerParams()
    sp.temperature = 0.0                      # greedy unless asked
    n_gen, n_ctx, batch, dtype, random_prompt = 16, 4096, 0, "bfloat16", 0
    i = 2
    while i < len(argv):
        a = argv[i]
        v = argv[i + 1] if i + 1 < len(argv) else "0"
        if a == "--temp": sp.temperature = float(v); i += 1
        elif a == "--top-k": sp.top_k = int(v); i += 1
        elif a == "--top-p": sp.top_p = float(v); i += 1
        elif a == "--min-p": sp.min_p = float(v); i += 1
        elif a == "--repeat-penalty": sp.repeat_penalty = float(v); i += 1
        elif a == "--seed": sp.seed = int(v); i += 1
        elif a == "--ctx": n_ctx = int(v); i += 1
        elif a == "--batch": batch = int(v); i += 1
        elif a == "--dtype": dtype = v; i += 1
        elif a == "--random-prompt": random_prompt = int(v); i += 1
        elif a in _NOT_BUILT:
            sys.stderr.write(f"qwen_demo: option {a} belongs to a part of the reference that this engine does not "
                             f"have\n")
            return 1
        elif a.startswith("--"):
            sys.stderr.write(f"qwen_demo: unknown option {a}\n{USAGE}")
            return 1
        else:
            n_gen = int(a)
        i += 1
    print(f"Sampling: temp {sp.temperature:g} top_k {sp.top_k} top_p {sp.top_p:g} min_p {sp.min_p:g} "
          f"repeat_penalty {sp.repeat_penalty:g} seed {sp.seed}")
    try:
        model = load_model(model_path, dtype=dtype)
        if random_prompt > 0:
            import torch
            g = torch.Generator().manual_seed(sp.seed)
            prompt = torch.randint(0, model.vocab_size(), (random_prompt,), generator=g).tolist()
        elif prompt_arg.startswith("@") and len(prompt_arg) > 1:
            try:
                with open(prompt_arg[1:]) as f:
                    prompt = parse_ids(f.read())
            except OSError:
                sys.stderr.write(f"cannot read prompt file {prompt_arg[1:]}\n")
                return 1
        else:
            prompt = parse_ids(prompt_arg)
        if not prompt:
            sys.stderr.write("qwen_demo: the prompt holds no token ids\n")
            return 1
        n_ctx = min(n_ctx, model._decoder.spec.max_position)
        model.kv_cache_init(n_ctx, max_sequences=1)
        if batch > 0:
            model.set_prefill_batch(batch)
        print(f"Prompt tokens ({len(prompt)}):", " ".join(str(t) for t in prompt[:32]) + (" ..." if len(prompt) > 32 else ""))
        import torch
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        model.prefill(prompt)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        out, reason = model.generate_stream([], GenOptions(sampler=sp, max_new_tokens=n_gen, ignore_eog=True,
                                                           on_token=lambda u, tok, text, n: print(tok, flush=True) or 0))
        torch.cuda.synchronize()
        t2 = time.perf_counter()
    except InferenceError as e:
        sys.stderr.write(f"qwen_demo: {e}\n")
        return 1
    pre_ms, gen_ms = (t1 - t0) * 1e3, (t2 - t1) * 1e3
    print(f"Timing: prefill {len(prompt)} tokens {pre_ms:.1f} ms ({len(prompt) / max(pre_ms, 1e-9) * 1e3:.1f} tok/s), "
          f"generation {len(out)} tokens {gen_ms:.1f} ms ({len(out) / max(gen_ms, 1e-9) * 1e3:.1f} tok/s), stop: {reason}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
