"""The C API from a plain C program (GPU): tests/capi_smoke.c includes api/inference.h, links libqengine.so and nothing
else, loads model folders of both tiny configurations and prints tokens; what it prints is compared with the plain
implementation.  (The reference checks its C API the same way: tests/capi_smoke.c:68-94 there.)"""
import os
import shutil
import subprocess

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
def program(tmp_path_factory):
    from purhie_b200.csrc.build import build_dir, build_library
    for lib in ("core", "flash", "gemm100", "qengine"):
        build_library(lib)
    cc = shutil.which("gcc") or shutil.which("cc")
    assert cc, "no C compiler"
    exe = str(tmp_path_factory.mktemp("capi") / "capi_smoke")
    cmd = [cc, "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "purhie_b200", "api"), os.path.join(ROOT, "tests", "capi_smoke.c"),
           "-o", exe, "-L", build_dir(), "-lqengine", "-Wl,-rpath," + build_dir()]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


@pytest.mark.parametrize("name,n_prompt,n_new", [("A", 17, 8), ("B0", 40, 12), ("B", 40, 12)])
def test_a_c_program_loads_a_model_and_generates_the_plain_implementation_s_tokens(program, name, n_prompt, n_new, tmp_path):
    cfg = make_model(tmp_path, *TINY[name], "float32")
    pc, pw = P.read_model(str(tmp_path))
    prompt = random_tokens(n_prompt, cfg.vocab_size, 7)
    want = plain_greedy(pc, pw, prompt, n_new)
    r = subprocess.run([program, str(tmp_path), "float32", str(n_new)] + [str(t) for t in prompt], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = dict(l.split(":", 1) for l in r.stdout.splitlines() if ":" in l)
    ids = lambda key: [int(x) for x in lines[key].split()]
    assert ids("generate_ex") == want and ids("decode_token") == want and ids("generate_stream") == want and ids("request") == want
    assert lines["n_past"].strip() == str(n_prompt + n_new - 1)              # the last token came back as an answer, it was not fed
    assert f"callback saw {n_new} tokens, stop reason 2" in r.stdout          # INFERENCE_STOP_MAX_TOKENS
    assert "finished 1 reason 2" in r.stdout
    assert f"engine_step: rows 1 vocab {cfg.vocab_size} length {n_prompt} argmax {want[0]}" in r.stdout
    assert f"vocab {cfg.vocab_size} hidden {cfg.hidden_size}" in r.stdout and r.stdout.strip().endswith("ok")


def test_the_c_program_in_bfloat16(program, tmp_path):
    """The serving precision through the same program: the tokens of the Python entry point on the same folder."""
    from purhie_b200.api import load_model
    cfg = make_model(tmp_path, *TINY["C"], "bfloat16")
    prompt = random_tokens(70, cfg.vocab_size, 11)
    model = load_model(str(tmp_path), dtype="bfloat16")
    model.kv_cache_init(256)
    want = model.generate_ex(prompt, 8)
    model.free()
    r = subprocess.run([program, str(tmp_path), "bfloat16", "8"] + [str(t) for t in prompt], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = dict(l.split(":", 1) for l in r.stdout.splitlines() if ":" in l)
    assert [int(x) for x in lines["generate_ex"].split()] == want
