"""The plain implementation and the host sampler against the reference's own CPU code (no GPU).

tests/golden/ref_ops.json holds what the reference's src/qwen_ops.cpp and src/sampler.cpp compute on fixed
inputs (made by tests/golden/make_golden.py).
"""
import json
import math
import os

import numpy as np
import pytest
import torch

from plain import qwen3_plain as P
from purhie_b200.sampling import Sampler, SamplerParams
from helpers import TINY_A, TINY_A_INIT, TINY_B, TINY_B_INIT, make_model, random_tokens

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "ref_ops.json")))


def t64(name):
    return torch.tensor(GOLD[name], dtype=torch.float64)


def test_rmsnorm_matches_the_reference():
    y = P.rmsnorm(t64("rms_x"), t64("rms_w"), 1e-5)
    assert (y - t64("rms_y")).abs().max() < 1e-6


@pytest.mark.parametrize("pos", [0, 7, 1234])
def test_rope_matches_the_reference(pos):
    v = t64("rope_in").view(1, 1, 32)
    full = P.rope_rotate_half(v, [pos], 1e6, 32).view(-1)
    half = P.rope_rotate_half(v, [pos], 10000.0, 16).view(-1)
    assert (full - t64(f"rope_full_theta1e6_pos{pos}")).abs().max() < 1e-6
    assert (half - t64(f"rope_half_theta1e4_pos{pos}")).abs().max() < 1e-6
    assert torch.equal(half[16:], v.view(-1)[16:])           # dims >= n_rot pass through


def test_attention_matches_the_reference():
    H, HKV, D, N = 8, 2, 32, 37
    q = t64("attn_q").view(1, H, D)
    k, v = t64("attn_k").view(N, HKV, D), t64("attn_v").view(N, HKV, D)
    # the reference attends one query over N cached positions: the last row of a causal pass over N rows
    qq = torch.zeros(N, H, D, dtype=torch.float64)
    qq[-1] = q[0]
    out = P.attention(qq, k, v, 0.17677669529663687)[-1].reshape(-1)
    assert (out - t64("attn_out")).abs().max() < 1e-5


def test_silu_matches_the_reference():
    x = t64("silu_x")
    assert (x / (1 + torch.exp(-x)) - t64("silu_y")).abs().max() < 1e-6


def test_window_masks_exactly_the_positions_before_it():
    torch.manual_seed(0)
    T, W = 12, 5
    q, k, v = (torch.randn(T, 2, 8, dtype=torch.float64) for _ in range(3))
    full, win = P.attention(q, k, v, 0.3), P.attention(q, k, v, 0.3, window=W)
    assert torch.allclose(full[:W], win[:W])                # the first W positions see everything
    z = T - 1
    manual = P.attention(q[z - W + 1:], k[z - W + 1:], v[z - W + 1:], 0.3)[-1]
    assert torch.allclose(win[z], manual)                   # a token at z sees positions > z - W only


def test_forward_is_causal_and_uses_the_tied_head(tmp_path):
    make_model(tmp_path, TINY_A, TINY_A_INIT)
    cfg, w = P.read_model(str(tmp_path))
    toks = random_tokens(20, 256, 1)
    full = P.forward(cfg, w, toks)
    assert full.shape == (20, 256)
    assert torch.allclose(P.forward(cfg, w, toks[:9]), full[:9], atol=1e-12)
    assert "lm_head.weight" not in w


def test_layer_windows_from_config_keys():
    assert P.layer_windows(TINY_B) == [None, 24, 24]
    assert P.layer_windows(TINY_A) == [None, None]
    assert P.layer_windows(dict(TINY_A, layer_types=["sliding_attention", "full_attention"], sliding_window=7)) == [7, None]


# ---- sampler -------------------------------------------------------------------------------------------
# The sampler under test is the host library's (sampling/sampler.cpp); the golden chains were drawn by the reference's
# own src/sampler.cpp with equal seeds, so equal tokens mean equal draws from the same generator.

def test_greedy_lowest_id_wins_ties():
    l = np.array(GOLD["samp_logits"], dtype=np.float32)
    assert Sampler(SamplerParams.greedy()).sample(l) == GOLD["samp_greedy"] == 11
    assert P.greedy(l) == 11


def test_defaults_are_the_reference_s():
    d = SamplerParams.defaults()
    assert (round(d.temperature, 6), d.top_k, round(d.top_p, 6), round(d.min_p, 6), d.repeat_penalty, d.repeat_last_n, d.seed,
            d.presence_penalty) == (0.8, 40, 0.95, 0.05, 1.0, 64, 0, 0.0)           # src/sampler.cpp:181-192


@pytest.mark.parametrize("name,params", [
    ("samp_default_seed3", SamplerParams(seed=3)),
    ("samp_temp_only_seed1", SamplerParams(temperature=0.7, top_k=0, top_p=1.0, min_p=0.0, seed=1)),
    ("samp_topp_only_seed5", SamplerParams(temperature=1.3, top_k=0, top_p=0.6, min_p=0.0, seed=5)),
    ("samp_penalty_seed9", SamplerParams(temperature=1.0, top_k=10, top_p=1.0, min_p=0.0, repeat_penalty=1.3,
                                         presence_penalty=0.5, seed=9)),
])
def test_sampler_chain_draws_the_reference_tokens(name, params):
    l = np.array(GOLD["samp_logits"], dtype=np.float32)
    s = Sampler(params)
    got = []
    for _ in range(40):
        t = s.sample(l)
        s.accept(t)
        got.append(t)
    assert got == GOLD[name]


def test_temperature_distribution():
    """200,000 draws against the exact probabilities, to 0.006: the reference's own bar (tests/sampler_verify.cpp:1-4)."""
    l = np.array(GOLD["samp_logits"], dtype=np.float32)
    p = P.temperature_probabilities(l, 0.7)
    s = Sampler(SamplerParams.pure_temperature(0.7, seed=2))
    n = 200000
    counts = s.histogram(l, n)
    assert counts.sum() == n and np.abs(counts / n - p).max() < 0.006
    # which kernel samples what: plain temperature, the chain with top-k on; the host keeps top-p without top-k,
    # more candidates than the kernel holds, and penalties
    assert s.device_mode() == "temperature" and Sampler(SamplerParams()).device_mode() == "chain"
    assert Sampler(SamplerParams(top_k=0)).device_mode() is None
    assert Sampler(SamplerParams(top_k=Sampler.chain_max_k() + 1)).device_mode() is None
    pen = Sampler(SamplerParams(repeat_penalty=1.1))
    pen.accept(3)
    assert pen.device_mode() is None and Sampler(SamplerParams(temperature=0.0)).device_mode() == "greedy"
    assert Sampler(SamplerParams.greedy()).device_mode() == "greedy"


def test_reset_reseeds_and_forgets():
    l = np.array(GOLD["samp_logits"], dtype=np.float32)
    s = Sampler(SamplerParams(seed=4, repeat_penalty=1.2))
    a = [s.sample(l) for _ in range(5)]
    s.accept(3)
    assert s.device_mode() is None                      # a token in the window: the penalty is live
    s.reset()
    assert [s.sample(l) for _ in range(5)] == a and s.device_mode() == "chain"
