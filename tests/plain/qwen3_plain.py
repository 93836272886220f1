"""A plain, slow Qwen3 dense forward pass: whole sequences, no cache, float64, one function per part.

It shares no code with ``purhie_b200``: it reads ``config.json`` with ``json`` and the weights with the
``safetensors`` package, and restates the reference's formulas.  The reference's own model code
(src/qwen_model.cpp, src/inference.cpp) calls the HIP runtime throughout and cannot be built on a CPU, and
it has no CPU forward pass for this architecture, so the composition below rests on the formulas (each
function cites where they stand); the three operators that the reference does have as plain CPU code
(src/qwen_ops.cpp) are compared with these functions in tests/golden/.
"""
import json
import math
import os

import numpy as np
import torch

F64 = torch.float64


def read_model(model_dir):
    """(config dict, {name: float64 tensor})."""
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    weights = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(F64)
    return cfg, weights


def layer_windows(cfg):
    """Per layer: None (all earlier positions) or the window W (positions > p - W).  Keys as in config.json:
    ``layer_types`` wins; else ``use_sliding_window`` makes layers >= ``max_window_layers`` windowed."""
    n = cfg["num_hidden_layers"]
    w = cfg.get("sliding_window")
    if cfg.get("layer_types"):
        return [w if t == "sliding_attention" else None for t in cfg["layer_types"]]
    if cfg.get("use_sliding_window") and w:
        first = cfg.get("max_window_layers", n)
        return [w if i >= first else None for i in range(n)]
    return [None] * n


def embedding(table, tokens):
    """x[t] = table[token[t]], no scaling.  src/qwen_model.cpp:1234-1244."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def rmsnorm(x, w, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w over the last axis; the weight multiplies after normalising.
    src/qwen_ops.cpp:8-13; src/gpu_ops.hip:34-53."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * w


def rope_rotate_half(v, positions, theta, n_rot):
    """v [T, H, D]; pair (i, i + n_rot/2) turns by positions[t] * theta^(-2i/n_rot); dims >= n_rot stay.
    src/qwen_ops.cpp:15-24; src/attention.hip:225-240."""
    half = n_rot // 2
    i = torch.arange(half, dtype=F64)
    ang = torch.as_tensor(positions, dtype=F64)[:, None] * torch.pow(torch.tensor(float(theta), dtype=F64),
                                                                     -2.0 * i / n_rot)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = v.clone()
    a, b = v[..., :half], v[..., half:n_rot]
    out[..., :half] = a * c - b * s
    out[..., half:n_rot] = a * s + b * c
    return out


def attention(q, k, v, scale, window=None):
    """q [T, HQ, D], k and v [T, HKV, D], all of one sequence from position 0.  Query head h uses kv head
    h // (HQ // HKV); scores * scale, causal (position z sees p <= z, and p > z - window with a window),
    max-subtracted softmax, weighted sum of v.  src/qwen_ops.cpp:26-51; src/attention.h:73;
    src/attention.cpp:197 (scale 1/sqrt(D))."""
    T, HQ, D = q.shape
    HKV = k.shape[1]
    grp = HQ // HKV
    out = torch.zeros_like(q)
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window:
        visible &= pos[None, :] > pos[:, None] - window
    for h in range(HQ):
        g = h // grp
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        p = torch.exp(s)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def attention_block(x, w, prefix, cfg, positions, window):
    """Projections (+ optional biases), per-head RMSNorm of q and k with the layer-norm eps, rotation, attention,
    output projection.  src/qwen_model.cpp:940-975; src/attention.hip:273-313 (bias, then norm, then rotation)."""
    T = x.shape[0]
    HQ, HKV = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    D = cfg.get("head_dim") or cfg["hidden_size"] // HQ
    eps = cfg.get("rms_norm_eps", 1e-6)
    q = x @ w[prefix + "self_attn.q_proj.weight"].T
    k = x @ w[prefix + "self_attn.k_proj.weight"].T
    v = x @ w[prefix + "self_attn.v_proj.weight"].T
    if cfg.get("attention_bias"):
        q = q + w[prefix + "self_attn.q_proj.bias"]
        k = k + w[prefix + "self_attn.k_proj.bias"]
        v = v + w[prefix + "self_attn.v_proj.bias"]
    q, k, v = q.view(T, HQ, D), k.view(T, HKV, D), v.view(T, HKV, D)
    q = rmsnorm(q, w[prefix + "self_attn.q_norm.weight"], eps)
    k = rmsnorm(k, w[prefix + "self_attn.k_norm.weight"], eps)
    theta = cfg.get("rope_theta")
    if theta is None:
        theta = (cfg.get("rope_parameters") or {}).get("rope_theta", 10000.0)
    q = rope_rotate_half(q, positions, theta, D)
    k = rope_rotate_half(k, positions, theta, D)
    o = attention(q, k, v, 1.0 / math.sqrt(D), window)
    return o.reshape(T, HQ * D) @ w[prefix + "self_attn.o_proj.weight"].T


def swiglu_mlp(x, w, prefix):
    """y = Wd (g / (1 + exp(-g)) * u), g = Wg x, u = Wu x.  src/qwen_model.cpp:1179-1183; src/gpu_ops.hip:109-111."""
    g = x @ w[prefix + "mlp.gate_proj.weight"].T
    u = x @ w[prefix + "mlp.up_proj.weight"].T
    return (g / (1.0 + torch.exp(-g)) * u) @ w[prefix + "mlp.down_proj.weight"].T


def forward(cfg, w, tokens, return_hidden=False, layer_outputs=None):
    """Logits [T, V] (float64) for one whole sequence starting at position 0.  Layer order and residuals:
    src/qwen_model.cpp:1196-1279; tied head when config says so: src/inference.cpp:1392-1396.  A list given as
    ``layer_outputs`` receives the residual stream after every layer (what the reference's per-layer callback sees,
    src/qwen_model.cpp:1262-1275)."""
    eps = cfg.get("rms_norm_eps", 1e-6)
    positions = list(range(len(tokens)))
    x = embedding(w["model.embed_tokens.weight"], tokens)
    windows = layer_windows(cfg)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        x = x + attention_block(rmsnorm(x, w[p + "input_layernorm.weight"], eps), w, p, cfg, positions, windows[l])
        x = x + swiglu_mlp(rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps), w, p)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    xn = rmsnorm(x, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    logits = xn @ head.T
    return (logits, x) if return_hidden else logits


# ---- sampling ---------------------------------------------------------------------------------------

def greedy(logits):
    """argmax, the lowest id wins ties.  src/sampler.cpp:60-68."""
    return int(np.argmax(np.asarray(logits)))


def temperature_probabilities(logits, temperature, logit_range=40.0):
    """The distribution the reference draws from with top-k, top-p and min-p off: tokens with
    logit >= max - 40 weigh exp((l - max) / T).  src/sampler.cpp:120-127, 155-162."""
    l = np.asarray(logits, dtype=np.float64)
    mx = l.max()
    p = np.where(l >= mx - logit_range, np.exp((l - mx) / temperature), 0.0)
    return p / p.sum()
