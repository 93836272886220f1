"""The bfloat16 engine against the float32 engine at real layer sizes (GPU).

The tiny configurations of the other tests leave paths untouched that only real sizes reach: a decode row whose
context is cut into more splits than it has blocks to fill, products on pairs of CTAs, K in parts, attention
tiles shared by several CTAs.  Two layers of an 8B-class shape (hidden 4096, 32 query heads over 8 kv heads of
128, feed-forward 12288), of a 0.6B-class shape (hidden 1024 under a query width of 2048, tied embeddings) and of a
32B-class shape (hidden 5120, groups of eight query heads, feed-forward 25600) with random weights: whatever way the
tokens are fed, the bfloat16 engine must stay as close to the float32 engine as it is for a whole prompt.
"""
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
    return float((a.double() - b.double()).norm() / b.double().norm())


@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_every_way_of_feeding_is_as_close_to_float32_as_a_whole_prompt(shape):
    from purhie_b200.api import load_model_random
    from purhie_b200.config import Qwen3Config
    from purhie_b200.engine import Engine, StepEntry
    cfg = Qwen3Config.from_dict(SHAPES[shape])
    g = torch.Generator().manual_seed(11)
    toks = torch.randint(0, cfg.vocab_size, (2700,), generator=g).tolist()
    others = [torch.randint(0, cfg.vocab_size, (n + 24,), generator=g).tolist() for n in (17, 300, 1000, 2047, 64, 129, 700)]
    out = {}
    for dtype in ("float32", "bfloat16"):
        m = load_model_random(cfg, 7, dtype, "cuda:0")
        eng = Engine(m._decoder, cfg, page_size=16, max_tokens=16384, max_requests=8)
        res = {}
        eng.add_request("w")
        res["whole"] = eng.step([StepEntry("w", toks[:2524], list(range(2499, 2524)))]).clone()      # from the prompt's last place on
        eng.release("w")
        # one request decoding alone at 2,500 tokens: its context is cut into more splits than it has blocks for
        eng.add_request("d")
        eng.step([StepEntry("d", toks[:2500], [])])
        res["decode"] = torch.cat([eng.step([StepEntry("d", [toks[2500 + k]], [0])]).clone() for k in range(24)])
        # ... then beside seven others of other lengths, and beside a prompt that comes in chunks
        for i, o in enumerate(others):
            eng.add_request(i)
            eng.step([StepEntry(i, o[:len(o) - 24], [])])
        rows = []
        for k in range(24):
            ent = [StepEntry("d", [toks[2524 + k]], [0])] + [StepEntry(i, [o[len(o) - 24 + k]], []) for i, o in enumerate(others)]
            rows.append(eng.step(ent).clone())
        res["batch"] = torch.cat(rows)
        for i in range(len(others)):
            eng.release(i)
        # a short portion late in the context: one attention tile that looks back over 2,600 keys, shared by several CTAs
        res["late"] = eng.step([StepEntry("d", toks[2548:2600], [0, 25, 51])]).clone()
        eng.add_request("c")
        for s in range(0, 2500, 500):
            lg = eng.step([StepEntry("c", toks[s:s + 500], [499] if s + 500 >= 2500 else [])])
        res["chunks"] = lg.clone()
        out[dtype] = res
        del eng, m
        torch.cuda.empty_cache()
    f32, b16 = out["float32"], out["bfloat16"]
    assert torch.equal(f32["whole"][1:], f32["decode"])               # float32: the same bits however it is fed
    assert torch.equal(f32["whole"][:1], f32["chunks"])
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
        assert not torch.isnan(b16[name]).any()
