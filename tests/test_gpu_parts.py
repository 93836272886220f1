"""Each part of a layer alone against the plain functions, and parts that the framework does not have:
a toy mixer with state of its own, a toy position encoding, a toy feed-forward with routing, a run order
that names a layer twice and lets a call read another call's cache (GPU).  The toys are defined here and
registered through the public registries; no file of the framework changes."""
import json
import math

import pytest
import torch

from plain import qwen3_plain as P
from helpers import TINY_B, TINY_B_INIT, make_model, random_tokens, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_ctx(segs, page_size, groups_tables, dtype):
    """A StepContext for segments [(ctx_len, q_len)] whose requests own pages 0.. in order."""
    from purhie_b200.parts import GroupStep, StepContext, Workspace
    toks, pos, row_seg, seg_start, ctx_lens, q_lens = [], [], [], [0], [], []
    for s, (ctx, ql) in enumerate(segs):
        pos += list(range(ctx - ql, ctx)); row_seg += [s] * ql; seg_start.append(seg_start[-1] + ql)
        ctx_lens.append(ctx); q_lens.append(ql)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    T = len(pos)
    groups = []
    for tables in groups_tables:
        w = max(len(t) for t in tables)
        bt = i32([t + [-1] * (w - len(t)) for t in tables])
        slots = [tables[s][p // page_size] * page_size + p % page_size for s, (ctx, ql) in enumerate(segs)
                 for p in range(ctx - ql, ctx)]
        groups.append(GroupStep(bt, i32(slots), page_size))
    dec = [seg_start[s] for s, q in enumerate(q_lens) if q == 1]
    tiles = [(s, f) for s, q in enumerate(q_lens) if q > 1 for f in range(0, q, 64)]
    return StepContext(T=T, S=len(segs), token_ids=i32([0] * T), positions=i32(pos), row_seg=i32(row_seg),
                       seg_start=i32(seg_start), seg_ctx_len=i32(ctx_lens), seg_slot=i32(list(range(len(segs)))),
                       q_lens=q_lens, ctx_lens=ctx_lens, groups=groups, workspace=Workspace(DEV), compute_dtype=dtype,
                       decode_only=not tiles, decode_rows=i32(dec or [0]) if tiles else None, n_decode_rows=len(dec),
                       decode_max_ctx=max([c for c, q in segs if q == 1] or [0]),
                       q_tile_seg=i32([t[0] for t in tiles] or [0]), q_tile_first=i32([t[1] for t in tiles] or [0]),
                       n_q_tiles=len(tiles))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part_folds_the_pending_addend(dtype):
    from purhie_b200.parts import Addend, BuildContext, PartSpec, ResidualStream, make_part
    n = make_part("norm", PartSpec("rmsnorm", {"size": 100, "eps": 1e-4, "names": {"weight": "w"}}), BuildContext(dtype))
    assert list(n.tensor_specs()) == ["w"] and n.tensor_specs()["w"].shape == (100,)
    w = torch.rand(100, device=DEV) + 0.5
    n.bind({"w": w}, DEV)
    ctx = make_ctx([(7, 7)], 16, [], dtype)
    x = torch.randn(7, 100, device=DEV)
    add = torch.randn(7, 100, device=DEV)
    stream = ResidualStream(x.clone())
    stream.add(Addend(add.clone()))
    y = n.forward(stream, ctx)
    v = (x + add).double()
    assert stream.pending is None and rel_err(stream.x, v) < 1e-6
    assert rel_err(y, P.rmsnorm(v, w.double(), 1e-4)) < (1e-5 if dtype == torch.float32 else 6e-3)


def test_rotary_table_is_made_in_double_precision():
    from purhie_b200.parts import BuildContext, PartSpec, make_part
    r = make_part("position", PartSpec("rope_neox", {"theta": 1e6, "n_rot": 32, "max_position": 300}), BuildContext())
    t = r.rotation_table(DEV).cpu()
    v = torch.randn(1, 1, 32, dtype=torch.float64)
    for pos in (0, 1, 255, 299):
        c, s = t[pos, :16].double(), t[pos, 16:].double()
        mine = torch.cat([v[0, 0, :16] * c - v[0, 0, 16:] * s, v[0, 0, :16] * s + v[0, 0, 16:] * c])
        assert (mine - P.rope_rotate_half(v, [pos], 1e6, 32).view(-1)).abs().max() < 1e-6


@pytest.mark.parametrize("dtype,window,HQ,HKV,D", [(torch.float32, None, 6, 3, 24), (torch.float32, 9, 4, 1, 16),
                                                   (torch.bfloat16, None, 8, 2, 64), (torch.bfloat16, 20, 4, 4, 128)])
def test_attention_part_alone(dtype, window, HQ, HKV, D):
    """One attention mixer, its own weights: a prompt portion in one step, then the rest in a second step that
    reads the first step's pages, against the plain attention block over the whole sequence."""
    from purhie_b200.parts import BuildContext, CacheView, PartSpec, make_part
    E, ps, n1, n2 = 80, 8, 37, 30
    names = {k: k for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm", "q_bias", "k_bias", "v_bias")}
    pos_spec = PartSpec("rope_neox", {"theta": 5e4, "n_rot": D, "max_position": 128})
    att = make_part("mixer", PartSpec("attention", {
        "hidden_size": E, "num_heads": HQ, "num_kv_heads": HKV, "head_dim": D, "qk_norm_eps": 1e-5, "bias": True,
        "position": pos_spec, "window": window, "names": names}), BuildContext(dtype))
    g = torch.Generator().manual_seed(0)
    w = {n: (torch.randn(s.shape, generator=g) * (0.2 if s.role == "matrix" else 0.3) + (1.0 if s.init == "scale" else 0.0))
         for n, s in att.tensor_specs().items()}
    att.bind({n: t.to(DEV).to(dtype if att.tensor_specs()[n].role == "matrix" else torch.float32) for n, t in w.items()}, DEV)
    need = att.cache_need()
    assert (need.kind, need.kv_heads, need.head_dim, need.window) == ("pages", HKV, D, window)
    pool = torch.full((16, 1, 2, HKV, ps, D), float("nan"), dtype=dtype, device=DEV)
    view = CacheView("pages", 0, pool[0, 0, 0], pool[0, 0, 1], pool.stride(0), ps, num_pages=16, writable=True)
    table = list(range(15, 15 - 9, -1))                       # pages in reverse order
    x = torch.randn(n1 + n2, E, generator=g)
    outs = []
    for ctx_len, ql in ((n1, n1), (n1 + n2, n2)):
        ctx = make_ctx([(ctx_len, ql)], ps, [[table[:-(-ctx_len // ps)]]], dtype)
        y = att.forward(x[ctx_len - ql:ctx_len].to(DEV).to(dtype).contiguous(), ctx, view)
        assert y.tensor.dtype == torch.float32
        outs.append(y.tensor.reshape(y.splits, ql, E).sum(0).clone())
    got = torch.cat(outs)
    wd = {("self_attn." + k.replace("_bias", "_proj.bias") if k.endswith("_bias") else
           "self_attn." + k + ".weight"): (t.to(dtype).double() if att.tensor_specs()[k].role == "matrix" else t.double())
          for k, t in w.items()}
    cfg = {"num_attention_heads": HQ, "num_key_value_heads": HKV, "head_dim": D, "hidden_size": E, "rms_norm_eps": 1e-5,
           "attention_bias": True, "rope_theta": 5e4}
    ref = P.attention_block(x.to(dtype).double(), wd, "", cfg, list(range(n1 + n2)), window)
    assert rel_err(got, ref) < (2e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part_alone(dtype):
    from purhie_b200.parts import BuildContext, PartSpec, make_part
    E, FF, T = 72, 200, 19
    ff = make_part("feed_forward", PartSpec("swiglu", {"hidden_size": E, "intermediate_size": FF, "names": {
        "gate_proj": "g", "up_proj": "u", "down_proj": "d"}}), BuildContext(dtype))
    g = torch.Generator().manual_seed(1)
    w = {n: torch.randn(s.shape, generator=g) * 0.2 for n, s in ff.tensor_specs().items()}
    ff.bind({n: t.to(DEV).to(dtype) for n, t in w.items()}, DEV)
    x = torch.randn(T, E, generator=g)
    ctx = make_ctx([(T, T)], 16, [], dtype)
    y = ff.forward(x.to(DEV).to(dtype), ctx)
    got = y.tensor.reshape(y.splits, T, E).sum(0)
    wd = {"mlp.gate_proj.weight": w["g"].to(dtype).double(), "mlp.up_proj.weight": w["u"].to(dtype).double(),
          "mlp.down_proj.weight": w["d"].to(dtype).double()}
    assert rel_err(got, P.swiglu_mlp(x.to(dtype).double(), wd, "")) < (1e-5 if dtype == torch.float32 else 2e-2)


def test_embedding_and_tied_head_parts():
    from purhie_b200.parts import BuildContext, PartSpec, make_part
    b = BuildContext(torch.float32)
    emb = make_part("embedding", PartSpec("embedding", {"vocab_size": 300, "hidden_size": 40, "names": {"weight": "e"}}), b)
    head = make_part("head", PartSpec("lm_head", {"hidden_size": 40, "vocab_size": 300, "tied_to": "e"}), b)
    assert head.tensor_specs() == {}
    table = torch.randn(300, 40, device=DEV)
    emb.bind({"e": table}, DEV); head.bind({"e": table}, DEV)
    ctx = make_ctx([(5, 5)], 16, [], torch.float32)
    ctx.token_ids = torch.tensor([3, 299, 0, 3, 17], dtype=torch.int32, device=DEV)
    x = emb.forward(ctx)
    assert torch.equal(x, table[ctx.token_ids.long()])
    logits = head.forward(x, ctx, 5)
    assert rel_err(logits, x.double() @ table.double().T) < 1e-5


# ---- toys: parts that are not in the framework ----------------------------------------------------------

def _register_toys():
    from purhie_b200.cache import CacheNeed
    from purhie_b200.csrc import ops
    from purhie_b200.parts import Addend, FeedForward, Mixer, PositionEncoding, register_part
    from purhie_b200.weights import TensorSpec

    class RunningMeanMixer(Mixer):
        """State of its own: per request the sum of all inputs so far and their count.  Output for a token =
        (mean of the request's inputs up to and including it) @ W.  Rows of a request arrive in order."""

        def __init__(self, params, build):
            super().__init__(params, build)
            self.size = params["hidden_size"]
            self.w = None

        def tensor_specs(self):
            n = self.names["weight"]
            return {n: TensorSpec(n, (self.size, self.size))}

        def bind(self, tensors, device):
            self.w = tensors[self.names["weight"]]

        def cache_need(self):
            return CacheNeed.state((self.size + 1,), "float32")

        def forward(self, x, ctx, cache):
            out = ctx.workspace.get("toy_mean", (ctx.T, self.size), torch.float32)
            slots = ctx.seg_slot.tolist()
            row = 0
            for s, n in enumerate(ctx.q_lens):
                st = cache.state[slots[s]]
                xs = x[row:row + n].float()
                sums = st[:self.size] + torch.cumsum(xs, 0)
                counts = st[self.size] + torch.arange(1, n + 1, device=x.device)
                out[row:row + n] = sums / counts[:, None]
                st[:self.size] = sums[-1]
                st[self.size] = counts[-1]
                row += n
            y = ctx.workspace.get("toy_mean_out", (ctx.T, self.size), torch.float32)
            ops.gemm_simple(out, self.w, y)
            return Addend(y)

    class ScaledRotary(PositionEncoding):
        """Another position encoding: rotate-half pairs with every frequency divided by ``factor``."""

        def __init__(self, params, build):
            super().__init__(params, build)
            self.n_rot, self.theta, self.factor, self.max_position = params["n_rot"], params["theta"], params["factor"], params["max_position"]

        def rotation_table(self, device):
            i = torch.arange(self.n_rot // 2, dtype=torch.float64)
            ang = torch.arange(self.max_position, dtype=torch.float64)[:, None] * (self.theta ** (-2 * i / self.n_rot) / self.factor)
            return torch.cat([ang.cos(), ang.sin()], 1).float().to(device)

    class Top1Routed(FeedForward):
        """A feed-forward with routing: the router's float32 logits pick one of ``experts`` matrices per token."""

        def __init__(self, params, build):
            super().__init__(params, build)
            self.size, self.experts = params["hidden_size"], params["experts"]

        def tensor_specs(self):
            specs = {"toy.router": TensorSpec("toy.router", (self.experts, self.size))}
            for e in range(self.experts):
                specs[f"toy.expert{e}"] = TensorSpec(f"toy.expert{e}", (self.size, self.size))
            return specs

        def bind(self, tensors, device):
            self.router = tensors["toy.router"].float()
            self.mats = [tensors[f"toy.expert{e}"] for e in range(self.experts)]

        def forward(self, x, ctx):
            logits = ctx.workspace.get("toy_router", (ctx.T, self.experts), torch.float32)
            ops.gemm_simple(x.float().contiguous(), self.router, logits)
            choice = logits.argmax(-1)
            y = ctx.workspace.get("toy_ff", (ctx.T, self.size), torch.float32)
            y.zero_()
            for e in range(self.experts):
                rows = torch.nonzero(choice == e).flatten()
                if rows.numel():
                    part = torch.empty(rows.numel(), self.size, dtype=torch.float32, device=x.device)
                    ops.gemm_simple(x[rows].contiguous(), self.mats[e], part)
                    y[rows] = part
            return Addend(y)

    register_part("mixer", "toy_running_mean", RunningMeanMixer)
    register_part("position", "toy_scaled_rope", ScaledRotary)
    register_part("feed_forward", "toy_top1", Top1Routed)


def _toy_spec(cfg):
    """A model nobody has: layer 0 attention with the toy position encoding and a routed feed-forward; layer 1
    the stateful toy mixer with SwiGLU.  Run order: layer 0, layer 1, layer 0 again (a cache of its own), and a
    fourth call of layer 0 that reads the first call's cache."""
    from purhie_b200.parts import LayerCall, LayerSpec, ModelSpec, PartSpec
    E = cfg["hidden_size"]
    norm = lambda n: PartSpec("rmsnorm", {"size": E, "eps": 1e-5, "names": {"weight": n}})
    att = PartSpec("attention", {"hidden_size": E, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "qk_norm_eps": 1e-5,
                                 "bias": False, "window": None,
                                 "position": PartSpec("toy_scaled_rope", {"theta": 1e4, "n_rot": 16, "factor": 4.0, "max_position": 128}),
                                 "names": {k: "l0." + k for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")}})
    layers = (
        LayerSpec(att, norm("l0.n1"), PartSpec("toy_top1", {"hidden_size": E, "experts": 3}), norm("l0.n2")),
        LayerSpec(PartSpec("toy_running_mean", {"hidden_size": E, "names": {"weight": "l1.mean"}}), norm("l1.n1"),
                  PartSpec("swiglu", {"hidden_size": E, "intermediate_size": 48,
                                      "names": {"gate_proj": "l1.g", "up_proj": "l1.u", "down_proj": "l1.d"}}), norm("l1.n2")))
    return ModelSpec(hidden_size=E, vocab_size=cfg["vocab_size"], max_position=128,
                     embedding=PartSpec("embedding", {"vocab_size": cfg["vocab_size"], "hidden_size": E, "names": {"weight": "emb"}}),
                     layers=layers, schedule=(LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(0, cache_from=0)),
                     final_norm=norm("final"), head=PartSpec("lm_head", {"hidden_size": E, "vocab_size": cfg["vocab_size"], "tied_to": "emb"}))


def test_toy_architecture_is_registered_built_and_stepped(tmp_path):
    from dataclasses import dataclass
    from purhie_b200.config import register_architecture, unregister_architecture
    from purhie_b200.config.base import ModelConfig
    from purhie_b200.engine import Engine, StepEntry
    from purhie_b200.parts import unregister_part
    from purhie_b200.weights import expected_tensors, write_random_model

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        hidden_size: int = 32
        vocab_size: int = 64

        @classmethod
        def from_dict(cls, d):
            return cls(d["architectures"][0], d["hidden_size"], d["vocab_size"])

        def to_dict(self):
            return {"architectures": [self.architecture], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size}

    _register_toys()
    register_architecture("ToyForCausalLM", ToyConfig, lambda c: _toy_spec(c.to_dict()))
    try:
        cfg = ToyConfig("ToyForCausalLM", 32, 64)
        assert "l1.mean" in expected_tensors(cfg) and "toy.expert2" in expected_tensors(cfg)
        write_random_model(str(tmp_path), cfg, 3, std=0.3, scale_low=0.8, scale_high=1.2, dtype="float32")
        toks = random_tokens(50, 64, 9)
        eng = Engine.from_folder(str(tmp_path), dtype="float32", page_size=8, max_tokens=256, max_requests=3, cuda_graphs=False)
        # the cache manager gave the stateful mixer a slot and the two owning attention calls one group
        assert [n.kind for n in eng.cache.needs] == ["pages", "state", "pages", "none"]
        assert len(eng.cache.groups) == 1 and eng.cache.groups[0].entries == [0, 2] and eng.cache.state_entries == [1]
        eng.add_request("whole")
        whole = eng.step([StepEntry("whole", toks, list(range(50)))]).clone()
        assert torch.isfinite(whole).all() and whole.std() > 0
        # cut into portions and mixed with another request: the same logits (the state carries over exactly)
        eng.add_request("cut"); eng.add_request("other")
        parts, i = [], 0
        for n in (7, 2, 1, 13, 1, 26):
            lg = eng.step([StepEntry("other", random_tokens(3, 64, i), []), StepEntry("cut", toks[i:i + n], list(range(n)))])
            parts.append(lg.clone()); i += n
        cut = torch.cat(parts)
        assert rel_err(cut, whole) < 1e-5
        # a new request in a reused slot starts from a zeroed state
        eng.release("whole"); eng.add_request("again")
        again = eng.step([StepEntry("again", toks, list(range(50)))])
        assert rel_err(again, whole) < 1e-5
        # the fourth call really reads the first call's cache: it owns no pages
        assert eng.views[3].writable is False and eng.views[3].k_base.data_ptr() == eng.views[0].k_base.data_ptr()
    finally:
        unregister_architecture("ToyForCausalLM")
        for fam, kind in (("mixer", "toy_running_mean"), ("position", "toy_scaled_rope"), ("feed_forward", "toy_top1")):
            unregister_part(fam, kind)
