"""Each kernel alone against a plain float64/float32 PyTorch restatement, at sizes other than the engine's
(GPU).  Sizes are deliberately awkward: widths and vocabularies that are no power of two, row counts that
do not fill tiles."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def rel(got, ref):
    return ((got.double() - ref.double()).abs().max() / ref.double().abs().max().clamp_min(1e-30)).item()


# ---- matrix products -----------------------------------------------------------------------------------

@pytest.mark.parametrize("M,N,K", [(1, 40, 24), (5, 100, 96), (64, 64, 64), (70, 130, 50), (200, 257, 333)])
@pytest.mark.parametrize("xd,wd,yd", [(torch.float32, torch.float32, torch.float32),
                                      (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                      (torch.float32, torch.bfloat16, torch.float32)])
def test_gemm_simple(M, N, K, xd, wd, yd):
    from purhie_b200.csrc import ops
    x, w = rnd(M, K, dtype=xd, seed=1), rnd(N, K, dtype=wd, seed=2)
    out = torch.full((M, N), float("nan"), dtype=yd, device=DEV)
    ops.gemm_simple(x, w, out)
    ref = x.double() @ w.double().T
    assert rel(out, ref) < (1e-5 if yd == torch.float32 else 6e-3)


def test_gemm_simple_sums_twelve_thousand_terms_in_float32():
    """The float32 path's product at the longest reduction of the model shapes (a feed-forward of 12,288) against
    float64."""
    from purhie_b200.csrc import ops
    x, w = rnd(5, 12288, seed=21), rnd(130, 12288, seed=22)
    out = torch.full((5, 130), float("nan"), device=DEV)
    ops.gemm_simple(x, w, out)
    assert rel(out, x.double() @ w.double().T) < 1e-5


def test_gemm_simple_rows_do_not_depend_on_the_batch():
    from purhie_b200.csrc import ops
    x, w = rnd(150, 200, seed=3), rnd(90, 200, seed=4)
    full = torch.empty(150, 90, device=DEV)
    ops.gemm_simple(x, w, full)
    for lo, hi in ((0, 1), (17, 18), (64, 150), (3, 70)):
        part = torch.empty(hi - lo, 90, device=DEV)
        ops.gemm_simple(x[lo:hi].contiguous(), w, part)
        assert torch.equal(part, full[lo:hi])


@pytest.mark.parametrize("M,N,K,swapped,block_n,splits", [
    (128, 256, 64, False, 256, 1),          # one tile, one block of K
    (128, 256, 512, False, 256, 1),         # the stage ring wraps
    (300, 520, 200, False, 256, 1),         # ragged tiles on every side, K not a multiple of 64
    (2048, 1024, 1024, False, 256, 1),      # many tiles per CTA: both accumulator buffers in use
    (130, 136, 72, False, 128, 1),
    (129, 72, 1000, False, 64, 1),
    (1, 128, 64, True, 16, 1),              # one token
    (8, 384, 256, True, 16, 1),
    (8, 1000, 4096, True, 16, 8),           # decode shape: K split over CTAs, partial sums
    (33, 520, 1000, True, 64, 3),
    (64, 300, 328, True, 64, 2),
    (100, 264, 512, True, 128, 1),
    (17, 96, 96, True, 32, 1),
    (200, 260, 136, True, 256, 1),
])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tcgen05(M, N, K, swapped, block_n, splits, out_dtype):
    from purhie_b200.csrc import gemm100
    if splits > 1 and out_dtype != torch.float32:
        pytest.skip("partial sums are float32")
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=5), rnd(N, K, dtype=torch.bfloat16, seed=6)
    out = torch.full((splits, M, N) if splits > 1 else (M, N), float("nan"), dtype=out_dtype, device=DEV)
    gemm100.gemm(x, w, out, swapped=swapped, block_n=block_n, splits=splits)
    gemm100.check_errors(DEV)
    got = out.double().sum(0) if splits > 1 else out.double()
    ref = x.double() @ w.double().T
    assert not torch.isnan(got).any()
    assert rel(got, ref) < (2e-5 if out_dtype == torch.float32 else 5e-3)


def test_gemm_tcgen05_against_the_plain_kernel_and_on_few_ctas():
    from purhie_b200.csrc import gemm100, ops
    x, w = rnd(384, 320, dtype=torch.bfloat16, seed=7), rnd(700, 320, dtype=torch.bfloat16, seed=8)
    a, b, c = (torch.empty(384, 700, device=DEV) for _ in range(3))
    gemm100.gemm(x, w, a, swapped=False, block_n=256)
    gemm100.gemm(x, w, c, swapped=False, block_n=256, max_ctas=2)       # every CTA walks many tiles
    ops.gemm_simple(x, w, b)
    gemm100.check_errors(DEV)
    assert rel(a, b) < 2e-5 and torch.equal(a, c)


@pytest.mark.parametrize("M,N,K", [(128, 512, 256), (300, 1000, 200), (2048, 2048, 512)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tcgen05_swiglu_epilogue(M, N, K, out_dtype):
    from purhie_b200.csrc import gemm100
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=9), rnd(N, K, dtype=torch.bfloat16, seed=10, scale=0.2)
    out = torch.full((M, N // 2), float("nan"), dtype=out_dtype, device=DEV)
    gemm100.gemm(x, w, out, swapped=False, block_n=256, swiglu=True)
    gemm100.check_errors(DEV)
    y = x.double() @ w.double().T
    g, u = y[:, 0::2], y[:, 1::2]
    assert rel(out, g / (1 + torch.exp(-g)) * u) < (3e-5 if out_dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("M,N,K,max_clusters,swiglu", [
    (256, 256, 64, 0, False),               # one tile, one block of K
    (256, 256, 1024, 0, False),             # the stage ring wraps
    (300, 520, 200, 0, False),              # ragged on every side, K not a multiple of 64; the second CTA's rows partly outside
    (130, 136, 72, 0, False),               # the second CTA of the pair has two rows and eight features
    (2048, 1024, 1024, 3, False),           # many tiles per pair: both accumulator buffers in use
    (1024, 2048, 512, 0, True),
    (2048, 6144, 256, 0, False),            # more tiles than pairs
])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tcgen05_pair(M, N, K, max_clusters, swiglu, out_dtype):
    """Two CTAs on one 256 x 256 tile (cta_group::2): each loads its half of both operands, the leader issues."""
    from purhie_b200.csrc import gemm100
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=13), rnd(N, K, dtype=torch.bfloat16, seed=14, scale=0.2)
    out = torch.full((M, N // 2) if swiglu else (M, N), float("nan"), dtype=out_dtype, device=DEV)
    gemm100.gemm_pair(x, w, out, max_clusters=max_clusters, swiglu=swiglu)
    gemm100.check_errors(DEV)
    y = x.double() @ w.double().T
    if swiglu:
        g, u = y[:, 0::2], y[:, 1::2]
        y = g / (1 + torch.exp(-g)) * u
    assert not torch.isnan(out).any()
    assert rel(out, y) < (3e-5 if out_dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("M,N,K,splits", [(512, 768, 2048, 2), (300, 520, 4104, 3), (1024, 1024, 8192, 8)])
def test_gemm_tcgen05_pair_with_k_in_parts(M, N, K, splits):
    from purhie_b200.csrc import gemm100
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=17), rnd(N, K, dtype=torch.bfloat16, seed=18, scale=0.2)
    out = torch.full((splits, M, N), float("nan"), device=DEV)
    gemm100.gemm_pair(x, w, out, splits=splits)
    gemm100.check_errors(DEV)
    assert rel(out.double().sum(0), x.double() @ w.double().T) < 3e-5


def test_plan_for_many_tokens_keeps_a_fused_epilogue_whole_and_fills_the_device():
    from purhie_b200 import native

    def plan(M, N, K, allow_split, fused=False):
        p = native.answer(native.lib().qe_plan_gemm(M, N, K, 148, int(allow_split), int(fused)))
        return p["pair"], p["splits"], p["swapped"]

    assert plan(2048, 24576, 4096, True, fused=True)[:2] == (True, 1)
    assert plan(512, 24576, 4096, True, fused=True)[1] == 1
    pair, splits, _ = plan(512, 4096, 12288, True)                   # 32 tiles of 256 x 256 on 74 pairs: K is cut
    assert splits > 1
    assert plan(512, 4096, 12288, False)[1] == 1
    assert plan(128, 4096, 4096, True)[0] is False                   # one tile high: no second CTA to pair with
    few = plan(8, 4096, 12288, True)                                 # few tokens: weights on the wide side, K in parts
    assert few[2] is True and few[1] > 1 and plan(8, 4096, 12288, False)[1] == 1


def test_gemm_tcgen05_pair_equals_one_cta_kernel():
    from purhie_b200.csrc import gemm100
    x, w = rnd(640, 448, dtype=torch.bfloat16, seed=15), rnd(1000, 448, dtype=torch.bfloat16, seed=16)
    a, b = torch.empty(640, 1000, device=DEV), torch.empty(640, 1000, device=DEV)
    gemm100.gemm(x, w, a, swapped=False, block_n=256)
    gemm100.gemm_pair(x, w, b)
    gemm100.check_errors(DEV)
    assert torch.equal(a, b)                # the same products added in the same order of K


@pytest.mark.parametrize("M,N,K,block_n", [(1, 256, 128, 16), (8, 1000, 328, 16), (33, 520, 200, 64), (100, 264, 512, 128)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tcgen05_swiglu_epilogue_with_few_tokens(M, N, K, block_n, out_dtype):
    """Swapped orientation: gate and up features are neighbouring accumulator rows, exchanged between lanes."""
    from purhie_b200.csrc import gemm100
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=19), rnd(N, K, dtype=torch.bfloat16, seed=20, scale=0.2)
    out = torch.full((M, N // 2), float("nan"), dtype=out_dtype, device=DEV)
    gemm100.gemm(x, w, out, swapped=True, block_n=block_n, swiglu=True)
    gemm100.check_errors(DEV)
    y = x.double() @ w.double().T
    g, u = y[:, 0::2], y[:, 1::2]
    assert rel(out, g / (1 + torch.exp(-g)) * u) < (3e-5 if out_dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("M,N,K", [(300, 520, 200), (2048, 1024, 512), (300, 522, 200), (131, 257, 64)])
def test_gemm_tcgen05_adds_into_the_output(M, N, K):
    """The residual sum in the epilogue: out += x w^T, on one CTA per tile and on pairs, with the bits of a product
    written out and added afterwards."""
    from purhie_b200.csrc import gemm100
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=27), rnd(N, K, dtype=torch.bfloat16, seed=28, scale=0.2)
    base = rnd(M, N, seed=29)
    prod = torch.empty(M, N, device=DEV)
    gemm100.gemm(x, w, prod, swapped=False, block_n=256)
    for pair in (False, True):
        out = base.clone()
        if pair:
            gemm100.gemm_pair(x, w, out, accumulate=True)
        else:
            gemm100.gemm(x, w, out, swapped=False, block_n=256, accumulate=True)
        gemm100.check_errors(DEV)
        assert torch.equal(out, base + prod)


@pytest.mark.parametrize("M,N,K", [(300, 1000, 192), (128, 256, 64), (515, 516, 104), (1024, 4096, 1024)])
def test_gemm_tcgen05_with_many_rows_does_the_work_of_the_norms_around_it(M, N, K):
    """Plain orientation, tiles of 256 columns, on one CTA per tile and on pairs.  (1) Adding into the output, the
    epilogue also leaves the new rows times the weight of the norm behind it, in bfloat16, and each row's sum of squares
    per tile; the accumulated output keeps the bits it has without that.  (2) A factor per row that the norm in front
    left out is applied before the store, the bfloat16 rounding and the activation."""
    from purhie_b200.csrc import gemm100
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=51, scale=0.5), rnd(N, K, dtype=torch.bfloat16, seed=52, scale=0.1)
    base = rnd(M, N, seed=53)
    wn = (torch.rand(N, generator=torch.Generator().manual_seed(54)) + 0.5).to(DEV)
    tiles = -(-N // 256)
    sq = (torch.rand(M, 3, generator=torch.Generator().manual_seed(55)) * 100 + 1).to(DEV)
    width, eps = 77, 1e-3
    factor = torch.rsqrt(sq.double().sum(-1, keepdim=True) / width + eps)
    prod = x.double() @ w.double().T
    for pair in (False, True):
        run = (lambda out, **kw: gemm100.gemm_pair(x, w, out, **kw)) if pair else \
              (lambda out, **kw: gemm100.gemm(x, w, out, swapped=False, block_n=256, **kw))
        plain = base.clone()
        run(plain, accumulate=True)
        out = base.clone()
        rows = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        sumsq = torch.full((M, 2 * tiles), float("nan"), device=DEV)            # per 128 columns: two entries per tile
        run(out, accumulate=True, norm_ahead=(wn, rows, sumsq))
        gemm100.check_errors(DEV)
        assert torch.equal(out, plain)
        assert torch.equal(rows, (out * wn).to(torch.bfloat16))
        padded = torch.zeros(M, tiles * 256, dtype=torch.float64, device=DEV)
        padded[:, :N] = out.double() ** 2
        assert rel(sumsq, padded.view(M, 2 * tiles, 128).sum(-1)) < 1e-6
        want = prod * factor
        o32 = torch.full((M, N), float("nan"), device=DEV)
        run(o32, row_sumsq=sq, row_width=width, row_eps=eps)
        assert rel(o32, want) < 1e-5
        ob = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        run(ob, row_sumsq=sq, row_width=width, row_eps=eps)
        assert rel(ob, want) < 4e-3
        act = torch.full((M, N // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
        run(act, swiglu=True, row_sumsq=sq, row_width=width, row_eps=eps)
        gemm100.check_errors(DEV)
        g, u = want[:, 0::2], want[:, 1::2]
        assert rel(act, g / (1 + torch.exp(-g)) * u) < 6e-3


def test_gemm_tcgen05_refuses_row_work_it_cannot_do():
    from purhie_b200.csrc import gemm100
    from purhie_b200.csrc.ops import KernelError
    x, w = rnd(128, 64, dtype=torch.bfloat16), rnd(256, 64, dtype=torch.bfloat16)
    out = torch.zeros(128, 256, device=DEV)
    ahead = (torch.ones(256, device=DEV), torch.empty(128, 256, dtype=torch.bfloat16, device=DEV), torch.empty(128, 2, device=DEV))
    sq = torch.ones(128, 2, device=DEV)
    with pytest.raises(KernelError, match="together with the addition"):
        gemm100.gemm_pair(x, w, out, norm_ahead=ahead)                                    # not adding into the output
    with pytest.raises(KernelError, match="tiles of 256"):
        gemm100.gemm(x, w, out, swapped=False, block_n=128, accumulate=True, norm_ahead=ahead)
    with pytest.raises(KernelError, match="plain orientation only"):
        gemm100.gemm(x, w, out, swapped=True, block_n=128, norm_ahead=ahead)
    with pytest.raises(KernelError, match="without accumulate"):
        gemm100.gemm_pair(x, w, out, accumulate=True, row_sumsq=sq, row_width=64, row_eps=1e-6)
    with pytest.raises(KernelError, match="norm_ahead wants"):
        gemm100.gemm_pair(x, w, out, accumulate=True, norm_ahead=(ahead[0], ahead[1], torch.empty(128, 3, device=DEV)))


@pytest.mark.parametrize("T,E,splits,yd", [(1, 512, 1, torch.bfloat16), (8, 4096, 9, torch.bfloat16), (5, 1000, 3, torch.bfloat16),
                                           (33, 5120, 6, torch.bfloat16), (3, 96, 2, torch.float32)])
def test_a_norm_that_leaves_the_row_factor_to_its_consumer(T, E, splits, yd):
    """add_weight_sumsq: x += the addends, y = x * weight, and the row's sum of squares in chunks of 512 columns; the
    consumer's factor rsqrt(sum / E + eps) times y is the RMSNorm.  Then the two consumers: the few-token product
    (with and without the SwiGLU) whose epilogue applies the factor, and the per-head norm behind a qkv product."""
    from purhie_b200.csrc import gemm100, ops
    x = rnd(T, E, seed=31)
    add = rnd(splits, T, E, seed=32, scale=0.3)
    w = (torch.rand(E, generator=torch.Generator().manual_seed(33)) + 0.5).to(DEV)
    v = x.double() + add.double().sum(0)
    y = torch.full((T, E), float("nan"), dtype=yd, device=DEV)
    sumsq = ops.add_weight_sumsq(x, add, w, y, add_splits=splits)
    assert sumsq.shape == (T, -(-E // 512))
    assert rel(x, v) < 1e-6                                             # the stream holds the sum
    assert rel(y, v * w.double()) < (4e-3 if yd == torch.bfloat16 else 1e-6)
    chunks = torch.stack([(v[:, c:c + 512] ** 2).sum(-1) for c in range(0, E, 512)], -1)
    assert rel(sumsq, chunks) < 1e-5
    if yd != torch.bfloat16 or E % 8:
        return
    eps = 1e-5
    factor = torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)          # float64
    N = 264
    wt = rnd(N, E, dtype=torch.bfloat16, seed=34, scale=0.2)
    block_n = 16 if T <= 16 else 64
    full = y.double() @ wt.double().T * factor                           # what the product of the finished rows would give
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    gemm100.gemm(y, wt, out, swapped=True, block_n=block_n, row_sumsq=sumsq, row_width=E, row_eps=eps)
    gemm100.check_errors(DEV)
    assert rel(out, full) < 6e-3
    act = torch.full((T, N // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
    gemm100.gemm(y, wt, act, swapped=True, block_n=block_n, swiglu=True, row_sumsq=sumsq, row_width=E, row_eps=eps)
    gemm100.check_errors(DEV)
    g, u = full[:, 0::2], full[:, 1::2]
    assert rel(act, g / (1 + torch.exp(-g)) * u) < 8e-3


@pytest.mark.parametrize("HQ,HKV,D,splits", [(4, 2, 128, 3), (3, 1, 48, 2)])
def test_qk_norm_rope_applies_the_row_factor_before_the_bias(HQ, HKV, D, splits):
    """The per-head norm kernel with a row factor: its result equals that of the same kernel fed rows that were
    multiplied by the factor beforehand (bias added after the factor; the v heads scaled too)."""
    from purhie_b200.csrc import ops
    T, ps = 9, 8
    width = (HQ + 2 * HKV) * D
    qkv = rnd(splits, T, width, seed=41)
    sumsq = (torch.rand(T, 3, generator=torch.Generator().manual_seed(42)) * 40 + 1).to(DEV)
    row_width, eps = 77, 1e-4
    factor = torch.rsqrt(sumsq.double().sum(-1) / row_width + eps).float()
    bias = rnd(width, seed=43, scale=0.1)
    qn, kn = rnd(D, seed=44).abs() + 0.5, rnd(D, seed=45).abs() + 0.5
    pos = torch.arange(3, 3 + T, dtype=torch.int32, device=DEV)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    ang = torch.arange(64, dtype=torch.float64)[:, None] * inv[None]
    table = torch.cat([ang.cos(), ang.sin()], -1).float().to(DEV)
    slots = torch.arange(T, dtype=torch.int32, device=DEV)
    res = []
    for scaled_before in (False, True):
        src = qkv * factor[None, :, None] if scaled_before else qkv
        pool = torch.zeros(2, 1, 2, HKV, ps, D, device=DEV)
        q = torch.empty(T, HQ, D, device=DEV)
        ops.qk_norm_rope_kv_write(src.contiguous(), q, pos, num_heads=HQ, num_kv_heads=HKV, head_dim=D, eps=1e-6, q_norm=qn, k_norm=kn,
                                  bias=bias, cos_sin=table, n_rot=D, slot_mapping=slots, k_base=pool[0, 0, 0], v_base=pool[0, 0, 1],
                                  page_stride=pool.stride(0), page_size=ps, splits=splits,
                                  row_sumsq=None if scaled_before else sumsq, row_width=row_width, row_eps=eps)
        res.append((q, pool))
    assert rel(res[0][0], res[1][0]) < 2e-6 and rel(res[0][1], res[1][1]) < 2e-6


def test_gemm_tcgen05_refuses_what_tma_cannot_address():
    from purhie_b200.csrc import gemm100
    from purhie_b200.csrc.ops import KernelError
    x, w = rnd(4, 100, dtype=torch.bfloat16), rnd(32, 100, dtype=torch.bfloat16)        # K % 8 != 0
    assert not gemm100.supports(w)
    with pytest.raises(KernelError):
        gemm100.gemm(x, w, torch.empty(4, 32, device=DEV), swapped=True, block_n=16)


# ---- norms, activation, embedding -----------------------------------------------------------------------

@pytest.mark.parametrize("T,E", [(1, 96), (7, 1000), (33, 4096), (3, 12289)])
@pytest.mark.parametrize("yd", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(T, E, yd):
    from purhie_b200.csrc import ops
    x, add, w = rnd(T, E, seed=1, scale=2.0), rnd(3, T, E, seed=2), rnd(E, seed=3) * 0.1 + 1.0
    x0 = x.clone()
    y = torch.empty(T, E, dtype=yd, device=DEV)
    ops.add_rmsnorm(x, add, w, 1e-5, y, add_splits=3)
    v = x0.double() + add.double().sum(0)
    ref = v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-5) * w.double()
    assert rel(x, v) < 1e-6
    assert rel(y, ref) < (1e-5 if yd == torch.float32 else 5e-3)
    # gathered rows: nothing is written back
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    x1 = x0.clone()
    y2 = torch.empty(2, E, dtype=yd, device=DEV)
    ops.add_rmsnorm(x1, add[0].contiguous().to(torch.bfloat16), w, 1e-5, y2, rows=rows)
    v2 = (x0.double() + add[0].to(torch.bfloat16).double())[[T - 1, 0]]
    ref2 = v2 / torch.sqrt((v2 * v2).mean(-1, keepdim=True) + 1e-5) * w.double()
    assert torch.equal(x1, x0) and rel(y2, ref2) < (1e-5 if yd == torch.float32 else 5e-3)


def test_add_rmsnorm_row_result_is_independent_of_the_batch():
    from purhie_b200.csrc import ops
    x, w = rnd(40, 1000, seed=4), rnd(1000, seed=5)
    y = torch.empty(40, 1000, device=DEV)
    ops.add_rmsnorm(x.clone(), None, w, 1e-6, y)
    y1 = torch.empty(1, 1000, device=DEV)
    ops.add_rmsnorm(x[23:24].clone(), None, w, 1e-6, y1)
    assert torch.equal(y1[0], y[23])


@pytest.mark.parametrize("T,FF,splits", [(1, 224, 1), (9, 1000, 1), (5, 352, 3)])
def test_swiglu(T, FF, splits):
    from purhie_b200.csrc import ops
    for dt, tol in ((torch.float32, 1e-6), (torch.bfloat16, 6e-3)):
        gu = rnd(splits, T, 2 * FF, dtype=torch.float32 if splits > 1 else dt, seed=6, scale=2.0)
        out = torch.empty(T, FF, dtype=dt, device=DEV)
        ops.swiglu(gu, out, splits=splits)
        s = gu.double().sum(0)
        g, u = s[:, 0::2], s[:, 1::2]                   # (gate, up) pairs side by side
        assert rel(out, g / (1 + torch.exp(-g)) * u) < tol


def test_embed_gather_and_cast():
    from purhie_b200.csrc import ops
    table = rnd(1000, 96, dtype=torch.bfloat16, seed=7)
    ids = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 96, device=DEV)
    ops.embed_gather(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())
    back = torch.empty(5, 96, dtype=torch.bfloat16, device=DEV)
    ops.cast(out, back)
    assert torch.equal(back, table[ids.long()])


# ---- sampling ------------------------------------------------------------------------------------------

def test_argmax_lowest_id_wins_ties():
    from purhie_b200.csrc import ops
    l = rnd(6, 151937, seed=8)
    l[0, 777] = l[0, 150000] = 50.0
    l[1, 151936] = 60.0
    l[2, 0] = 70.0
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.argmax(l, out)
    ref = [int(torch.nonzero(r == r.max())[0]) for r in l]
    assert out.tolist() == ref and ref[:3] == [777, 151936, 0]
    # rows that start on a 16-byte boundary are read four values at a time: ties inside one vector, across vectors
    # that different threads read, in the last place, a row of equal values and a row of -inf
    l = rnd(8, 151936, seed=9)
    l[0, 4097] = l[0, 4098] = l[0, 90001] = 50.0
    l[1, 151935] = 60.0
    l[2, 3] = l[2, 4 * 1024 * 5 + 3] = 70.0
    l[3, :] = 1.25
    l[4, :] = float("-inf")
    l[5, 151932] = l[5, 151933] = 80.0
    out = torch.empty(8, dtype=torch.int32, device=DEV)
    ops.argmax(l, out)
    ref = [int(torch.nonzero(r == r.max())[0]) for r in l]
    assert out.tolist() == ref and ref[:6] == [4097, 151935, 3, 0, 0, 151932]
    # several CTAs per row (the form the engine runs): the same choices, call after call on the same scratch, for
    # one row, for rows that do not start on a 16-byte boundary and for more rows than fill the device
    for rows, V in ((8, 151936), (1, 151936), (6, 151937), (300, 5000), (3, 100)):
        m = rnd(rows, V, seed=10 + rows)
        if V > 4200:
            m[0, 4095] = m[0, 4096] = m[0, V - 1] = 90.0                   # a tie across the boundary of two parts
        if rows == 8:
            m = l
        scratch = torch.zeros(rows * (4 + 64 * 8), dtype=torch.uint8, device=DEV)
        want = [int(torch.nonzero(r == r.max())[0]) for r in m]
        for _ in range(3):
            got = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
            ops.argmax(m, got, scratch=scratch)
            assert got.tolist() == want, (rows, V)
        assert int(scratch[:4 * rows].view(torch.int32).abs().sum()) == 0     # the counters are back at zero
    # one scratch for calls of changing numbers of rows, as a server's steps have them
    scratch = torch.zeros(64 * (4 + 64 * 8), dtype=torch.uint8, device=DEV)
    for rows in (24, 3, 64, 10, 24, 1, 17):
        m = rnd(rows, 151936, seed=40 + rows)
        got = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
        ops.argmax(m, got, scratch=scratch)
        assert got.tolist() == m.argmax(-1).tolist(), rows


def test_sample_temperature_follows_the_distribution_and_the_host_chain():
    from purhie_b200.csrc import ops
    from purhie_b200.sampling import Sampler, SamplerParams
    from plain import qwen3_plain as P
    V = 1000
    row = rnd(V, seed=9, scale=3.0)
    n = 4096
    logits = row[None, :].expand(n, V).contiguous()
    g = torch.Generator().manual_seed(0)
    u = torch.rand(n, generator=g, dtype=torch.float64)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample_temperature(logits, torch.full((n,), 0.7, device=DEV), u.to(DEV), out)
    p = P.temperature_probabilities(row.cpu().numpy(), 0.7)
    counts = torch.bincount(out.long().cpu(), minlength=V).double() / n
    assert (counts - torch.from_numpy(p)).abs().max() < 0.02
    # the same uniform numbers give the tokens of the host chain
    s = Sampler(SamplerParams.pure_temperature(0.7, seed=5))
    s2 = Sampler(SamplerParams.pure_temperature(0.7, seed=5))
    us = torch.tensor([s2.uniform() for _ in range(64)], dtype=torch.float64)
    host = [s.sample(row.cpu().numpy()) for _ in range(64)]
    dev = torch.empty(64, dtype=torch.int32, device=DEV)
    ops.sample_temperature(logits[:64].contiguous(), torch.full((64,), 0.7, device=DEV), us.to(DEV), dev)
    assert dev.tolist() == host


# ---- attention over pages ----------------------------------------------------------------------------------

def paged_case(segs, HQ, HKV, D, page_size, dtype, seed=0, poison=True):
    """segs: [(ctx_len, q_len)].  Returns everything the attention kernels take plus the dense K, V per segment.
    Pages are handed out in a shuffled order and every slot that holds no key is NaN."""
    import random
    rng = random.Random(seed)
    n_pages = sum(-(-c // page_size) for c, _ in segs) + 3
    order = list(range(n_pages))
    rng.shuffle(order)
    pool = torch.full((n_pages, 1, 2, HKV, page_size, D), float("nan") if poison else 0.0, dtype=dtype, device=DEV)
    width = max(-(-c // page_size) for c, _ in segs)
    table = torch.full((len(segs), width), -1, dtype=torch.int32)
    dense, rows_seg, positions, seg_start = [], [], [], [0]
    for s, (ctx, ql) in enumerate(segs):
        k, v = rnd(ctx, HKV, D, dtype=dtype, seed=seed * 100 + 2 * s), rnd(ctx, HKV, D, dtype=dtype, seed=seed * 100 + 2 * s + 1)
        dense.append((k, v))
        for b in range(-(-ctx // page_size)):
            page = order.pop()
            table[s, b] = page
            n = min(page_size, ctx - b * page_size)
            pool[page, 0, 0, :, :n] = k[b * page_size:b * page_size + n].transpose(0, 1)
            pool[page, 0, 1, :, :n] = v[b * page_size:b * page_size + n].transpose(0, 1)
        rows_seg += [s] * ql
        positions += list(range(ctx - ql, ctx))
        seg_start.append(seg_start[-1] + ql)
    T = len(positions)
    q = rnd(T, HQ, D, dtype=dtype, seed=seed * 100 + 99)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return dict(q=q, pool=pool, k_base=pool[0, 0, 0], v_base=pool[0, 0, 1], page_stride=pool.stride(0), table=table.to(DEV),
                row_seg=i32(rows_seg), positions=i32(positions), seg_start=i32(seg_start),
                seg_ctx=i32([c for c, _ in segs]), dense=dense, T=T, segs=segs)


def dense_attention(case, HQ, HKV, D, window, scale):
    out = torch.zeros(case["T"], HQ, D, dtype=torch.float64)
    row = 0
    for (ctx, ql), (k, v) in zip(case["segs"], case["dense"]):
        k, v = k.double().cpu(), v.double().cpu()
        for i in range(ql):
            z = ctx - ql + i
            lo = max(0, z - window + 1) if window else 0
            for h in range(HQ):
                g = h // (HQ // HKV)
                s = (k[lo:z + 1, g] @ case["q"][row, h].double().cpu()) * scale
                p = torch.softmax(s, 0)
                out[row, h] = p @ v[lo:z + 1, g]
            row += 1
    return out.view(case["T"], HQ * D)


def run_generic(case, HQ, HKV, D, page_size, window, scale, out_dtype):
    from purhie_b200.csrc import ops
    out = torch.full((case["T"], HQ * D), float("nan"), dtype=out_dtype, device=DEV)
    ops.attention_generic(case["q"], case["k_base"], case["v_base"], case["page_stride"], page_size, case["table"],
                          case["row_seg"], case["positions"], out, num_heads=HQ, num_kv_heads=HKV, head_dim=D,
                          window=window, scale=scale)
    return out


def run_flash(case, HQ, HKV, D, page_size, window, scale, splits=None, bulk=True, max_ctas=0, tc5=True, tile_splits=1):
    from purhie_b200.csrc import flash
    from purhie_b200.csrc.ops import Workspace
    out = torch.full((case["T"], HQ * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    tile_seg, tile_first, dec_rows, start = [], [], [], 0
    for s, (ctx, ql) in enumerate(case["segs"]):
        if ql == 1:
            dec_rows.append(start)
        else:
            for f in range(0, ql, 64):
                tile_seg.append(s); tile_first.append(f)
        start += ql
    i32 = lambda x: torch.tensor(x or [0], dtype=torch.int32, device=DEV)
    if tile_seg and tc5 and flash.tc5_supports(D, page_size):
        big = [(s, f) for s, (ctx, ql) in enumerate(case["segs"]) if ql > 1 for f in range(0, ql, 128)]
        flash.prefill_tc5(case["q"], case["T"], case["k_base"], case["v_base"], case["page_stride"], page_size,
                          case["pool"].shape[0], case["table"], case["seg_start"], case["seg_ctx"], i32([b[0] for b in big]),
                          i32([b[1] for b in big]), len(big), out, num_heads=HQ, num_kv_heads=HKV, head_dim=D,
                          window=window, scale=scale, splits=tile_splits, workspace=Workspace(DEV))
        flash.check_errors(DEV)
    elif tile_seg:
        flash.prefill(case["q"], case["k_base"], case["v_base"], case["page_stride"], page_size, case["table"],
                      case["seg_start"], case["seg_ctx"], i32(tile_seg), i32(tile_first), len(tile_seg), out,
                      num_heads=HQ, num_kv_heads=HKV, head_dim=D, window=window, scale=scale)
    if dec_rows:
        max_ctx = max(c for c, ql in case["segs"] if ql == 1)
        head = (case["q"], case["k_base"], case["v_base"], case["page_stride"], page_size)
        tail = (case["table"], None if len(dec_rows) == case["T"] else i32(dec_rows), len(dec_rows), case["row_seg"],
                case["positions"], out, Workspace(DEV))
        args = head + tail
        kw = dict(num_heads=HQ, num_kv_heads=HKV, head_dim=D, window=window, scale=scale)
        if bulk and flash.bulk_supports(page_size):
            sp = splits or flash.bulk_splits(len(dec_rows), HKV, max_ctx, 148, window)
            flash.decode_bulk(*head, case["pool"].shape[0], *tail, splits=sp, max_ctas=max_ctas, **kw)
            flash.check_errors(DEV)
        else:
            sp = splits or flash.decode_splits(len(dec_rows), HKV, max_ctx, 148, window)
            flash.decode(*args, splits=sp, **kw)
    return out


@pytest.mark.parametrize("HQ,HKV,D,page_size,window", [
    (4, 2, 16, 16, None), (8, 2, 32, 8, 24), (6, 3, 48, 5, 7), (3, 1, 80, 16, None), (2, 2, 256, 32, 100)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_generic(HQ, HKV, D, page_size, window, dtype):
    segs = [(1, 1), (33, 33), (70, 1), (129, 17), (40, 2)]
    case = paged_case(segs, HQ, HKV, D, page_size, dtype, seed=1)
    scale = 1.0 / math.sqrt(D)
    out = run_generic(case, HQ, HKV, D, page_size, window, scale, dtype)
    ref = dense_attention(case, HQ, HKV, D, window, scale)
    assert rel(out.cpu(), ref) < (2e-6 if dtype == torch.float32 else 8e-3)


def test_attention_generic_float32_over_2500_keys():
    """The float32 path's attention at a context of the length the real-size tests decode at, against float64."""
    HQ, HKV, D, ps = 8, 2, 128, 16
    case = paged_case([(2500, 1), (2500, 3), (2437, 1)], HQ, HKV, D, ps, torch.float32, seed=5)
    scale = 1.0 / math.sqrt(D)
    for window in (None, 2048):
        out = run_generic(case, HQ, HKV, D, ps, window, scale, torch.float32)
        assert rel(out.cpu(), dense_attention(case, HQ, HKV, D, window, scale)) < 5e-6


@pytest.mark.parametrize("HQ,HKV,D,page_size,window", [
    (8, 2, 128, 16, None), (4, 4, 64, 16, None), (6, 2, 64, 8, 40), (16, 1, 128, 64, 200), (32, 8, 128, 16, None),
    (2, 1, 128, 3, 65), (4, 2, 128, 8, 150), (3, 3, 128, 16, 77), (8, 2, 128, 32, None), (4, 1, 128, 64, None)])
def test_attention_flash_prefill_and_decode(HQ, HKV, D, page_size, window):
    # portions that start mid-page, cross many blocks, end inside a tile; decode rows short and long
    segs = [(1, 1), (64, 64), (200, 130), (300, 1), (65, 2), (700, 1), (513, 257), (63, 1), (128, 1)]
    case = paged_case(segs, HQ, HKV, D, page_size, torch.bfloat16, seed=2)
    scale = 1.0 / math.sqrt(D)
    ref = dense_attention(case, HQ, HKV, D, window, scale)
    out = run_flash(case, HQ, HKV, D, page_size, window, scale)
    assert not torch.isnan(out.float()).any()
    assert rel(out.cpu(), ref) < 1e-2
    plain = run_generic(case, HQ, HKV, D, page_size, window, scale, torch.bfloat16)
    assert rel(out.cpu(), plain.cpu()) < 1e-2
    legacy = run_flash(case, HQ, HKV, D, page_size, window, scale, tc5=False)      # the mma.sync prefill kernel
    assert rel(legacy.cpu(), ref) < 1e-2
    for sp in (1, 3, 32):                                  # any number of splits, more than there are blocks too
        for bulk in (True, False):                         # the persistent bulk-copy kernel and the cp.async kernel
            o2 = run_flash(case, HQ, HKV, D, page_size, window, scale, splits=sp, bulk=bulk)
            assert not torch.isnan(o2.float()).any()
            assert rel(o2.cpu(), ref) < 1e-2
    # several CTAs on the keys of one prompt tile, more than a short tile has blocks too
    from purhie_b200.csrc import flash
    if flash.tc5_supports(D, page_size):
        for ts in (2, 5, 16):
            o4 = run_flash(case, HQ, HKV, D, page_size, window, scale, tile_splits=ts)
            assert not torch.isnan(o4.float()).any()
            assert rel(o4.cpu(), ref) < 1e-2, ts
    # few CTAs: each walks many items, the stage ring and the query buffers wrap many times
    for sp, ctas in ((2, 3), (2, 1), (3, 1), (1, 2)):
        o3 = run_flash(case, HQ, HKV, D, page_size, window, scale, splits=sp, max_ctas=ctas)
        assert rel(o3.cpu(), ref) < 1e-2, (sp, ctas)


@pytest.mark.parametrize("kernel", ["generic32", "generic16", "flash", "flash_cp_async"])
def test_attention_finds_one_far_key_and_respects_the_window_edge(kernel):
    """Random keys would hide a lost key among hundreds: make one key match the query so that it carries all the
    weight, then put it first in the context, on a page's edge, just inside and just outside the window."""
    HQ, HKV, D, ps = 4, 2, 64, 16
    scale = 1.0 / math.sqrt(D)
    dtype = torch.float32 if kernel == "generic32" else torch.bfloat16
    ctx = 600
    for window, key_pos, visible in [(None, 0, True), (None, 15, True), (None, 16, True), (None, 599, True),
                                     (100, 500, True), (100, 499, False), (100, 599, True), (584, 16, True), (584, 15, False)]:
        for ql in (1, 90):                       # the last row is a decode row or the end of a portion
            case = paged_case([(ctx, ql)], HQ, HKV, D, ps, dtype, seed=3)
            k, v = case["dense"][0]
            qrow = case["T"] - 1
            spike = torch.zeros(D, device=DEV); spike[5] = 60.0
            case["q"][qrow, :] = spike.to(dtype)
            page, off = int(case["table"][0, key_pos // ps]), key_pos % ps
            case["pool"][page, 0, 0, :, off] = spike.to(dtype)       # K[key_pos] for both kv heads
            k[key_pos] = spike.to(dtype)
            marker = torch.full((D,), 7.0, device=DEV)
            case["pool"][page, 0, 1, :, off] = marker.to(dtype)      # V[key_pos]
            v[key_pos] = marker.to(dtype)
            if kernel.startswith("flash"):
                out = run_flash(case, HQ, HKV, D, ps, window, scale, bulk=kernel == "flash")
            else:
                out = run_generic(case, HQ, HKV, D, ps, window, scale, dtype)
            got = out[qrow].float().view(HQ, D)
            if visible:
                assert (got - 7.0).abs().max() < 0.05, (kernel, window, key_pos, ql)
            else:
                assert got.abs().max() < 4.0, (kernel, window, key_pos, ql)
            ref = dense_attention(case, HQ, HKV, D, window, scale)
            assert rel(out.cpu(), ref) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("kernel,kw", [
    ("generic", {}), ("bulk", {"splits": 1}), ("bulk", {"splits": 3}), ("bulk", {"splits": 8}), ("cp_async", {"splits": 1}),
    ("cp_async", {"splits": 4}), ("tc5", {"tile_splits": 1}), ("tc5", {"tile_splits": 3}), ("mma", {})])
def test_attention_window_edge_between_two_matching_keys(kernel, kw):
    """Two keys match the query equally: the one at z - window (just outside the window, value 3) and the one at
    z - window + 1 (just inside, value 7).  The right answer is 7; a kernel that lets the outer key in answers 5, one
    that drops the inner key answers noise.  The edge is put inside a page, on a page's first slot and on a block's
    first key, for a decode row, for both rows of a 2-token portion and for the first and last row of longer
    portions (head size 128: the TMA decode kernel, the cp.async one, the tcgen05 and the mma.sync prefill kernels)."""
    HQ, HKV, D, ps = 4, 2, 128, 16
    scale = 1.0 / math.sqrt(D)
    dtype = torch.bfloat16
    ctx = 600
    decode = kernel in ("bulk", "cp_async")
    for window in (100, 88, 104, 64):            # 599 - 88 + 1 = 512 (a block's first key), 599 - 104 + 1 = 496 (a page's)
        for ql in ((1,) if decode else (1, 2, 90, 200) if kernel == "generic" else (2, 90, 200)):
            for which in sorted({0, ql - 1}):     # the portion's first and last row
                case = paged_case([(ctx, ql)], HQ, HKV, D, ps, dtype, seed=4)
                k, v = case["dense"][0]
                z = ctx - ql + which
                spike = torch.zeros(D, device=DEV); spike[9] = 60.0
                case["q"][which, :] = spike.to(dtype)
                for key_pos, value in ((z - window, 3.0), (z - window + 1, 7.0)):
                    page, off = int(case["table"][0, key_pos // ps]), key_pos % ps
                    case["pool"][page, 0, 0, :, off] = spike.to(dtype)
                    case["pool"][page, 0, 1, :, off] = value
                    k[key_pos] = spike.to(dtype)
                    v[key_pos] = value
                if kernel == "generic":
                    out = run_generic(case, HQ, HKV, D, ps, window, scale, dtype)
                else:
                    out = run_flash(case, HQ, HKV, D, ps, window, scale, bulk=kernel != "cp_async", tc5=kernel != "mma", **kw)
                got = out[which].float()
                assert (got - 7.0).abs().max() < 0.05, (kernel, kw, window, ql, which, float(got.mean()))
                ref = dense_attention(case, HQ, HKV, D, window, scale)
                assert rel(out.cpu(), ref) < 1e-2


# ---- per-head norm, rotation and cache write ---------------------------------------------------------------

@pytest.mark.parametrize("HQ,HKV,D,n_rot,interleaved,splits,dtype", [
    (4, 2, 16, 16, False, 1, torch.float32), (8, 2, 32, 32, False, 3, torch.float32), (3, 1, 48, 24, False, 1, torch.float32),
    (6, 3, 64, 64, True, 1, torch.bfloat16), (32, 8, 128, 128, False, 1, torch.bfloat16),
    (32, 8, 128, 128, False, 5, torch.bfloat16), (4, 4, 128, 64, False, 1, torch.bfloat16), (2, 1, 256, 256, False, 2, torch.float32)])
def test_qk_norm_rope_kv_write(HQ, HKV, D, n_rot, interleaved, splits, dtype):
    from purhie_b200.csrc import ops
    T, ps, n_pages, max_pos, eps = 9, 8, 6, 64, 1e-5
    width = (HQ + 2 * HKV) * D
    in_dtype = torch.float32 if splits > 1 else dtype
    qkv = rnd(splits, T, width, dtype=in_dtype, seed=1)
    bias, qw, kw = rnd(width, seed=2) * 0.1, rnd(D, seed=3) * 0.2 + 1.0, rnd(D, seed=4) * 0.2 + 1.0
    pos = torch.tensor([0, 1, 7, 8, 9, 31, 40, 62, 63], dtype=torch.int32, device=DEV)
    slots = torch.tensor([3, 47, 0, 8, 9, 17, 40, -1, 22], dtype=torch.int32, device=DEV)
    half = n_rot // 2
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * (1e4 ** (-2.0 * torch.arange(half, dtype=torch.float64) / n_rot))[None, :]
    table = torch.cat([ang.cos(), ang.sin()], 1).float().to(DEV)
    pool = torch.full((n_pages, 1, 2, HKV, ps, D), float("nan"), dtype=dtype, device=DEV)
    q = torch.full((T, HQ, D), float("nan"), dtype=dtype, device=DEV)
    ops.qk_norm_rope_kv_write(qkv, q, pos, num_heads=HQ, num_kv_heads=HKV, head_dim=D, eps=eps, q_norm=qw, k_norm=kw,
                              bias=bias, cos_sin=table, n_rot=n_rot, slot_mapping=slots, k_base=pool[0, 0, 0],
                              v_base=pool[0, 0, 1], page_stride=pool.stride(0), page_size=ps, splits=splits,
                              interleaved=interleaved)
    x = (qkv.double().sum(0) + bias.double()).cpu().view(T, HQ + 2 * HKV, D)
    def norm_rot(v, w):
        v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * w.double().cpu()
        c, s = ang[pos.long().cpu()].cos()[:, None, :], ang[pos.long().cpu()].sin()[:, None, :]
        out = v.clone()
        if interleaved:
            a, b = v[..., 0:n_rot:2], v[..., 1:n_rot:2]
            out[..., 0:n_rot:2], out[..., 1:n_rot:2] = a * c - b * s, a * s + b * c
        else:
            a, b = v[..., :half], v[..., half:n_rot]
            out[..., :half], out[..., half:n_rot] = a * c - b * s, a * s + b * c
        return out
    tol = 1e-5 if dtype == torch.float32 else 8e-3
    assert rel(q.cpu(), norm_rot(x[:, :HQ], qw)) < tol
    k_ref, v_ref = norm_rot(x[:, HQ:HQ + HKV], kw), x[:, HQ + HKV:]
    written = torch.zeros(n_pages * ps, dtype=torch.bool)
    for t in range(T):
        sl = int(slots[t])
        if sl < 0:
            continue
        written[sl] = True
        assert rel(pool[sl // ps, 0, 0, :, sl % ps].cpu(), k_ref[t]) < tol
        assert rel(pool[sl // ps, 0, 1, :, sl % ps].cpu(), v_ref[t]) < tol
    # nothing but the mapped slots was touched
    untouched = pool.float().cpu().permute(0, 4, 1, 2, 3, 5).reshape(n_pages * ps, -1)[~written]
    assert torch.isnan(untouched).all()


@pytest.mark.parametrize("HQ,HKV,splits,dtype,with_bias", [(32, 8, 1, torch.bfloat16, False), (5, 3, 2, torch.bfloat16, True),
                                                          (32, 8, 1, torch.float32, False)])
def test_qk_norm_rope_of_many_tokens_gives_the_bits_of_few(HQ, HKV, splits, dtype, with_bias):
    """Many tokens run a kernel with eight dimensions per lane; a token's result must not depend on how many
    tokens share its launch, so it is compared bit by bit with launches of a few tokens (the four-per-lane kernel)."""
    from purhie_b200.csrc import ops
    D, ps, eps = 128, 16, 1e-6
    n_heads = HQ + 2 * HKV
    T = -(-16384 // n_heads) + 37                 # enough for the wide kernel, and not a round number
    n_pages, max_pos = -(-T // ps) + 1, T + 5
    in_dtype = torch.float32 if splits > 1 else dtype
    qkv = rnd(splits, T, n_heads * D, dtype=in_dtype, seed=21)
    bias = rnd(n_heads * D, seed=22) * 0.1 if with_bias else None
    qw, kw = rnd(D, seed=23) * 0.2 + 1.0, rnd(D, seed=24) * 0.2 + 1.0
    g = torch.Generator().manual_seed(5)
    pos = torch.randint(0, max_pos, (T,), generator=g).int().to(DEV)
    slots = torch.randperm(n_pages * ps, generator=g)[:T].int().to(DEV)
    slots[7] = -1
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * (1e6 ** (-2.0 * torch.arange(D // 2, dtype=torch.float64) / D))[None, :]
    table = torch.cat([ang.cos(), ang.sin()], 1).float().to(DEV)

    def run(rows):
        pool = torch.full((n_pages, 1, 2, HKV, ps, D), float("nan"), dtype=dtype, device=DEV)
        q = torch.full((len(rows), HQ, D), float("nan"), dtype=dtype, device=DEV)
        ops.qk_norm_rope_kv_write(qkv[:, rows].contiguous(), q, pos[rows].contiguous(), num_heads=HQ, num_kv_heads=HKV,
                                  head_dim=D, eps=eps, q_norm=qw, k_norm=kw, bias=bias, cos_sin=table, n_rot=D,
                                  slot_mapping=slots[rows].contiguous(), k_base=pool[0, 0, 0], v_base=pool[0, 0, 1],
                                  page_stride=pool.stride(0), page_size=ps, splits=splits, interleaved=False)
        return q, pool

    q_all, pool_all = run(torch.arange(T, device=DEV))
    assert not torch.isnan(q_all.float()).any()
    few = torch.tensor([0, 7, 100, T - 1], device=DEV)
    q_few, pool_few = run(few)
    assert torch.equal(q_all[few], q_few)
    for t in few.tolist():
        sl = int(slots[t])
        if sl >= 0:
            assert torch.equal(pool_all[sl // ps, 0, :, :, sl % ps], pool_few[sl // ps, 0, :, :, sl % ps])
    written = torch.zeros(n_pages * ps, dtype=torch.bool)
    written[slots[slots >= 0].long().cpu()] = True
    untouched = pool_all.float().cpu().permute(0, 4, 1, 2, 3, 5).reshape(n_pages * ps, -1)[~written]
    assert torch.isnan(untouched).all()


@pytest.mark.parametrize("V", [1000, 151936])
def test_sample_chain_equals_the_host_chain(V):
    """top-k -> top-p -> min-p -> temperature -> draw on the device picks the token the host chain picks, for the
    same uniform number: rows with ties at the k-th place, flat rows, peaked rows, every filter on and off."""
    import numpy as np
    from purhie_b200.csrc import ops
    from purhie_b200.sampling import Sampler, SamplerParams
    g = torch.Generator().manual_seed(V)
    cases = []
    for top_k in (2, 40, 256):
        for top_p in (0.5, 0.95, 1.0):
            for min_p in (0.0, 0.05):
                for temperature in (0.7, 1.3):
                    cases.append((top_k, top_p, min_p, temperature))
    R = len(cases)
    logits = torch.randn(R, V, generator=g) * 3.0
    logits[1] = torch.round(logits[1])                        # many equal logits: ties at the k-th place and inside
    logits[2] = 0.25                                          # all equal
    logits[3, 17] = 40.0                                      # one token has all the mass
    logits[4] = -logits[4].abs()
    logits[4, ::7] = -0.0
    logits[5] = torch.round(logits[5] * 2) / 2
    dev = logits.to(DEV)
    for seed in (0, 1, 2):
        host, device = [], []
        rec = np.zeros(R, dtype=ops.CHAIN_ROW)
        for r, (top_k, top_p, min_p, temperature) in enumerate(cases):
            prm = SamplerParams(temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p, seed=seed * 1000 + r)
            a, b = Sampler(prm), Sampler(prm)
            assert b.device_mode() == "chain"
            host.append(a.sample(logits[r].numpy()))
            rec[r:r + 1] = np.frombuffer(b.chain_record(), dtype=ops.CHAIN_ROW)
        out = torch.empty(R, dtype=torch.int32, device=DEV)
        ops.sample_chain(dev, torch.from_numpy(rec.view(np.uint8).reshape(R, 24)).to(DEV), out)
        device = out.cpu().tolist()
        assert device == host, [(i, cases[i], host[i], device[i]) for i in range(R) if host[i] != device[i]]


@pytest.mark.parametrize("ctx,splits", [(130, 4), (130, 1), (200, 3), (64, 2)])
def test_decode_attention_sees_the_key_written_by_the_kernel_in_front(ctx, splits):
    """The decode kernel starts under the kernel that writes the token's own key and value and requests older
    blocks before it waits for that kernel; the block with the token's own position must wait, also when it is not
    in the last split (130 tokens = 3 blocks in 4 splits: the last split is empty).  As in a model's step the three
    kernels (a product, the writer, the attention) are replayed as a graph, with no host between them; the writer
    works through 2,048 rows first to last while the attention takes them last first, and the slot is NaN until it
    is written, so a request issued too early finds NaN (seen in a handful of rows per run with the check on the
    split instead of on the block)."""
    from purhie_b200.csrc import flash, ops
    from purhie_b200.csrc.ops import Workspace
    HQ, HKV, D, ps, R = 32, 8, 128, 16, 2048
    scale = 1.0 / math.sqrt(D)
    pages_per = -(-ctx // ps)
    n_pages = R * pages_per + 1
    g = torch.Generator(device=DEV).manual_seed(ctx)
    pool = torch.randn(n_pages, 1, 2, HKV, ps, D, device=DEV, generator=g).bfloat16()
    table = (torch.randperm(n_pages - 1, device=DEV, generator=g).int() + 1).view(R, pages_per).contiguous()
    z = ctx - 1
    own_page = table[:, z // ps].long()
    slots = (own_page * ps + z % ps).int()
    qkv = torch.randn(2, R, (HQ + 2 * HKV) * D, device=DEV, generator=g)         # two partial sums, as after a split product
    q = torch.empty(R, HQ, D, dtype=torch.bfloat16, device=DEV)
    out = torch.full((R, HQ * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    pos = torch.full((R,), z, dtype=torch.int32, device=DEV)
    row_seg = torch.arange(R, dtype=torch.int32, device=DEV)
    last_first = torch.arange(R - 1, -1, -1, dtype=torch.int32, device=DEV)
    ws = Workspace(DEV)
    from purhie_b200.csrc import gemm100
    gx, gw = rnd(8, 8192, dtype=torch.bfloat16, seed=1), rnd(16384, 8192, dtype=torch.bfloat16, seed=2)
    gout = torch.empty(8, 16384, device=DEV)

    def chain():
        gemm100.gemm(gx, gw, gout, swapped=True, block_n=16, max_ctas=74)
        ops.qk_norm_rope_kv_write(qkv, q, pos, num_heads=HQ, num_kv_heads=HKV, head_dim=D, eps=1e-6, q_norm=None, k_norm=None,
                                  bias=None, cos_sin=None, n_rot=0, slot_mapping=slots, k_base=pool[0, 0, 0],
                                  v_base=pool[0, 0, 1], page_stride=pool.stride(0), page_size=ps, splits=2, interleaved=False)
        flash.decode_bulk(q, pool[0, 0, 0], pool[0, 0, 1], pool.stride(0), ps, n_pages, table, last_first, R, row_seg, pos, out, ws,
                          num_heads=HQ, num_kv_heads=HKV, head_dim=D, window=None, scale=scale, splits=splits)

    chain()                                                  # first use of every kernel, outside the capture
    flash.check_errors(DEV)
    ws.frozen = True
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph), ops.on_current_stream():
        chain()
    for _ in range(3):
        pool.view(-1, 2, HKV, ps, D)[own_page, :, :, z % ps] = float("nan")        # not written yet
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        graph.replay()                                       # as a step does: no host between the launches
        flash.check_errors(DEV)
        assert not torch.isnan(out.float()).any()
    # and it is the right answer for a row
    r = R - 3
    gemm100.check_errors(DEV)
    idx = table[r].long()
    K = pool[idx, 0, 0].permute(0, 2, 1, 3).reshape(-1, HKV, D)[:ctx].double()
    V = pool[idx, 0, 1].permute(0, 2, 1, 3).reshape(-1, HKV, D)[:ctx].double()
    ref = []
    for h in range(HQ):
        kv = h // (HQ // HKV)
        p = torch.softmax((K[:, kv] @ q[r, h].double()) * scale, 0)
        ref.append(p @ V[:, kv])
    assert rel(out[r].double(), torch.cat(ref)) < 5e-3
