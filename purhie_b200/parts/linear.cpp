#include "linear.h"

namespace qe {

namespace {
constexpr int kBlockK = 64;
inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Few tokens: the product is weight streaming.  The work items (128-feature tile, split of K) should fill whole
// waves of the SMs, so the number of splits is the one with the best wave efficiency (items / (waves * SMs)),
// the fewest splits winning among near-equals, each split keeping at least four blocks of K.
GemmPlan plan_few(int M, int N, int K, int sms, bool allow_split) {
    GemmPlan p;
    p.swapped = true;
    p.block_n = 16;
    while (p.block_n < M) p.block_n *= 2;
    p.splits = 1;
    if (allow_split) {
        const int kblocks = ceil_div(K, kBlockK), a_tiles = ceil_div(N, 128);
        const int slots = sms * (p.block_n <= 64 ? 2 : 1);        // the kernel runs two CTAs per SM for small tiles
        double best = -1.0;
        const int most = std::min(16, std::max(1, kblocks / 4));
        for (int s = 1; s <= most; s++) {
            const int items = a_tiles * s;
            const double eff = (double)items / ((double)ceil_div(items, slots) * slots);
            if (eff > best + 0.03) { best = eff; p.splits = s; }
        }
    }
    return p;
}

// Many tokens, plain orientation: the one-CTA kernel (tiles of 128 tokens x 256 features) or the pair kernel
// (256 x 256 on two SMs), and into how many parts K is cut.  Estimated cost in units of one block of K on one
// SM's tile: rounds of the CTAs (or pairs) times the item's blocks (the pair spends 0.87 of a block's time per
// block: half the shared-memory traffic per flop) plus six for an item's start and epilogue, plus the float32
// partial results' way to memory and back when K is split.  A fused epilogue needs the whole sum in one place.
void plan_many(int M, int N, int K, int sms, bool allow_split, bool fused_epilogue, GemmPlan& p) {
    const int kblocks = ceil_div(K, kBlockK);
    static const int kAll[] = {1, 2, 3, 4, 6, 8};
    const int n_options = (allow_split && !fused_epilogue) ? 6 : 1;
    double best = -1.0;
    p.pair = false;
    p.splits = 1;
    for (int pair = 0; pair < 2; pair++) {
        if (pair && (M <= 128 || N <= 128)) continue;
        const int tiles = (pair ? ceil_div(M, 256) : ceil_div(M, 128)) * ceil_div(N, 256);
        const int slots = pair ? sms / 2 : sms;
        for (int o = 0; o < n_options; o++) {
            const int s = kAll[o];
            if (s > 1 && kblocks / s < 8) continue;
            const int rounds = ceil_div((long long)tiles * s, slots);
            double cost = rounds * ((pair ? 0.87 : 1.0) * kblocks / s + 6.0);
            if (s > 1) cost += 2.0 * s * (double)M * N * 4 / 4.0e12 / 0.33e-6;
            if (best < 0 || cost < best - 1e-9) { best = cost; p.pair = pair != 0; p.splits = s; }
        }
    }
}
}  // namespace

GemmPlan plan_gemm(int M, int N, int K, int sms, bool allow_split, bool fused_epilogue) {
    if (M < 128) return plan_few(M, N, K, sms, allow_split);
    GemmPlan p;
    p.swapped = false;
    p.block_n = N > 128 ? 256 : N > 64 ? 128 : 64;
    p.splits = 1;
    if (p.block_n == 256) plan_many(M, N, K, sms, allow_split, fused_epilogue, p);
    return p;
}

Linear::Linear(Tensor weight, std::string label, const std::string& gemm) : weight_(std::move(weight)), label_(std::move(label)) {
    if (weight_.shape.size() != 2)
        throw ConfigError(label_ + ": a linear weight must be a matrix, got " + shape_text(weight_.shape));
    const bool takes = weight_.dtype == DType::BF16 && weight_.shape[1] % 8 == 0 && ((uintptr_t)weight_.data % 16) == 0;
    if (weight_.dtype == DType::BF16 && (gemm == "auto" || gemm == "tcgen05")) {
        fast_ = takes;
        if (!takes && gemm == "tcgen05")
            throw KernelError(label_ + ": the tcgen05 kernel does not take a weight of shape " + shape_text(weight_.shape));
    }
}

std::vector<std::string> Linear::required_libraries() const {
    return fast_ ? std::vector<std::string>{"core", "gemm100"} : std::vector<std::string>{"core"};
}

bool Linear::swapped_for(int rows, bool allow_split, bool fused_epilogue) const {
    if (!fast_) return false;
    const GemmPlan p = plan_gemm(rows, (int)weight_.shape[0], (int)weight_.shape[1], sm_count(), allow_split, fused_epilogue);
    return p.swapped && !p.pair;
}

bool Linear::applies_row_scale(int rows, DType out_dtype, bool fuse_swiglu, bool allow_split) const {
    if (!fast_) return false;
    const bool fused = fuse_swiglu && weight_.shape[0] % 2 == 0;
    const GemmPlan p = plan_gemm(rows, (int)weight_.shape[0], (int)weight_.shape[1], sm_count(), allow_split, fused);
    // few rows: the fused activation keeps K whole and writes bfloat16 from the swapped epilogue, which is where the factor goes
    if (p.swapped) return out_dtype == DType::BF16 && fused;
    // many rows: the epilogue of the 256-feature tiles, whenever it holds whole sums
    return p.block_n == 256 && p.splits == 1;
}

bool Linear::gives_partial_sums(int rows, bool allow_split) const {
    if (!fast_) return false;
    return plan_gemm(rows, (int)weight_.shape[0], (int)weight_.shape[1], sm_count(), allow_split, false).splits > 1;
}

Addend Linear::operator()(const Tensor& x_in, StepContext& ctx, const std::string& out_name, DType out_dtype, int rows,
                          bool allow_split, bool fuse_swiglu, float* add_into, const RowScale* scale, NormAhead* ahead) const {
    const int M = rows, N = (int)weight_.shape[0], K = (int)weight_.shape[1];
    Workspace& ws = *ctx.workspace;
    const CoreKernels& core = core_kernels();
    Tensor x = x_in;
    if (weight_.dtype == DType::F32 && x.dtype != DType::F32) {
        Tensor x32 = ws.get("linear_x32", {M, K}, DType::F32);
        QE_LAUNCH(core, core.cast(x.data, x.code(), x32.data, x32.code(), (long long)M * K, ctx.stream));
        x = x32;
    }
    const bool scaled = scale && scale->defined();
    if (scaled && !(fast_ && x.dtype == DType::BF16 && !add_into && applies_row_scale(M, out_dtype, fuse_swiglu, allow_split)))
        throw KernelError(label_ + ": rows without their factor reached a product that cannot apply it");
    if (!(fast_ && x.dtype == DType::BF16)) {
        Tensor out = ws.get(out_name, {M, N}, out_dtype);
        if (LaunchProfile::get().on())
            LaunchProfile::get().note_cost((double)weight_.bytes() + (double)x.bytes() + (double)out.bytes(), 2.0 * M * N * K);
        QE_LAUNCH(core, core.gemm_simple(x.data, x.code(), weight_.data, weight_.code(), out.data, out.code(), M, N, K, ctx.stream));
        return Addend(out, 1);
    }
    const GemmKernels& g = gemm_kernels();
    const bool fused = fuse_swiglu && N % 2 == 0;
    GemmPlan p = plan_gemm(M, N, K, sm_count(), allow_split, fused);
    auto run = [&](Tensor& out, int splits, bool swiglu, bool accumulate, NormAhead* work_ahead = nullptr) {
        if (LaunchProfile::get().on())      // what the product has to move and to compute: the weight once, x, and its result
            LaunchProfile::get().note_cost(2.0 * N * K + 2.0 * M * K + (double)out.bytes(), 2.0 * M * N * K);
        const float* sumsq = scaled ? scale->sumsq : nullptr;
        const int chunks = scaled ? scale->chunks : 0, width = scaled ? scale->width : 0;
        const float eps = scaled ? scale->eps : 0.0f;
        const float* ahead_weight = nullptr;
        void* ahead_rows = nullptr;
        float* ahead_sumsq = nullptr;
        if (work_ahead) {
            // the norm behind this addition: its weighted rows and their sums of squares per 128 features (two per tile)
            const int tiles = 2 * ceil_div(N, 256);
            work_ahead->rows = ws.get("norm_ahead_rows", {M, N}, DType::BF16);
            Tensor sums = ws.get("norm_ahead_sumsq", {M, tiles}, DType::F32);
            work_ahead->scale.sumsq = sums.as<float>(); work_ahead->scale.chunks = tiles;
            work_ahead->scale.width = N; work_ahead->scale.eps = work_ahead->eps;
            ahead_weight = work_ahead->weight; ahead_rows = work_ahead->rows.data; ahead_sumsq = sums.as<float>();
        }
        if (p.pair)
            QE_LAUNCH(g, g.gemm_pair(x.data, weight_.data, out.data, out.code(), M, N, K, splits, 0, swiglu, accumulate, sumsq, chunks,
                                     width, eps, ahead_weight, ahead_rows, ahead_sumsq, ctx.gemm_error, ctx.stream));
        else
            QE_LAUNCH(g, g.gemm(x.data, weight_.data, out.data, out.code(), M, N, K, p.swapped, p.block_n, splits, 0, swiglu,
                                accumulate, sumsq, chunks, width, eps, ahead_weight, ahead_rows, ahead_sumsq, ctx.gemm_error,
                                ctx.stream));
    };
    if (fused && (p.swapped || p.splits == 1)) {
        // K stays whole, so that the epilogue holds whole sums and can apply the activation; with few tokens the
        // weight tiles alone (N / 128 of them) keep the SMs streaming
        Tensor out = ws.get(out_name + "_act", {M, N / 2}, out_dtype);
        run(out, 1, true, false);
        return Addend(out, 1, true);
    }
    if (add_into && !p.swapped && p.splits == 1 && ctx.residual_width == N) {
        // many tokens, K whole: the residual sum happens in the epilogue and the product never goes to memory
        Tensor target(add_into, DType::F32, {M, N});
        const bool work_ahead = ahead && ahead->offered() && ahead->width == N && p.block_n == 256 && N % 4 == 0;
        run(target, 1, false, true, work_ahead ? ahead : nullptr);
        return Addend();
    }
    Tensor out = p.splits > 1 ? ws.get(out_name + "_partial", {p.splits, M, N}, DType::F32) : ws.get(out_name, {M, N}, out_dtype);
    run(out, p.splits, false, false);
    return Addend(out, p.splits);
}

}  // namespace qe
