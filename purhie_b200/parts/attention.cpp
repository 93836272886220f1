// Grouped-query attention over cache pages, with per-head RMSNorm on q and k and a position encoding.
//
// q = Wq x, k = Wk x, v = Wv x (+ optional biases, added before the norms); each q and k head is RMS-normalised
// over head_dim with a weight shared by all heads (same eps as the layer norms), then rotated; k and v go into
// the request's pages; query head h attends with kv head h / (HQ / HKV), scale 1 / sqrt(head_dim), causally,
// optionally only over the last `window` positions; then y = Wo o.
// Reference: src/qwen_model.cpp:940-975 (full_attention), src/attention.hip:273-313 (prep),
// src/attention.cpp:139-288 (host side; scale at :197), src/attention.h:73 (window),
// src/inference.cpp:623-646 (tensors and shapes).
//
// K and V are written to pages before attention runs, and attention reads everything, the current step's keys
// included, from pages: a whole prompt, a portion and a decoded token are one algorithm per kernel.
//
// Which kernel: float32, or a head size the tensor-core kernels do not take -> attention_generic (any size, fixed
// order).  bfloat16 with head size 64 or 128 and groups up to 16: single-token segments go to the persistent
// TMA-fed split-key kernel (pages of 8..64 tokens; else the cp.async one), prompt portions to the tcgen05 kernel
// (head size 128, pages of 8 to 64) or the mma.sync tiled kernel.  The tile lists those two want are this
// part's own metadata: prepare_step() adds them to the step.
#include <algorithm>
#include <cmath>

#include "linear.h"
#include "parts.h"

namespace qe {

namespace {
constexpr int kBlockKeys = 64, kMaxSplits = 32;
constexpr int kTile = 64;          // rows of a query tile of the mma.sync prefill kernel
constexpr int kTileLarge = 128;    // rows of a query tile of the tcgen05 prefill kernel
constexpr int kCtasPerSm = 3;      // cp.async decode CTAs that fit one SM (68 KB of shared memory each at head_dim 128)
inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Splits of the key range for the cp.async decode kernel.  CTAs run in waves of kCtasPerSm per SM; the number of
// splits is the one that minimises waves x (fixed cost + blocks per split).
int decode_splits(int n_rows, int kv_heads, int max_ctx, int sms, int window) {
    const int span = window ? std::min(max_ctx, window) : max_ctx;
    const int blocks = std::max(1, ceil_div(span, kBlockKeys)), pairs = std::max(1, n_rows * kv_heads), slots = kCtasPerSm * sms;
    int best = 1;
    double best_cost = -1;
    for (int s = 1; s <= std::min(blocks, kMaxSplits); s++) {
        const int per = ceil_div(blocks, s);
        if (s > 1 && ceil_div(blocks, per) != s) continue;        // the same blocks per split as a smaller s
        const double cost = (double)ceil_div((long long)pairs * s, slots) * (4.0 + per);
        if (best_cost < 0 || cost < best_cost - 1e-9) { best = s; best_cost = cost; }
    }
    return best;
}

// Splits for the persistent kernel: two CTAs per SM take items in turn, so the time is (items per CTA, rounded
// up) x (blocks of 64 keys per item + what an item costs beside its blocks), plus the merge kernel when the keys
// are split.  A split item costs about a block and a half more (its partial result goes to memory), a whole one
// next to nothing, and the merge grows with the number of parts it reads: measured at 1 to 128 rows of 1,024 to
// 8,192 keys.
int bulk_splits(int n_rows, int kv_heads, int max_ctx, int sms, int window) {
    const int span = window ? std::min(max_ctx, window) : max_ctx;
    const int blocks = std::max(1, ceil_div(span, kBlockKeys)), pairs = std::max(1, n_rows * kv_heads);
    int best = 1;
    double best_cost = -1;
    for (int s = 1; s <= std::min(blocks, kMaxSplits); s++) {
        const int per = ceil_div(blocks, s);
        if (s > 1 && ceil_div(blocks, per) != s) continue;
        const double cost = (double)ceil_div((long long)pairs * s, 2 * sms) * (per + (s > 1 ? 1.5 : 0.25)) + (s > 1 ? 2.0 + 0.15 * s : 0.0);
        if (best_cost < 0 || cost < best_cost - 1e-9) { best = s; best_cost = cost; }
    }
    return best;
}

// CTAs per tile of the tcgen05 prefill kernel.  The time is about (rounds of the CTAs over two slots per SM) x
// (blocks of 64 keys per CTA + a few for its start) plus, when tiles are shared, what writing and merging the
// partial results costs.  Many tiles, or tiles that look back over few keys, stay whole; a short portion late
// in a long context is cut so that its CTAs fill the device once.
int tc5_splits(int n_tiles, int heads, int max_ctx, int sms, int window) {
    const int span = window ? std::min(max_ctx, window + 128) : max_ctx;
    const int blocks = std::max(1, ceil_div(span, 64)), ctas = std::max(1, n_tiles * heads);
    int best = 1;
    double best_cost = -1;
    for (int s = 1; s <= std::min(16, blocks); s++) {
        double cost = (double)ceil_div((long long)ctas * s, 2 * sms) * (ceil_div(blocks, s) + 4);
        if (s > 1) cost += 8 + 0.5 * s + 0.024 * ctas * s;
        if (best_cost < 0 || cost < best_cost - 1e-9) { best = s; best_cost = cost; }
    }
    return best;
}

// The prompt portions of a step cut into tiles of `rows` rows: segment and first row (within the portion) of
// each tile.  The tiles that look furthest back come first: the grid starts them first and the short ones fill
// the tail.
void add_tiles(StepPlan& plan, int rows, const std::string& name) {
    if (plan.has(name + ".seg")) return;
    struct Tile { int seg, first, reach; };
    std::vector<Tile> tiles;
    for (int s = 0; s < plan.S; s++) {
        const int n = plan.q_lens[s];
        if (n == 1) continue;
        for (int first = 0; first < n; first += rows)
            tiles.push_back({s, first, plan.ctx_lens[s] - n + std::min(first + rows, n)});
    }
    std::stable_sort(tiles.begin(), tiles.end(), [](const Tile& a, const Tile& b) { return a.reach > b.reach; });
    std::vector<int32_t> seg, first;
    for (const Tile& t : tiles) { seg.push_back(t.seg); first.push_back(t.first); }
    plan.add(name + ".seg", std::move(seg));
    plan.add(name + ".first", std::move(first));
}
}  // namespace

// params: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm_eps (null: no q/k norm), bias, position
// (a PartSpec as {kind, params}, or null), window (null: all positions), scale (null: 1/sqrt(head_dim)),
// names{q_proj, k_proj, v_proj, o_proj, q_norm, k_norm, q_bias, k_bias, v_bias}.
class Attention : public Mixer {
public:
    Attention(const Json& p, BuildContext& b) : Mixer(p, b) {
        hidden_ = p.at("hidden_size").as_int();
        heads_ = (int)p.at("num_heads").as_int();
        kv_heads_ = (int)p.at("num_kv_heads").as_int();
        head_dim_ = (int)p.at("head_dim").as_int();
        if (heads_ < 1 || kv_heads_ < 1 || heads_ % kv_heads_)
            throw ConfigError(std::to_string(heads_) + " query heads are not a multiple of " + std::to_string(kv_heads_) + " kv heads");
        const Json* eps = p.find("qk_norm_eps");
        has_norm_ = eps && !eps->is_null();
        eps_ = has_norm_ ? eps->as_double() : 0.0;
        has_bias_ = p.get_bool("bias", false);
        window_ = (int)p.get_int("window", 0);
        const Json* sc = p.find("scale");
        scale_ = (sc && !sc->is_null()) ? sc->as_double() : 1.0 / std::sqrt((double)head_dim_);
        if (const Json* pos = p.find("position")) {
            if (!pos->is_null()) {
                PartSpec spec = PartSpec::from_json(*pos);
                Json key_params = Json::object();
                for (const auto& m : spec.params.members()) if (m.first != "names") key_params.set(m.first, m.second);
                auto part = b.shared("position:" + spec.kind + ":" + key_params.dump(), [&] { return make_part("position", spec, b); });
                position_ = std::dynamic_pointer_cast<PositionEncoding>(part);
                if (!position_) throw ConfigError("part '" + spec.kind + "' is not a position encoding");
            }
        }
        gemm_ = b.options.get_string("gemm", "auto");
        attention_ = b.options.get_string("attention", "auto");
        q_width_ = (int64_t)heads_ * head_dim_;
        kv_width_ = (int64_t)kv_heads_ * head_dim_;
    }

    // ---- weights ----------------------------------------------------------------------------------------------
    std::vector<TensorSpec> tensor_specs() const override {
        std::vector<TensorSpec> s = {{name_of("q_proj"), {q_width_, hidden_}, Role::Matrix, Init::Normal},
                                     {name_of("k_proj"), {kv_width_, hidden_}, Role::Matrix, Init::Normal},
                                     {name_of("v_proj"), {kv_width_, hidden_}, Role::Matrix, Init::Normal},
                                     {name_of("o_proj"), {hidden_, q_width_}, Role::Matrix, Init::Normal}};
        if (has_norm_) {
            s.push_back({name_of("q_norm"), {head_dim_}, Role::Vector, Init::Scale});
            s.push_back({name_of("k_norm"), {head_dim_}, Role::Vector, Init::Scale});
        }
        if (has_bias_) {
            s.push_back({name_of("q_bias"), {q_width_}, Role::Vector, Init::Normal});
            s.push_back({name_of("k_bias"), {kv_width_}, Role::Vector, Init::Normal});
            s.push_back({name_of("v_bias"), {kv_width_}, Role::Vector, Init::Normal});
        }
        return s;
    }

    void bind(WeightSource& src) override {
        // one matrix [q | k | v] so that the three projections are one product (a layout choice only)
        Tensor parts[3] = {src.fetch(name_of("q_proj")), src.fetch(name_of("k_proj")), src.fetch(name_of("v_proj"))};
        if (parts[0].dtype != parts[1].dtype || parts[0].dtype != parts[2].dtype)
            throw WeightError(name_of("q_proj") + ", " + name_of("k_proj") + " and " + name_of("v_proj") + " are stored in different precisions");
        Tensor qkv = src.arena().alloc(parts[0].dtype, {q_width_ + 2 * kv_width_, hidden_});
        size_t off = 0;
        for (Tensor& t : parts) {
            QE_CUDA(cudaMemcpyAsync(static_cast<char*>(qkv.data) + off, t.data, t.bytes(), cudaMemcpyDeviceToDevice, src.stream()));
            off += t.bytes();
        }
        if (has_bias_) {
            Tensor b[3] = {src.fetch(name_of("q_bias")), src.fetch(name_of("k_bias")), src.fetch(name_of("v_bias"))};
            bias_ = src.arena().alloc(DType::F32, {q_width_ + 2 * kv_width_});
            off = 0;
            for (Tensor& t : b) {
                QE_CUDA(cudaMemcpyAsync(static_cast<char*>(bias_.data) + off, t.data, t.bytes(), cudaMemcpyDeviceToDevice, src.stream()));
                off += t.bytes();
            }
            QE_CUDA(cudaStreamSynchronize(src.stream()));
            for (Tensor& t : b) src.release(t);
        }
        QE_CUDA(cudaStreamSynchronize(src.stream()));
        for (Tensor& t : parts) src.release(t);
        qkv_proj_ = Linear(qkv, "qkv_proj", gemm_);
        q_only_proj_ = Linear(qkv.rows(0, q_width_), "q_proj", gemm_);
        o_proj_ = Linear(src.fetch(name_of("o_proj")), "o_proj", gemm_);
        if (has_norm_) {
            q_norm_ = src.fetch(name_of("q_norm"));
            k_norm_ = src.fetch(name_of("k_norm"));
        }
        if (position_) {
            position_->bind(src);
            table_ = position_->rotation_table();
        }
    }

    std::vector<std::string> required_libraries() const override {
        std::vector<std::string> libs = {"core"};
        if (qkv_proj_.fast() || o_proj_.fast()) libs.push_back("gemm100");
        if (use_flash()) libs.push_back("flash");
        return libs;
    }
    std::vector<Part*> children() override { return position_ ? std::vector<Part*>{position_.get()} : std::vector<Part*>{}; }
    // rows per tile of the products for many tokens (the tcgen05 pair kernel): a scheduler may end a step there
    int preferred_row_multiple() const override { return (qkv_proj_.fast() || o_proj_.fast()) ? 256 : 0; }

    bool use_flash() const {
        if (compute_dtype != DType::BF16 || attention_ == "generic") return false;
        const int group = heads_ / kv_heads_;
        const bool ok = (head_dim_ == 64 || head_dim_ == 128) && group >= 1 && group <= 16;
        if (!ok && attention_ == "flash")
            throw KernelError("the flash attention kernels do not take head_dim " + std::to_string(head_dim_) + " with " +
                              std::to_string(group) + " query heads per kv head");
        return ok;
    }

    // ---- cache and step metadata ------------------------------------------------------------------------------
    CacheNeed cache_need() const override { return CacheNeed::pages(kv_heads_, head_dim_, window_); }

    void prepare_step(StepPlan& plan) override {
        if (!use_flash()) return;
        bool portions = false;
        for (int n : plan.q_lens) portions |= n > 1;
        if (!portions) return;
        add_tiles(plan, kTile, "attention.tiles64");
        add_tiles(plan, kTileLarge, "attention.tiles128");
    }

    // Few rows in bfloat16: the qkv product's float32 sums are linear in the rows, and the kernel that adds them up
    // (per-head norm, rotation, cache write) multiplies by the factor the norm in front left out.
    // Many rows: either the qkv product's epilogue applies the factor (K whole), or K is cut and the same kernel as
    // above adds up the parts.
    bool takes_unscaled_rows(const StepContext& ctx) const override {
        auto takes = [&](const Linear& proj) {
            return proj.swapped_for(ctx.T, true, false) || proj.applies_row_scale(ctx.T, compute_dtype, false, true) ||
                   proj.gives_partial_sums(ctx.T, true);
        };
        return compute_dtype == DType::BF16 && takes(qkv_proj_) && (!q_only_proj_.defined() || takes(q_only_proj_));
    }

    // ---- step ----------------------------------------------------------------------------------------------------
    Addend forward(const Tensor& x, StepContext& ctx, const CacheView& cache) override {
        const int T = ctx.T;
        Workspace& ws = *ctx.workspace;
        const DType dt = compute_dtype;
        const GroupStep& g = ctx.groups.at(cache.group);
        const CoreKernels& core = core_kernels();
        const Linear& proj = cache.writable ? qkv_proj_ : q_only_proj_;
        // rows without their factor (RowScale): the product's epilogue applies it where it can, else the kernel behind it
        const bool scale_in_product = ctx.row_scale.defined() && proj.applies_row_scale(T, dt, false, true);
        Addend qkv = proj(x, ctx, "qkv", dt, T, true, false, nullptr, scale_in_product ? &ctx.row_scale : nullptr);
        const RowScale later = scale_in_product ? RowScale() : ctx.row_scale;
        const int kv_heads_written = cache.writable ? kv_heads_ : 0;
        Tensor q = ws.get("q", {T, heads_, head_dim_}, dt);
        const int column = position_ ? position_->position_column() : 0;
        const int32_t* positions = ctx.position_column(column);
        QE_LAUNCH(core, core.qk_norm_rope_kv_write(
            qkv.tensor.data, qkv.tensor.code(), qkv.splits, (long long)T * (q_width_ + 2 * (int64_t)kv_heads_written * head_dim_),
            bias_.defined() ? bias_.as<float>() : nullptr, has_norm_ ? q_norm_.as<float>() : nullptr,
            has_norm_ ? k_norm_.as<float>() : nullptr, (float)eps_, table_.defined() ? table_.as<float>() : nullptr,
            position_ ? position_->n_rot() : 0, table_.defined() ? (int)table_.shape[0] : 0, positions,
            cache.writable ? g.slot_mapping : nullptr, q.data, q.code(), cache.k_base, cache.v_base, (int)cache.kv_dtype,
            cache.page_stride, cache.page_size, T, heads_, kv_heads_written, head_dim_,
            position_ && position_->interleaved() ? 1 : 0, later.sumsq, later.chunks, later.width, later.eps, ctx.stream));
        Tensor out = ws.get("attn_out", {T, q_width_}, dt);
        const int32_t* abs_positions = ctx.position_column(0);       // the mask always follows the index in the request
        if (use_flash()) {
            if (cache.kv_dtype != DType::BF16) throw KernelError("attention_flash: the cache must be bfloat16");
            flash(q, cache, g, ctx, out, abs_positions);
        } else {
            QE_LAUNCH(core, core.attention_generic(q.data, q.code(), cache.k_base, cache.v_base, (int)cache.kv_dtype, cache.page_stride,
                                                   cache.page_size, g.block_table, g.table_width, ctx.row_seg, abs_positions, out.data,
                                                   out.code(), T, heads_, kv_heads_, head_dim_, window_, (float)scale_, ctx.stream));
        }
        return o_proj_(out, ctx, "o_out", DType::F32, T, true, false, ctx.residual, nullptr, &ctx.norm_ahead);
    }

private:
    // All rows of the step: q [T, HQ, D] bfloat16 -> out [T, HQ * D] bfloat16.
    void flash(const Tensor& q, const CacheView& cache, const GroupStep& g, StepContext& ctx, Tensor& out, const int32_t* positions) {
        const FlashKernels& f = flash_kernels();
        Workspace& ws = *ctx.workspace;
        const int sms = sm_count();
        StepArray t64 = ctx.array("attention.tiles64.seg"), t64f = ctx.array("attention.tiles64.first");
        StepArray t128 = ctx.array("attention.tiles128.seg"), t128f = ctx.array("attention.tiles128.first");
        const bool tc5_ok = head_dim_ == 128 && (cache.page_size == 8 || cache.page_size == 16 || cache.page_size == 32 || cache.page_size == 64) && cache.num_pages > 0;
        if (t64.count && t128.count && tc5_ok && ctx.option("prefill_kernel") != "mma_sync") {
            int splits = (int)ctx.option_int("prefill_splits");
            if (!splits) splits = tc5_splits(t128.count, heads_, ctx.prefill_max_ctx, sms, window_);
            float *part_o = nullptr, *part_ml = nullptr;
            if (splits > 1) {
                part_o = ws.get("attn_tile_part_o", {ctx.T, heads_, splits, head_dim_}, DType::F32).as<float>();
                part_ml = ws.get("attn_tile_part_ml", {ctx.T, heads_, splits, 2}, DType::F32).as<float>();
            }
            QE_LAUNCH(f, f.prefill_tc5(q.data, ctx.T, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, cache.num_pages,
                                       g.block_table, g.table_width, ctx.seg_start, ctx.seg_ctx_len, t128.data, t128f.data, t128.count,
                                       out.data, heads_, kv_heads_, head_dim_, window_, (float)scale_, splits, part_o, part_ml,
                                       ctx.attention_error, ctx.stream));
        } else if (t64.count) {
            QE_LAUNCH(f, f.prefill(q.data, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, g.block_table, g.table_width,
                                   ctx.seg_start, ctx.seg_ctx_len, t64.data, t64f.data, t64.count, out.data, heads_, kv_heads_,
                                   head_dim_, window_, (float)scale_, ctx.stream));
        }
        if (!ctx.n_decode_rows) return;
        const int n = ctx.n_decode_rows;
        const bool bulk_ok = cache.page_size % 8 == 0 && kBlockKeys % cache.page_size == 0 && cache.num_pages > 0;
        const bool bulk = bulk_ok && ctx.option("decode_kernel") != "cp_async";
        int splits = (int)ctx.option_int("decode_splits");            // a test's choice, else what the cost model picks
        if (splits < 1 || splits > kMaxSplits)
            splits = bulk ? bulk_splits(n, kv_heads_, ctx.decode_max_ctx, sms, window_)
                          : decode_splits(n, kv_heads_, ctx.decode_max_ctx, sms, window_);
        float *part_o = nullptr, *part_ml = nullptr;
        if (splits > 1) {
            part_o = ws.get("attn_part_o", {n, heads_, splits, head_dim_}, DType::F32).as<float>();
            part_ml = ws.get("attn_part_ml", {n, heads_, splits, 2}, DType::F32).as<float>();
        }
        if (bulk)
            QE_LAUNCH(f, f.decode_bulk(q.data, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, cache.num_pages, g.block_table,
                                       g.table_width, ctx.decode_rows, n, ctx.row_seg, positions, part_o, part_ml, out.data, heads_,
                                       kv_heads_, head_dim_, splits, window_, (float)scale_, 0, ctx.attention_error, ctx.stream));
        else
            QE_LAUNCH(f, f.decode(q.data, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, g.block_table, g.table_width,
                                  ctx.decode_rows, n, ctx.row_seg, positions, part_o, part_ml, out.data, heads_, kv_heads_, head_dim_,
                                  splits, window_, (float)scale_, ctx.stream));
    }

    int64_t hidden_, q_width_, kv_width_;
    int heads_, kv_heads_, head_dim_, window_;
    bool has_norm_, has_bias_;
    double eps_, scale_;
    std::string gemm_, attention_;
    std::shared_ptr<PositionEncoding> position_;
    Linear qkv_proj_, q_only_proj_, o_proj_;
    Tensor q_norm_, k_norm_, bias_, table_;
};

void register_mixer_parts() {
    register_part("mixer", "attention", [](const Json& p, BuildContext& b) { return std::make_shared<Attention>(p, b); });
}

}  // namespace qe
