// Parts that the framework does not have, defined by a test and registered through the public registries when this
// shared object is loaded: a mixer with state of its own (and step metadata of its own), a mixer that keeps values
// narrower than its keys in the cache manager's pages, another position encoding, a
// feed-forward with routing, an arrangement with a third norm, and an architecture nobody has that strings them
// together with the framework's own attention and SwiGLU.  No file of the framework changes for any of it; the only
// header a part needs is parts/parts.h (config/config.h for an architecture).
#include <cuda_bf16.h>

#include <cmath>

#include "purhie_b200/config/config.h"
#include "purhie_b200/parts/parts.h"

using namespace qe;

namespace {

// ---- a mixer with state of its own -------------------------------------------------------------------------------
// Per request the sum of all inputs so far and their count.  Output for a token = (mean of the request's inputs up
// to and including it) @ W.  Rows of a request arrive in order; the state carries over from step to step.
// One block per segment walks the segment's rows in order; the segments come from an array this mixer adds to the
// step itself ("toy_mean.segments": first row, rows, state slot per segment).
__global__ void running_mean_kernel(const void* x, int x_is_bf16, const int32_t* segments, float* state, int E, float* out) {
    const int32_t first = segments[3 * blockIdx.x], rows = segments[3 * blockIdx.x + 1], slot = segments[3 * blockIdx.x + 2];
    float* st = state + (size_t)slot * (E + 1);
    const float count0 = st[E];
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        float sum = st[e];
        for (int r = 0; r < rows; r++) {
            const size_t i = (size_t)(first + r) * E + e;
            sum += x_is_bf16 ? __bfloat162float(((const __nv_bfloat16*)x)[i]) : ((const float*)x)[i];
            out[i] = sum / (count0 + (float)(r + 1));
        }
        st[e] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) st[E] = count0 + (float)rows;
}

class RunningMeanMixer : public Mixer {
public:
    RunningMeanMixer(const Json& p, BuildContext& b) : Mixer(p, b), size_(p.at("hidden_size").as_int()) {}
    std::vector<TensorSpec> tensor_specs() const override { return {{name_of("weight"), {size_, size_}, Role::Matrix, Init::Normal}}; }
    void bind(WeightSource& src) override { w_ = src.fetch(name_of("weight")); }
    CacheNeed cache_need() const override { return CacheNeed::state({size_ + 1}, DType::F32); }
    void prepare_step(StepPlan& plan) override {
        if (plan.has("toy_mean.segments")) return;
        std::vector<int32_t> seg;
        int row = 0;
        for (int s = 0; s < plan.S; s++) {
            seg.push_back(row); seg.push_back(plan.q_lens[s]); seg.push_back(plan.slots[s]);
            row += plan.q_lens[s];
        }
        plan.add("toy_mean.segments", seg);
    }
    Addend forward(const Tensor& x, StepContext& ctx, const CacheView& cache) override {
        StepArray seg = ctx.array("toy_mean.segments");             // what prepare_step added, on the device now
        if (seg.count != 3 * ctx.S) throw Error(kInvalidState, "toy_mean.segments is not in the step");
        Tensor mean = ctx.workspace->get("toy_mean", {ctx.T, size_}, DType::F32);
        running_mean_kernel<<<ctx.S, 128, 0, ctx.stream>>>(x.data, x.dtype == DType::BF16, seg.data, cache.state.as<float>(),
                                                           (int)size_, mean.as<float>());
        Tensor y = ctx.workspace->get("toy_mean_out", {ctx.T, size_}, DType::F32);
        const CoreKernels& k = core_kernels();
        QE_LAUNCH(k, k.gemm_simple(mean.data, mean.code(), w_.data, w_.code(), y.data, y.code(), ctx.T, (int)size_, (int)size_, ctx.stream));
        return Addend(y, 1);
    }
private:
    int64_t size_;
    Tensor w_;
};

// ---- a mixer whose values are narrower than its keys ----------------------------------------------------------------
// One head: keys of key_dim, values of value_dim < key_dim (a "compressed" value), both kept in the cache manager's
// pages: the mixer states the two widths in its CacheNeed and gets pages laid out [K: page_size x key_dim][V: page_size
// x value_dim].  Plain causal attention over the request's pages, float32.
__global__ void narrow_write_kernel(const float* k, const float* v, const int32_t* slot_mapping, float* k_base, float* v_base,
                                    long long page_stride, int page_size, int Dk, int Dv) {
    const int t = blockIdx.x;
    const int slot = slot_mapping[t], page = slot / page_size, off = slot % page_size;
    for (int d = threadIdx.x; d < Dk; d += blockDim.x) k_base[(size_t)page * page_stride + (size_t)off * Dk + d] = k[(size_t)t * Dk + d];
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) v_base[(size_t)page * page_stride + (size_t)off * Dv + d] = v[(size_t)t * Dv + d];
}
__global__ void narrow_attend_kernel(const float* q, const int32_t* row_seg, const int32_t* positions, const int32_t* block_table,
                                     int table_width, const float* k_base, const float* v_base, long long page_stride,
                                     int page_size, int Dk, int Dv, float* out) {
    extern __shared__ float score[];                      // one per visible key
    __shared__ float red[2];
    const int t = blockIdx.x, z = positions[t];
    const int32_t* table = block_table + (size_t)row_seg[t] * table_width;
    for (int p = threadIdx.x; p <= z; p += blockDim.x) {
        const float* kp = k_base + (size_t)table[p / page_size] * page_stride + (size_t)(p % page_size) * Dk;
        float s = 0.0f;
        for (int d = 0; d < Dk; d++) s += q[(size_t)t * Dk + d] * kp[d];
        score[p] = s * rsqrtf((float)Dk);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = -INFINITY, l = 0.0f;
        for (int p = 0; p <= z; p++) m = fmaxf(m, score[p]);
        for (int p = 0; p <= z; p++) l += expf(score[p] - m);
        red[0] = m; red[1] = l;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        float acc = 0.0f;
        for (int p = 0; p <= z; p++)
            acc += expf(score[p] - red[0]) * v_base[(size_t)table[p / page_size] * page_stride + (size_t)(p % page_size) * Dv + d];
        out[(size_t)t * Dv + d] = acc / red[1];
    }
}

class NarrowValueAttention : public Mixer {
public:
    NarrowValueAttention(const Json& p, BuildContext& b)
        : Mixer(p, b), size_(p.at("hidden_size").as_int()), dk_((int)p.at("key_dim").as_int()), dv_((int)p.at("value_dim").as_int()) {}
    std::vector<TensorSpec> tensor_specs() const override {
        return {{name_of("wq"), {dk_, size_}, Role::Matrix, Init::Normal}, {name_of("wk"), {dk_, size_}, Role::Matrix, Init::Normal},
                {name_of("wv"), {dv_, size_}, Role::Matrix, Init::Normal}, {name_of("wo"), {size_, dv_}, Role::Matrix, Init::Normal}};
    }
    void bind(WeightSource& src) override {
        wq_ = src.fetch(name_of("wq")); wk_ = src.fetch(name_of("wk")); wv_ = src.fetch(name_of("wv")); wo_ = src.fetch(name_of("wo"));
    }
    CacheNeed cache_need() const override { return CacheNeed::pages(1, dk_, 0, dv_); }
    Addend forward(const Tensor& x, StepContext& ctx, const CacheView& cache) override {
        if (cache.kv_dtype != DType::F32 || x.dtype != DType::F32) throw Error(kInvalidState, "the toy attention runs in float32");
        if (cache.key_dim != dk_ || cache.value_dim != dv_ || cache.kv_heads != 1) throw Error(kInvalidState, "the cache is not laid out for this mixer");
        const CoreKernels& kn = core_kernels();
        const GroupStep& g = ctx.groups.at(cache.group);
        Workspace& ws = *ctx.workspace;
        auto product = [&](const Tensor& in, const Tensor& w, const char* name, int n_out) {
            Tensor out = ws.get(name, {ctx.T, n_out}, DType::F32);
            QE_LAUNCH(kn, kn.gemm_simple(in.data, in.code(), w.data, w.code(), out.data, out.code(), ctx.T, n_out, (int)w.shape[1], ctx.stream));
            return out;
        };
        Tensor q = product(x, wq_, "toy_narrow_q", dk_), k = product(x, wk_, "toy_narrow_k", dk_), v = product(x, wv_, "toy_narrow_v", dv_);
        narrow_write_kernel<<<ctx.T, 32, 0, ctx.stream>>>(k.as<float>(), v.as<float>(), g.slot_mapping, (float*)cache.k_base,
                                                          (float*)cache.v_base, cache.page_stride, cache.page_size, dk_, dv_);
        int longest = 1;
        for (int c : ctx.ctx_lens) longest = std::max(longest, c);
        Tensor o = ws.get("toy_narrow_o", {ctx.T, dv_}, DType::F32);
        narrow_attend_kernel<<<ctx.T, 64, (size_t)longest * sizeof(float), ctx.stream>>>(
            q.as<float>(), ctx.row_seg, ctx.position_column(0), g.block_table, g.table_width, (const float*)cache.k_base,
            (const float*)cache.v_base, cache.page_stride, cache.page_size, dk_, dv_, o.as<float>());
        return Addend(product(o, wo_, "toy_narrow_y", (int)size_), 1);
    }
private:
    int64_t size_;
    int dk_, dv_;
    Tensor wq_, wk_, wv_, wo_;
};

// ---- another position encoding --------------------------------------------------------------------------------------
// Rotate-half pairs with every frequency divided by `factor`.
class ScaledRotary : public PositionEncoding {
public:
    ScaledRotary(const Json& p, BuildContext& b) : PositionEncoding(p, b) {
        n_rot_ = (int)p.at("n_rot").as_int();
        theta_ = p.at("theta").as_double();
        factor_ = p.at("factor").as_double();
        max_position_ = p.at("max_position").as_int();
    }
    int n_rot() const override { return n_rot_; }
    void bind(WeightSource& src) override {
        if (table_.defined()) return;
        const int half = n_rot_ / 2;
        std::vector<float> host((size_t)max_position_ * n_rot_);
        for (int64_t pos = 0; pos < max_position_; pos++)
            for (int i = 0; i < half; i++) {
                const double a = (double)pos * std::pow(theta_, -2.0 * i / n_rot_) / factor_;
                host[(size_t)pos * n_rot_ + i] = (float)std::cos(a);
                host[(size_t)pos * n_rot_ + half + i] = (float)std::sin(a);
            }
        table_ = src.arena().alloc(DType::F32, {max_position_, n_rot_});
        QE_CUDA(cudaMemcpy(table_.data, host.data(), host.size() * 4, cudaMemcpyHostToDevice));
    }
    Tensor rotation_table() override { return table_; }
private:
    int n_rot_;
    double theta_, factor_;
    int64_t max_position_;
    Tensor table_;
};

// ---- a feed-forward with routing ----------------------------------------------------------------------------------------
// The router's float32 logits pick one of `experts` matrices per token (the lowest index on ties).
__global__ void top1_kernel(const float* logits, int experts, int32_t* choice) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    int best = 0;
    for (int e = 1; e < experts; e++)
        if (logits[(size_t)t * experts + e] > logits[(size_t)t * experts + best]) best = e;
    choice[t] = best;
}
__global__ void routed_matvec_kernel(const float* x, const void* const* mats, int mats_are_bf16, const int32_t* choice, int E, float* y) {
    const int t = blockIdx.x;
    const void* w = mats[choice[t]];
    for (int o = threadIdx.x; o < E; o += blockDim.x) {
        float acc = 0.0f;
        for (int i = 0; i < E; i++) {
            const float wv = mats_are_bf16 ? __bfloat162float(((const __nv_bfloat16*)w)[(size_t)o * E + i]) : ((const float*)w)[(size_t)o * E + i];
            acc = fmaf(x[(size_t)t * E + i], wv, acc);
        }
        y[(size_t)t * E + o] = acc;
    }
}

class Top1Routed : public FeedForward {
public:
    Top1Routed(const Json& p, BuildContext& b) : FeedForward(p, b), size_(p.at("hidden_size").as_int()), experts_((int)p.at("experts").as_int()) {}
    std::vector<TensorSpec> tensor_specs() const override {
        std::vector<TensorSpec> s = {{"toy.router", {experts_, size_}, Role::Vector, Init::Normal}};     // float32 always
        for (int e = 0; e < experts_; e++) s.push_back({"toy.expert" + std::to_string(e), {size_, size_}, Role::Matrix, Init::Normal});
        return s;
    }
    void bind(WeightSource& src) override {
        router_ = src.fetch("toy.router");
        std::vector<const void*> ptrs;
        for (int e = 0; e < experts_; e++) {
            mats_.push_back(src.fetch("toy.expert" + std::to_string(e)));
            ptrs.push_back(mats_.back().data);
        }
        table_ = src.arena().alloc(DType::I64, {experts_});
        QE_CUDA(cudaMemcpy(table_.data, ptrs.data(), ptrs.size() * sizeof(void*), cudaMemcpyHostToDevice));
    }
    Addend forward(const Tensor& x, StepContext& ctx) override {
        Workspace& ws = *ctx.workspace;
        const CoreKernels& k = core_kernels();
        Tensor x32 = x;
        if (x.dtype != DType::F32) {
            x32 = ws.get("toy_x32", {ctx.T, size_}, DType::F32);
            QE_LAUNCH(k, k.cast(x.data, x.code(), x32.data, x32.code(), (long long)ctx.T * size_, ctx.stream));
        }
        Tensor logits = ws.get("toy_router", {ctx.T, experts_}, DType::F32);
        QE_LAUNCH(k, k.gemm_simple(x32.data, x32.code(), router_.data, router_.code(), logits.data, logits.code(), ctx.T, experts_,
                                   (int)size_, ctx.stream));
        Tensor choice = ws.get("toy_choice", {ctx.T}, DType::I32);
        top1_kernel<<<1, ctx.T, 0, ctx.stream>>>(logits.as<float>(), experts_, choice.as<int32_t>());       // a toy: T <= 1024
        Tensor y = ws.get("toy_ff", {ctx.T, size_}, DType::F32);
        routed_matvec_kernel<<<ctx.T, 64, 0, ctx.stream>>>(x32.as<float>(), (const void* const*)table_.data, mats_[0].dtype == DType::BF16,
                                                            choice.as<int32_t>(), (int)size_, y.as<float>());
        return Addend(y, 1);
    }
private:
    int64_t size_;
    int experts_;
    Tensor router_, table_;
    std::vector<Tensor> mats_;
};

// ---- an arrangement with a third norm ------------------------------------------------------------------------------------
// x += post_norm(mixer(norm1(x))); x += feed_forward(norm2(x)).  Sub-parts: mixer_norm, mixer, mixer_post_norm,
// feed_forward_norm, feed_forward.  The post norm runs over the mixer's addend alone: a scratch stream of zeros takes
// the addend as its pending sum.
class SandwichBlock : public Arrangement {
public:
    SandwichBlock(const LayerSpec& layer, BuildContext& build) {
        n1_ = make_part_as<Norm>("norm", layer.part("mixer_norm"), build);
        mixer_ = make_part_as<Mixer>("mixer", layer.part("mixer"), build);
        post_ = make_part_as<Norm>("norm", layer.part("mixer_post_norm"), build);
        n2_ = make_part_as<Norm>("norm", layer.part("feed_forward_norm"), build);
        ff_ = make_part_as<FeedForward>("feed_forward", layer.part("feed_forward"), build);
    }
    std::vector<Part*> parts() override { return {n1_.get(), mixer_.get(), post_.get(), n2_.get(), ff_.get()}; }
    CacheNeed cache_need() const override { return mixer_->cache_need(); }
    void forward(ResidualStream& stream, StepContext& ctx, const CacheView& cache) override {
        ctx.residual = nullptr;                                  // nobody adds into the stream behind this block's back
        Tensor xn = n1_->forward(stream, ctx);
        Addend mixed = mixer_->forward(xn, ctx, cache);
        const int64_t E = stream.x.shape[1];
        ResidualStream scratch;
        scratch.x = ctx.workspace->get("toy_sandwich_zero", {ctx.T, E}, DType::F32);
        QE_CUDA(cudaMemsetAsync(scratch.x.data, 0, scratch.x.bytes(), ctx.stream));
        scratch.add(mixed);
        Tensor normed = post_->forward(scratch, ctx);
        // the normed rows live in the norm's own scratch ("normed"), which the next norm overwrites: keep a copy
        Tensor kept = ctx.workspace->get("toy_sandwich_kept", {ctx.T, E}, normed.dtype);
        QE_CUDA(cudaMemcpyAsync(kept.data, normed.data, normed.bytes(), cudaMemcpyDeviceToDevice, ctx.stream));
        stream.add(Addend(kept, 1));
        xn = n2_->forward(stream, ctx);
        stream.add(ff_->forward(xn, ctx));
    }
private:
    std::shared_ptr<Norm> n1_, post_, n2_;
    std::shared_ptr<Mixer> mixer_;
    std::shared_ptr<FeedForward> ff_;
};

// ---- an architecture nobody has -----------------------------------------------------------------------------------------------
// Layer 0: the framework's attention with the toy position encoding, and the routed feed-forward.  Layer 1: the
// stateful toy mixer with the framework's SwiGLU, in the sandwich arrangement.  Run order: layer 0, layer 1, layer 0
// again (a cache of its own), and a fourth call of layer 0 that reads the first call's cache.
class ToyConfig : public ModelConfig {
public:
    long long hidden = 32, vocab = 64;
    static std::unique_ptr<ModelConfig> read(const Json& d) {
        std::unique_ptr<ToyConfig> c(new ToyConfig());
        c->hidden = take_int(d, "hidden_size");
        c->vocab = take_int(d, "vocab_size");
        return std::unique_ptr<ModelConfig>(c.release());
    }
    Json to_json() const override {
        Json d = Json::object();
        Json a = Json::array();
        a.push("ToyForCausalLM");
        d.set("architectures", a);
        d.set("hidden_size", hidden);
        d.set("vocab_size", vocab);
        return d;
    }
    ModelSpec build_spec() const override {
        auto names = [](std::initializer_list<std::pair<const char*, std::string>> l) {
            Json n = Json::object();
            for (const auto& kv : l) n.set(kv.first, kv.second);
            return n;
        };
        auto norm = [&](const std::string& w) {
            Json p = Json::object();
            p.set("size", hidden); p.set("eps", 1e-5); p.set("names", names({{"weight", w}}));
            return PartSpec("rmsnorm", p);
        };
        Json pos = Json::object();
        pos.set("theta", 1e4); pos.set("n_rot", 16); pos.set("factor", 4.0); pos.set("max_position", 128);
        Json att = Json::object();
        att.set("hidden_size", hidden); att.set("num_heads", 4); att.set("num_kv_heads", 2); att.set("head_dim", 16);
        att.set("qk_norm_eps", 1e-5); att.set("bias", false); att.set("window", Json());
        att.set("position", PartSpec("toy_scaled_rope", pos).to_json());
        att.set("names", names({{"q_proj", "l0.q_proj"}, {"k_proj", "l0.k_proj"}, {"v_proj", "l0.v_proj"}, {"o_proj", "l0.o_proj"},
                                {"q_norm", "l0.q_norm"}, {"k_norm", "l0.k_norm"}}));
        Json routed = Json::object();
        routed.set("hidden_size", hidden); routed.set("experts", 3);
        Json mean = Json::object();
        mean.set("hidden_size", hidden); mean.set("names", names({{"weight", "l1.mean"}}));
        Json glu = Json::object();
        glu.set("hidden_size", hidden); glu.set("intermediate_size", 48);
        glu.set("names", names({{"gate_proj", "l1.g"}, {"up_proj", "l1.u"}, {"down_proj", "l1.d"}}));
        ModelSpec spec;
        spec.hidden_size = hidden; spec.vocab_size = vocab; spec.max_position = 128;
        LayerSpec l0;
        l0.arrangement = "pre_norm";
        l0.parts = {{"mixer_norm", norm("l0.n1")}, {"mixer", PartSpec("attention", att)}, {"feed_forward_norm", norm("l0.n2")},
                    {"feed_forward", PartSpec("toy_top1", routed)}};
        LayerSpec l1;
        l1.arrangement = "toy_sandwich";
        l1.parts = {{"mixer_norm", norm("l1.n1")}, {"mixer", PartSpec("toy_running_mean", mean)}, {"mixer_post_norm", norm("l1.post")},
                    {"feed_forward_norm", norm("l1.n2")}, {"feed_forward", PartSpec("swiglu", glu)}};
        spec.layers = {l0, l1};
        spec.schedule = {{0, -1}, {1, -1}, {0, -1}, {0, 0}};
        Json emb = Json::object();
        emb.set("vocab_size", vocab); emb.set("hidden_size", hidden); emb.set("names", names({{"weight", "emb"}}));
        spec.embedding = PartSpec("embedding", emb);
        Json head = Json::object();
        head.set("hidden_size", hidden); head.set("vocab_size", vocab); head.set("tied_to", "emb");
        spec.head = PartSpec("lm_head", head);
        spec.final_norm = norm("final");
        return spec;
    }
};

}  // namespace

extern "C" __attribute__((visibility("default"))) int qe_plugin_init(void) {
    try {
        register_part("mixer", "toy_running_mean", [](const Json& p, BuildContext& b) { return std::make_shared<RunningMeanMixer>(p, b); });
        register_part("mixer", "toy_narrow_value_attention", [](const Json& p, BuildContext& b) { return std::make_shared<NarrowValueAttention>(p, b); });
        register_part("position", "toy_scaled_rope", [](const Json& p, BuildContext& b) { return std::make_shared<ScaledRotary>(p, b); });
        register_part("feed_forward", "toy_top1", [](const Json& p, BuildContext& b) { return std::make_shared<Top1Routed>(p, b); });
        register_arrangement("toy_sandwich", [](const LayerSpec& l, BuildContext& b) { return std::unique_ptr<Arrangement>(new SandwichBlock(l, b)); });
        register_architecture("ToyForCausalLM", ToyConfig::read);
        return 0;
    } catch (...) {
        return 1;
    }
}

extern "C" __attribute__((visibility("default"))) int qe_plugin_exit(void) {
    unregister_part("mixer", "toy_running_mean");
    unregister_part("mixer", "toy_narrow_value_attention");
    unregister_part("position", "toy_scaled_rope");
    unregister_part("feed_forward", "toy_top1");
    unregister_arrangement("toy_sandwich");
    unregister_architecture("ToyForCausalLM");
    return 0;
}
