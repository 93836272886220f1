// Entry points for tests that run ONE part alone on the device: build it from {kind, params} through the
// registries, bind it to a folder of tensors or to seeded random values, and call its forward on inputs from the
// host.  A mixer gets a cache manager of its own (one run-order entry), and its steps are laid out by the very
// functions the engine uses (lay_out_step, context_from_layout), so what it sees is what it sees in a model.
#include <algorithm>

#include "capi_internal.h"

using namespace qe;
using namespace qe::capi;

namespace {
thread_local std::string g_text;
template <typename F> const char* guarded_text(F&& body) {
    const char* out = nullptr;
    guarded([&] {
        g_text = body();
        out = g_text.c_str();
        return 0;
    });
    return out;
}

struct PartProbe {
    std::string family;
    DType dtype = DType::F32;
    std::unique_ptr<BuildContext> build;
    std::shared_ptr<Part> part;
    DeviceArena arena;
    Workspace ws;
    cudaStream_t stream = nullptr;
    DeviceBuffer errors;
    std::unique_ptr<CacheManager> cache;      // mixers
    PinnedBuffer pinned;
    ~PartProbe() {
        if (stream) { cudaStreamSynchronize(stream); cudaStreamDestroy(stream); }
    }
};

// host float32 -> a device tensor of `dtype` (float32 or bfloat16) in the probe's workspace
Tensor upload(PartProbe& p, const std::string& name, const float* host, std::vector<int64_t> shape, DType dtype) {
    Tensor t = p.ws.get(name, shape, dtype);
    const size_t n = (size_t)t.numel();
    if (dtype == DType::F32) {
        QE_CUDA(cudaMemcpyAsync(t.data, host, n * 4, cudaMemcpyHostToDevice, p.stream));
    } else {
        std::vector<uint16_t> h(n);
        for (size_t i = 0; i < n; i++) h[i] = f32_to_bf16(host[i]);
        QE_CUDA(cudaMemcpyAsync(t.data, h.data(), n * 2, cudaMemcpyHostToDevice, p.stream));
        QE_CUDA(cudaStreamSynchronize(p.stream));
    }
    return t;
}
// a device tensor -> host float32, summing `splits` stacked copies (split-K partial sums)
void download(PartProbe& p, const Tensor& t, int splits, float* host) {
    QE_CUDA(cudaStreamSynchronize(p.stream));
    const size_t n = (size_t)t.numel(), each = n / (size_t)std::max(splits, 1);
    std::vector<uint8_t> raw(t.bytes());
    QE_CUDA(cudaMemcpy(raw.data(), t.data, raw.size(), cudaMemcpyDeviceToHost));
    std::vector<double> acc(each, 0.0);
    for (size_t i = 0; i < n; i++) {
        float v;
        if (t.dtype == DType::F32) memcpy(&v, raw.data() + 4 * i, 4);
        else { uint16_t h; memcpy(&h, raw.data() + 2 * i, 2); v = bf16_to_f32(h); }
        acc[i % each] += v;
    }
    for (size_t i = 0; i < each; i++) host[i] = (float)acc[i];
}
void fill_context(PartProbe& p, StepContext& ctx) {
    ctx.workspace = &p.ws;
    ctx.compute_dtype = p.dtype;
    ctx.stream = p.stream;
    ctx.gemm_error = static_cast<int*>(p.errors.data());
    ctx.attention_error = static_cast<int*>(p.errors.data()) + 1;
}
void check_errors(PartProbe& p) {
    int words[2] = {0, 0};
    QE_CUDA(cudaStreamSynchronize(p.stream));
    QE_CUDA(cudaMemcpy(words, p.errors.data(), 8, cudaMemcpyDeviceToHost));
    if (words[0] || words[1]) throw KernelError("a kernel gave up on a wait (status " + std::to_string(words[0] ? words[0] : words[1]) + ")");
}
// a context of T rows in one segment and no cache, for parts that only look at rows
void rows_context(PartProbe& p, int T, StepContext& ctx) {
    ctx.T = T; ctx.S = 1;
    ctx.q_lens = {T}; ctx.ctx_lens = {T}; ctx.slots = {0};
    ctx.decode_only = false;
    fill_context(p, ctx);
}
#define PROBE(h) (*static_cast<PartProbe*>(h))
}  // namespace

// family: norm, position, mixer, feed_forward, embedding, head.  spec_json: {"kind", "params"}.
API void* qe_part_create(const char* family, const char* spec_json, const char* dtype, const char* options_json) {
    void* h = nullptr;
    guarded([&] {
        register_builtin_parts();
        std::unique_ptr<PartProbe> p(new PartProbe());
        p->family = family;
        p->dtype = parse_compute_dtype(dtype);
        p->build.reset(new BuildContext(p->dtype, options_json && *options_json ? Json::parse(options_json) : Json::object()));
        p->part = make_part(family, PartSpec::from_json(Json::parse(spec_json)), *p->build);
        h = p.release();
        return 0;
    });
    return h;
}
API void qe_part_free(void* h) { delete static_cast<PartProbe*>(h); }

API const char* qe_part_tensor_specs(void* h) {
    return guarded_text([&] {
        Json a = Json::array();
        std::function<void(Part*)> visit = [&](Part* part) {
            for (const TensorSpec& s : part->tensor_specs()) {
                Json e = Json::object();
                e.set("name", s.name);
                Json shape = Json::array();
                for (auto d : s.shape) shape.push((long long)d);
                e.set("shape", shape);
                e.set("role", role_name(s.role));
                e.set("init", s.init == Init::Scale ? "scale" : "normal");
                a.push(e);
            }
            for (Part* c : part->children()) visit(c);
        };
        visit(PROBE(h).part.get());
        return a.dump();
    });
}

static void start_device(PartProbe& p) {
    if (p.stream) return;
    QE_CUDA(cudaStreamCreateWithFlags(&p.stream, cudaStreamNonBlocking));
    p.ws.stream = p.stream;
    p.errors = DeviceBuffer(16);
    QE_CUDA(cudaMemset(p.errors.data(), 0, 16));
}
static std::vector<TensorSpec> all_specs(Part* part) {
    std::vector<TensorSpec> out = part->tensor_specs();
    for (Part* c : part->children())
        for (const TensorSpec& s : all_specs(c)) out.push_back(s);
    return out;
}

// Bind to the tensors of a folder (model.safetensors holding at least the part's tensors; others are ignored).
API int qe_part_bind_folder(void* h, const char* model_dir) {
    return guarded([&] {
        PartProbe& p = PROBE(h);
        start_device(p);
        std::vector<TensorSpec> specs = all_specs(p.part.get());
        SafetensorsFolder probe(model_dir);
        std::vector<std::string> ignore;
        for (const std::string& n : probe.names()) ignore.push_back(n);
        FolderSource src(model_dir, specs, ignore, p.dtype, p.arena, p.stream);
        p.part->bind(src);
        QE_CUDA(cudaStreamSynchronize(p.stream));
        return 0;
    });
}
API int qe_part_bind_random(void* h, uint64_t seed, double std_, double lo, double hi) {
    return guarded([&] {
        PartProbe& p = PROBE(h);
        start_device(p);
        RandomInit init;
        init.seed = seed; init.std = std_; init.scale_low = lo; init.scale_high = hi;
        RandomSource src(all_specs(p.part.get()), init, p.dtype, p.dtype, p.arena, p.stream);
        p.part->bind(src);
        QE_CUDA(cudaStreamSynchronize(p.stream));
        return 0;
    });
}

API const char* qe_part_cache_need(void* h) {
    return guarded_text([&] {
        auto* mixer = dynamic_cast<Mixer*>(PROBE(h).part.get());
        if (!mixer) throw Error(kInvalidArg, "only a mixer has a cache need");
        CacheNeed n = mixer->cache_need();
        Json j = Json::object();
        j.set("kind", n.kind == CacheNeed::Pages ? "pages" : n.kind == CacheNeed::State ? "state" : "none");
        j.set("kv_heads", n.kv_heads);
        j.set("head_dim", n.head_dim);
        if (n.kind == CacheNeed::Pages && n.value_dim) j.set("value_dim", n.value_dim);
        j.set("window", n.window ? Json(n.window) : Json());
        Json shape = Json::array();
        for (auto d : n.state_shape) shape.push((long long)d);
        j.set("state_shape", shape);
        return j.dump();
    });
}

// Norm: the stream holds x [T, E]; `add` (optional) is its pending addend.  out_x: the stream afterwards (x + add),
// out_y: the normed rows as float32.
API int qe_part_norm(void* h, const float* x, const float* add, int T, int E, float* out_x, float* out_y) {
    return guarded([&] {
        PartProbe& p = PROBE(h);
        auto* norm = dynamic_cast<Norm*>(p.part.get());
        if (!norm) throw Error(kInvalidArg, "not a norm");
        StepContext ctx;
        rows_context(p, T, ctx);
        ResidualStream stream;
        stream.x = upload(p, "probe_x", x, {T, E}, DType::F32);
        if (add) stream.add(Addend(upload(p, "probe_add", add, {T, E}, DType::F32), 1));
        Tensor y = norm->forward(stream, ctx);
        if (stream.has_pending) throw Error(kInvalidState, "the norm left the pending addend in the stream");
        download(p, stream.x, 1, out_x);
        download(p, y, 1, out_y);
        return 0;
    });
}

// Position encoding: n_rot, pairing, column and the rotation table's shape; the table itself with qe_part_position_table.
API const char* qe_part_position_info(void* h) {
    return guarded_text([&] {
        auto* pos = dynamic_cast<PositionEncoding*>(PROBE(h).part.get());
        if (!pos) throw Error(kInvalidArg, "not a position encoding");
        Tensor t = pos->rotation_table();
        Json j = Json::object();
        j.set("n_rot", pos->n_rot());
        j.set("interleaved", pos->interleaved());
        j.set("position_column", pos->position_column());
        j.set("rows", t.defined() ? (long long)t.shape[0] : 0LL);
        j.set("width", t.defined() ? (long long)t.shape[1] : 0LL);
        return j.dump();
    });
}
API int qe_part_position_table(void* h, float* out, long long capacity) {
    return guarded([&] {
        PartProbe& p = PROBE(h);
        auto* pos = dynamic_cast<PositionEncoding*>(p.part.get());
        if (!pos) throw Error(kInvalidArg, "not a position encoding");
        Tensor t = pos->rotation_table();
        if (!t.defined() || t.numel() > capacity) throw Error(kInvalidArg, "no table, or the buffer is too small");
        QE_CUDA(cudaMemcpy(out, t.data, t.bytes(), cudaMemcpyDeviceToHost));
        return 0;
    });
}

API int qe_part_embedding(void* h, const int32_t* ids, int T, int E, float* out) {
    return guarded([&] {
        PartProbe& p = PROBE(h);
        auto* emb = dynamic_cast<Embedding*>(p.part.get());
        if (!emb) throw Error(kInvalidArg, "not an embedding");
        StepContext ctx;
        rows_context(p, T, ctx);
        Tensor dev = p.ws.get("probe_ids", {T}, DType::I32);
        QE_CUDA(cudaMemcpyAsync(dev.data, ids, (size_t)T * 4, cudaMemcpyHostToDevice, p.stream));
        ctx.token_ids = dev.as<int32_t>();
        Tensor x = emb->forward(ctx);
        if (x.shape[1] != E) throw Error(kInvalidArg, "the embedding's width is " + std::to_string(x.shape[1]));
        download(p, x, 1, out);
        return 0;
    });
}

API int qe_part_head(void* h, const float* xn, int T, int E, float* out) {
    return guarded([&] {
        PartProbe& p = PROBE(h);
        auto* head = dynamic_cast<Head*>(p.part.get());
        if (!head) throw Error(kInvalidArg, "not a head");
        StepContext ctx;
        rows_context(p, T, ctx);
        Tensor x = upload(p, "probe_x", xn, {T, E}, p.dtype);
        Tensor logits = head->forward(x, ctx, T);
        download(p, logits, 1, out);
        check_errors(p);
        return 0;
    });
}

// Feed-forward: x [T, E] (rounded to the compute dtype) -> the addend, partial sums added up, as float32 [T, E].
API int qe_part_feed_forward(void* h, const float* x, int T, int E, float* out) {
    return guarded([&] {
        PartProbe& p = PROBE(h);
        auto* ff = dynamic_cast<FeedForward*>(p.part.get());
        if (!ff) throw Error(kInvalidArg, "not a feed-forward");
        StepContext ctx;
        rows_context(p, T, ctx);
        Tensor xin = upload(p, "probe_x", x, {T, E}, p.dtype);
        Addend y = ff->forward(xin, ctx);
        if (!y.tensor.defined()) throw Error(kInvalidState, "the part added into a residual that was not there");
        download(p, y.tensor, y.splits, out);
        check_errors(p);
        return 0;
    });
}

// Mixer: a cache of its own first, then steps.
API int qe_part_mixer_cache(void* h, int page_size, int num_pages, int max_requests, int poison) {
    return guarded([&] {
        PartProbe& p = PROBE(h);
        auto* mixer = dynamic_cast<Mixer*>(p.part.get());
        if (!mixer) throw Error(kInvalidArg, "not a mixer");
        start_device(p);
        p.cache.reset(new CacheManager({mixer->cache_need()}, page_size, {num_pages}, max_requests));
        p.cache->materialize(p.dtype, poison != 0, p.stream);
        return 0;
    });
}
API int qe_part_mixer_add_request(void* h, long long id) { return guarded([&] { PROBE(h).cache->add_request(id); return 0; }); }
API int qe_part_mixer_release(void* h, long long id) { return guarded([&] { PROBE(h).cache->release(id); return 0; }); }
// One step: segment s brings n_new[s] new rows of request requests[s]; x holds all rows [T, E] in segment order.
// out: the mixer's addend, partial sums added up, float32 [T, E].
API int qe_part_mixer_step(void* h, const long long* requests, const int* n_new, int n_segments, const float* x, int E, float* out) {
    return guarded([&] {
        PartProbe& p = PROBE(h);
        auto* mixer = dynamic_cast<Mixer*>(p.part.get());
        if (!mixer || !p.cache) throw Error(kInvalidState, "qe_part_mixer_cache first");
        std::vector<StepEntry> entries((size_t)n_segments);
        int T = 0, longest = 1;
        for (int s = 0; s < n_segments; s++) T += n_new[s];
        std::vector<int32_t> zeros((size_t)T, 0);
        for (int s = 0, at = 0; s < n_segments; s++) {
            entries[s].request = requests[s];
            entries[s].tokens = zeros.data() + at;
            entries[s].n_tokens = n_new[s];
            at += n_new[s];
            longest = std::max(longest, (p.cache->length(requests[s]) + n_new[s] + p.cache->page_size() - 1) / p.cache->page_size());
        }
        int width = 8;
        while (width < longest) width *= 2;
        StepLayout lay;
        lay_out_step(*p.cache, 1, entries, width, false, [&](StepPlan& plan) { mixer->prepare_step(plan); }, lay);
        try {
            Tensor meta = p.ws.get("probe_meta", {(int64_t)lay.flat.size()}, DType::I32);
            p.pinned.ensure(lay.flat.size() * 4);
            QE_CUDA(cudaStreamSynchronize(p.stream));
            memcpy(p.pinned.data(), lay.flat.data(), lay.flat.size() * 4);
            QE_CUDA(cudaMemcpyAsync(meta.data, p.pinned.data(), lay.flat.size() * 4, cudaMemcpyHostToDevice, p.stream));
            StepContext ctx;
            const int32_t* want = nullptr;
            context_from_layout(lay, *p.cache, 1, meta.as<int32_t>(), ctx, &want);
            fill_context(p, ctx);
            Tensor xin = upload(p, "probe_x", x, {T, E}, p.dtype);
            CacheView view = p.cache->view(0, 0);
            Addend y = mixer->forward(xin, ctx, view);
            if (!y.tensor.defined()) throw Error(kInvalidState, "the part added into a residual that was not there");
            download(p, y.tensor, y.splits, out);
            check_errors(p);
        } catch (...) {
            for (const StepEntry& e : entries) p.cache->unreserve(e.request);
            throw;
        }
        for (const StepEntry& e : entries) p.cache->advance(e.request, e.n_tokens);
        return 0;
    });
}
