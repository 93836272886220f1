// Entry points for tests and tools: the pieces of the host library that the C API of inference.h does not show
// on their own (configuration reading, the weight check, the cache manager's bookkeeping, the scheduler's
// decisions with a stand-in runner, a look inside a live engine).  Answers that are more than a number come as
// JSON text in a per-thread buffer that the next call on the thread overwrites.  None of these needs a device
// unless it says so.
#include <algorithm>

#include "../parts/linear.h"
#include "capi_internal.h"

using namespace qe;
using namespace qe::capi;

namespace {
thread_local std::string g_text;
const char* text(const std::string& s) {
    g_text = s;
    return g_text.c_str();
}
template <typename F> const char* guarded_text(F&& body) {
    const char* out = nullptr;
    guarded([&] {
        out = text(body());
        return 0;
    });
    return out;
}
Json ints(const std::vector<int>& v) {
    Json a = Json::array();
    for (int x : v) a.push(x);
    return a;
}
Json spec_json(const ModelSpec& spec) {
    Json j = Json::object();
    j.set("hidden_size", (long long)spec.hidden_size);
    j.set("vocab_size", (long long)spec.vocab_size);
    j.set("max_position", (long long)spec.max_position);
    j.set("position_columns", spec.position_columns);
    j.set("embedding", spec.embedding.to_json());
    Json layers = Json::array();
    for (const LayerSpec& l : spec.layers) {
        Json lj = Json::object();
        lj.set("arrangement", l.arrangement);
        Json parts = Json::object();
        for (const auto& p : l.parts) parts.set(p.first, p.second.to_json());
        lj.set("parts", parts);
        layers.push(lj);
    }
    j.set("layers", layers);
    Json sched = Json::array();
    for (const LayerCall& c : spec.schedule) {
        Json cj = Json::object();
        cj.set("layer", c.layer);
        cj.set("cache_from", c.cache_from >= 0 ? Json(c.cache_from) : Json());
        sched.push(cj);
    }
    j.set("schedule", sched);
    j.set("final_norm", spec.final_norm.to_json());
    j.set("head", spec.head.to_json());
    return j;
}
Json tensor_specs_json(const std::vector<TensorSpec>& specs) {
    Json a = Json::array();
    for (const TensorSpec& s : specs) {
        Json e = Json::object();
        e.set("name", s.name);
        Json shape = Json::array();
        for (auto d : s.shape) shape.push((long long)d);
        e.set("shape", shape);
        e.set("role", role_name(s.role));
        e.set("init", s.init == Init::Scale ? "scale" : "normal");
        a.push(e);
    }
    return a;
}
}  // namespace

// ---- configuration ---------------------------------------------------------------------------------------------------
// The typed configuration read from config.json text, written back as JSON (every default filled in), with
// "parameter_count" added for architectures that can tell.  NULL on error (inference_get_last_error).
API const char* qe_config_read(const char* config_json) {
    return guarded_text([&] {
        std::unique_ptr<ModelConfig> c = config_from_json(Json::parse(config_json));
        Json j = c->to_json();
        if (auto* q = dynamic_cast<Qwen3Config*>(c.get())) {
            j.set("parameter_count", q->parameter_count());
            Json lt = Json::array();
            for (const auto& t : q->layer_types) lt.push(t);
            j.set("layer_types", lt);
            j.set("sliding_window", q->sliding_window ? Json(q->sliding_window) : Json());
        }
        return j.dump();
    });
}
API const char* qe_config_load(const char* model_dir) {
    return guarded_text([&] { return load_config(model_dir)->to_json().dump(); });
}
API const char* qe_registered_architectures(void) {
    return guarded_text([&] {
        register_builtin_architectures();
        Json a = Json::array();
        for (const auto& n : registered_architectures()) a.push(n);
        return a.dump();
    });
}
API const char* qe_registered_parts(const char* family) {
    return guarded_text([&] {
        register_builtin_parts();
        Json a = Json::array();
        for (const auto& n : registered_parts(family)) a.push(n);
        return a.dump();
    });
}
API const char* qe_model_spec(const char* config_json) {
    return guarded_text([&] { return spec_json(config_from_json(Json::parse(config_json))->build_spec()).dump(); });
}
API const char* qe_expected_tensors(const char* config_json) {
    return guarded_text([&] { return tensor_specs_json(expected_tensors(*config_from_json(Json::parse(config_json)))).dump(); });
}

// ---- weights ---------------------------------------------------------------------------------------------------------
// Check a folder against its own config.json without copying anything.  0, or an error whose details
// qe_weight_error_details gives as {"missing": [...], "unexpected": [...], "wrong_shape": [...], "wrong_type": [...]}.
namespace { thread_local std::string g_weight_details = "{}"; }
API int qe_check_model_folder(const char* model_dir) {
    g_weight_details = "{}";
    return guarded([&] {
        std::unique_ptr<ModelConfig> config = load_config(model_dir);
        DecoderModel model(config->build_spec(), DType::F32);
        SafetensorsFolder folder(model_dir);
        try {
            check_folder(folder, model.tensor_specs(), model.ignored_tensors());
        } catch (const WeightError& e) {
            Json d = Json::object();
            auto list = [](const std::vector<std::string>& v) { Json a = Json::array(); for (const auto& s : v) a.push(s); return a; };
            d.set("missing", list(e.missing));
            d.set("unexpected", list(e.unexpected));
            d.set("wrong_shape", list(e.wrong_shape));
            d.set("wrong_type", list(e.wrong_type));
            g_weight_details = d.dump();
            throw;
        }
        return 0;
    });
}
API const char* qe_weight_error_details(void) { return g_weight_details.c_str(); }
// The tensors of a folder as [{"name", "dtype", "shape", "bytes"}], in file order.
API const char* qe_safetensors_list(const char* model_dir) {
    return guarded_text([&] {
        SafetensorsFolder folder(model_dir);
        Json a = Json::array();
        for (const std::string& n : folder.names()) {
            const TensorEntry& e = folder.at(n);
            Json j = Json::object();
            j.set("name", n);
            j.set("dtype", e.dtype_name);
            Json shape = Json::array();
            for (auto d : e.shape) shape.push((long long)d);
            j.set("shape", shape);
            j.set("bytes", (long long)e.bytes);
            a.push(j);
        }
        return a.dump();
    });
}
// Copy one tensor's bytes out of a folder (as stored).  Returns the byte count, negative on error.
API long long qe_safetensors_read(const char* model_dir, const char* name, void* dst, long long capacity) {
    long long n = -1;
    int rc = guarded([&] {
        SafetensorsFolder folder(model_dir);
        const TensorEntry& e = folder.at(name);
        if ((long long)e.bytes > capacity) throw Error(kInvalidArg, "the buffer is too small");
        memcpy(dst, e.data, e.bytes);
        n = (long long)e.bytes;
        return 0;
    });
    return rc < 0 ? rc : n;
}
// What dtype a stored tensor gets on the device: names as in common.h ("bfloat16", "float32", "int32").
API const char* qe_device_dtype(const char* stored, const char* role, const char* compute) {
    return guarded_text([&] {
        bool ok = false;
        std::string st = stored;
        DType s = st == "float32" ? DType::F32 : st == "float64" ? DType::F64 : st == "float16" ? DType::F16 : st == "bfloat16" ? DType::BF16
                : st == "int64" ? DType::I64 : st == "int32" ? DType::I32 : (ok = true, DType::U8);
        (void)ok;
        std::string r = role;
        Role ro = r == "matrix" ? Role::Matrix : r == "vector" ? Role::Vector : Role::Table;
        return std::string(dtype_name(device_dtype(s, ro, parse_compute_dtype(compute))));
    });
}
// One tensor of a random model as float32 values on the host (n floats into dst).
API int qe_random_tensor(const char* name, const char* init, long long n, uint64_t seed, double std_, double lo, double hi, float* dst) {
    return guarded([&] {
        TensorSpec spec;
        spec.name = name;
        spec.shape = {n};
        spec.init = std::string(init) == "scale" ? Init::Scale : Init::Normal;
        RandomInit ri;
        ri.seed = seed; ri.std = std_; ri.scale_low = lo; ri.scale_high = hi;
        std::vector<float> v = random_tensor_host(spec, ri);
        memcpy(dst, v.data(), v.size() * 4);
        return 0;
    });
}

// ---- samplers ----------------------------------------------------------------------------------------------------------
// Which device kernel gives what this sampler gives on the host: "greedy", "temperature", "chain", or "" (none).
API const char* qe_sampler_device_mode(sampler_t* s) {
    switch (s->s.device_mode()) {
        case Sampler::DeviceMode::Greedy: return "greedy";
        case Sampler::DeviceMode::Temperature: return "temperature";
        case Sampler::DeviceMode::Chain: return "chain";
        default: return "";
    }
}
API int qe_sampler_chain_max_k(void) { return Sampler::kChainMaxK; }
// The sampler's next uniform number, and the 24-byte record the device's chain kernel takes for its next token
// (either one draws from the generator, as sampling a token does).
API double qe_sampler_uniform(sampler_t* s) { return s->s.uniform(); }
API void qe_sampler_chain_record(sampler_t* s, void* out24) {
    ChainRecord r = s->s.chain_record();
    memcpy(out24, &r, sizeof r);
}
// The shape the engine picks for the tcgen05 product of M tokens with an [N, K] weight:
// {"swapped", "block_n", "splits", "pair"}.
API const char* qe_plan_gemm(int M, int N, int K, int sms, int allow_split, int fused_epilogue) {
    return guarded_text([&] {
        GemmPlan p = plan_gemm(M, N, K, sms, allow_split != 0, fused_epilogue != 0);
        Json j = Json::object();
        j.set("swapped", p.swapped);
        j.set("block_n", p.block_n);
        j.set("splits", p.splits);
        j.set("pair", p.pair);
        return j.dump();
    });
}
// `draws` tokens sampled from one row of logits (none accepted); counts[token] is incremented for each.
API int qe_sampler_histogram(sampler_t* s, const float* logits, int n_vocab, long long draws, long long* counts) {
    return guarded([&] {
        for (long long i = 0; i < draws; i++) counts[s->s.sample(logits, n_vocab)]++;
        return 0;
    });
}

// The kernel libraries a loaded model launches from, as a JSON list ("core", "flash", "gemm100"): a binding that
// compiles libraries by need builds these before inference_kv_cache_init.
API const char* qe_model_required_libraries(inference_model_t* m) {
    return guarded_text([&] {
        if (!m) throw Error(kInvalidArg, "no model");
        Json a = Json::array();
        for (const auto& l : m->decoder->required_libraries()) a.push(l);
        return a.dump();
    });
}
// ---- a look inside a live engine (needs a device) -----------------------------------------------------------------------
API const char* qe_engine_info(inference_model_t* m) {
    return guarded_text([&] {
        Engine& eng = need_engine(m);
        const CacheManager& c = eng.cache();
        Json j = Json::object();
        j.set("free_pages", ints(c.free_pages()));
        j.set("total_pages", ints(c.total_pages()));
        Json groups = Json::array();
        for (const PageGroup& g : c.groups()) {
            Json gj = Json::object();
            gj.set("entries", ints(g.entries));
            gj.set("kv_heads", g.kv_heads);
            gj.set("head_dim", g.head_dim);
            gj.set("window", g.window ? Json(g.window) : Json());
            groups.push(gj);
        }
        j.set("groups", groups);
        Json needs = Json::array();
        for (const CacheNeed& n : c.needs()) needs.push(n.kind == CacheNeed::Pages ? "pages" : n.kind == CacheNeed::State ? "state" : "none");
        j.set("needs", needs);
        j.set("state_entries", ints(c.state_entries()));
        Json views = Json::array();
        for (const CacheView& v : eng.views()) {
            Json vj = Json::object();
            vj.set("writable", v.writable);
            vj.set("k_base", (long long)(uintptr_t)v.k_base);
            vj.set("group", v.group);
            views.push(vj);
        }
        j.set("views", views);
        j.set("graphs", (long long)eng.graphs());
        j.set("graph_replays", eng.graph_replays());
        j.set("launches", g_launches);
        j.set("pool_bytes", (long long)c.pool_bytes());
        j.set("weight_bytes", (long long)eng.model().weight_bytes());
        j.set("row_multiple", eng.row_multiple());
        j.set("upload_bytes", (long long)eng.last_upload_bytes());
        j.set("free_slots", c.slots().num_free());
        j.set("scheduler_steps", m->scheduler->steps);
        j.set("preemptions", m->scheduler->preemptions);
        return j.dump();
    });
}
API int qe_engine_cache_check(inference_model_t* m) {
    return guarded([&] {
        need_engine(m).cache().check();
        return 0;
    });
}
// Make the next kernel-error check fire as if a kernel had given up on a wait (which: 0 products, 1 attention).
API int qe_engine_set_error_word(inference_model_t* m, int which, int code) {
    return guarded([&] {
        need_engine(m).inject_error_word(which, code);
        return 0;
    });
}
// ---- timing on the device, for the benchmark ---------------------------------------------------------------------------
// `warmup + steps` decode steps of n requests (live, each with its prefix in the cache): step k feeds request i the
// token tokens[i * (warmup + steps) + k] from the host, and, with `sample`, every step's logits go through the greedy
// sampling kernel with the ids copied to the host, nobody waiting for them.  The last `steps` steps are bracketed
// by CUDA events on the engine's stream; *ms_per_step is their mean, *launches the launcher calls they made.
API int qe_time_decode_steps(inference_model_t* m, const long long* requests, int n, const int32_t* tokens, int warmup, int steps,
                             int sample, double* ms_per_step, long long* launches) {
    return guarded([&] {
        Engine& eng = need_engine(m);
        const int total = warmup + steps;
        std::vector<Sampler> greedy((size_t)n, Sampler(SamplerParams::greedy()));
        std::vector<Sampler*> samplers;
        for (Sampler& s : greedy) samplers.push_back(&s);
        static const int32_t kFirst[1] = {0};
        cudaEvent_t t0, t1;
        QE_CUDA(cudaEventCreate(&t0));
        QE_CUDA(cudaEventCreate(&t1));
        long long before = 0;
        for (int k = 0; k < total; k++) {
            if (k == warmup) {
                QE_CUDA(cudaStreamSynchronize(eng.stream()));
                before = g_launches;
                QE_CUDA(cudaEventRecord(t0, eng.stream()));
            }
            std::vector<StepEntry> entries((size_t)n);
            for (int i = 0; i < n; i++) {
                entries[i].request = requests[i];
                entries[i].tokens = tokens + (size_t)i * total + k;
                entries[i].n_tokens = 1;
                entries[i].want = kFirst;
                entries[i].n_want = 1;
            }
            Tensor logits = eng.step(entries);
            if (sample) eng.sample_async(logits, samplers);
        }
        QE_CUDA(cudaEventRecord(t1, eng.stream()));
        QE_CUDA(cudaEventSynchronize(t1));
        float ms = 0;
        QE_CUDA(cudaEventElapsedTime(&ms, t0, t1));
        cudaEventDestroy(t0);
        cudaEventDestroy(t1);
        eng.check_kernel_errors();
        if (ms_per_step) *ms_per_step = (double)ms / steps;
        if (launches) *launches = g_launches - before;
        return 0;
    });
}
// One batch through the step function, bracketed by CUDA events on the engine's stream (the logits stay on the
// device).  *ms: the device time of the step.
API int qe_time_step(inference_model_t* m, const engine_step_batch* batch, double* ms) {
    return guarded([&] {
        Engine& eng = need_engine(m);
        std::vector<StepEntry> entries((size_t)batch->n_entries);
        for (int i = 0; i < batch->n_entries; i++) {
            const engine_step_entry& e = batch->entries[i];
            entries[i].request = e.request;
            entries[i].tokens = e.tokens; entries[i].n_tokens = e.n_tokens;
            entries[i].want = e.want; entries[i].n_want = e.n_want;
        }
        cudaEvent_t t0, t1;
        QE_CUDA(cudaEventCreate(&t0));
        QE_CUDA(cudaEventCreate(&t1));
        QE_CUDA(cudaStreamSynchronize(eng.stream()));
        QE_CUDA(cudaEventRecord(t0, eng.stream()));
        eng.step(entries);
        QE_CUDA(cudaEventRecord(t1, eng.stream()));
        QE_CUDA(cudaEventSynchronize(t1));
        float f = 0;
        QE_CUDA(cudaEventElapsedTime(&f, t0, t1));
        cudaEventDestroy(t0);
        cudaEventDestroy(t1);
        eng.check_kernel_errors();
        if (ms) *ms = f;
        return 0;
    });
}

// Time per kernel class (see LaunchProfile in host/device.h): on with PURHIE_PROFILE=1 in the environment or with
// qe_profile_enable(1).  The report is {"launcher": {"calls", "ms", "bytes", "flops"}} since the last reset.
API void qe_profile_enable(int on) { LaunchProfile::get().set_enabled(on != 0); }
API int qe_profile_enabled(void) { return LaunchProfile::get().on() ? 1 : 0; }
// Timing by omission: the launchers named (comma separated; "" for none) are skipped from now on.  For finding what
// a kernel class costs inside a graph; the results of a step are meaningless while anything is left out.
API void qe_profile_leave_out(const char* names) { LaunchProfile::get().leave_out(names); }
API const char* qe_profile_report(int reset) {
    return guarded_text([&] { return LaunchProfile::get().report_json(reset != 0); });
}

API long long qe_launches(void) { return g_launches; }
API void qe_set_library_dir(const char* dir) { set_library_dir(dir ? dir : ""); }

// After every run-order entry of the following engine_step calls, `fn(user, entry, residual, rows, width)` is called
// with a host copy of the float32 residual stream (its pending addend folded in).  NULL turns it off.
typedef void (*qe_layer_dump_fn)(void* user, int entry, const float* residual, int rows, int width);
API int qe_engine_set_layer_dump(inference_model_t* m, qe_layer_dump_fn fn, void* user) {
    return guarded([&] {
        Engine& eng = need_engine(m);
        if (fn) eng.set_layer_dump([fn, user](int entry, const float* x, int T, int E) { fn(user, entry, x, T, E); });
        else eng.set_layer_dump(nullptr);
        return 0;
    });
}
