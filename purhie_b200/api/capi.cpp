// The C interface (api/inference.h) over the host library: handles, error codes, and the bookkeeping of
// sequences and streams.  All generation goes through the one Scheduler and the one Engine::step; this file
// only translates.  The shape follows the reference's C API (src/inference.h there: load :40, cache :115, prefill
// :183, decode :203, generate :223-275, sequences :284-287, streams :297-317, logits :459, errors :18-33, 479).
#include <fstream>
#include <sstream>

#include "capi_internal.h"

using namespace qe;
using namespace qe::capi;

namespace {
thread_local std::string g_last_error, g_last_kind;
}  // namespace

namespace qe {
namespace capi {
void set_last_error(const char* kind, const std::string& text) { g_last_error = text; g_last_kind = kind; }

SamplerParams to_params(const sampler_params& p) {
    SamplerParams s;
    s.temperature = p.temperature; s.top_k = p.top_k; s.top_p = p.top_p; s.min_p = p.min_p;
    s.repeat_penalty = p.repeat_penalty; s.repeat_last_n = p.repeat_last_n; s.seed = p.seed;
    s.presence_penalty = p.presence_penalty;
    return s;
}
}  // namespace capi
}  // namespace qe

namespace qe {
namespace capi {
Engine& need_engine(inference_model* m) {
    if (!m) throw Error(kInvalidArg, "no model");
    if (!m->engine) throw Error(kInvalidState, "inference_kv_cache_init has not been called");
    return *m->engine;
}

Sequence& sequence(inference_model* m, int idx) {
    need_engine(m);
    auto it = m->seqs.find(idx);
    if (it == m->seqs.end()) {
        if (idx != 0) throw Error(kInvalidArg, "no sequence " + std::to_string(idx));
        m->engine->add_request(0);              // sequence 0 comes into being with its first use
        Sequence& s = m->seqs[0];
        s.index = 0;
        return s;
    }
    return it->second;
}
Sequence& current(inference_model* m) { return sequence(m, m->current); }

void must_be_idle(const Sequence& s) {
    if (s.active) throw Error(kInvalidState, "sequence " + std::to_string(s.index) + " has a stream in progress");
}

// Bring the cache up to the sequence's tokens and, when `extra` is given, append and feed those too.  The logits
// of the last token are kept; with all_logits the logits after every one of the extra tokens go to the host.
void feed(inference_model* m, Sequence& s, const int32_t* extra, int n_extra, float* all_logits) {
    Engine& eng = need_engine(m);
    if ((long long)s.tokens.size() + n_extra > m->n_ctx)
        throw Error(kContextFull, std::to_string(s.tokens.size()) + " + " + std::to_string(n_extra) + " tokens do not fit a context of " +
                                      std::to_string(m->n_ctx));
    const size_t before = s.tokens.size();
    s.tokens.insert(s.tokens.end(), extra, extra + n_extra);
    const int64_t V = eng.vocab_size();
    try {
        std::vector<int32_t> want;
        while (eng.length(s.index) < (int)s.tokens.size()) {
            const int at = eng.length(s.index);
            const int n = std::min<int>(m->prefill_batch, (int)s.tokens.size() - at);
            const bool last = at + n == (int)s.tokens.size();
            want.clear();
            if (all_logits) {
                for (int i = 0; i < n; i++) if (at + i >= (int)before) want.push_back(i);
            } else if (last) {
                want.push_back(n - 1);
            }
            StepEntry e;
            e.request = s.index; e.tokens = s.tokens.data() + at; e.n_tokens = n;
            e.want = want.data(); e.n_want = (int)want.size();
            Tensor lg = eng.step({e});
            if (lg.defined()) {
                if (all_logits) {
                    const int first = std::max(at, (int)before) - (int)before;
                    eng.read_logits(lg, all_logits + (size_t)first * V);
                }
                if (last) {
                    if (!s.logits.data()) s.logits = DeviceBuffer((size_t)V * 4);
                    QE_CUDA(cudaMemcpyAsync(s.logits.data(), lg.as<float>() + (size_t)(lg.shape[0] - 1) * V, (size_t)V * 4,
                                            cudaMemcpyDeviceToDevice, eng.stream()));
                    s.logits_valid = true;
                }
            }
        }
    } catch (...) {
        // what was not fed is forgotten; the tokens never fall behind the cache
        s.tokens.resize(std::max<size_t>(before, (size_t)eng.length(s.index)));
        s.logits_valid = false;
        throw;
    }
}

}  // namespace capi
}  // namespace qe

namespace {
std::vector<int> read_eos_ids(const std::string& model_dir, const ModelConfig& config) {
    std::set<int> ids;
    std::ifstream f(model_dir + "/generation_config.json", std::ios::binary);
    if (f) {
        std::ostringstream ss;
        ss << f.rdbuf();
        try {
            Json g = Json::parse(ss.str());
            if (const Json* e = g.find("eos_token_id")) {
                if (e->is_int()) ids.insert((int)e->as_int());
                else if (e->is_array())
                    for (const Json& v : e->items()) if (v.is_int()) ids.insert((int)v.as_int());
            }
        } catch (const JsonError&) {
        }
    }
    if (ids.empty())
        for (int id : config.eos_token_ids()) ids.insert(id);
    return std::vector<int>(ids.begin(), ids.end());
}

std::string base_name(std::string path) {
    while (path.size() > 1 && path.back() == '/') path.pop_back();
    size_t slash = path.rfind('/');
    return slash == std::string::npos ? path : path.substr(slash + 1);
}
}  // namespace

// ---- errors ----------------------------------------------------------------------------------------------------------
API const char* inference_strerror(inference_error_t err) {
    switch (err) {
        case INFERENCE_OK: return "success";
        case INFERENCE_ERR_INVALID_ARG: return "invalid argument";
        case INFERENCE_ERR_OUT_OF_MEMORY: return "out of memory";
        case INFERENCE_ERR_MODEL_LOAD: return "model load failed";
        case INFERENCE_ERR_KV_CACHE: return "KV cache error";
        case INFERENCE_ERR_TOKENIZER: return "tokenizer error";
        case INFERENCE_ERR_KERNEL_LAUNCH: return "kernel launch failed";
        case INFERENCE_ERR_INVALID_STATE: return "invalid state";
        case INFERENCE_ERR_NOT_IMPLEMENTED: return "not implemented";
        case INFERENCE_ERR_CONTEXT_FULL: return "context full";
        case INFERENCE_ERR_CANCELLED: return "cancelled";
    }
    return "unknown error";
}
API const char* inference_get_last_error(void) { return g_last_error.c_str(); }
// The kind of the last error on this thread ("ConfigError", "WeightError", "OutOfPages", ...), for bindings that
// map errors to exception classes.
API const char* qe_last_error_kind(void) { return g_last_kind.c_str(); }

// ---- sampler -------------------------------------------------------------------------------------------------------------
API sampler_params sampler_default_params(void) {
    SamplerParams d;
    sampler_params p;
    p.temperature = d.temperature; p.top_k = d.top_k; p.top_p = d.top_p; p.min_p = d.min_p;
    p.repeat_penalty = d.repeat_penalty; p.repeat_last_n = d.repeat_last_n; p.seed = d.seed; p.presence_penalty = d.presence_penalty;
    return p;
}
API sampler_t* sampler_create(const sampler_params* params) {
    return new sampler(params ? to_params(*params) : SamplerParams());
}
API void sampler_free(sampler_t* s) { delete s; }
API int sampler_sample(sampler_t* s, const float* logits, int n_vocab) { return s->s.sample(logits, n_vocab); }
API void sampler_accept(sampler_t* s, int token) { s->s.accept(token); }
API void sampler_reset(sampler_t* s) { s->s.reset(); }

// ---- models ----------------------------------------------------------------------------------------------------------------
API inference_model_t* inference_load_model_ex(const char* model_dir, const char* dtype, const char* options_json) {
    inference_model_t* m = nullptr;
    int rc = guarded([&] {
        if (!model_dir) throw Error(kInvalidArg, "no model folder");
        std::unique_ptr<inference_model> fresh(new inference_model());
        fresh->dtype = parse_compute_dtype(dtype ? dtype : "bfloat16");
        Json options = options_json && *options_json ? Json::parse(options_json) : Json::object();
        fresh->decoder = load_model_folder(model_dir, fresh->dtype, options, &fresh->config);
        fresh->name = base_name(model_dir);
        fresh->eos_ids = read_eos_ids(model_dir, *fresh->config);
        m = fresh.release();
        return 0;
    });
    return rc == 0 ? m : nullptr;
}
API inference_model_t* inference_load_model(const char* model_dir) { return inference_load_model_ex(model_dir, "bfloat16", nullptr); }

API inference_model_t* inference_load_model_random_ex(const char* config_json, uint64_t seed, const char* dtype, double std_,
                                                      double scale_low, double scale_high, const char* options_json) {
    inference_model_t* m = nullptr;
    int rc = guarded([&] {
        if (!config_json) throw Error(kInvalidArg, "no configuration");
        std::unique_ptr<inference_model> fresh(new inference_model());
        fresh->dtype = parse_compute_dtype(dtype ? dtype : "bfloat16");
        Json options = options_json && *options_json ? Json::parse(options_json) : Json::object();
        Json cfg;
        try {
            cfg = Json::parse(config_json);
        } catch (const JsonError& e) {
            throw ConfigError(std::string("the configuration is not valid JSON (") + e.what() + ")");
        }
        fresh->config = config_from_json(cfg);
        RandomInit init;
        init.seed = seed; init.std = std_; init.scale_low = scale_low; init.scale_high = scale_high;
        fresh->decoder = load_model_random(*fresh->config, init, fresh->dtype, options);
        fresh->name = "random";
        fresh->eos_ids = fresh->config->eos_token_ids();
        m = fresh.release();
        return 0;
    });
    return rc == 0 ? m : nullptr;
}
API inference_model_t* inference_load_model_random(const char* config_json, uint64_t seed, const char* dtype) {
    return inference_load_model_random_ex(config_json, seed, dtype, 0.02, 1.0, 1.0, nullptr);
}

API int inference_write_random_model(const char* model_dir, const char* config_json, uint64_t seed, double std_, double scale_low,
                                     double scale_high, const char* stored_dtype) {
    return guarded([&] {
        if (!model_dir || !config_json) throw Error(kInvalidArg, "a folder and a configuration are needed");
        Json cfg;
        try {
            cfg = Json::parse(config_json);
        } catch (const JsonError& e) {
            throw ConfigError(std::string("the configuration is not valid JSON (") + e.what() + ")");
        }
        std::unique_ptr<ModelConfig> config = config_from_json(cfg);
        RandomInit init;
        init.seed = seed; init.std = std_; init.scale_low = scale_low; init.scale_high = scale_high;
        const std::string d = stored_dtype ? stored_dtype : "bfloat16";
        if (d != "bfloat16" && d != "float32") throw Error(kInvalidArg, "random models are stored as bfloat16 or float32");
        write_random_model(model_dir, *config, init, d == "bfloat16" ? DType::BF16 : DType::F32, DType::F32);
        return 0;
    });
}

API void inference_free_model(inference_model_t* model) {
    if (!model) return;
    inference_kv_cache_free(model);
    delete model;
}

// ---- the cache ---------------------------------------------------------------------------------------------------------------
API int inference_kv_cache_init_ex(inference_model_t* m, int n_ctx, int max_sequences, int page_size, long long kv_tokens,
                                   const char* engine_options_json) {
    return guarded([&] {
        if (!m) throw Error(kInvalidArg, "no model");
        if (n_ctx == 0) n_ctx = (int)m->decoder->spec().max_position;          // _ex only: as long as the model allows
        if (n_ctx < 1) throw Error(kInvalidArg, "n_ctx must be positive");
        if (n_ctx > m->decoder->spec().max_position)
            throw Error(kInvalidArg, "n_ctx " + std::to_string(n_ctx) + " exceeds the model's max_position_embeddings " +
                                         std::to_string(m->decoder->spec().max_position));
        if (max_sequences < 1 || page_size < 1) throw Error(kInvalidArg, "max_sequences and page_size must be positive");
        inference_kv_cache_free(m);
        Json o = engine_options_json && *engine_options_json ? Json::parse(engine_options_json) : Json::object();
        EngineOptions eo;
        eo.page_size = page_size;
        eo.max_requests = max_sequences;
        const long long per_seq = (n_ctx + page_size - 1) / page_size * (long long)page_size;
        eo.max_tokens = kv_tokens > 0 ? kv_tokens : per_seq * max_sequences;
        eo.poison_cache = o.get_bool("poison_cache", false);
        eo.cuda_graphs = o.get_bool("cuda_graphs", true);
        eo.max_graph_batch = (int)o.get_int("max_graph_batch", eo.max_graph_batch);
        eo.max_graphs = (int)o.get_int("max_graphs", eo.max_graphs);
        if (const Json* np = o.find("num_pages")) {
            if (np->is_array()) for (const Json& v : np->items()) eo.num_pages.push_back((int)v.as_int());
            else if (!np->is_null()) eo.num_pages.push_back((int)np->as_int());
        }
        if (const Json* st = o.find("step")) eo.step_options = *st;
        m->engine.reset(new Engine(m->decoder, eo));
        m->runner.reset(new EngineRunner(*m->engine));
        SchedulerOptions so;
        so.n_ctx = n_ctx;
        so.max_batch_tokens = (int)o.get_int("max_batch_tokens", so.max_batch_tokens);
        so.prefill_chunk = (int)o.get_int("prefill_chunk", so.prefill_chunk);
        so.run_ahead = o.get_bool("run_ahead", true);
        if (o.has("align_rows")) so.align_rows = (int)o.get_int("align_rows", -1);
        m->scheduler.reset(new Scheduler(*m->runner, so));
        m->n_ctx = n_ctx;
        m->max_sequences = max_sequences;
        m->current = 0;
        return 0;
    });
}
API int inference_kv_cache_init(inference_model_t* model, int n_ctx) {
    if (n_ctx < 1) { set_last_error("Error", "n_ctx must be positive"); return INFERENCE_ERR_INVALID_ARG; }
    return inference_kv_cache_init_ex(model, n_ctx, 4, 16, 0, nullptr);
}

API void inference_kv_cache_free(inference_model_t* m) {
    if (!m) return;
    m->queued.clear();
    m->done.clear();
    m->seqs.clear();
    m->scheduler.reset();
    m->runner.reset();
    m->engine.reset();
    m->n_ctx = 0;
}

API int inference_synchronize(inference_model_t* m) {
    return guarded([&] {
        need_engine(m).synchronize();
        return 0;
    });
}

API int inference_set_eog_tokens(inference_model_t* m, const int32_t* ids, int n) {
    return guarded([&] {
        if (!m || n < 0 || (n > 0 && !ids)) throw Error(kInvalidArg, "a model and n token ids are needed");
        m->eos_ids.assign(ids, ids + n);
        return 0;
    });
}

API void inference_set_seed(inference_model_t* m, unsigned int seed) { if (m) m->seed = seed; }
API void inference_set_prefill_batch(inference_model_t* m, int n) { if (m) m->prefill_batch = n < 1 ? 1 : n; }

// ---- facts ---------------------------------------------------------------------------------------------------------------------
API int inference_n_ctx(const inference_model_t* m) { return m ? m->n_ctx : 0; }
API int inference_batch_size(const inference_model_t* m) { return m ? m->max_sequences : 0; }
API const char* inference_model_name(const inference_model_t* m) { return m ? m->name.c_str() : ""; }
API int inference_vocab_size(const inference_model_t* m) { return m ? (int)m->decoder->spec().vocab_size : 0; }
API int inference_hidden_size(const inference_model_t* m) { return m ? (int)m->decoder->spec().hidden_size : 0; }
API int inference_max_position(const inference_model_t* m) { return m ? (int)m->decoder->spec().max_position : 0; }

// ---- sequences -----------------------------------------------------------------------------------------------------------------
API int inference_seq_new(inference_model_t* m) {
    int idx = -1;
    int rc = guarded([&] {
        Engine& eng = need_engine(m);
        sequence(m, 0);                                   // sequence 0 exists before any other
        int i = 0;
        while (m->seqs.count(i)) i++;
        try {
            eng.add_request(i);
        } catch (const OutOfSlots&) {
            return 0;
        }
        m->seqs[i].index = i;
        idx = i;
        return 0;
    });
    return rc == 0 ? idx : -1;
}
API int inference_seq_select(inference_model_t* m, int seq) {
    return guarded([&] {
        sequence(m, seq);
        m->current = seq;
        return 0;
    });
}
API int inference_seq_current(const inference_model_t* m) { return m ? m->current : 0; }
API int inference_seq_free(inference_model_t* m, int seq) {
    return guarded([&] {
        Engine& eng = need_engine(m);
        if (seq == 0 || !m->seqs.count(seq)) throw Error(kInvalidArg, "sequence " + std::to_string(seq) + " cannot be freed");
        must_be_idle(m->seqs[seq]);
        if (eng.has_request(seq)) eng.release(seq);
        m->seqs.erase(seq);
        if (m->current == seq) m->current = 0;
        return 0;
    });
}

API void inference_reset(inference_model_t* m) {
    guarded([&] {
        Engine& eng = need_engine(m);
        Sequence& s = current(m);
        must_be_idle(s);
        if (eng.has_request(s.index)) eng.release(s.index);
        eng.add_request(s.index);
        s.tokens.clear();
        s.logits_valid = false;
        return 0;
    });
}
API int inference_n_past(const inference_model_t* m) {
    if (!m) return 0;
    auto it = m->seqs.find(m->current);
    return it == m->seqs.end() ? 0 : (int)(it->second.active ? it->second.active->tokens.size() : it->second.tokens.size());
}

// ---- forward passes on the current sequence ------------------------------------------------------------------------------------
API int inference_prefill(inference_model_t* m, const int32_t* tokens, int n) {
    return guarded([&] {
        Sequence& s = current(m);
        must_be_idle(s);
        if (n < 0 || (n > 0 && !tokens)) throw Error(kInvalidArg, "no tokens");
        if (n > 0) feed(m, s, tokens, n, nullptr);
        return 0;
    });
}
API int inference_prefill_logits(inference_model_t* m, const int32_t* tokens, int n, float* logits) {
    return guarded([&] {
        Sequence& s = current(m);
        must_be_idle(s);
        if (n < 1 || !tokens || !logits) throw Error(kInvalidArg, "tokens and room for their logits are needed");
        feed(m, s, tokens, n, logits);
        return 0;
    });
}
API int inference_decode_token(inference_model_t* m, int token_id, int* next_token_out) {
    return guarded([&] {
        Sequence& s = current(m);
        must_be_idle(s);
        const int32_t t = token_id;
        feed(m, s, &t, 1, nullptr);
        if (next_token_out) {
            Sampler greedy(SamplerParams::greedy());
            Tensor row(s.logits.data(), DType::F32, {1, need_engine(m).vocab_size()});
            *next_token_out = need_engine(m).sample(row, {&greedy})[0];
        }
        return 0;
    });
}
API int inference_get_logits(inference_model_t* m, int* vocab_ids, float* logits) {
    return guarded([&] {
        Engine& eng = need_engine(m);
        Sequence& s = current(m);
        must_be_idle(s);
        if (s.tokens.empty()) throw Error(kInvalidState, "nothing decoded yet");
        if (!s.logits_valid || eng.length(s.index) < (int)s.tokens.size()) {
            if (eng.length(s.index) == (int)s.tokens.size()) {
                // everything is in the cache but the logits are gone: run the last token again
                if (!eng.cache().can_rewind()) throw Error(kInvalidState, "the logits of this sequence are not at hand");
                eng.cache().truncate(s.index, (int)s.tokens.size() - 1);
            }
            feed(m, s, nullptr, 0, nullptr);
        }
        const int V = (int)eng.vocab_size();
        if (vocab_ids) for (int i = 0; i < V; i++) vocab_ids[i] = i;
        if (logits) eng.read_logits(Tensor(s.logits.data(), DType::F32, {1, V}), logits);
        return 0;
    });
}
