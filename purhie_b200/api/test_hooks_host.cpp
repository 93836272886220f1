// Entry points for tests that need no device: the cache manager's bookkeeping on its own, and the scheduler's
// decisions with a stand-in for the engine that keeps the real cache bookkeeping but runs no model.
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
Json ints(const std::vector<int>& v) {
    Json a = Json::array();
    for (int x : v) a.push(x);
    return a;
}

std::vector<CacheNeed> needs_from_json(const Json& list) {
    std::vector<CacheNeed> needs;
    for (const Json& n : list.items()) {
        const std::string kind = n.get_string("kind", "none");
        if (kind == "pages") needs.push_back(CacheNeed::pages((int)n.at("kv_heads").as_int(), (int)n.at("head_dim").as_int(), (int)n.get_int("window", 0), (int)n.get_int("value_dim", 0)));
        else if (kind == "state") {
            std::vector<int64_t> shape;
            for (const Json& d : n.at("shape").items()) shape.push_back(d.as_int());
            needs.push_back(CacheNeed::state(shape));
        } else needs.push_back(CacheNeed());
    }
    return needs;
}
std::vector<int> ints_from_json(const Json& j) {
    std::vector<int> out;
    if (j.is_array()) for (const Json& v : j.items()) out.push_back((int)v.as_int());
    else out.push_back((int)j.as_int());
    return out;
}

Json cache_info(const CacheManager& c) {
    Json j = Json::object();
    j.set("free_pages", ints(c.free_pages()));
    j.set("total_pages", ints(c.total_pages()));
    Json groups = Json::array();
    for (const PageGroup& g : c.groups()) {
        Json gj = Json::object();
        gj.set("entries", ints(g.entries));
        gj.set("window", g.window ? Json(g.window) : Json());
        gj.set("kv_heads", g.kv_heads);
        gj.set("head_dim", g.head_dim);
        gj.set("value_dim", g.value_dim);
        gj.set("page_stride", (long long)g.page_stride);
        gj.set("used", g.allocator.num_pages() - g.allocator.num_free());
        groups.push(gj);
    }
    j.set("groups", groups);
    j.set("state_entries", ints(c.state_entries()));
    j.set("free_slots", c.slots().num_free());
    Json entry_group = Json::object();
    for (int e = 0; e < (int)c.needs().size(); e++)
        if (c.entry_group(e) >= 0) entry_group.set(std::to_string(e), c.entry_group(e));
    j.set("entry_group", entry_group);
    Json reqs = Json::object();
    for (const auto& kv : c.requests()) {
        Json r = Json::object();
        r.set("length", kv.second.length);
        r.set("slot", kv.second.slot);
        Json tables = Json::array();
        for (const auto& t : kv.second.tables) tables.push(ints(t));
        r.set("tables", tables);
        reqs.set(std::to_string(kv.first), r);
    }
    j.set("requests", reqs);
    return j;
}

// Runs no model: the logits of a row put all weight on (sum of the request's tokens so far * 7 + their count) %
// vocab, so the generated tokens are a pure function of the request's history and any change of order or cut shows.
class FakeRunner : public StepRunner {
public:
    FakeRunner(std::vector<CacheNeed> needs, int page_size, std::vector<int> pages, int max_requests, int vocab, long long max_pos, bool ahead)
        : cache_(std::move(needs), page_size, std::move(pages), max_requests), vocab_(vocab), max_pos_(max_pos), ahead_(ahead) {}
    CacheManager& cache() override { return cache_; }
    int64_t max_position() const override { return max_pos_; }
    bool decodes_as_graph(int) const override { return ahead_; }

    std::vector<int> run(const std::vector<StepEntry>& entries, const std::vector<Sampler*>& samplers) override {
        size_t done = 0;
        try {
            for (; done < entries.size(); done++) cache_.reserve(entries[done].request, entries[done].n_tokens);
        } catch (const OutOfPages&) {
            for (size_t i = 0; i < done; i++) cache_.unreserve(entries[i].request);
            throw;
        }
        std::vector<int> toks;
        size_t next_sampler = 0;
        Json batch = Json::array();
        for (const StepEntry& e : entries) {
            if (cache_.length(e.request) == 0) history_[e.request].clear();       // new, or preempted and starting over
            std::vector<int>& h = history_[e.request];
            if ((int)h.size() != cache_.length(e.request)) throw CheckError("the stand-in's history and the cache disagree");
            Json want = Json::array();
            for (int i = 0; i < e.n_tokens; i++) {
                h.push_back(e.tokens[i]);
                bool wanted = false;
                for (int w = 0; w < e.n_want; w++) wanted |= e.want[w] == i;
                if (!wanted) continue;
                want.push(i);
                long long sum = 0;
                for (int t : h) sum += t;
                std::vector<float> row((size_t)vocab_, 0.0f);
                row[(size_t)((sum * 7 + (long long)h.size()) % vocab_)] = 5.0f;
                toks.push_back(samplers.at(next_sampler++)->sample(row.data(), vocab_));
            }
            cache_.advance(e.request, e.n_tokens);
            Json b = Json::array();
            b.push((long long)e.request); b.push(e.n_tokens); b.push(want);
            batch.push(b);
        }
        batches.push(batch);
        cache_.check();
        return toks;
    }
    PendingTokens* run_async(const std::vector<StepEntry>& entries, const std::vector<Sampler*>& samplers, const int32_t* device_tokens) override {
        std::vector<StepEntry> real = entries;
        std::vector<int32_t> fed(entries.size());
        if (device_tokens)
            for (size_t i = 0; i < entries.size(); i++) { fed[i] = device_tokens[i]; real[i].tokens = &fed[i]; }
        std::vector<int> toks = run(real, samplers);
        turn_ ^= 1;
        ids_[turn_].assign(toks.begin(), toks.end());
        pend_[turn_].rows = (int)toks.size();
        pend_[turn_].ids = ids_[turn_].data();           // "on the device"
        pend_[turn_].host = ids_[turn_].data();
        return &pend_[turn_];
    }
    std::vector<int> wait(PendingTokens* p) override { return std::vector<int>(p->host, p->host + p->rows); }
    std::vector<int> sample_only(const Tensor&, Sampler&) override { throw Error(kNotImplemented, "the stand-in has no stored logits"); }

    Json batches = Json::array();
private:
    CacheManager cache_;
    int vocab_;
    long long max_pos_;
    bool ahead_;
    std::map<int64_t, std::vector<int>> history_;
    PendingTokens pend_[2];
    std::vector<int32_t> ids_[2];
    int turn_ = 0;
};

struct SchedProbe {
    std::unique_ptr<FakeRunner> runner;
    std::unique_ptr<Scheduler> sched;
    std::map<int64_t, std::unique_ptr<GenRequest>> finished;
    std::vector<int64_t> order;
    void collect() {
        for (int64_t id : order)
            if (!finished.count(id))
                if (auto r = sched->take_finished(id)) finished[id] = std::move(r);
    }
};
const char* kReasons[] = {"none", "eog", "max_tokens", "stop_string", "callback", "context_full", "cancelled"};
}  // namespace

// ---- the page and slot allocators -------------------------------------------------------------------------------------
API void* qe_pages_create(int num_pages) {
    void* h = nullptr;
    guarded([&] { h = new PageAllocator(num_pages); return 0; });
    return h;
}
API void qe_pages_free_handle(void* h) { delete static_cast<PageAllocator*>(h); }
API const char* qe_pages_alloc(void* h, int n) { return guarded_text([&] { return ints(static_cast<PageAllocator*>(h)->alloc(n)).dump(); }); }
API const char* qe_pages_release(void* h, const char* pages_json) {
    return guarded_text([&] { return ints(static_cast<PageAllocator*>(h)->free(ints_from_json(Json::parse(pages_json)))).dump(); });
}
API int qe_pages_share(void* h, int page) { return guarded([&] { static_cast<PageAllocator*>(h)->share(page); return 0; }); }
API int qe_pages_num_free(void* h) { return static_cast<PageAllocator*>(h)->num_free(); }
API int qe_pages_check(void* h) { return guarded([&] { static_cast<PageAllocator*>(h)->check(); return 0; }); }
API void* qe_slots_create(int n) { return new SlotAllocator(n); }
API void qe_slots_free_handle(void* h) { delete static_cast<SlotAllocator*>(h); }
API int qe_slots_alloc(void* h) { return guarded([&] { return static_cast<SlotAllocator*>(h)->alloc(); }); }
API int qe_slots_release(void* h, int slot) { return guarded([&] { static_cast<SlotAllocator*>(h)->free(slot); return 0; }); }
API int qe_slots_check(void* h) { return guarded([&] { static_cast<SlotAllocator*>(h)->check(); return 0; }); }

// ---- the cache manager (bookkeeping only: nothing is allocated on a device) -----------------------------------------------
API void* qe_cache_create(const char* needs_json, int page_size, const char* num_pages_json, int max_requests) {
    void* h = nullptr;
    guarded([&] {
        h = new CacheManager(needs_from_json(Json::parse(needs_json)), page_size, ints_from_json(Json::parse(num_pages_json)), max_requests);
        return 0;
    });
    return h;
}
API void qe_cache_free_handle(void* h) { delete static_cast<CacheManager*>(h); }
#define CACHE(h) (*static_cast<CacheManager*>(h))
API int qe_cache_add_request(void* h, long long id) { return guarded([&] { CACHE(h).add_request(id); return 0; }); }
API int qe_cache_release(void* h, long long id) { return guarded([&] { CACHE(h).release(id); return 0; }); }
API int qe_cache_reserve(void* h, long long id, int n) { return guarded([&] { CACHE(h).reserve(id, n); return 0; }); }
API int qe_cache_unreserve(void* h, long long id) { return guarded([&] { CACHE(h).unreserve(id); return 0; }); }
API int qe_cache_advance(void* h, long long id, int n) { return guarded([&] { CACHE(h).advance(id, n); return 0; }); }
API int qe_cache_truncate(void* h, long long id, int n) { return guarded([&] { CACHE(h).truncate(id, n); return 0; }); }
API int qe_cache_length(void* h, long long id) { return guarded([&] { return CACHE(h).length(id); }); }
API int qe_cache_can_reserve(void* h, long long id, int n) { return guarded([&] { return CACHE(h).can_reserve(id, n) ? 1 : 0; }); }
API int qe_cache_check(void* h) { return guarded([&] { CACHE(h).check(); return 0; }); }
API const char* qe_cache_info(void* h) { return guarded_text([&] { return cache_info(CACHE(h)).dump(); }); }
API const char* qe_cache_pages_needed(void* h, long long id, int n) { return guarded_text([&] { return ints(CACHE(h).pages_needed(id, n)).dump(); }); }
API const char* qe_cache_token_slots(void* h, long long id, int group, int start, int n) {
    return guarded_text([&] {
        std::vector<int32_t> out;
        CACHE(h).token_slots(id, group, start, n, out);
        return ints(std::vector<int>(out.begin(), out.end())).dump();
    });
}

// ---- the scheduler over the stand-in -------------------------------------------------------------------------------------------
// options_json: {"num_pages", "page_size", "max_requests", "window", "max_position", "vocab", "ahead" (the stand-in
// takes token ids "from the device"), and the scheduler's max_batch_tokens, prefill_chunk, n_ctx, align_rows, run_ahead}.
API void* qe_sched_create(const char* options_json) {
    void* h = nullptr;
    guarded([&] {
        Json o = Json::parse(options_json);
        std::unique_ptr<SchedProbe> p(new SchedProbe());
        std::vector<CacheNeed> needs = {CacheNeed::pages(1, 8, (int)o.get_int("window", 0))};
        p->runner.reset(new FakeRunner(needs, (int)o.get_int("page_size", 4), {(int)o.get_int("num_pages", 64)},
                                       (int)o.get_int("max_requests", 4), (int)o.get_int("vocab", 50),
                                       o.get_int("max_position", 1 << 20), o.get_bool("ahead", false)));
        SchedulerOptions so;
        so.max_batch_tokens = (int)o.get_int("max_batch_tokens", so.max_batch_tokens);
        so.prefill_chunk = (int)o.get_int("prefill_chunk", so.prefill_chunk);
        so.n_ctx = o.get_int("n_ctx", 0);
        so.align_rows = (int)o.get_int("align_rows", 0);
        so.run_ahead = o.get_bool("run_ahead", true);
        p->sched.reset(new Scheduler(*p->runner, so));
        h = p.release();
        return 0;
    });
    return h;
}
API void qe_sched_free_handle(void* h) { delete static_cast<SchedProbe*>(h); }
// stop_after: the request's token callback asks to stop once it has seen this many tokens (0: no callback).
API int qe_sched_add(void* h, long long id, const int32_t* tokens, int n, const sampler_params* params, int max_new_tokens,
                     const int32_t* eos, int n_eos, int ignore_eos, int stop_after) {
    return guarded([&] {
        SchedProbe& p = *static_cast<SchedProbe*>(h);
        std::unique_ptr<GenRequest> r(new GenRequest());
        r->id = id;
        r->tokens.assign(tokens, tokens + n);
        r->n_prompt = (size_t)n;
        r->sampler = Sampler(params ? to_params(*params) : SamplerParams::greedy());
        for (int32_t t : r->tokens) r->sampler.accept(t);
        r->max_new_tokens = max_new_tokens;
        r->eos_ids.assign(eos, eos + n_eos);
        r->ignore_eos = ignore_eos != 0;
        if (stop_after > 0) r->on_token = [stop_after](GenRequest& req, int) { return req.n_output() >= stop_after; };
        p.sched->add(std::move(r));
        p.order.push_back(id);
        return 0;
    });
}
API int qe_sched_step(void* h) {
    return guarded([&] {
        SchedProbe& p = *static_cast<SchedProbe*>(h);
        p.sched->step();
        p.collect();
        return 0;
    });
}
API int qe_sched_decode_ahead(void* h) {
    return guarded([&] {
        SchedProbe& p = *static_cast<SchedProbe*>(h);
        int n = (int)p.sched->decode_ahead(1 << 30).size();
        p.collect();
        return n;
    });
}
API int qe_sched_cancel(void* h, long long id) {
    return guarded([&] {
        SchedProbe& p = *static_cast<SchedProbe*>(h);
        int ok = p.sched->cancel(id) ? 1 : 0;
        p.collect();
        return ok;
    });
}
API int qe_sched_has_work(void* h) { return static_cast<SchedProbe*>(h)->sched->has_work() ? 1 : 0; }
API const char* qe_sched_state(void* h) {
    return guarded_text([&] {
        SchedProbe& p = *static_cast<SchedProbe*>(h);
        Json j = Json::object();
        Json running = Json::array(), waiting = Json::array();
        for (GenRequest* r : p.sched->running()) running.push((long long)r->id);
        for (GenRequest* r : p.sched->waiting()) waiting.push((long long)r->id);
        j.set("running", running);
        j.set("waiting", waiting);
        Json fin = Json::object();
        for (const auto& kv : p.finished) {
            Json r = Json::object();
            Json out = Json::array();
            for (int32_t t : kv.second->output()) out.push(t);
            r.set("output", out);
            r.set("n_tokens", (long long)kv.second->tokens.size());
            r.set("stop_reason", kReasons[kv.second->stop_reason]);
            r.set("preemptions", kv.second->preemptions);
            fin.set(std::to_string(kv.first), r);
        }
        j.set("finished", fin);
        j.set("batches", p.runner->batches);
        j.set("preemptions", p.sched->preemptions);
        j.set("steps", p.sched->steps);
        j.set("cache", cache_info(p.runner->cache()));
        return j.dump();
    });
}
