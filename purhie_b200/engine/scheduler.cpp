#include "scheduler.h"

#include <algorithm>

namespace qe {

Scheduler::Scheduler(StepRunner& runner, const SchedulerOptions& opts) : options(opts), runner_(runner), cache_(runner.cache()) {
    align_rows_ = opts.align_rows >= 0 ? opts.align_rows : runner.row_multiple();
    n_ctx_ = opts.n_ctx > 0 ? opts.n_ctx : runner.max_position();
    max_running_ = opts.max_running > 0 ? opts.max_running : cache_.max_requests();
}

// ---- requests ----------------------------------------------------------------------------------------------------
GenRequest* Scheduler::add(std::unique_ptr<GenRequest> request) {
    if (request->tokens.empty()) throw Error(kInvalidArg, "a request needs at least one prompt token");
    if (all_.count(request->id)) throw Error(kInvalidArg, "request " + std::to_string(request->id) + " is already scheduled");
    GenRequest* r = request.get();
    r->status = GenRequest::Waiting;
    all_[r->id] = std::move(request);
    waiting_.push_back(r);
    return r;
}

GenRequest* Scheduler::adopt(std::unique_ptr<GenRequest> request) {
    if (!cache_.has_request(request->id)) throw Error(kInvalidState, "adopt() needs a request whose cache is live");
    if (all_.count(request->id)) throw Error(kInvalidArg, "request " + std::to_string(request->id) + " is already scheduled");
    GenRequest* r = request.get();
    r->status = GenRequest::Running;
    r->admitted_at = admissions_++;
    all_[r->id] = std::move(request);
    running_.push_back(r);
    return r;
}

GenRequest* Scheduler::find(int64_t id) {
    auto it = all_.find(id);
    return it == all_.end() ? nullptr : it->second.get();
}

std::unique_ptr<GenRequest> Scheduler::take_finished(int64_t id) {
    auto it = all_.find(id);
    if (it == all_.end() || it->second->status != GenRequest::Finished) return nullptr;
    std::unique_ptr<GenRequest> r = std::move(it->second);
    all_.erase(it);
    just_finished_.erase(std::remove(just_finished_.begin(), just_finished_.end(), r.get()), just_finished_.end());
    return r;
}

bool Scheduler::cancel(int64_t id) {
    GenRequest* r = find(id);
    if (!r || r->status == GenRequest::Finished) return false;
    if (r->status == GenRequest::Waiting) {
        waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), r), waiting_.end());
        finish(r, kStopCancelled, false);
    } else {
        finish(r, kStopCancelled);
    }
    return true;
}

// ---- planning ------------------------------------------------------------------------------------------------------
int Scheduler::computed(const GenRequest& r) const { return cache_.has_request(r.id) ? cache_.length(r.id) : 0; }

bool Scheduler::decoding(const GenRequest& r) const {
    return (int)r.tokens.size() - computed(r) == 1 && r.n_output() > 0;
}

void Scheduler::take(const GenRequest& r, int n_new, std::vector<int>& free) const {
    std::vector<int> need = cache_.pages_needed(r.id, n_new);
    for (size_t i = 0; i < need.size(); i++) free[i] -= need[i];
}

// The most tokens <= want for which pages are free.
int Scheduler::largest_portion(const GenRequest& r, int want, const std::vector<int>& free) const {
    const int ps = cache_.page_size(), len = cache_.length(r.id);
    int best = want;
    for (const PageGroup& g : cache_.groups()) {
        const int room = ((int)cache_.block_table(r.id, g.index).size() + free[g.index]) * ps - len;
        best = std::min(best, room);
    }
    return std::max(best, 0);
}

// The portion of n tokens (of `rest` that the request still has) after `used` rows of the step: when the prompt
// goes on after it and the step would end past a multiple of align_rows, the portion ends there instead, unless
// that takes more than half of it.  (The products run in tiles of that many rows: a step of 544 rows costs what
// one of 768 does.)
int Scheduler::aligned(int n, int rest, int used) const {
    const int a = align_rows_;
    if (!a || n >= rest || used + n < a) return n;
    const int over = (used + n) % a;
    return (over && n - over >= std::max(n / 2, 1)) ? n - over : n;
}

void Scheduler::preempt(GenRequest* r) {
    cache_.release(r->id);
    running_.erase(std::remove(running_.begin(), running_.end(), r), running_.end());
    r->status = GenRequest::Waiting;
    r->preemptions++;
    preemptions++;
    waiting_.push_front(r);
}

void Scheduler::finish(GenRequest* r, StopReason reason, bool live) {
    if (live) {
        if (!r->keep_cache && cache_.has_request(r->id)) cache_.release(r->id);
        running_.erase(std::remove(running_.begin(), running_.end(), r), running_.end());
    }
    r->status = GenRequest::Finished;
    r->stop_reason = reason;
    just_finished_.push_back(r);
}

std::vector<Scheduler::Planned> Scheduler::plan(const std::set<GenRequest*>* only) {
    auto takes_part = [&](GenRequest* r) { return !only || only->count(r); };
    while (true) {
        std::vector<int> free = cache_.free_pages();
        int budget = options.max_batch_tokens;
        std::vector<Planned> plan;
        std::vector<GenRequest*> pool, decoders;
        for (GenRequest* r : running_)
            if (takes_part(r) && !r->first_logits.defined()) pool.push_back(r);
        for (GenRequest* r : pool)
            if (decoding(*r)) decoders.push_back(r);
        auto newest = [&] { return *std::max_element(running_.begin(), running_.end(), [](GenRequest* a, GenRequest* b) { return a->admitted_at < b->admitted_at; }); };
        // 1. decode rows; make room by preempting the newest running request
        std::vector<int> need(free.size(), 0);
        for (GenRequest* r : decoders) {
            std::vector<int> n = cache_.pages_needed(r->id, 1);
            for (size_t i = 0; i < n.size(); i++) need[i] += n[i];
        }
        bool short_of = (int)decoders.size() > budget;
        for (size_t i = 0; i < free.size(); i++) short_of |= need[i] > free[i];
        if (short_of) {
            GenRequest* victim = newest();
            if (running_.size() == 1) finish(victim, kStopContextFull);
            else preempt(victim);
            continue;
        }
        for (GenRequest* r : decoders) {
            take(*r, 1, free);
            plan.push_back({r, (int)r->tokens.size() - 1, 1, true});
            budget--;
        }
        // 2. portions of what the other running requests still have to feed, oldest admission first
        std::vector<GenRequest*> by_age = pool;
        std::sort(by_age.begin(), by_age.end(), [](GenRequest* a, GenRequest* b) { return a->admitted_at < b->admitted_at; });
        for (GenRequest* r : by_age) {
            if (budget <= 0 || std::find(decoders.begin(), decoders.end(), r) != decoders.end()) continue;
            const int rest = (int)r->tokens.size() - computed(*r);
            if (rest <= 0) continue;
            const int cap = r->chunk > 0 ? r->chunk : options.prefill_chunk;
            int n = largest_portion(*r, std::min({rest, budget, cap}), free);
            if (n <= 0) continue;
            n = aligned(n, rest, options.max_batch_tokens - budget);
            take(*r, n, free);
            plan.push_back({r, computed(*r), n, n == rest});
            budget -= n;
        }
        // 3. admissions, first come first served
        for (size_t w = 0; w < waiting_.size() && budget > 0 && (int)running_.size() < max_running_ && cache_.slots().num_free() > 0;) {
            GenRequest* r = waiting_[w];
            if (!takes_part(r)) {
                if (!only) break;
                w++;
                continue;
            }
            const int known = (int)r->tokens.size();
            std::vector<int> whole = cache_.pages_for_new_request(known + 1), total = cache_.total_pages();
            bool too_big = known + 1 > n_ctx_;
            for (size_t i = 0; i < whole.size(); i++) too_big |= whole[i] > total[i];
            if (too_big) {
                // even an empty pool (or the context) cannot hold this request and one more token
                waiting_.erase(waiting_.begin() + (long)w);
                finish(r, kStopContextFull, false);
                continue;
            }
            const int cap = r->chunk > 0 ? r->chunk : options.prefill_chunk;
            int n = std::min({known, budget, cap});
            const int pages = (n + cache_.page_size() - 1) / cache_.page_size();
            int least = free.empty() ? pages : *std::min_element(free.begin(), free.end());
            if (pages > least) {
                n = least * cache_.page_size();
                if (n <= 0) break;
            }
            n = aligned(n, known, options.max_batch_tokens - budget);
            waiting_.erase(waiting_.begin() + (long)w);
            cache_.add_request(r->id);
            r->status = GenRequest::Running;
            r->admitted_at = admissions_++;
            running_.push_back(r);
            take(*r, n, free);
            plan.push_back({r, 0, n, n == known});
            budget -= n;
        }
        bool stuck = plan.empty() && !pool.empty();
        if (stuck) {
            // nobody can move: the pages are spread over half-done prompts; make room for the oldest
            GenRequest* victim = newest();
            if (running_.size() == 1) finish(victim, kStopContextFull);
            else preempt(victim);
            continue;
        }
        return plan;
    }
}

// ---- one step --------------------------------------------------------------------------------------------------------
void Scheduler::note_finished(std::vector<StepEvent>& events) {
    for (GenRequest* r : just_finished_) {
        bool told = false;
        for (const StepEvent& e : events) told |= (e.request == r && e.finished);
        if (!told) events.push_back({r, -1, true, r->stop_reason});
    }
    just_finished_.clear();
}

StepEvent Scheduler::emit(GenRequest* r, int tok) {
    if (!r->ignore_eos && std::find(r->eos_ids.begin(), r->eos_ids.end(), tok) != r->eos_ids.end()) {
        finish(r, kStopEog);                        // the end-of-generation token is not emitted
        return {r, -1, true, kStopEog};
    }
    r->tokens.push_back(tok);
    r->sampler.accept(tok);
    const bool stop = r->on_token ? r->on_token(*r, tok) : false;
    StopReason reason;
    if (stop) reason = kStopCallback;
    else if (r->n_output() >= r->max_new_tokens) reason = kStopMaxTokens;
    else if ((long long)r->tokens.size() >= n_ctx_) reason = kStopContextFull;
    else return {r, tok, false, kStopNone};
    finish(r, reason);
    return {r, tok, true, reason};
}

std::vector<StepEvent> Scheduler::step(const std::set<GenRequest*>* only) {
    std::vector<StepEvent> events;
    just_finished_.clear();
    // requests that continue from logits they already have: sample, feed nothing
    for (GenRequest* r : std::vector<GenRequest*>(running_)) {
        if ((only && !only->count(r)) || !r->first_logits.defined()) continue;
        Tensor lg = r->first_logits;
        r->first_logits = Tensor();
        events.push_back(emit(r, runner_.sample_only(lg, r->sampler)[0]));
    }
    std::set<GenRequest*> sampled_now;
    for (const StepEvent& e : events) sampled_now.insert(e.request);
    std::set<GenRequest*> rest_set;
    const std::set<GenRequest*>* filter = only;
    if (!sampled_now.empty()) {
        // a request that was just sampled from stored logits takes its forward pass in the next step
        for (GenRequest* r : running_) if ((!only || only->count(r)) && !sampled_now.count(r)) rest_set.insert(r);
        for (GenRequest* r : waiting_) if (!only || only->count(r)) rest_set.insert(r);
        filter = &rest_set;
        if (rest_set.empty()) { note_finished(events); return events; }
    }
    std::vector<Planned> planned = plan(filter);
    if (planned.empty()) { note_finished(events); return events; }
    std::vector<StepEntry> entries;
    std::vector<Sampler*> samplers;
    std::vector<GenRequest*> sampled;
    std::vector<std::vector<int32_t>> want_store(planned.size());
    for (size_t i = 0; i < planned.size(); i++) {
        const Planned& p = planned[i];
        StepEntry e;
        e.request = p.request->id;
        e.tokens = p.request->tokens.data() + p.start;
        e.n_tokens = p.count;
        if (p.samples) {
            want_store[i] = {p.count - 1};
            e.want = want_store[i].data();
            e.n_want = 1;
            samplers.push_back(&p.request->sampler);
            sampled.push_back(p.request);
        }
        entries.push_back(e);
    }
    std::vector<int> toks = runner_.run(entries, samplers);
    steps++;
    for (size_t i = 0; i < sampled.size(); i++) events.push_back(emit(sampled[i], toks[i]));
    note_finished(events);
    return events;
}

std::vector<std::vector<StepEvent>> Scheduler::decode_ahead(int max_steps, const std::set<GenRequest*>* only) {
    std::vector<std::vector<StepEvent>> results;
    if (!options.run_ahead) return results;
    std::vector<GenRequest*> run;
    for (GenRequest* r : running_) if (!only || only->count(r)) run.push_back(r);
    for (GenRequest* r : waiting_) if (!only || only->count(r)) return results;      // somebody waits: an ordinary step admits
    if (run.empty() || (int)run.size() > options.max_batch_tokens) return results;
    long long horizon = 1LL << 40;
    for (GenRequest* r : run) {
        if (r->first_logits.defined() || (int)r->tokens.size() - computed(*r) != 1) return results;
        if (r->sampler.device_mode() == Sampler::DeviceMode::None || r->sampler.device_mode() != run[0]->sampler.device_mode()) return results;
        // an end-of-generation token is found out after the next step has put it into the cache: a cache that
        // outlives the request must be able to take it back
        if (r->keep_cache && !r->ignore_eos && !r->eos_ids.empty() && !cache_.can_rewind()) return results;
        horizon = std::min<long long>(horizon, std::min<long long>(r->max_new_tokens - r->n_output(), n_ctx_ - (long long)r->tokens.size()));
    }
    const int n = (int)std::min<long long>(max_steps, horizon);
    if (n < 2 || !runner_.decodes_as_graph((int)run.size())) return results;
    std::vector<Sampler*> samplers;
    for (GenRequest* r : run) samplers.push_back(&r->sampler);
    static const int32_t kZero[1] = {0};
    std::vector<int32_t> first_tokens(run.size());
    PendingTokens* prev = nullptr;
    just_finished_.clear();

    // settle the tokens of a step; `fed`: the step after it has already put them into the cache
    auto settle = [&](const std::vector<int>& toks, bool fed, std::vector<StepEvent>& events) {
        bool ended = false;
        for (size_t i = 0; i < run.size(); i++) {
            GenRequest* r = run[i];
            if (r->status != GenRequest::Running) continue;
            StepEvent e = emit(r, toks[i]);
            if (e.finished && e.reason == kStopEog && fed && r->keep_cache && cache_.has_request(r->id))
                cache_.truncate(r->id, (int)r->tokens.size());          // the step in flight fed it: take it back
            ended |= e.finished;
            events.push_back(e);
        }
        return ended;
    };

    for (int step = 0; step < n; step++) {
        std::vector<StepEntry> entries(run.size());
        for (size_t i = 0; i < run.size(); i++) {
            entries[i].request = run[i]->id;
            if (step == 0) { first_tokens[i] = run[i]->tokens.back(); entries[i].tokens = &first_tokens[i]; }
            else entries[i].tokens = kZero;                              // placeholders: the ids come from the device
            entries[i].n_tokens = 1;
            entries[i].want = kZero;
            entries[i].n_want = 1;
        }
        PendingTokens* pend;
        try {
            pend = runner_.run_async(entries, samplers, prev ? prev->ids : nullptr);
        } catch (const OutOfPages&) {
            break;                                                       // the ordinary step decides whom to preempt
        }
        steps++;
        if (prev) {
            // PendingTokens slots are reused in turn; copy what wait() returns before the next launch
            std::vector<int> toks = runner_.wait(prev);
            std::vector<StepEvent> events;
            const bool ended = settle(toks, true, events);
            note_finished(events);
            results.push_back(events);
            if (ended) {
                // the batch changes: the step in flight stands for the requests that go on
                std::vector<int> toks2 = runner_.wait(pend);
                std::vector<StepEvent> events2;
                settle(toks2, false, events2);
                note_finished(events2);
                results.push_back(events2);
                return results;
            }
        }
        prev = pend;
    }
    if (prev) {
        std::vector<StepEvent> events;
        settle(runner_.wait(prev), false, events);
        note_finished(events);
        results.push_back(events);
    }
    return results;
}

void Scheduler::run() {
    while (has_work()) {
        if (decode_ahead(1 << 30).empty()) step();
    }
}

// ---- the engine as a runner ----------------------------------------------------------------------------------------------
bool EngineRunner::decodes_as_graph(int batch) const {
    std::vector<StepEntry> probe((size_t)batch);
    for (StepEntry& e : probe) e.n_tokens = 1;
    return engine_.decodes_as_graph(probe);
}

std::vector<int> EngineRunner::run(const std::vector<StepEntry>& entries, const std::vector<Sampler*>& samplers) {
    Tensor logits = engine_.step(entries);
    if (samplers.empty()) return {};
    return engine_.sample(logits, samplers);
}

PendingTokens* EngineRunner::run_async(const std::vector<StepEntry>& entries, const std::vector<Sampler*>& samplers, const int32_t* device_tokens) {
    Tensor logits = engine_.step(entries, device_tokens);
    PendingTokens* p = engine_.sample_async(logits, samplers);
    if (!p) throw Error(kInvalidState, "the samplers of a run-ahead batch must share one device kernel");
    return p;
}

std::vector<int> EngineRunner::sample_only(const Tensor& logits, Sampler& sampler) {
    Tensor row(logits.data, DType::F32, {1, logits.numel()});
    return engine_.sample(row, {&sampler});
}

}  // namespace qe
