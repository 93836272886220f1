// Generation through the C interface: generate calls, streams and the request queue, all as GenRequests in the
// model's one Scheduler; and engine_step, the step function itself.  A stream borrows its sequence's tokens for as
// long as it runs; the sequence's cache outlives it.  The last token a generation emits is not fed at once: the
// next call on the sequence brings the cache up to the tokens first (the reference decodes it right away,
// src/inference.h:266-274; what a caller sees is the same).
#include <algorithm>

#include "capi_internal.h"

using namespace qe;
using namespace qe::capi;

namespace {

inference_stop_reason to_reason(StopReason r) { return (inference_stop_reason)(int)r; }

// reuse_prefix: keep the longest common prefix of the sequence and `prompt`; return how much of the prompt is
// left to feed from (src/inference.cpp:2514-2574 in the reference).
size_t sync_prompt(inference_model* m, Sequence& s, const int32_t* prompt, int n) {
    Engine& eng = need_engine(m);
    size_t keep = 0;
    while (keep < s.tokens.size() && keep < (size_t)n && s.tokens[keep] == prompt[keep]) keep++;
    if (keep == (size_t)n && keep > 0) keep--;              // at least one token must run to give logits
    const int cached = std::min<int>(eng.length(s.index), (int)keep);
    if (eng.cache().can_rewind() || cached == eng.length(s.index)) {
        eng.cache().truncate(s.index, cached);
        s.tokens.resize(keep);
    } else {
        eng.release(s.index);
        eng.add_request(s.index);
        s.tokens.clear();
        keep = 0;
    }
    s.logits_valid = false;
    m->reused = (int)keep;
    m->prefilled = n - (int)keep;
    return keep;
}

// A request on sequence `s` that continues it with the prompt; running in the scheduler when this returns.
GenRequest* begin_on_sequence(inference_model* m, Sequence& s, const int32_t* prompt, int n_prompt, const inference_gen_options& o,
                              bool whole_prompt_now, std::function<bool(GenRequest&, int)> on_token) {
    Engine& eng = need_engine(m);
    must_be_idle(s);
    if (n_prompt < 0 || (n_prompt > 0 && !prompt)) throw Error(kInvalidArg, "no prompt tokens");
    size_t from = 0;
    if (o.reuse_prefix) from = sync_prompt(m, s, prompt, n_prompt);
    else { m->reused = 0; m->prefilled = n_prompt; }
    if ((long long)s.tokens.size() + (n_prompt - (int)from) > m->n_ctx)
        throw Error(kContextFull, "the prompt does not fit a context of " + std::to_string(m->n_ctx));
    if (whole_prompt_now) {
        if (n_prompt - (int)from > 0 || eng.length(s.index) < (int)s.tokens.size()) feed(m, s, prompt + from, n_prompt - (int)from, nullptr);
    } else {
        s.tokens.insert(s.tokens.end(), prompt + from, prompt + n_prompt);
        if (eng.length(s.index) < (int)s.tokens.size()) s.logits_valid = false;
    }
    std::unique_ptr<GenRequest> r(new GenRequest());
    r->id = s.index;
    r->sampler = Sampler(to_params(o.sampler));
    for (int32_t t : s.tokens) r->sampler.accept(t);       // the penalty window covers the prompt (src/inference.cpp:2791-2792)
    r->max_new_tokens = o.max_new_tokens;
    r->eos_ids = m->eos_ids;
    r->ignore_eos = o.ignore_eog != 0;
    r->keep_cache = true;
    r->chunk = o.prefill_chunk > 0 ? o.prefill_chunk : 0;
    r->on_token = std::move(on_token);
    if (eng.length(s.index) == (int)s.tokens.size()) {
        if (!s.logits_valid) {
            if (s.tokens.empty()) throw Error(kInvalidState, "nothing to continue from: the sequence is empty");
            if (!eng.cache().can_rewind()) throw Error(kInvalidState, "the logits of this sequence are not at hand");
            eng.cache().truncate(s.index, (int)s.tokens.size() - 1);       // run the last token again
        } else {
            r->first_logits = Tensor(s.logits.data(), DType::F32, {eng.vocab_size()});
        }
    }
    r->tokens = std::move(s.tokens);
    r->n_prompt = r->tokens.size();
    s.tokens.clear();
    GenRequest* raw = m->scheduler->adopt(std::move(r));
    s.active = raw;
    s.logits_valid = false;
    return raw;
}

// The request has ended (or is taken away): the sequence gets its tokens back.
void end_on_sequence(inference_model* m, Sequence& s) {
    GenRequest* r = s.active;
    if (!r) return;
    if (r->status != GenRequest::Finished) m->scheduler->cancel(r->id);
    std::unique_ptr<GenRequest> owned = m->scheduler->take_finished(r->id);
    s.tokens = std::move(owned->tokens);
    s.active = nullptr;
    s.logits_valid = false;
    Engine& eng = need_engine(m);
    if (!eng.has_request(s.index)) eng.add_request(s.index);        // a preempted request gave its cache up
}

void fill_result(inference_stream* st, const std::vector<StepEvent>& events, inference_step_result& out) {
    out.token = -1; out.text = ""; out.text_len = 0; out.reason = st->reason; out.rc = st->finished ? 0 : 1;
    if (st->finished) return;
    for (const StepEvent& e : events) {
        if (e.request != st->request) continue;
        if (e.token >= 0) { out.token = e.token; st->emitted++; }
        if (e.finished) {
            st->finished = true;
            st->reason = out.reason = to_reason(e.reason);
            out.rc = 0;
        }
    }
    if (st->finished) end_on_sequence(st->model, st->model->seqs[st->seq]);
}

std::set<GenRequest*> requests_of(inference_stream_t* const* streams, int n, inference_model** model) {
    std::set<GenRequest*> only;
    *model = nullptr;
    for (int i = 0; i < n; i++) {
        if (!streams[i]) throw Error(kInvalidArg, "a stream is NULL");
        if (*model && streams[i]->model != *model) throw Error(kInvalidArg, "the streams belong to different models");
        *model = streams[i]->model;
        if (!streams[i]->finished) only.insert(streams[i]->request);
    }
    return only;
}
}  // namespace

// ---- generate ----------------------------------------------------------------------------------------------------------
API inference_gen_options inference_gen_default_options(void) {
    inference_gen_options o;
    memset(&o, 0, sizeof o);
    o.sampler = sampler_default_params();
    o.max_new_tokens = 256;
    o.checkpoint_tail = 16;
    return o;
}

API int inference_generate_stream(inference_model_t* m, const int32_t* prompt_ids, int n_prompt, const inference_gen_options* options,
                                  int32_t* out_ids, int max_out, int* n_out, inference_stop_reason* reason) {
    return guarded([&] {
        need_engine(m);
        inference_gen_options o = options ? *options : inference_gen_default_options();
        Sequence& s = current(m);
        std::function<bool(GenRequest&, int)> cb;
        if (o.on_token) cb = [o](GenRequest&, int tok) { return o.on_token(o.user, tok, "", 0) != 0; };
        GenRequest* r = begin_on_sequence(m, s, prompt_ids, n_prompt, o, false, cb);
        std::set<GenRequest*> only = {r};
        try {
            while (r->status != GenRequest::Finished)
                if (m->scheduler->decode_ahead(1 << 30, &only).empty()) m->scheduler->step(&only);
        } catch (...) {
            end_on_sequence(m, s);
            throw;
        }
        const int n = r->n_output();
        if (out_ids) for (int i = 0; i < std::min(n, max_out); i++) out_ids[i] = r->tokens[r->n_prompt + i];
        if (n_out) *n_out = n;
        if (reason) *reason = to_reason(r->stop_reason);
        end_on_sequence(m, s);
        return 0;
    });
}

API int inference_generate_ex(inference_model_t* m, const int32_t* prompt_ids, int prompt_len, int max_new_tokens,
                              const sampler_params* params, int32_t* out_ids, int* out_len) {
    return guarded([&] {
        need_engine(m);
        inference_reset(m);
        inference_gen_options o = inference_gen_default_options();
        if (params) o.sampler = *params;
        else { o.sampler.temperature = 0.0f; o.sampler.seed = m->seed; }
        o.max_new_tokens = max_new_tokens;
        int n = 0;
        int rc = inference_generate_stream(m, prompt_ids, prompt_len, &o, out_ids, max_new_tokens, &n, nullptr);
        if (out_len) *out_len = std::min(n, max_new_tokens);
        return rc;
    });
}

API int inference_last_prompt_stats(const inference_model_t* m, int* reused, int* prefilled) {
    if (!m) return INFERENCE_ERR_INVALID_ARG;
    if (reused) *reused = m->reused;
    if (prefilled) *prefilled = m->prefilled;
    return 0;
}

// ---- streams -------------------------------------------------------------------------------------------------------------
API inference_stream_t* inference_stream_begin(inference_model_t* m, const int32_t* prompt_ids, int n_prompt,
                                               const inference_gen_options* options) {
    inference_stream_t* st = nullptr;
    int rc = guarded([&] {
        need_engine(m);
        inference_gen_options o = options ? *options : inference_gen_default_options();
        Sequence& s = current(m);
        GenRequest* r = begin_on_sequence(m, s, prompt_ids, n_prompt, o, o.prefill_chunk <= 0, nullptr);
        st = new inference_stream();
        st->model = m; st->seq = s.index; st->request = r;
        return 0;
    });
    return rc == 0 ? st : nullptr;
}

API int inference_stream_step_batch(inference_stream_t* const* streams, int n, inference_step_result* results) {
    return guarded([&] {
        if (n < 1 || !streams || !results) throw Error(kInvalidArg, "streams and room for their results are needed");
        inference_model* m = nullptr;
        std::set<GenRequest*> only = requests_of(streams, n, &m);
        std::vector<StepEvent> events;
        if (!only.empty()) events = m->scheduler->step(&only);
        for (int i = 0; i < n; i++) fill_result(streams[i], events, results[i]);
        return 0;
    });
}

API int inference_stream_step(inference_stream_t* stream, int32_t* token, const char** text, int* text_len, inference_stop_reason* reason) {
    inference_step_result res;
    int rc = inference_stream_step_batch(&stream, 1, &res);
    if (rc < 0) return rc;
    if (token) *token = res.token;
    if (text) *text = "";
    if (text_len) *text_len = 0;
    if (reason) *reason = res.reason;
    return res.rc;
}

API int inference_stream_run(inference_stream_t* const* streams, int n, int n_steps, inference_step_result* results) {
    int taken = 0;
    int rc = guarded([&] {
        if (n < 1 || !streams || !results) throw Error(kInvalidArg, "streams and room for their results are needed");
        inference_model* m = nullptr;
        while (taken < n_steps) {
            std::set<GenRequest*> only = requests_of(streams, n, &m);
            if (only.empty()) break;
            std::vector<std::vector<StepEvent>> run = m->scheduler->decode_ahead(n_steps - taken, &only);
            if (run.empty()) run.push_back(m->scheduler->step(&only));
            for (const auto& events : run) {
                for (int i = 0; i < n; i++) fill_result(streams[i], events, results[(size_t)taken * n + i]);
                taken++;
            }
        }
        return 0;
    });
    return rc < 0 ? rc : taken;
}

API int inference_stream_tokens(const inference_stream_t* st) { return st ? st->emitted : 0; }
API int inference_stream_seq(const inference_stream_t* st) { return st ? st->seq : -1; }
API void inference_stream_free(inference_stream_t* st) {
    if (!st) return;
    guarded([&] {
        if (!st->finished && st->model->engine) end_on_sequence(st->model, st->model->seqs[st->seq]);
        return 0;
    });
    delete st;
}

// ---- the request queue -------------------------------------------------------------------------------------------------------
API long long inference_request_add(inference_model_t* m, const int32_t* tokens, int n, const inference_request_options* options) {
    long long id = -1;
    int rc = guarded([&] {
        need_engine(m);
        if (n < 1 || !tokens) throw Error(kInvalidArg, "a request needs at least one prompt token");
        std::unique_ptr<GenRequest> r(new GenRequest());
        r->id = m->next_request++;
        r->tokens.assign(tokens, tokens + n);
        r->n_prompt = (size_t)n;
        SamplerParams sp = options ? to_params(options->sampler) : SamplerParams::greedy();
        r->sampler = Sampler(sp);
        for (int32_t t : r->tokens) r->sampler.accept(t);
        r->max_new_tokens = options ? options->max_new_tokens : 256;
        r->eos_ids = m->eos_ids;
        r->ignore_eos = options ? options->ignore_eog != 0 : false;
        GenRequest* raw = m->scheduler->add(std::move(r));
        m->queued.insert(raw);
        id = raw->id;
        return 0;
    });
    return rc == 0 ? id : rc;
}

API int inference_step(inference_model_t* m) {
    return guarded([&] {
        need_engine(m);
        auto settle = [&] {
            for (auto it = m->queued.begin(); it != m->queued.end();) {
                if ((*it)->status == GenRequest::Finished) {
                    const long long id = (*it)->id;
                    it = m->queued.erase(it);
                    m->done[id] = m->scheduler->take_finished(id);
                } else ++it;
            }
        };
        if (!m->queued.empty()) {
            std::set<GenRequest*> only = m->queued;
            if (m->scheduler->decode_ahead(64, &only).empty()) m->scheduler->step(&only);
        }
        settle();
        return (int)m->queued.size();
    });
}

API int inference_request_poll(inference_model_t* m, long long request, int32_t* out, int max_out, int* n_out, int* finished,
                               inference_stop_reason* reason) {
    return guarded([&] {
        need_engine(m);
        const GenRequest* r = nullptr;
        auto d = m->done.find(request);
        if (d != m->done.end()) r = d->second.get();
        else r = m->scheduler->find(request);
        if (!r || request < kQueueBase) throw Error(kInvalidArg, "no request " + std::to_string(request));
        const int n = r->n_output();
        if (out) for (int i = 0; i < std::min(n, max_out); i++) out[i] = r->tokens[r->n_prompt + i];
        if (n_out) *n_out = n;
        if (finished) *finished = r->status == GenRequest::Finished;
        if (reason) *reason = to_reason(r->stop_reason);
        return 0;
    });
}

API int inference_request_cancel(inference_model_t* m, long long request) {
    return guarded([&] {
        need_engine(m);
        GenRequest* r = m->scheduler->find(request);
        if (!r || !m->queued.count(r)) throw Error(kInvalidArg, "no running request " + std::to_string(request));
        m->scheduler->cancel(request);
        m->queued.erase(r);
        m->done[request] = m->scheduler->take_finished(request);
        return 0;
    });
}

API int inference_request_free(inference_model_t* m, long long request) {
    return guarded([&] {
        need_engine(m);
        if (!m->done.erase(request)) throw Error(kInvalidArg, "request " + std::to_string(request) + " is not finished (cancel it first)");
        return 0;
    });
}

// ---- the step function itself ----------------------------------------------------------------------------------------------------
API int engine_request_add(inference_model_t* m, long long request) {
    return guarded([&] {
        need_engine(m).add_request(request);
        return 0;
    });
}
API int engine_request_release(inference_model_t* m, long long request) {
    return guarded([&] {
        Engine& eng = need_engine(m);
        if (!eng.has_request(request)) throw Error(kInvalidArg, "request " + std::to_string(request) + " is not live");
        eng.release(request);
        return 0;
    });
}
API int engine_request_length(const inference_model_t* m, long long request) {
    if (!m || !m->engine || !m->engine->has_request(request)) return -1;
    return m->engine->length(request);
}

API int engine_step(inference_model_t* m, const engine_step_batch* batch, engine_step_output* out) {
    return guarded([&] {
        Engine& eng = need_engine(m);
        if (!batch || !out || batch->n_entries < 0 || (batch->n_entries && !batch->entries)) throw Error(kInvalidArg, "no batch");
        std::vector<StepEntry> entries((size_t)batch->n_entries);
        long long wanted = 0;
        for (int i = 0; i < batch->n_entries; i++) {
            const engine_step_entry& e = batch->entries[i];
            entries[i].request = e.request;
            entries[i].tokens = e.tokens; entries[i].n_tokens = e.n_tokens;
            entries[i].want = e.want; entries[i].n_want = e.n_want;
            wanted += e.n_want > 0 ? e.n_want : 0;
        }
        const long long V = eng.vocab_size();
        if (wanted * V > out->logits_capacity || (wanted && !out->logits))
            throw Error(kInvalidArg, "engine_step: " + std::to_string(wanted) + " rows of " + std::to_string(V) +
                                         " logits do not fit logits_capacity " + std::to_string(out->logits_capacity));
        Tensor lg = eng.step(entries);
        out->n_rows = lg.defined() ? (int)lg.shape[0] : 0;
        out->vocab_size = (int)V;
        if (lg.defined()) eng.read_logits(lg, out->logits);
        else eng.check_kernel_errors();
        const StepStats& st = eng.last_stats();
        out->tokens = st.tokens; out->prompt_rows = st.prompt_rows; out->decode_rows = st.decode_rows;
        out->replayed_graph = st.replayed_graph ? 1 : 0;
        return 0;
    });
}
