#include "engine.h"

#include <algorithm>
#include <set>

#include "../weights/weights.h"

namespace qe {

namespace {
// 0, or the power of two (at least 256) that n fits.
int bucket(int n) {
    if (n <= 0) return 0;
    int b = 256;
    while (b < n) b *= 2;
    return b;
}
int pow2_at_least(int need, int start) {
    int w = start;
    while (w < need) w *= 2;
    return w;
}
const char* kGemmErrors[] = {"the TMA producer waited too long for a free stage", "the MMA warp waited too long",
                             "the epilogue waited too long for an accumulator"};
std::string flag_text(int which, int code) {
    if (which == 0) {
        const char* t = (code >= 101 && code <= 103) ? kGemmErrors[code - 101] : "error";
        return "gemm_tcgen05: " + std::string(t) + " (status " + std::to_string(code) + ")";
    }
    const char* t = code == 111 ? "the attention producer waited too long for a free stage"
                  : code == 112 ? "an attention consumer waited too long for keys"
                  : code == 121 ? "the prefill attention producer waited too long"
                  : code == 122 ? "the prefill attention tensor-core warp waited too long"
                  : code == 123 ? "a prefill attention softmax warp waited too long" : "error";
    return "attention kernel: " + std::string(t) + " (status " + std::to_string(code) + ")";
}
}  // namespace

// ---- construction -----------------------------------------------------------------------------------------------
Engine::Engine(std::shared_ptr<DecoderModel> model, const EngineOptions& options) : model_(std::move(model)), options_(options) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count < 1)
        throw Error(kInvalidState, "purhie_b200 runs on a CUDA device only; no GPU is visible and there is no host path");
    for (const std::string& lib : model_->required_libraries()) require_library(lib);     // fail now if one is missing
    QE_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    workspace_.stream = stream_;
    std::vector<int> pages = options_.num_pages;
    if (pages.empty()) pages = {(int)((options_.max_tokens + options_.page_size - 1) / options_.page_size)};
    cache_.reset(new CacheManager(model_->cache_needs(), options_.page_size, pages, options_.max_requests));
    cache_->materialize(model_->compute_dtype(), options_.poison_cache, stream_);
    views_ = model_->cache_views(*cache_);
    row_multiple_ = model_->compute_dtype() == DType::BF16 ? model_->preferred_row_multiple() : 0;
    for (int i = 0; i < 2; i++) QE_CUDA(cudaEventCreateWithFlags(&meta_event_[i], cudaEventDisableTiming));
    error_words_ = DeviceBuffer(16);
    QE_CUDA(cudaMemsetAsync(error_words_.data(), 0, 16, stream_));
    error_host_.ensure(16);
    QE_CUDA(cudaStreamSynchronize(stream_));
}

Engine::~Engine() {
    if (stream_) cudaStreamSynchronize(stream_);
    for (auto& g : graphs_)
        if (g.second->exec) cudaGraphExecDestroy(g.second->exec);
    for (auto& s : pending_)
        if (s.p.event) cudaEventDestroy(s.p.event);
    for (int i = 0; i < 2; i++)
        if (meta_event_[i]) cudaEventDestroy(meta_event_[i]);
    LaunchProfile::get().forget_stream(stream_);
    if (stream_) cudaStreamDestroy(stream_);
}

// ---- the step ------------------------------------------------------------------------------------------------------
void Engine::validate(const std::vector<StepEntry>& entries) const {
    std::set<int64_t> seen;
    const int64_t vocab = vocab_size();
    for (const StepEntry& e : entries) {
        const std::string who = "request " + std::to_string(e.request);
        if (!seen.insert(e.request).second) throw StepError(who + " is in the batch twice");
        if (!cache_->has_request(e.request)) throw StepError(who + " is not live (add_request first)");
        if (e.n_tokens < 1 || !e.tokens) throw StepError(who + " brings no tokens");
        for (int i = 0; i < e.n_tokens; i++)
            if (e.tokens[i] < 0 || e.tokens[i] >= vocab)
                throw StepError(who + ": token id " + std::to_string(e.tokens[i]) + " is outside the vocabulary of " + std::to_string(vocab));
        if (cache_->length(e.request) + e.n_tokens > max_position())
            throw StepError(who + " would reach position " + std::to_string(cache_->length(e.request) + e.n_tokens) +
                            ", the model's limit is " + std::to_string(max_position()));
        for (int i = 0; i < e.n_want; i++)
            if (e.want[i] < 0 || e.want[i] >= e.n_tokens)
                throw StepError(who + ": wanted place " + std::to_string(e.want[i]) + " is outside its " + std::to_string(e.n_tokens) + " tokens");
    }
}

// Reserve pages for the batch and lay its metadata out as one int32 buffer:
//   tokens [T] | positions [columns, T] | row_seg [T] | seg_start [S + 1] | ctx_len [S] | slot [S] | want [>= 1]
//   | per group block_table [S, width] | per group slot_mapping [T] | decode_rows [>= 1] | what the parts added
void Engine::layout(const std::vector<StepEntry>& entries, int table_width, bool all_rows_wanted, Layout& lay) {
    lay_out_step(*cache_, model_->spec().position_columns, entries, table_width, all_rows_wanted,
                 [&](StepPlan& plan) { model_->prepare_step(plan); }, lay);
}

void lay_out_step(CacheManager& cache, int cols, const std::vector<StepEntry>& entries, int table_width, bool all_rows_wanted,
                  const std::function<void(StepPlan&)>& prepare, StepLayout& lay) {
    size_t reserved = 0;
    try {
        for (; reserved < entries.size(); reserved++) cache.reserve(entries[reserved].request, entries[reserved].n_tokens);
    } catch (const OutOfPages&) {
        // give back what this step took, so that a refused step changes nothing
        for (size_t i = 0; i < reserved; i++) cache.unreserve(entries[i].request);
        throw;
    }
    const int S = (int)entries.size(), G = (int)cache.groups().size();
    int T = 0;
    for (const StepEntry& e : entries) T += e.n_tokens;
    lay.T = T; lay.S = S;
    std::vector<int32_t> want_rows, decode_rows, seg_start = {0};
    std::vector<int> starts;
    for (int s = 0; s < S; s++) {
        const StepEntry& e = entries[s];
        const int start = cache.length(e.request), base = seg_start.back();
        starts.push_back(start);
        lay.q_lens.push_back(e.n_tokens);
        lay.ctx_lens.push_back(start + e.n_tokens);
        lay.slots.push_back(cache.slot_of(e.request));
        seg_start.push_back(base + e.n_tokens);
        if (all_rows_wanted) want_rows.push_back(base);
        else for (int i = 0; i < e.n_want; i++) want_rows.push_back(base + e.want[i]);
        if (e.n_tokens == 1) {
            decode_rows.push_back(base);
            lay.decode_max_ctx = std::max(lay.decode_max_ctx, start + 1);
        } else {
            lay.n_portions++;
            lay.prefill_max_ctx = std::max(lay.prefill_max_ctx, start + e.n_tokens);
        }
    }
    lay.n_want = (int)want_rows.size();
    lay.n_decode = (int)decode_rows.size();
    for (int g = 0; g < G; g++) {
        int w = 0;
        for (const StepEntry& e : entries) w = std::max(w, (int)cache.block_table(e.request, g).size());
        lay.widths.push_back(std::max(table_width, (w + 7) / 8 * 8));
    }
    // what the parts want to add
    StepPlan plan;
    plan.T = T; plan.S = S; plan.q_lens = lay.q_lens; plan.ctx_lens = lay.ctx_lens; plan.starts = starts; plan.slots = lay.slots;
    if (prepare) prepare(plan);

    std::vector<int32_t>& f = lay.flat;
    f.clear();
    auto mark = [&] { lay.offset.push_back(f.size()); };
    mark();                                                            // 0: tokens
    for (const StepEntry& e : entries) f.insert(f.end(), e.tokens, e.tokens + e.n_tokens);
    mark();                                                            // 1: positions, every column the index in the request
    for (int c = 0; c < cols; c++)
        for (int s = 0; s < S; s++)
            for (int i = 0; i < lay.q_lens[s]; i++) f.push_back(starts[s] + i);
    mark();                                                            // 2: row_seg
    for (int s = 0; s < S; s++) f.insert(f.end(), (size_t)lay.q_lens[s], s);
    mark(); f.insert(f.end(), seg_start.begin(), seg_start.end());     // 3
    mark(); f.insert(f.end(), lay.ctx_lens.begin(), lay.ctx_lens.end());   // 4
    mark(); f.insert(f.end(), lay.slots.begin(), lay.slots.end());     // 5
    mark();                                                            // 6: want
    if (want_rows.empty()) f.push_back(0); else f.insert(f.end(), want_rows.begin(), want_rows.end());
    for (int g = 0; g < G; g++) {                                      // 7 .. 7 + G - 1: block tables
        mark();
        for (const StepEntry& e : entries) {
            const std::vector<int>& table = cache.block_table(e.request, g);
            f.insert(f.end(), table.begin(), table.end());
            f.insert(f.end(), (size_t)(lay.widths[g] - (int)table.size()), -1);
        }
    }
    for (int g = 0; g < G; g++) {                                      // 7 + G ..: slot mappings
        mark();
        for (int s = 0; s < S; s++) cache.token_slots(entries[s].request, g, starts[s], lay.q_lens[s], f);
    }
    mark();                                                            // 7 + 2G: decode rows
    if (decode_rows.empty()) f.push_back(0); else f.insert(f.end(), decode_rows.begin(), decode_rows.end());
    for (auto& a : plan.arrays) {
        lay.extra.push_back({a.first, {f.size(), (int)a.second.size()}});
        if (a.second.empty()) f.push_back(0); else f.insert(f.end(), a.second.begin(), a.second.end());
    }
}

// One copy of the metadata to the device, through two pinned buffers used in turn: a buffer is rewritten only
// after the copy that last read it is done.
void Engine::upload(const Layout& lay, void* device) {
    const size_t bytes = lay.flat.size() * sizeof(int32_t);
    last_upload_bytes_ = bytes;
    meta_turn_ ^= 1;
    PinnedBuffer& buf = meta_host_[meta_turn_];
    if (buf.bytes() < bytes) {
        QE_CUDA(cudaEventSynchronize(meta_event_[meta_turn_]));
        buf.ensure(std::max<size_t>(2 * bytes, 16384));
    } else {
        QE_CUDA(cudaEventSynchronize(meta_event_[meta_turn_]));
    }
    memcpy(buf.data(), lay.flat.data(), bytes);
    QE_CUDA(cudaMemcpyAsync(device, buf.data(), bytes, cudaMemcpyHostToDevice, stream_));
    QE_CUDA(cudaEventRecord(meta_event_[meta_turn_], stream_));
}

void Engine::context(const Layout& lay, const int32_t* dev, Workspace& ws, StepContext& ctx, const int32_t** want_rows) {
    context_from_layout(lay, *cache_, model_->spec().position_columns, dev, ctx, want_rows);
    ctx.workspace = &ws;
    ctx.compute_dtype = model_->compute_dtype();
    ctx.stream = stream_;
    ctx.gemm_error = static_cast<int*>(error_words_.data());
    ctx.attention_error = static_cast<int*>(error_words_.data()) + 1;
    ctx.options = &options_.step_options;
}

void context_from_layout(const StepLayout& lay, const CacheManager& cache, int position_columns, const int32_t* dev, StepContext& ctx,
                         const int32_t** want_rows) {
    const int G = (int)cache.groups().size();
    auto at = [&](int i) { return dev + lay.offset[i]; };
    ctx.T = lay.T; ctx.S = lay.S;
    ctx.token_ids = at(0);
    ctx.positions = at(1);
    ctx.position_columns = position_columns;
    ctx.row_seg = at(2);
    ctx.seg_start = at(3);
    ctx.seg_ctx_len = at(4);
    ctx.seg_slot = at(5);
    *want_rows = at(6);
    ctx.q_lens = lay.q_lens; ctx.ctx_lens = lay.ctx_lens; ctx.slots = lay.slots;
    ctx.groups.clear();
    for (int g = 0; g < G; g++) {
        GroupStep gs;
        gs.block_table = at(7 + g);
        gs.table_width = lay.widths[g];
        gs.slot_mapping = at(7 + G + g);
        gs.page_size = cache.page_size();
        ctx.groups.push_back(gs);
    }
    ctx.decode_only = lay.n_portions == 0;
    ctx.decode_rows = ctx.decode_only ? nullptr : at(7 + 2 * G);
    ctx.n_decode_rows = lay.n_decode;
    ctx.decode_max_ctx = bucket(lay.decode_max_ctx);
    ctx.prefill_max_ctx = bucket(lay.prefill_max_ctx);
    ctx.arrays.clear();
    for (const auto& a : lay.extra) ctx.arrays[a.first] = StepArray{dev + a.second.first, a.second.second};
}

Tensor Engine::forward(StepContext& ctx, const int32_t* want_rows, int n_want) {
    if (LaunchProfile::get().on()) LaunchProfile::get().set_stream(stream_);
    if (!layer_dump_) return model_->forward(ctx, views_, want_rows, n_want);
    auto dump = [&](int entry, ResidualStream& stream, StepContext& c) {
        const int T = c.T, E = (int)stream.x.shape[1];
        std::vector<float> x((size_t)T * E);
        QE_CUDA(cudaStreamSynchronize(stream_));
        QE_CUDA(cudaMemcpy(x.data(), stream.x.data, x.size() * 4, cudaMemcpyDeviceToHost));
        if (stream.has_pending) {
            const Tensor& p = stream.pending.tensor;
            const size_t n = (size_t)stream.pending.splits * T * E;
            std::vector<uint8_t> raw(n * dtype_size(p.dtype));
            QE_CUDA(cudaMemcpy(raw.data(), p.data, raw.size(), cudaMemcpyDeviceToHost));
            for (int s = 0; s < stream.pending.splits; s++)
                for (size_t i = 0; i < (size_t)T * E; i++) {
                    const size_t j = (size_t)s * T * E + i;
                    float v;
                    if (p.dtype == DType::F32) memcpy(&v, raw.data() + 4 * j, 4);
                    else { uint16_t h; memcpy(&h, raw.data() + 2 * j, 2); v = bf16_to_f32(h); }
                    x[i] += v;
                }
        }
        layer_dump_(entry, x.data(), T, E);
    };
    return model_->forward(ctx, views_, want_rows, n_want, dump);
}

bool Engine::decodes_as_graph(const std::vector<StepEntry>& entries) const {
    if (!options_.cuda_graphs || layer_dump_ || LaunchProfile::get().on() || (int)entries.size() > options_.max_graph_batch) return false;
    for (const StepEntry& e : entries) if (e.n_tokens != 1) return false;
    return true;
}

Tensor Engine::step(const std::vector<StepEntry>& entries, const int32_t* device_tokens) {
    if (entries.empty()) return Tensor();
    validate(entries);
    Layout lay;
    Tensor logits;
    if (decodes_as_graph(entries)) logits = step_graph(entries, device_tokens, lay);
    else if (device_tokens) throw StepError("token ids from the device need a batch of single tokens that runs as a graph");
    else logits = step_any(entries, lay);
    for (const StepEntry& e : entries) cache_->advance(e.request, e.n_tokens);
    stats_.tokens = lay.T;
    stats_.prompt_rows = stats_.decode_rows = 0;
    for (int q : lay.q_lens) (q > 1 ? stats_.prompt_rows : stats_.decode_rows) += q;
    stats_.wanted = logits.defined() ? (int)logits.shape[0] : 0;
    stats_.pages_free = cache_->free_pages();
    return logits;
}

// A batch with prompt portions (or with graphs off): launched kernel by kernel.
Tensor Engine::step_any(const std::vector<StepEntry>& entries, Layout& lay) {
    int need = 1;
    if (!cache_->groups().empty())
        for (const StepEntry& e : entries)
            need = std::max(need, (cache_->length(e.request) + e.n_tokens + cache_->page_size() - 1) / cache_->page_size());
    layout(entries, pow2_at_least(need, 8), false, lay);
    Tensor dev = workspace_.get("step_meta", {(int64_t)lay.flat.size()}, DType::I32);
    upload(lay, dev.data);
    StepContext ctx;
    const int32_t* want_rows = nullptr;
    context(lay, dev.as<int32_t>(), workspace_, ctx, &want_rows);
    stats_.replayed_graph = false;
    try {
        return forward(ctx, want_rows, lay.n_want);
    } catch (...) {
        for (const StepEntry& e : entries) cache_->unreserve(e.request);
        throw;
    }
}

// A batch of single tokens: the launches of the whole model are captured once per (batch size, block table
// widths, context bucket, what the parts added) and replayed.  Each graph owns its scratch memory and metadata
// buffer, so nothing it points at ever moves.  The graph computes every row's logits; the wanted ones are picked
// afterwards.
Tensor Engine::step_graph(const std::vector<StepEntry>& entries, const int32_t* device_tokens, Layout& lay) {
    const int S = (int)entries.size();
    int need = 1;
    for (const StepEntry& e : entries)
        for (const PageGroup& g : cache_->groups()) need = std::max(need, (int)cache_->block_table(e.request, g.index).size() + 1);
    layout(entries, pow2_at_least(need, 8), true, lay);
    const int ctx_bucket = pow2_at_least(lay.decode_max_ctx, 256);
    std::string key = std::to_string(S) + "|" + std::to_string(ctx_bucket);
    for (int w : lay.widths) key += "|w" + std::to_string(w);
    for (const auto& a : lay.extra) key += "|" + a.first + ":" + std::to_string(a.second.second);
    Graph* g = nullptr;
    for (auto it = graphs_.begin(); it != graphs_.end(); ++it)
        if (it->first == key) {
            graphs_.splice(graphs_.end(), graphs_, it);          // most recently used last
            g = graphs_.back().second.get();
            break;
        }
    try {
        if (!g) {
            if ((int)graphs_.size() >= options_.max_graphs) {
                QE_CUDA(cudaStreamSynchronize(stream_));
                if (graphs_.front().second->exec) cudaGraphExecDestroy(graphs_.front().second->exec);
                graphs_.pop_front();
            }
            std::unique_ptr<Graph> fresh(new Graph());
            fresh->workspace.stream = stream_;
            fresh->meta = DeviceBuffer(lay.flat.size() * sizeof(int32_t));
            graphs_.emplace_back(key, std::move(fresh));
            g = graphs_.back().second.get();
        }
        if (g->meta.bytes() != lay.flat.size() * sizeof(int32_t))
            throw Error(kInvalidState, "a decode graph's metadata changed size under the same key");
        upload(lay, g->meta.data());
        if (device_tokens)                                           // the token ids lead the metadata
            QE_CUDA(cudaMemcpyAsync(g->meta.data(), device_tokens, (size_t)S * 4, cudaMemcpyDeviceToDevice, stream_));
        if (!g->exec) {
            StepContext ctx;
            const int32_t* rows = nullptr;
            context(lay, static_cast<const int32_t*>(g->meta.data()), g->workspace, ctx, &rows);
            ctx.decode_max_ctx = ctx_bucket;                         // the number of attention splits must not change between replays
            // the first time: run the launches directly (this is the step's result, and whatever a kernel sets up
            // on first use is set up), then capture the same launches for the next time
            g->logits = forward(ctx, rows, S);
            g->workspace.frozen = true;
            const long long before = g_launches;
            QE_CUDA(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeRelaxed));
            cudaGraph_t graph = nullptr;
            try {
                forward(ctx, rows, S);
            } catch (...) {
                cudaStreamEndCapture(stream_, &graph);
                if (graph) cudaGraphDestroy(graph);
                throw;
            }
            QE_CUDA(cudaStreamEndCapture(stream_, &graph));
            g->launches = g_launches - before;
            g_launches = before;
            cudaError_t e = cudaGraphInstantiate(&g->exec, graph, 0);
            cudaGraphDestroy(graph);
            if (e != cudaSuccess) { g->exec = nullptr; throw KernelError(std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e)); }
            stats_.replayed_graph = false;
        } else {
            QE_CUDA(cudaGraphLaunch(g->exec, stream_));
            g_launches += g->launches;
            stats_.replayed_graph = true;
            graph_replays_++;
        }
    } catch (...) {
        for (const StepEntry& e : entries) cache_->unreserve(e.request);
        if (g && !g->exec) graphs_.pop_back();                        // a graph that was never finished is not kept
        throw;
    }
    // pick the wanted rows
    std::vector<int> want;
    for (int s = 0; s < S; s++) if (entries[s].n_want) want.push_back(s);
    if ((int)want.size() == S) return g->logits;
    if (want.empty()) return Tensor();
    const int64_t V = g->logits.shape[1];
    Tensor picked = workspace_.get("logits_picked", {(int64_t)want.size(), V}, DType::F32);
    for (size_t i = 0; i < want.size(); i++)
        QE_CUDA(cudaMemcpyAsync(picked.as<float>() + i * V, g->logits.as<float>() + (size_t)want[i] * V, (size_t)V * 4,
                                cudaMemcpyDeviceToDevice, stream_));
    return picked;
}

// ---- results and errors ------------------------------------------------------------------------------------------------
void Engine::flags_to_host_async(int32_t* pinned_dst) {
    QE_CUDA(cudaMemcpyAsync(pinned_dst, error_words_.data(), 8, cudaMemcpyDeviceToHost, stream_));
}

void Engine::raise_flags(const int32_t* words) {
    for (int which = 0; which < 2; which++)
        if (words[which]) {
            const int code = words[which];
            cudaMemsetAsync(error_words_.data(), 0, 16, stream_);
            throw KernelError(flag_text(which, code) + "; the step's results are not valid");
        }
}

void Engine::check_kernel_errors() {
    int32_t* host = static_cast<int32_t*>(error_host_.data());
    flags_to_host_async(host);
    QE_CUDA(cudaStreamSynchronize(stream_));
    raise_flags(host);
}
void Engine::synchronize() { check_kernel_errors(); }

void Engine::inject_error_word(int which, int code) {
    if (which < 0 || which > 1) throw Error(kInvalidArg, "there are two error words: 0 products, 1 attention");
    QE_CUDA(cudaMemcpyAsync(static_cast<int*>(error_words_.data()) + which, &code, 4, cudaMemcpyHostToDevice, stream_));
    QE_CUDA(cudaStreamSynchronize(stream_));
}

void Engine::read_logits(const Tensor& logits, float* host) {
    if (!logits.defined()) return;
    QE_CUDA(cudaMemcpyAsync(host, logits.data, logits.bytes(), cudaMemcpyDeviceToHost, stream_));
    check_kernel_errors();
}

// ---- sampling --------------------------------------------------------------------------------------------------------------
PendingTokens* Engine::sample_async(const Tensor& logits, const std::vector<Sampler*>& samplers) {
    const int R = (int)samplers.size();
    if (!logits.defined() || logits.shape[0] != R)
        throw StepError(std::to_string(R) + " samplers for " + std::to_string(logits.defined() ? logits.shape[0] : 0) + " rows of logits");
    if (R == 0) return nullptr;
    Sampler::DeviceMode mode = samplers[0]->device_mode();
    for (Sampler* s : samplers) if (s->device_mode() != mode) return nullptr;
    if (mode == Sampler::DeviceMode::None) return nullptr;
    pending_turn_ = (pending_turn_ + 1) % 4;
    PendingSlot& slot = pending_[pending_turn_];
    if (!slot.p.event) QE_CUDA(cudaEventCreateWithFlags(&slot.p.event, cudaEventDisableTiming));
    QE_CUDA(cudaEventSynchronize(slot.p.event));          // its last copies are done: the pinned buffers may be rewritten
    if (slot.capacity < R) {
        QE_CUDA(cudaStreamSynchronize(stream_));          // a step in flight may still read the old ids
        slot.capacity = std::max(R, 64);
        slot.host.ensure((size_t)(slot.capacity + 2) * 4);
        slot.params.ensure((size_t)slot.capacity * 24);
        slot.ids = DeviceBuffer((size_t)slot.capacity * 4);
        // the greedy kernel's scratch (partial results of the CTAs that share a row; its counters start at zero)
        slot.scratch = DeviceBuffer((size_t)core_kernels().argmax_scratch_bytes(slot.capacity));
        QE_CUDA(cudaMemsetAsync(slot.scratch.data(), 0, slot.scratch.bytes(), stream_));
    }
    const CoreKernels& k = core_kernels();
    const int V = (int)logits.shape[1];
    int32_t* ids = static_cast<int32_t*>(slot.ids.data());
    if (mode == Sampler::DeviceMode::Greedy) {
        QE_LAUNCH(k, k.argmax(logits.as<float>(), R, V, ids, slot.scratch.data(), (long long)slot.scratch.bytes(), stream_));
    } else if (mode == Sampler::DeviceMode::Chain) {
        ChainRecord* rec = static_cast<ChainRecord*>(slot.params.data());
        for (int i = 0; i < R; i++) rec[i] = samplers[i]->chain_record();
        Tensor rows = workspace_.get("sample_rows", {R, 24}, DType::U8);
        QE_CUDA(cudaMemcpyAsync(rows.data, rec, (size_t)R * 24, cudaMemcpyHostToDevice, stream_));
        QE_LAUNCH(k, k.sample_chain(logits.as<float>(), R, V, rows.data, ids, stream_));
    } else {
        double* unis = static_cast<double*>(slot.params.data());
        float* temps = reinterpret_cast<float*>(unis + R);
        for (int i = 0; i < R; i++) { unis[i] = samplers[i]->uniform(); temps[i] = samplers[i]->params().temperature; }
        Tensor dev = workspace_.get("sample_params", {(int64_t)R * 12}, DType::U8);
        QE_CUDA(cudaMemcpyAsync(dev.data, unis, (size_t)R * 12, cudaMemcpyHostToDevice, stream_));
        QE_LAUNCH(k, k.sample_temperature(logits.as<float>(), R, V, reinterpret_cast<float*>(dev.as<double>() + R), dev.as<double>(),
                                          Sampler::kLogitRange, ids, stream_));
    }
    int32_t* host = static_cast<int32_t*>(slot.host.data());
    QE_CUDA(cudaMemcpyAsync(host, ids, (size_t)R * 4, cudaMemcpyDeviceToHost, stream_));
    flags_to_host_async(host + R);                        // the error words travel with the ids: no extra wait
    QE_CUDA(cudaEventRecord(slot.p.event, stream_));
    slot.p.rows = R; slot.p.ids = ids; slot.p.host = host;
    return &slot.p;
}

std::vector<int> Engine::wait(PendingTokens* pending) {
    QE_CUDA(cudaEventSynchronize(pending->event));
    raise_flags(pending->host + pending->rows);
    return std::vector<int>(pending->host, pending->host + pending->rows);
}

std::vector<int> Engine::sample(const Tensor& logits, const std::vector<Sampler*>& samplers) {
    const int R = (int)samplers.size();
    if (!logits.defined() || logits.shape[0] != R)
        throw StepError(std::to_string(R) + " samplers for " + std::to_string(logits.defined() ? logits.shape[0] : 0) + " rows of logits");
    if (PendingTokens* p = sample_async(logits, samplers)) return wait(p);
    // mixed kinds: row by row, each through the kernel its sampler allows, the rest on the host over a copy
    std::vector<int> out(R, 0);
    const int V = (int)logits.shape[1];
    std::vector<float> row;
    for (int i = 0; i < R; i++) {
        Tensor one(logits.as<float>() + (size_t)i * V, DType::F32, {1, V});
        if (samplers[i]->device_mode() != Sampler::DeviceMode::None) {
            out[i] = wait(sample_async(one, {samplers[i]}))[0];
        } else {
            row.resize(V);
            read_logits(one, row.data());
            out[i] = samplers[i]->sample(row.data(), V);
        }
    }
    return out;
}

// ---- construction helpers -------------------------------------------------------------------------------------------------
std::shared_ptr<DecoderModel> load_model_folder(const std::string& model_dir, DType dtype, const Json& options,
                                                std::unique_ptr<ModelConfig>* config_out) {
    std::unique_ptr<ModelConfig> config = load_config(model_dir);
    auto model = std::make_shared<DecoderModel>(config->build_spec(), dtype, options);
    cudaStream_t stream = nullptr;
    {
        FolderSource src(model_dir, model->tensor_specs(), model->ignored_tensors(), dtype, model->arena(), stream);
        model->bind(src);
    }
    QE_CUDA(cudaDeviceSynchronize());
    if (config_out) *config_out = std::move(config);
    return model;
}

std::shared_ptr<DecoderModel> load_model_random(const ModelConfig& config, const RandomInit& init, DType dtype, const Json& options) {
    auto model = std::make_shared<DecoderModel>(config.build_spec(), dtype, options);
    RandomSource src(model->tensor_specs(), init, dtype, dtype, model->arena(), nullptr);
    model->bind(src);
    QE_CUDA(cudaDeviceSynchronize());
    return model;
}

}  // namespace qe
