// The engine: a model, its cache and the one step function.
//
// Engine::step(entries) takes a batch of (request, its next tokens, the places whose logits are wanted):
// portions of prompts beside single decoded tokens, cut anywhere.  It runs only the tokens it is given, as one
// batch, against the cache that earlier steps left, and returns float32 logits at the wanted places.  The
// scheduler, the C API, the Python entry point and the trace replay tool all drive this function; there is no
// other forward pass.  The reference has three entry points instead (one decode row, consecutive rows of one
// sequence, one decode row of each of n sequences: src/qwen_model.h:36-42, 150-161) and never mixes prompt
// portions with decode rows in one pass (src/inference.cpp:3071-3143).
//
// A step: validate the batch on the host, reserve pages (all or nothing), let the parts add their own metadata
// (StepPlan), pack everything into one int32 buffer and send it with one pinned copy, run the model's launches
// on the engine's stream, advance the requests.  A batch of single tokens replays a CUDA graph captured once
// per (batch size, block-table width, context bucket); every other batch is launched kernel by kernel, which
// costs the host a few microseconds per launch.
#pragma once

#include <functional>
#include <list>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../cache/cache.h"
#include "../config/config.h"
#include "../parts/model.h"
#include "../sampling/sampler.h"
#include "../weights/weights.h"

namespace qe {

struct StepEntry {
    int64_t request = 0;
    const int32_t* tokens = nullptr;
    int n_tokens = 0;
    const int32_t* want = nullptr;       // places among the tokens whose logits are returned
    int n_want = 0;
};

struct StepStats {
    int tokens = 0, prompt_rows = 0, decode_rows = 0, wanted = 0;
    bool replayed_graph = false;
    std::vector<int> pages_free;
};

struct EngineOptions {
    int page_size = 16;
    long long max_tokens = 4096;         // tokens the pool of each page group holds (each request rounded up to whole pages)
    int max_requests = 4;
    std::vector<int> num_pages;          // overrides max_tokens: one count, or one per group
    bool poison_cache = false;           // NaN in pages at the start and whenever they are freed
    bool cuda_graphs = true;
    int max_graph_batch = 256;
    int max_graphs = 24;
    Json step_options = Json::object();  // kernel choices handed to the parts ("decode_kernel": "cp_async", ...)
};

// Tokens being sampled on the device: `ids` (int32 on the device, valid in stream order at once) and their copy
// to pinned host memory, complete when `event` is.
struct PendingTokens {
    int rows = 0;
    int32_t* ids = nullptr;              // device
    int32_t* host = nullptr;             // pinned: rows ids, then the two error words
    cudaEvent_t event = nullptr;
};

// A step as the host lays it out: one int32 buffer
//   tokens [T] | positions [columns, T] | row_seg [T] | seg_start [S + 1] | ctx_len [S] | slot [S] | want [>= 1]
//   | per group block_table [S, width] | per group slot_mapping [T] | decode_rows [>= 1] | what the parts added
// and the host's own copies of what launch decisions need.
struct StepLayout {
    std::vector<int32_t> flat;
    std::vector<size_t> offset;                      // of each fixed array in flat
    std::vector<std::pair<std::string, std::pair<size_t, int>>> extra;    // part arrays: name -> (offset, count)
    int T = 0, S = 0, n_want = 0, n_decode = 0, n_portions = 0, decode_max_ctx = 0, prefill_max_ctx = 0;
    std::vector<int> widths, q_lens, ctx_lens, slots;
};
// Reserve pages for the batch (all or nothing: OutOfPages leaves the cache as it was), let `prepare` add the parts'
// own arrays, and lay everything out.  all_rows_wanted: the wanted rows are every entry's first row (a batch of
// single tokens whose graph computes all logits).
QE_API void lay_out_step(CacheManager& cache, int position_columns, const std::vector<StepEntry>& entries, int table_width,
                         bool all_rows_wanted, const std::function<void(StepPlan&)>& prepare, StepLayout& lay);
// The step context over a layout that lies at `dev` on the device (workspace, stream, dtype and error words are the
// caller's to fill in).
QE_API void context_from_layout(const StepLayout& lay, const CacheManager& cache, int position_columns, const int32_t* dev,
                                StepContext& ctx, const int32_t** want_rows);

class QE_API Engine {
public:
    Engine(std::shared_ptr<DecoderModel> model, const EngineOptions& options);
    ~Engine();
    Engine(const Engine&) = delete;
    Engine& operator=(const Engine&) = delete;

    // ---- requests
    void add_request(int64_t id) { cache_->add_request(id); }
    bool has_request(int64_t id) const { return cache_->has_request(id); }
    void release(int64_t id) { cache_->release(id); }
    int length(int64_t id) const { return cache_->length(id); }

    // ---- the step
    // Returns float32 logits [wanted places, vocab] on the device, in the order of the entries and of each
    // entry's want (undefined when nothing is wanted); they live in scratch memory that the next step reuses.
    // Throws OutOfPages, leaving everything as it was, when the cache cannot hold the batch; StepError for a
    // batch that cannot be run.  device_tokens (int32 on the device, one per entry): a batch of single tokens
    // takes its token ids from there instead of from the entries, whose ids are then placeholders; that lets a
    // caller launch a step with the tokens the step before sampled without waiting for them.
    Tensor step(const std::vector<StepEntry>& entries, const int32_t* device_tokens = nullptr);
    bool decodes_as_graph(const std::vector<StepEntry>& entries) const;
    // Copy logits to the host (waits for the stream) and raise if a kernel reported giving up on a wait.
    void read_logits(const Tensor& logits, float* host);
    void synchronize();                                  // wait for the stream, then check_kernel_errors()
    void check_kernel_errors();                          // synchronises; throws KernelError when a kernel gave up on a wait
    void inject_error_word(int which, int code);         // for tests: as if a kernel had reported `code` (0 products, 1 attention)
    // After every run-order entry of the next steps, call `fn(entry index, residual [T, E] float32 with its
    // pending addend folded in, T, E)` with a host copy (for layer-by-layer comparison; turns graphs off while set).
    void set_layer_dump(std::function<void(int, const float*, int, int)> fn) { layer_dump_ = std::move(fn); }

    // ---- sampling
    // One token per row of logits with the row's sampler.  Greedy, plain temperature sampling and the chain with
    // top-k on run in the device kernels (the uniform number still comes from the sampler's generator, one per
    // token); penalties, and top-p or min-p without top-k, run on the host over a copy of the row.
    std::vector<int> sample(const Tensor& logits, const std::vector<Sampler*>& samplers);
    // Start sampling on the device and the ids' copy to the host without waiting for either.  Returns nullptr when
    // the rows' samplers do not all run the same device kernel.  Each sampler draws its uniform number now.
    PendingTokens* sample_async(const Tensor& logits, const std::vector<Sampler*>& samplers);
    std::vector<int> wait(PendingTokens* pending);       // the ids on the host; throws if a kernel gave up on a wait

    // ---- facts
    CacheManager& cache() { return *cache_; }
    const CacheManager& cache() const { return *cache_; }
    DecoderModel& model() { return *model_; }
    const std::vector<CacheView>& views() const { return views_; }
    int64_t vocab_size() const { return model_->spec().vocab_size; }
    int64_t max_position() const { return model_->spec().max_position; }
    DType dtype() const { return model_->compute_dtype(); }
    int row_multiple() const { return row_multiple_; }   // a step's rows are cheapest in multiples of this (0: no preference)
    cudaStream_t stream() const { return stream_; }
    const StepStats& last_stats() const { return stats_; }
    size_t last_upload_bytes() const { return last_upload_bytes_; }
    size_t graphs() const { return graphs_.size(); }
    long long graph_replays() const { return graph_replays_; }
    Workspace& workspace() { return workspace_; }
    EngineOptions& options() { return options_; }

private:
    using Layout = StepLayout;
    struct Graph {
        Workspace workspace;
        DeviceBuffer meta;
        cudaGraphExec_t exec = nullptr;
        Tensor logits;
        long long launches = 0;
        std::string signature;
    };
    void validate(const std::vector<StepEntry>& entries) const;
    void layout(const std::vector<StepEntry>& entries, int table_width, bool all_rows_wanted, Layout& lay);
    void upload(const Layout& lay, void* device);
    void context(const Layout& lay, const int32_t* dev, Workspace& ws, StepContext& ctx, const int32_t** want_rows);
    Tensor forward(StepContext& ctx, const int32_t* want_rows, int n_want);
    Tensor step_any(const std::vector<StepEntry>& entries, Layout& lay);
    Tensor step_graph(const std::vector<StepEntry>& entries, const int32_t* device_tokens, Layout& lay);
    void flags_to_host_async(int32_t* pinned_dst);
    void raise_flags(const int32_t* words);

    std::shared_ptr<DecoderModel> model_;
    EngineOptions options_;
    std::unique_ptr<CacheManager> cache_;
    std::vector<CacheView> views_;
    Workspace workspace_;
    cudaStream_t stream_ = nullptr;
    int row_multiple_ = 0;
    StepStats stats_;
    long long graph_replays_ = 0;
    size_t last_upload_bytes_ = 0;
    // metadata upload: two pinned buffers used in turn
    PinnedBuffer meta_host_[2];
    cudaEvent_t meta_event_[2] = {nullptr, nullptr};
    int meta_turn_ = 0;
    // error words: [0] products, [1] attention
    DeviceBuffer error_words_;
    PinnedBuffer error_host_;
    // graphs of single-token batches, most recently used last
    std::list<std::pair<std::string, std::unique_ptr<Graph>>> graphs_;
    // sampling
    struct PendingSlot { PendingTokens p; int capacity = 0; PinnedBuffer host, params; DeviceBuffer ids, scratch; };
    PendingSlot pending_[4];
    int pending_turn_ = 0;
    std::function<void(int, const float*, int, int)> layer_dump_;
};

// ---- construction -----------------------------------------------------------------------------------------------
// A model bound to the tensors of a folder (config.json chooses the architecture).
QE_API std::shared_ptr<DecoderModel> load_model_folder(const std::string& model_dir, DType dtype, const Json& options,
                                                       std::unique_ptr<ModelConfig>* config_out = nullptr);
// A model of `config` with seeded random weights made on the device: the values write_random_model stores.
QE_API std::shared_ptr<DecoderModel> load_model_random(const ModelConfig& config, const RandomInit& init, DType dtype,
                                                       const Json& options);

}  // namespace qe
