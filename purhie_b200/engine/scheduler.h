// The scheduler: admits requests, cuts prompts into portions under a token budget, decodes, finishes and frees;
// and decides what happens when pages run out.  It is the one driver of generation: the C API's generate calls,
// its streams and its request queue all put GenRequests here.
//
// Every step() plans one batch and runs it through the engine's one step function:
//   1. one decode row for every running request whose known tokens are all but one in the cache;
//   2. portions of the known tokens of the other running requests, oldest first (portion = min(rest, rest of
//      the token budget, the chunk cap), cut down to the pages that are free);
//   3. newly admitted requests from the waiting queue, first come first served, while a state slot, pages and
//      budget are left.
// When the decode rows need more pages than are free, the most recently admitted running request is preempted:
// its pages and slot are given back and it returns to the front of the waiting queue; its known tokens (prompt
// plus what it generated so far) are recomputed on re-admission, and its sampler, and so its random stream, is
// kept, so the continuation is the same.  If the one remaining request still cannot get a page, it is finished
// with reason context_full.  Decisions depend on the order of arrival only.
//
// The reference's scheduler lives in its server (tick, bin/rocm-inference-server:1818-1871): a FIFO queue, a
// fixed pool of sequences each with a whole-context cache, a prefill chunk of --prefill-chunk tokens (default
// 512, :1648) per tick beside batched decoding, no token budget and no preemption; stop reasons are those of
// src/inference.h:229-236.
#pragma once

#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <set>
#include <vector>

#include "../sampling/sampler.h"
#include "engine.h"

namespace qe {

// Stop reasons, numbered as src/inference.h:229-236 numbers them; cancelled is this library's own.
enum StopReason { kStopNone = 0, kStopEog = 1, kStopMaxTokens = 2, kStopString = 3, kStopCallback = 4, kStopContextFull = 5, kStopCancelled = 6 };

struct GenRequest {
    int64_t id = 0;                          // the request's id in the cache manager
    std::vector<int32_t> tokens;             // everything known: what came before, the prompt, what was generated
    size_t n_prompt = 0;                     // tokens.size() when the request was added: output = tokens[n_prompt:]
    Sampler sampler;
    int max_new_tokens = 256;
    std::vector<int> eos_ids;
    bool ignore_eos = false;
    std::function<bool(GenRequest&, int)> on_token;   // a true return stops the request after this token
    int chunk = 0;                           // cap on this request's prompt portions (0: the scheduler's)
    bool keep_cache = false;                 // the cache outlives the request (a sequence owns it): finishing does not release
    Tensor first_logits;                     // float32 [vocab] on the device: sample the first token from these, feed nothing
    // state
    enum Status { Waiting, Running, Finished } status = Waiting;
    StopReason stop_reason = kStopNone;
    long long admitted_at = -1;
    int preemptions = 0;
    std::vector<int32_t> output() const { return std::vector<int32_t>(tokens.begin() + (long)n_prompt, tokens.end()); }
    int n_output() const { return (int)(tokens.size() - n_prompt); }
};

struct StepEvent {
    GenRequest* request = nullptr;
    int token = -1;                          // the token emitted in this step (-1: none)
    bool finished = false;
    StopReason reason = kStopNone;
};

// What the scheduler needs from an engine; tests drive the scheduler's decisions with a stand-in.
class QE_API StepRunner {
public:
    virtual ~StepRunner() = default;
    virtual CacheManager& cache() = 0;
    virtual int row_multiple() const { return 0; }
    virtual int64_t max_position() const = 0;
    virtual bool decodes_as_graph(int batch) const { return false; }
    // run the batch and sample one token for every entry that wants its last row, with the sampler given for it
    virtual std::vector<int> run(const std::vector<StepEntry>& entries, const std::vector<Sampler*>& samplers) = 0;
    // the same without waiting: ids stay on the device and feed the next call's single-token batch
    virtual PendingTokens* run_async(const std::vector<StepEntry>&, const std::vector<Sampler*>&, const int32_t*) { return nullptr; }
    virtual std::vector<int> wait(PendingTokens*) { return {}; }
    virtual std::vector<int> sample_only(const Tensor& logits, Sampler& sampler) = 0;
};

struct SchedulerOptions {
    int max_batch_tokens = 2048;
    int prefill_chunk = 512;
    int max_running = 0;                     // 0: the cache's state slots
    long long n_ctx = 0;                     // 0: the model's max_position
    int align_rows = -1;                     // -1: the engine's row multiple; 0: off
    bool run_ahead = true;
};

class QE_API Scheduler {
public:
    Scheduler(StepRunner& runner, const SchedulerOptions& options);

    // ---- requests
    GenRequest* add(std::unique_ptr<GenRequest> request);       // to the back of the waiting queue
    GenRequest* adopt(std::unique_ptr<GenRequest> request);     // a request whose cache is live already (a sequence's): running at once
    bool cancel(int64_t id);
    bool has_work() const { return !waiting_.empty() || !running_.empty(); }
    GenRequest* find(int64_t id);
    std::unique_ptr<GenRequest> take_finished(int64_t id);      // hand a finished request back to its owner

    // ---- steps
    // Plan a batch, run it, sample, and finish what is done.  `only`: take part in this step with these requests
    // alone (streams that a caller steps by hand); waiting requests outside it are not admitted.
    std::vector<StepEvent> step(const std::set<GenRequest*>* only = nullptr);
    // While nothing waits and every running request is decoding with a device sampler: decode steps each launched
    // with the token ids the step before left on the device, the host reading them one step behind.  Returns the
    // events step by step (empty: not applicable, take an ordinary step).
    std::vector<std::vector<StepEvent>> decode_ahead(int max_steps, const std::set<GenRequest*>* only = nullptr);
    void run();                                                 // step until nothing is waiting or running

    // ---- what tests look at
    struct Planned { GenRequest* request; int start, count; bool samples; };
    std::vector<Planned> plan(const std::set<GenRequest*>* only = nullptr);
    const std::deque<GenRequest*>& waiting() const { return waiting_; }
    const std::vector<GenRequest*>& running() const { return running_; }
    long long steps = 0, preemptions = 0;
    SchedulerOptions options;

private:
    int computed(const GenRequest& r) const;
    bool decoding(const GenRequest& r) const;
    int largest_portion(const GenRequest& r, int want, const std::vector<int>& free) const;
    int aligned(int n, int rest, int used) const;
    void take(const GenRequest& r, int n_new, std::vector<int>& free) const;
    void preempt(GenRequest* r);
    void finish(GenRequest* r, StopReason reason, bool live = true);
    StepEvent emit(GenRequest* r, int token);
    void note_finished(std::vector<StepEvent>& events);

    StepRunner& runner_;
    CacheManager& cache_;
    std::deque<GenRequest*> waiting_;
    std::vector<GenRequest*> running_;
    std::map<int64_t, std::unique_ptr<GenRequest>> all_;
    std::vector<GenRequest*> just_finished_;
    long long admissions_ = 0;
    int align_rows_ = 0;
    long long n_ctx_ = 0;
    int max_running_ = 0;
};

// The engine as the scheduler drives it.
class QE_API EngineRunner : public StepRunner {
public:
    explicit EngineRunner(Engine& engine) : engine_(engine) {}
    CacheManager& cache() override { return engine_.cache(); }
    int row_multiple() const override { return engine_.row_multiple(); }
    int64_t max_position() const override { return engine_.max_position(); }
    bool decodes_as_graph(int batch) const override;
    std::vector<int> run(const std::vector<StepEntry>& entries, const std::vector<Sampler*>& samplers) override;
    PendingTokens* run_async(const std::vector<StepEntry>& entries, const std::vector<Sampler*>& samplers, const int32_t* device_tokens) override;
    std::vector<int> wait(PendingTokens* p) override { return engine_.wait(p); }
    std::vector<int> sample_only(const Tensor& logits, Sampler& sampler) override;
private:
    Engine& engine_;
};

}  // namespace qe
