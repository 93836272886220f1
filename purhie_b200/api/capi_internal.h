// What the files of the C interface share: the handles' contents and the error plumbing.
#pragma once

#include <map>
#include <set>
#include <string>

#include "../engine/engine.h"
#include "../engine/scheduler.h"
#include "../weights/weights.h"
#include "inference.h"

#define API extern "C" QE_API

namespace qe {
namespace capi {

// The thread's last error: its text and the name of its kind ("ConfigError", "OutOfPages", ...; "Error" otherwise).
void set_last_error(const char* kind, const std::string& text);

// Run `body`; an exception becomes its error code and the thread's last error.
template <typename F> int guarded(F&& body) {
    try {
        return body();
    }
#define QE_CATCH(KIND) catch (const KIND& e) { set_last_error(#KIND, e.what()); return e.code; }
    QE_CATCH(ConfigError) QE_CATCH(SafetensorsError) QE_CATCH(WeightError) QE_CATCH(StepError) QE_CATCH(OutOfPages)
    QE_CATCH(OutOfSlots) QE_CATCH(KernelError) QE_CATCH(CheckError) QE_CATCH(Error)
#undef QE_CATCH
    catch (const JsonError& e) {
        set_last_error("Error", std::string("bad JSON: ") + e.what());
        return kInvalidArg;
    } catch (const std::bad_alloc&) {
        set_last_error("Error", "out of host memory");
        return kOutOfMemory;
    } catch (const std::exception& e) {
        set_last_error("Error", e.what());
        return kInvalidState;
    }
}

constexpr long long kQueueBase = 1LL << 32;     // ids of queue requests; sequences use their small numbers

struct Sequence {
    int index = 0;
    std::vector<int32_t> tokens;                // everything the sequence holds; the cache may lag behind by a tail
    DeviceBuffer logits;                        // float32 [vocab] of the last token, when valid
    bool logits_valid = false;
    GenRequest* active = nullptr;               // a stream that has the tokens on loan
};

SamplerParams to_params(const sampler_params& p);
Engine& need_engine(inference_model* m);
Sequence& sequence(inference_model* m, int idx);
Sequence& current(inference_model* m);
void must_be_idle(const Sequence& s);
void feed(inference_model* m, Sequence& s, const int32_t* extra, int n_extra, float* all_logits);

}  // namespace capi
}  // namespace qe

struct inference_model {
    std::shared_ptr<qe::DecoderModel> decoder;
    std::unique_ptr<qe::ModelConfig> config;
    qe::DType dtype = qe::DType::BF16;
    std::string name;
    std::vector<int> eos_ids;
    std::unique_ptr<qe::Engine> engine;
    std::unique_ptr<qe::EngineRunner> runner;
    std::unique_ptr<qe::Scheduler> scheduler;
    int n_ctx = 0, prefill_batch = 1024, current = 0, reused = 0, prefilled = 0, max_sequences = 0;
    unsigned seed = 0;
    std::map<int, qe::capi::Sequence> seqs;
    long long next_request = qe::capi::kQueueBase;
    std::set<qe::GenRequest*> queued;           // live queue requests
    std::map<long long, std::unique_ptr<qe::GenRequest>> done;
};

struct sampler {
    qe::Sampler s;
    explicit sampler(const qe::SamplerParams& p) : s(p) {}
};

struct inference_stream {
    inference_model* model = nullptr;
    int seq = 0;
    qe::GenRequest* request = nullptr;          // owned by the scheduler while it runs
    int emitted = 0;
    bool finished = false;
    inference_stop_reason reason = INFERENCE_STOP_NONE;
};
