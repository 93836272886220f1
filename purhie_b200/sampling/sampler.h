// Next-token sampling: the reference's chain on the host, plus the choice of a device kernel.
//
// Chain (src/sampler.h:1-6, src/sampler.cpp:58-170): repetition / presence penalty over the last repeat_last_n
// accepted tokens -> top-k -> top-p -> min-p -> temperature -> one draw.  temperature <= 0 (or top_k == 1) is
// greedy: argmax after the penalty, the lowest id wins ties.  Defaults are the reference's
// (src/sampler.cpp:181-192).  The generator is std::mt19937_64 seeded with `seed`, one uniform number from its
// top 53 bits per sampled token, so equal seeds give the reference's draws.  When only greedy, plain temperature
// sampling or the chain with top-k on is asked for, the engine samples with its device kernels instead of
// copying logits to the host; the uniform number still comes from this sampler's generator.
#pragma once

#include <cstdint>
#include <deque>
#include <random>
#include <vector>

#include "../host/common.h"

namespace qe {

struct SamplerParams {
    float temperature = 0.8f;      // <= 0: greedy
    int top_k = 40;                // keep the k most likely tokens; <= 0: off
    float top_p = 0.95f;           // smallest set with cumulative probability >= top_p; >= 1: off
    float min_p = 0.05f;           // keep tokens with p >= min_p * p_max; <= 0: off
    float repeat_penalty = 1.0f;   // positive logits / r, negative * r, for recent tokens; 1: off
    int repeat_last_n = 64;        // how many accepted tokens the penalty looks back over
    uint64_t seed = 0;
    float presence_penalty = 0.0f; // subtracted from the logit of each recent token, after repeat_penalty

    static SamplerParams greedy() { SamplerParams p; p.temperature = 0.0f; return p; }
    static SamplerParams pure_temperature(float t, uint64_t seed = 0) {
        SamplerParams p; p.temperature = t; p.top_k = 0; p.top_p = 1.0f; p.min_p = 0.0f; p.seed = seed; return p;
    }
};

// One row of the device chain kernel's parameters (24 bytes, see csrc/sampling.cu).
struct ChainRecord {
    double uniform;
    float top_p, log_min_p, temperature;
    int32_t top_k;
};
static_assert(sizeof(ChainRecord) == 24, "the chain kernel reads 24-byte records");

class QE_API Sampler {
public:
    enum class DeviceMode { None, Greedy, Temperature, Chain };
    static constexpr int kChainMaxK = 256;         // most candidates the device's chain kernel keeps
    static constexpr float kLogitRange = 40.0f;    // without a filter, tokens more than this below the maximum are not candidates

    explicit Sampler(const SamplerParams& params = SamplerParams());
    const SamplerParams& params() const { return params_; }

    bool penalised() const;
    bool is_greedy() const { return params_.temperature <= 0.0f || params_.top_k == 1; }
    // The device kernel that gives the same result as the chain on the host; None: penalties, or top-p / min-p
    // without top-k, or top-k beyond kChainMaxK.
    DeviceMode device_mode() const;
    ChainRecord chain_record();                    // draws the token's uniform number
    double uniform();                              // [0, 1) from the generator's top 53 bits

    int sample(const float* logits, int n);        // does not record the token; see accept()
    void accept(int token);
    void reset();                                  // forget the history and re-seed

    using Snapshot = std::mt19937_64;              // take back draws: restore(snapshot()) undoes what came between
    Snapshot snapshot() const { return rng_; }
    void restore(const Snapshot& s) { rng_ = s; }

private:
    SamplerParams params_;
    std::mt19937_64 rng_;
    std::deque<int> history_;
    std::vector<float> scratch_;
};

}  // namespace qe
