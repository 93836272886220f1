#include "sampler.h"

#include <algorithm>
#include <cmath>
#include <numeric>

namespace qe {

namespace {
struct Candidate {
    int id;
    float logit;
};
// by logit descending, the lower id first among equals
inline bool better(const Candidate& a, const Candidate& b) { return a.logit > b.logit || (a.logit == b.logit && a.id < b.id); }

float max_logit(const std::vector<Candidate>& c) {
    float m = -INFINITY;
    for (const Candidate& x : c) m = std::max(m, x.logit);
    return m;
}
}  // namespace

Sampler::Sampler(const SamplerParams& params) : params_(params), rng_(params.seed) {}

bool Sampler::penalised() const {
    return (params_.repeat_penalty != 1.0f || params_.presence_penalty != 0.0f) && !history_.empty();
}

Sampler::DeviceMode Sampler::device_mode() const {
    if (penalised()) return DeviceMode::None;
    if (is_greedy()) return DeviceMode::Greedy;
    if (params_.top_k <= 0 && params_.top_p >= 1.0f && params_.min_p <= 0.0f) return DeviceMode::Temperature;
    if (params_.top_k > 0 && params_.top_k <= kChainMaxK) return DeviceMode::Chain;
    return DeviceMode::None;
}

double Sampler::uniform() { return (double)(rng_() >> 11) * (1.0 / 9007199254740992.0); }

ChainRecord Sampler::chain_record() {
    ChainRecord r;
    r.uniform = uniform();
    r.top_p = params_.top_p;
    r.log_min_p = params_.min_p > 0.0f ? std::log(params_.min_p) : -INFINITY;
    r.temperature = params_.temperature;
    r.top_k = params_.top_k;
    return r;
}

void Sampler::accept(int token) {
    if (params_.repeat_last_n <= 0) return;
    history_.push_back(token);
    while ((int)history_.size() > params_.repeat_last_n) history_.pop_front();
}

void Sampler::reset() {
    history_.clear();
    rng_.seed(params_.seed);
}

int Sampler::sample(const float* raw, int n) {
    const SamplerParams& p = params_;
    // stage 0: penalties on a copy of the row (each recent token once)
    const float* logits = raw;
    if (penalised()) {
        scratch_.assign(raw, raw + n);
        std::vector<int> recent(history_.begin(), history_.end());
        std::sort(recent.begin(), recent.end());
        recent.erase(std::unique(recent.begin(), recent.end()), recent.end());
        for (int t : recent) {
            if (t < 0 || t >= n) continue;
            float v = scratch_[t];
            if (p.repeat_penalty != 1.0f) v = v > 0.0f ? v / p.repeat_penalty : v * p.repeat_penalty;
            scratch_[t] = v - p.presence_penalty;
        }
        logits = scratch_.data();
    }
    if (is_greedy()) return (int)(std::max_element(logits, logits + n) - logits);      // the first maximum: lowest id

    std::vector<Candidate> cand;
    bool ordered = false;
    double z_vocab = 0.0;            // softmax normaliser over the whole vocabulary, when top-p without top-k made it
    if (p.top_k > 0) {
        // stage 1a: the k best, ties keeping the lower id, best first
        const int k = std::min(p.top_k, n);
        cand.resize(n);
        for (int i = 0; i < n; i++) cand[i] = {i, logits[i]};
        std::partial_sort(cand.begin(), cand.begin() + k, cand.end(), better);
        cand.resize(k);
        ordered = true;
    } else {
        const float top = *std::max_element(logits, logits + n);
        if (p.top_p < 1.0f) {
            // stage 1b: top-p over the whole vocabulary without sorting it: every token's mass goes into one of
            // 1,024 buckets by its distance below the maximum (everything 40 or more below shares the last);
            // the nucleus lies within the buckets up to the one where the running mass reaches top_p
            constexpr int kBuckets = 1024;
            const float per_unit = kBuckets / kLogitRange;
            std::vector<double> mass(kBuckets, 0.0);
            auto bucket_of = [&](float v) { return std::min(kBuckets - 1, (int)((top - v) * per_unit)); };
            for (int i = 0; i < n; i++) {
                const double e = std::exp(-(double)(top - logits[i]));
                z_vocab += e;
                mass[bucket_of(logits[i])] += e;
            }
            int last = kBuckets - 1;
            double running = 0.0;
            for (int b = 0; b < kBuckets; b++) {
                running += mass[b];
                if (running >= p.top_p * z_vocab) { last = b; break; }
            }
            for (int i = 0; i < n; i++)
                if (bucket_of(logits[i]) <= last) cand.push_back({i, logits[i]});
            std::sort(cand.begin(), cand.end(), better);
            ordered = true;
        } else {
            // stage 1c: no order needed; the floor is min-p's cut, or 40 below the maximum
            const float floor = p.min_p > 0.0f ? top + std::log(p.min_p) : top - kLogitRange;
            for (int i = 0; i < n; i++)
                if (logits[i] >= floor) cand.push_back({i, logits[i]});
        }
    }
    // stage 2: top-p on ordered candidates: the shortest prefix whose probability reaches top_p
    if (p.top_p < 1.0f && ordered) {
        const float top = cand.front().logit;
        double z = z_vocab;
        if (z == 0.0)
            for (const Candidate& c : cand) z += std::exp((double)c.logit - top);
        double running = 0.0;
        size_t keep = cand.size();
        for (size_t i = 0; i < cand.size(); i++) {
            running += std::exp((double)cand[i].logit - top);
            if (running >= p.top_p * z) { keep = i + 1; break; }
        }
        cand.resize(keep);
    }
    // stage 3: min-p relative to the best candidate left
    if (p.min_p > 0.0f) {
        const float cut = max_logit(cand) + std::log(p.min_p);
        size_t w = 0;
        for (size_t i = 0; i < cand.size(); i++)
            if (!(cand[i].logit < cut)) cand[w++] = cand[i];
        cand.resize(w);
    }
    // stage 4: temperature and one draw, walking the candidates in the order they stand
    const float top = max_logit(cand);
    std::vector<float> weight(cand.size());
    double z = 0.0;
    for (size_t i = 0; i < cand.size(); i++) {
        weight[i] = (float)std::exp((double)(cand[i].logit - top) / p.temperature);
        z += weight[i];
    }
    const double r = uniform() * z;
    double running = 0.0;
    for (size_t i = 0; i < cand.size(); i++) {
        running += weight[i];
        if (r < running) return cand[i].id;
    }
    return cand.back().id;
}

}  // namespace qe
