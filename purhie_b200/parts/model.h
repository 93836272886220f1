// The generic decoder: embedding, layers in the order the description gives, final norm, head.
//
// It is assembled from a ModelSpec through the part registries and knows no architecture.  One forward serves
// every kind of step: it runs the rows it is given against the cache views and returns float32 logits for the
// wanted rows only (the reference computes the head for the last row or for all rows:
// src/qwen_model.cpp:1421-1486, 1358-1371).
#pragma once

#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "../cache/cache.h"
#include "parts.h"

namespace qe {

class QE_API DecoderModel {
public:
    DecoderModel(ModelSpec spec, DType compute_dtype, Json options = Json::object());

    // ---- weights
    std::vector<TensorSpec> tensor_specs() const;            // in part order; two parts may read one tensor
    std::vector<std::string> ignored_tensors() const;
    void bind(WeightSource& src);
    std::vector<std::string> required_libraries() const;
    size_t weight_bytes() const { return arena_.bytes(); }
    DeviceArena& arena() { return arena_; }

    // ---- cache
    std::vector<CacheNeed> cache_needs() const;              // one per entry of the run order (a borrower needs nothing itself)
    std::vector<CacheView> cache_views(const CacheManager& manager) const;

    // ---- step
    int preferred_row_multiple() const;
    void prepare_step(StepPlan& plan);
    // Run the rows of ctx.  want_rows (int32, device) are the rows whose logits are returned as float32
    // [n_want, vocab]; with n_want 0 the head is skipped and an undefined tensor is returned.  after_entry, when
    // set, is called after every run-order entry with its index and the residual stream (for dumps).
    Tensor forward(StepContext& ctx, const std::vector<CacheView>& views, const int32_t* want_rows, int n_want,
                   const std::function<void(int, ResidualStream&, StepContext&)>& after_entry = nullptr);

    const ModelSpec& spec() const { return spec_; }
    DType compute_dtype() const { return build_.compute_dtype; }
    std::vector<Part*> all_parts() const;

private:
    ModelSpec spec_;
    BuildContext build_;
    std::shared_ptr<Embedding> embedding_;
    std::vector<std::unique_ptr<Arrangement>> layers_;
    std::shared_ptr<Norm> final_norm_;
    std::shared_ptr<Head> head_;
    DeviceArena arena_;
};

}  // namespace qe
