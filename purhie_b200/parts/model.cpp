#include "model.h"

#include <algorithm>
#include <set>

namespace qe {

DecoderModel::DecoderModel(ModelSpec spec, DType compute_dtype, Json options)
    : spec_(std::move(spec)), build_(compute_dtype, std::move(options)) {
    register_builtin_parts();
    spec_.validate();
    embedding_ = make_part_as<Embedding>("embedding", spec_.embedding, build_);
    for (const LayerSpec& layer : spec_.layers) layers_.push_back(make_arrangement(layer, build_));
    final_norm_ = make_part_as<Norm>("norm", spec_.final_norm, build_);
    head_ = make_part_as<Head>("head", spec_.head, build_);
}

std::vector<Part*> DecoderModel::all_parts() const {
    std::vector<Part*> out = {embedding_.get()};
    for (const auto& layer : layers_)
        for (Part* p : layer->parts()) out.push_back(p);
    out.push_back(final_norm_.get());
    out.push_back(head_.get());
    return out;
}

std::vector<TensorSpec> DecoderModel::tensor_specs() const {
    std::vector<TensorSpec> out;
    std::map<std::string, size_t> seen;
    std::function<void(Part*)> visit = [&](Part* p) {
        for (const TensorSpec& s : p->tensor_specs()) {
            auto it = seen.find(s.name);
            if (it != seen.end()) {
                if (!(out[it->second] == s)) throw ConfigError("two parts read '" + s.name + "' with different shapes or roles");
                continue;
            }
            seen[s.name] = out.size();
            out.push_back(s);
        }
        for (Part* c : p->children()) visit(c);
    };
    for (Part* p : all_parts()) visit(p);
    return out;
}

std::vector<std::string> DecoderModel::ignored_tensors() const {
    std::set<std::string> names;
    for (Part* p : all_parts())
        for (const std::string& n : p->ignored_tensors()) names.insert(n);
    return std::vector<std::string>(names.begin(), names.end());
}

void DecoderModel::bind(WeightSource& src) {
    for (Part* p : all_parts()) p->bind(src);
}

std::vector<std::string> DecoderModel::required_libraries() const {
    std::set<std::string> libs;
    for (Part* p : all_parts())
        for (const std::string& l : p->required_libraries()) libs.insert(l);
    return std::vector<std::string>(libs.begin(), libs.end());
}

std::vector<CacheNeed> DecoderModel::cache_needs() const {
    std::vector<CacheNeed> needs;
    for (const LayerCall& call : spec_.schedule)
        needs.push_back(call.cache_from >= 0 ? CacheNeed() : layers_[call.layer]->cache_need());
    return needs;
}

std::vector<CacheView> DecoderModel::cache_views(const CacheManager& manager) const {
    std::vector<CacheView> views;
    for (int i = 0; i < (int)spec_.schedule.size(); i++) {
        const int owner = spec_.schedule[i].cache_from >= 0 ? spec_.schedule[i].cache_from : i;
        views.push_back(manager.view(i, owner));
    }
    return views;
}

int DecoderModel::preferred_row_multiple() const {
    int m = 0;
    for (Part* p : all_parts()) m = std::max(m, p->preferred_row_multiple());
    return m;
}

void DecoderModel::prepare_step(StepPlan& plan) {
    for (Part* p : all_parts()) p->prepare_step(plan);
}

Tensor DecoderModel::forward(StepContext& ctx, const std::vector<CacheView>& views, const int32_t* want_rows, int n_want,
                             const std::function<void(int, ResidualStream&, StepContext&)>& after_entry) {
    ResidualStream stream;
    stream.x = embedding_->forward(ctx);
    for (size_t i = 0; i < spec_.schedule.size(); i++) {
        // a layer learns which norm the next entry of the run order starts with: its last product may work ahead for it
        ctx.next_layer_norm = i + 1 < spec_.schedule.size() ? layers_[spec_.schedule[i + 1].layer]->first_norm(ctx) : NormAhead();
        layers_[spec_.schedule[i].layer]->forward(stream, ctx, views[i]);
        if (after_entry) after_entry((int)i, stream, ctx);
    }
    ctx.next_layer_norm = NormAhead();
    if (n_want == 0) return Tensor();
    Tensor xn = final_norm_->forward(stream, ctx, want_rows, n_want);
    return head_->forward(xn, ctx, n_want);
}

}  // namespace qe
