// How a layer's parts are strung together.
//
// pre_norm: x += mixer(norm1(x)); x += feed_forward(norm2(x)), with each addition folded into the norm that
// follows it (the reference fuses them the same way: src/qwen_model.cpp:1175-1187, 1248, 1260).  Sub-parts by
// name: mixer_norm, mixer, feed_forward_norm, feed_forward.
#include "parts.h"

namespace qe {

class PreNormBlock : public Arrangement {
public:
    PreNormBlock(const LayerSpec& layer, BuildContext& build) {
        mixer_norm_ = make_part_as<Norm>("norm", layer.part("mixer_norm"), build);
        mixer_ = make_part_as<Mixer>("mixer", layer.part("mixer"), build);
        ff_norm_ = make_part_as<Norm>("norm", layer.part("feed_forward_norm"), build);
        ff_ = make_part_as<FeedForward>("feed_forward", layer.part("feed_forward"), build);
    }
    std::vector<Part*> parts() override { return {mixer_norm_.get(), mixer_.get(), ff_norm_.get(), ff_.get()}; }
    CacheNeed cache_need() const override { return mixer_->cache_need(); }
    void forward(ResidualStream& stream, StepContext& ctx, const CacheView& cache) override {
        ctx.residual = stream.x.as<float>();
        ctx.residual_width = stream.x.shape[1];
        // a consumer that applies the row's factor itself lets the norm in front leave it out (RowScale)
        // (the option "row_factor": "norm" keeps the factor in the norm, for comparing the two forms)
        const bool may_defer = ctx.option("row_factor") != "norm";
        // and a part whose last product adds into the residual itself may do the pass of the norm behind it there
        // (NormAhead; the option "norm_ahead": "off" keeps every norm a kernel of its own)
        const bool may_work_ahead = may_defer && ctx.option("norm_ahead") != "off";
        const bool ff_unscaled = may_defer && ff_->takes_unscaled_rows(ctx);
        ctx.row_scale = RowScale();
        Tensor xn = may_defer && mixer_->takes_unscaled_rows(ctx) ? mixer_norm_->forward_unscaled(stream, ctx, &ctx.row_scale)
                                                                  : mixer_norm_->forward(stream, ctx);
        ctx.norm_ahead = may_work_ahead && ff_unscaled ? ff_norm_->offer(ctx) : NormAhead();
        stream.add(mixer_->forward(xn, ctx, cache));
        stream.prepare(ctx.norm_ahead);
        ctx.row_scale = RowScale();
        xn = ff_unscaled ? ff_norm_->forward_unscaled(stream, ctx, &ctx.row_scale) : ff_norm_->forward(stream, ctx);
        ctx.norm_ahead = may_work_ahead ? ctx.next_layer_norm : NormAhead();
        stream.add(ff_->forward(xn, ctx));
        stream.prepare(ctx.norm_ahead);
        ctx.row_scale = RowScale();
        ctx.norm_ahead = NormAhead();
    }
    NormAhead first_norm(const StepContext& ctx) const override {
        const bool may_defer = ctx.option("row_factor") != "norm";
        return may_defer && mixer_->takes_unscaled_rows(ctx) ? mixer_norm_->offer(ctx) : NormAhead();
    }
private:
    std::shared_ptr<Norm> mixer_norm_, ff_norm_;
    std::shared_ptr<Mixer> mixer_;
    std::shared_ptr<FeedForward> ff_;
};

void register_norm_parts();
void register_position_parts();
void register_mixer_parts();
void register_feed_forward_parts();
void register_embedding_parts();

void register_builtin_parts() {
    static bool done = false;
    if (done) return;
    done = true;
    register_norm_parts();
    register_position_parts();
    register_mixer_parts();
    register_feed_forward_parts();
    register_embedding_parts();
    register_arrangement("pre_norm", [](const LayerSpec& layer, BuildContext& build) {
        return std::unique_ptr<Arrangement>(new PreNormBlock(layer, build));
    });
}

}  // namespace qe
