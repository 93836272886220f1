// SwiGLU feed-forward: y = Wd (silu(Wg x) * (Wu x)).
//
// Reference: src/qwen_model.cpp:1170-1189 (gate and up as one grouped product, the activation, down),
// src/gpu_ops.hip:103-114 (silu(g) * u with g / (1 + exp(-g))).
#include "linear.h"
#include "parts.h"

namespace qe {

// params: hidden_size, intermediate_size, names{gate_proj, up_proj, down_proj}.
class SwiGLU : public FeedForward {
public:
    SwiGLU(const Json& p, BuildContext& b)
        : FeedForward(p, b), hidden_(p.at("hidden_size").as_int()), inter_(p.at("intermediate_size").as_int()),
          gemm_(b.options.get_string("gemm", "auto")) {}

    std::vector<TensorSpec> tensor_specs() const override {
        return {{name_of("gate_proj"), {inter_, hidden_}, Role::Matrix, Init::Normal},
                {name_of("up_proj"), {inter_, hidden_}, Role::Matrix, Init::Normal},
                {name_of("down_proj"), {hidden_, inter_}, Role::Matrix, Init::Normal}};
    }

    void bind(WeightSource& src) override {
        Tensor gate = src.fetch(name_of("gate_proj")), up = src.fetch(name_of("up_proj"));
        if (gate.dtype != up.dtype) throw WeightError(name_of("gate_proj") + " and " + name_of("up_proj") + " are stored in different precisions");
        // gate and up rows interleaved (g0, u0, g1, u1, ...) in one matrix: one product, and matching pairs sit
        // side by side, so the activation can run in the product's epilogue (a layout choice only)
        Tensor both = src.arena().alloc(gate.dtype, {2 * inter_, hidden_});
        const size_t row = (size_t)hidden_ * dtype_size(gate.dtype);
        QE_CUDA(cudaMemcpy2DAsync(both.data, 2 * row, gate.data, row, row, (size_t)inter_, cudaMemcpyDeviceToDevice, src.stream()));
        QE_CUDA(cudaMemcpy2DAsync(static_cast<char*>(both.data) + row, 2 * row, up.data, row, row, (size_t)inter_,
                                  cudaMemcpyDeviceToDevice, src.stream()));
        QE_CUDA(cudaStreamSynchronize(src.stream()));
        src.release(gate);
        src.release(up);
        gate_up_ = Linear(both, "gate_up_proj", gemm_);
        down_ = Linear(src.fetch(name_of("down_proj")), "down_proj", gemm_);
    }

    std::vector<std::string> required_libraries() const override {
        return (gate_up_.fast() || down_.fast()) ? std::vector<std::string>{"core", "gemm100"} : std::vector<std::string>{"core"};
    }

    // bfloat16: the gate/up product's epilogue applies the norm's factor per row before the activation
    bool takes_unscaled_rows(const StepContext& ctx) const override {
        return compute_dtype == DType::BF16 && gate_up_.applies_row_scale(ctx.T, compute_dtype, true);
    }

    Addend forward(const Tensor& x, StepContext& ctx) override {
        const int T = ctx.T;
        Addend gu = gate_up_(x, ctx, "gate_up", compute_dtype, T, true, true, nullptr, &ctx.row_scale);
        Tensor act;
        if (gu.activated) act = gu.tensor;
        else {
            act = ctx.workspace->get("ff_act", {T, inter_}, compute_dtype);
            const CoreKernels& k = core_kernels();
            QE_LAUNCH(k, k.swiglu(gu.tensor.data, gu.tensor.code(), gu.splits, (long long)T * 2 * inter_, act.data, act.code(), T,
                                  (int)inter_, ctx.stream));
        }
        return down_(act, ctx, "ff_out", DType::F32, T, true, false, ctx.residual, nullptr, &ctx.norm_ahead);
    }

private:
    int64_t hidden_, inter_;
    std::string gemm_;
    Linear gate_up_, down_;
};

void register_feed_forward_parts() {
    register_part("feed_forward", "swiglu", [](const Json& p, BuildContext& b) { return std::make_shared<SwiGLU>(p, b); });
}

}  // namespace qe
