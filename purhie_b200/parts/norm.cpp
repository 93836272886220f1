// RMSNorm with the residual add folded in.
//
// y = v * rsqrt(mean(v^2) + eps) * w, v = x + pending addend; the weight multiplies after normalising (plain w,
// not 1 + w).  Reference: src/gpu_ops.hip:24-56 (add + norm in one kernel), src/qwen_ops.cpp:8-13.
#include "parts.h"

namespace qe {

// params: size, eps, names{weight}.
class RMSNorm : public Norm {
public:
    RMSNorm(const Json& p, BuildContext& b) : Norm(p, b), size_(p.at("size").as_int()), eps_(p.at("eps").as_double()) {
        if (size_ < 1 || !(eps_ > 0)) throw ConfigError("rmsnorm: size must be positive and eps > 0");
    }
    std::vector<TensorSpec> tensor_specs() const override { return {{name_of("weight"), {size_}, Role::Vector, Init::Scale}}; }
    void bind(WeightSource& src) override { weight_ = src.fetch(name_of("weight")); }

    Tensor forward(ResidualStream& stream, StepContext& ctx, const int32_t* rows, int n_rows) override {
        const int n = rows ? n_rows : ctx.T;
        Tensor out = ctx.workspace->get(rows ? "normed_rows" : "normed", {n, size_}, compute_dtype);
        const CoreKernels& k = core_kernels();
        const Addend* pend = stream.has_pending ? &stream.pending : nullptr;
        QE_LAUNCH(k, k.add_rmsnorm(stream.x.as<float>(), pend ? pend->tensor.data : nullptr, pend ? pend->tensor.code() : 0,
                                   pend ? pend->splits : 1, pend ? (long long)ctx.T * size_ : 0, weight_.as<float>(),
                                   (float)eps_, rows, n, (int)size_, out.data, out.code(), rows ? 0 : 1, ctx.stream));
        if (!rows) stream.clear();
        return out;
    }

    // The few-row form: x += addend, y = x * weight, and the row's sum of squares in chunks for the consumer to turn
    // into the factor (bfloat16 model, rows of a multiple of four elements; else the ordinary form).
    Tensor forward_unscaled(ResidualStream& stream, StepContext& ctx, RowScale* scale) override {
        *scale = RowScale();
        if (stream.prepared.done() && stream.prepared.norm == this && !stream.has_pending) {
            // the product that added into the stream did this norm's pass in its epilogue
            Tensor rows = stream.prepared.rows;
            *scale = stream.prepared.scale;
            stream.clear();
            return rows;
        }
        if (compute_dtype != DType::BF16 || size_ % 4) return forward(stream, ctx, nullptr, 0);
        constexpr int kChunk = 512;                                   // columns per CTA of the kernel
        const int chunks = (int)((size_ + kChunk - 1) / kChunk);
        Tensor out = ctx.workspace->get("normed", {ctx.T, size_}, compute_dtype);
        Tensor sumsq = ctx.workspace->get("normed_sumsq", {ctx.T, chunks}, DType::F32);
        const CoreKernels& k = core_kernels();
        const Addend* pend = stream.has_pending ? &stream.pending : nullptr;
        QE_LAUNCH(k, k.add_weight_sumsq(stream.x.as<float>(), pend ? pend->tensor.data : nullptr, pend ? pend->tensor.code() : 0,
                                        pend ? pend->splits : 1, pend ? (long long)ctx.T * size_ : 0, weight_.as<float>(), ctx.T,
                                        (int)size_, out.data, out.code(), sumsq.as<float>(), chunks, ctx.stream));
        stream.clear();
        scale->sumsq = sumsq.as<float>(); scale->chunks = chunks; scale->width = (int)size_; scale->eps = (float)eps_;
        return out;
    }

    NormAhead offer(const StepContext&) const override {
        NormAhead a;
        if (compute_dtype != DType::BF16 || size_ % 4) return a;
        a.weight = weight_.as<float>(); a.norm = this; a.width = (int)size_; a.eps = (float)eps_;
        return a;
    }

private:
    int64_t size_;
    double eps_;
    Tensor weight_;
};

void register_norm_parts() {
    register_part("norm", "rmsnorm", [](const Json& p, BuildContext& b) { return std::make_shared<RMSNorm>(p, b); });
}

}  // namespace qe
