// y = x W^T for a weight stored [out_features, in_features], and the choice of the kernel that does it.
//
// float32 weights go through the exact-order CUDA-core kernel (the 32-bit path; also a 32-bit tensor met in a
// bfloat16 model).  bfloat16 weights go through the tcgen05 tensor-core kernel when it takes the shape, else
// through the plain kernel.  The reference picks a kernel by weight type and batch size the same way
// (qmatvec_launch, src/qmatvec.cpp:274; matvec / matvec_multi, src/qwen_model.cpp:855-922).
#pragma once

#include <string>

#include "parts.h"

namespace qe {

struct GemmPlan {
    bool swapped = false;    // weights on the 128-row side of the instruction, tokens on the other (few tokens)
    int block_n = 256;
    int splits = 1;          // parts of K, float32 partial sums
    bool pair = false;       // 256 x 256 tiles on pairs of CTAs
};
// The shape of the tcgen05 product for M tokens and an [N, K] weight on a device of `sms` SMs.
QE_API GemmPlan plan_gemm(int M, int N, int K, int sms, bool allow_split, bool fused_epilogue);

class QE_API Linear {
public:
    Linear() = default;
    // gemm: "auto" (tcgen05 where it takes the shape), "tcgen05" (demand it), "simple" (never)
    Linear(Tensor weight, std::string label, const std::string& gemm);
    bool defined() const { return weight_.defined(); }
    bool fast() const { return fast_; }
    int64_t out_features() const { return weight_.shape[0]; }
    int64_t in_features() const { return weight_.shape[1]; }
    const Tensor& weight() const { return weight_; }
    std::vector<std::string> required_libraries() const;
    // x [rows, in] -> Addend of [rows, out] in out_dtype (float32 partial sums [splits, rows, out] when K is
    // split).  fuse_swiglu: the weight holds (gate, up) row pairs; where the kernel can, it applies the activation
    // in its epilogue and the result [rows, out / 2] comes back marked activated.  add_into (float32 [rows, out]):
    // where the kernel can add the product there in its epilogue it does, and the addend comes back empty.
    // scale: the rows of x lack a factor per row (RowScale); only where applies_row_scale() is true, and then the
    // kernel's epilogue multiplies by it.  ahead (with add_into, for a part's last product): the norm that follows
    // the addition; where the kernel adds in its epilogue and can, it fills ahead->rows and ahead->scale (NormAhead).
    Addend operator()(const Tensor& x, StepContext& ctx, const std::string& out_name, DType out_dtype, int rows,
                      bool allow_split = false, bool fuse_swiglu = false, float* add_into = nullptr,
                      const RowScale* scale = nullptr, NormAhead* ahead = nullptr) const;
    // Few rows on the tensor-core kernel: the weight fills the wide side of the instruction (what plan_gemm calls
    // swapped).  Its partial sums are linear in the rows, and its bfloat16 epilogue can apply a factor per row.
    bool swapped_for(int rows, bool allow_split, bool fused_epilogue) const;
    // The product's own epilogue multiplies by the rows' factor: few rows with the fused activation; many rows
    // (tiles of 256 features) whenever K stays whole and nothing is added into the output.
    bool applies_row_scale(int rows, DType out_dtype, bool fuse_swiglu, bool allow_split = true) const;
    // Many rows, K cut into parts: float32 partial sums, linear in the rows, so whoever adds them up can apply the factor.
    bool gives_partial_sums(int rows, bool allow_split) const;
private:
    Tensor weight_;
    std::string label_;
    bool fast_ = false;
};

}  // namespace qe
