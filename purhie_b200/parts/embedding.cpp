// Token embedding and output head.
//
// x[t] = table[token[t]] without scaling (src/qwen_model.cpp:1234-1244); logits = W_out xn for the rows that are
// asked for only (src/qwen_model.cpp:1421-1486).  A tied head shares the embedding table
// (src/inference.cpp:1392-1396).
#include "linear.h"
#include "parts.h"

namespace qe {

// params: vocab_size, hidden_size, names{weight}.
class TokenEmbedding : public Embedding {
public:
    TokenEmbedding(const Json& p, BuildContext& b)
        : Embedding(p, b), vocab_(p.at("vocab_size").as_int()), hidden_(p.at("hidden_size").as_int()) {}
    std::vector<TensorSpec> tensor_specs() const override { return {{name_of("weight"), {vocab_, hidden_}, Role::Matrix, Init::Normal}}; }
    void bind(WeightSource& src) override { table_ = src.fetch(name_of("weight")); }
    Tensor forward(StepContext& ctx) override {
        Tensor x = ctx.workspace->get("residual", {ctx.T, hidden_}, DType::F32);
        const CoreKernels& k = core_kernels();
        QE_LAUNCH(k, k.embed_gather(table_.data, table_.code(), ctx.token_ids, x.as<float>(), ctx.T, (int)hidden_, (int)vocab_, ctx.stream));
        return x;
    }
private:
    int64_t vocab_, hidden_;
    Tensor table_;
};

// params: hidden_size, vocab_size, and either names{weight} or tied_to (a tensor another part reads); ignore: names
// that may be present in a checkpoint and are not read (a stray lm_head.weight beside a tied head).
class LMHead : public Head {
public:
    LMHead(const Json& p, BuildContext& b) : Head(p, b), hidden_(p.at("hidden_size").as_int()), vocab_(p.at("vocab_size").as_int()) {
        tied_to_ = p.get_string("tied_to", "");
        if (const Json* ig = p.find("ignore"))
            for (const Json& n : ig->items()) ignore_.push_back(n.as_string());
        gemm_ = b.options.get_string("gemm", "auto");
    }
    std::vector<TensorSpec> tensor_specs() const override {
        if (!tied_to_.empty()) return {};
        return {{name_of("weight"), {vocab_, hidden_}, Role::Matrix, Init::Normal}};
    }
    std::vector<std::string> ignored_tensors() const override { return ignore_; }
    void bind(WeightSource& src) override { proj_ = Linear(src.fetch(tied_to_.empty() ? name_of("weight") : tied_to_), "lm_head", gemm_); }
    std::vector<std::string> required_libraries() const override { return proj_.defined() ? proj_.required_libraries() : std::vector<std::string>{"core"}; }
    Tensor forward(const Tensor& xn, StepContext& ctx, int n_rows) override {
        return proj_(xn, ctx, "logits", DType::F32, n_rows).tensor;
    }
private:
    int64_t hidden_, vocab_;
    std::string tied_to_, gemm_;
    std::vector<std::string> ignore_;
    Linear proj_;
};

void register_embedding_parts() {
    register_part("embedding", "embedding", [](const Json& p, BuildContext& b) { return std::make_shared<TokenEmbedding>(p, b); });
    register_part("head", "lm_head", [](const Json& p, BuildContext& b) { return std::make_shared<LMHead>(p, b); });
}

}  // namespace qe
