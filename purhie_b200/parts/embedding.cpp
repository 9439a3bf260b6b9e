// Token embedding and output head.
//
// x[t] = table[token[t]] (src/qwen_model.cpp:1234-1244), times `scale` where a design has one; logits = W_out xn for the rows that are
// asked for only (src/qwen_model.cpp:1421-1486).  A tied head shares the embedding table
// (src/inference.cpp:1392-1396).
#include "linear.h"
#include "parts.h"

namespace qe {

// params: vocab_size, hidden_size, scale (default 1), norm (null, or a norm as {kind, params} that the gathered rows pass
// through, in float32 and in place, before they become the residual stream), names{weight}.
class TokenEmbedding : public Embedding {
public:
    TokenEmbedding(const Json& p, BuildContext& b)
        : Embedding(p, b), vocab_(p.at("vocab_size").as_int()), hidden_(p.at("hidden_size").as_int()), scale_(p.get_double("scale", 1.0)) {
        if (const Json* n = p.find("norm"))
            if (!n->is_null()) norm_ = make_part_as<Norm>("norm", PartSpec::from_json(*n), b);
    }
    std::vector<TensorSpec> tensor_specs() const override { return {{name_of("weight"), {vocab_, hidden_}, Role::Matrix, Init::Normal}}; }
    void bind(WeightSource& src) override {
        table_ = src.fetch(name_of("weight"));
        if (norm_) norm_->bind(src);
    }
    std::vector<Part*> children() override { return norm_ ? std::vector<Part*>{norm_.get()} : std::vector<Part*>{}; }
    Tensor forward(StepContext& ctx) override {
        Tensor x = ctx.workspace->get("residual", {ctx.T, hidden_}, DType::F32);
        const CoreKernels& k = core_kernels();
        if (scale_ == 1.0)
            QE_LAUNCH(k, k.embed_gather(table_.data, table_.code(), ctx.token_ids, x.as<float>(), ctx.T, (int)hidden_, (int)vocab_, ctx.stream));
        else
            QE_LAUNCH(k, k.embed_gather_scaled(table_.data, table_.code(), ctx.token_ids, x.as<float>(), ctx.T, (int)hidden_, (int)vocab_,
                                               (float)scale_, ctx.stream));
        if (norm_) norm_->apply_in_place(x, ctx, ctx.T);
        return x;
    }
private:
    int64_t vocab_, hidden_;
    double scale_;
    Tensor table_;
    std::shared_ptr<Norm> norm_;
};

// params: hidden_size, vocab_size, and either names{weight} or tied_to (a tensor another part reads); ignore: names
// that may be present in a checkpoint and are not read (a stray lm_head.weight beside a tied head); scale (default 1)
// and softcap (null: none): logits <- softcap * tanh(logits * scale / softcap), in float32.
class LMHead : public Head {
public:
    LMHead(const Json& p, BuildContext& b) : Head(p, b), hidden_(p.at("hidden_size").as_int()), vocab_(p.at("vocab_size").as_int()) {
        tied_to_ = p.get_string("tied_to", "");
        scale_ = p.get_double("scale", 1.0);
        if (const Json* cap = p.find("softcap"))
            if (!cap->is_null()) softcap_ = cap->as_double();
        if (softcap_ < 0.0) throw ConfigError("lm_head: softcap must be positive");
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
        Tensor logits = proj_(xn, ctx, "logits", DType::F32, n_rows).tensor;
        if (scale_ != 1.0 || softcap_ > 0.0) {
            const CoreKernels& k = core_kernels();
            if (LaunchProfile::get().on()) LaunchProfile::get().note_cost(8.0 * n_rows * vocab_, 0.0);
            QE_LAUNCH(k, k.scale_softcap(logits.as<float>(), (long long)n_rows * vocab_, (float)scale_, (float)softcap_, ctx.stream));
        }
        return logits;
    }
private:
    int64_t hidden_, vocab_;
    double scale_ = 1.0, softcap_ = 0.0;
    std::string tied_to_, gemm_;
    std::vector<std::string> ignore_;
    Linear proj_;
};

void register_embedding_parts() {
    register_part("embedding", "embedding", [](const Json& p, BuildContext& b) { return std::make_shared<TokenEmbedding>(p, b); });
    register_part("head", "lm_head", [](const Json& p, BuildContext& b) { return std::make_shared<LMHead>(p, b); });
}

}  // namespace qe
