// How a layer's parts are strung together.
//
// pre_norm: x += mixer(norm1(x)); x += feed_forward(norm2(x)), with each addition folded into the norm that
// follows it (the reference fuses them the same way: src/qwen_model.cpp:1175-1187, 1248, 1260).  Sub-parts by
// name: mixer_norm, mixer, feed_forward_norm, feed_forward (a layer may come without the last two).  With the layer
// param "residual_factor" m != 1 the layer is x += m * mixer(norm1(x)); x += m * feed_forward(norm2(x)): the factor
// travels with each part's addend as its transform, and whoever folds the addend in applies it.
//
// sandwich_norm: x += m * post_norm(mixer(norm1(x))); x += m * post_norm2(feed_forward(norm2(x))), a norm in front of
// and behind each part and a factor m on what is added (layer param "residual_factor", default 1).  The norm behind
// a part and the factor travel with the part's addend as its transform, and the next norm's kernel applies them in
// the pass in which it adds and norms, so a layer still launches two norm kernels.  Sub-parts by name: mixer_norm,
// mixer, mixer_post_norm, and, unless the layer has no feed-forward, feed_forward_norm, feed_forward,
// feed_forward_post_norm.
//
// parallel: h = norm(x); x += mixer(h) + feed_forward(h): one norm, and both parts read what it gives (the feed-forward is
// optional).  The two addends wait side by side in the stream and the next norm folds both in its one pass.  Sub-parts
// by name: norm, mixer, feed_forward.
//
// reinject: x <- W [x ; e] + step[pass], e the rows the embedding gave (the model keeps them: ModelSpec::
// keep_embedding_output), W [E, 2E], step [passes, E] and pass the run-order entry's LayerCall::pass.  It has no mixer,
// keeps nothing in the cache, and stands in the run order in front of each round of a stretch of layers that runs
// several times.  Layer params: hidden_size, passes, names{weight, step}.
#include "linear.h"
#include "parts.h"

namespace qe {

class PreNormBlock : public Arrangement {
public:
    PreNormBlock(const LayerSpec& layer, BuildContext& build) {
        mixer_norm_ = make_part_as<Norm>("norm", layer.part("mixer_norm"), build);
        mixer_ = make_part_as<Mixer>("mixer", layer.part("mixer"), build);
        if (layer.has("feed_forward")) {
            ff_norm_ = make_part_as<Norm>("norm", layer.part("feed_forward_norm"), build);
            ff_ = make_part_as<FeedForward>("feed_forward", layer.part("feed_forward"), build);
        }
        factor_ = (float)layer.params.get_double("residual_factor", 1.0);
    }
    std::vector<Part*> parts() override {
        std::vector<Part*> p = {mixer_norm_.get(), mixer_.get()};
        if (ff_) { p.push_back(ff_norm_.get()); p.push_back(ff_.get()); }
        return p;
    }
    CacheNeed cache_need() const override { return mixer_->cache_need(); }
    void forward(ResidualStream& stream, StepContext& ctx, const CacheView& cache) override {
        if (factor_ != 1.0f) return forward_scaled(stream, ctx, cache);
        ctx.residual = stream.x.as<float>();
        ctx.residual_width = stream.x.shape[1];
        // a consumer that applies the row's factor itself lets the norm in front leave it out (RowScale)
        // (the option "row_factor": "norm" keeps the factor in the norm, for comparing the two forms)
        const bool may_defer = ctx.option("row_factor") != "norm";
        // and a part whose last product adds into the residual itself may do the pass of the norm behind it there
        // (NormAhead; the option "norm_ahead": "off" keeps every norm a kernel of its own)
        const bool may_work_ahead = may_defer && ctx.option("norm_ahead") != "off";
        const bool ff_unscaled = ff_ && may_defer && ff_->takes_unscaled_rows(ctx);
        ctx.row_scale = RowScale();
        Tensor xn = may_defer && mixer_->takes_unscaled_rows(ctx) ? mixer_norm_->forward_unscaled(stream, ctx, &ctx.row_scale)
                                                                  : mixer_norm_->forward(stream, ctx);
        ctx.norm_ahead = may_work_ahead && ff_unscaled ? ff_norm_->offer(ctx) : (!ff_ && may_work_ahead) ? ctx.next_layer_norm : NormAhead();
        stream.add(mixer_->forward(xn, ctx, cache));
        stream.prepare(ctx.norm_ahead);
        ctx.row_scale = RowScale();
        if (!ff_) { ctx.norm_ahead = NormAhead(); return; }
        xn = ff_unscaled ? ff_norm_->forward_unscaled(stream, ctx, &ctx.row_scale) : ff_norm_->forward(stream, ctx);
        ctx.norm_ahead = may_work_ahead ? ctx.next_layer_norm : NormAhead();
        stream.add(ff_->forward(xn, ctx));
        stream.prepare(ctx.norm_ahead);
        ctx.row_scale = RowScale();
        ctx.norm_ahead = NormAhead();
    }
    NormAhead first_norm(const StepContext& ctx) const override {
        const bool may_defer = ctx.option("row_factor") != "norm";
        return factor_ == 1.0f && may_defer && mixer_->takes_unscaled_rows(ctx) ? mixer_norm_->offer(ctx) : NormAhead();
    }
private:
    // What a part gives is multiplied by the factor on its way into the residual, so no product adds into the residual
    // itself and no norm's work is handed to a product: every part returns its addend, which carries the factor.
    void forward_scaled(ResidualStream& stream, StepContext& ctx, const CacheView& cache) {
        ctx.residual = nullptr;
        ctx.residual_width = 0;
        ctx.row_scale = RowScale();
        ctx.norm_ahead = NormAhead();
        Tensor xn = mixer_norm_->forward(stream, ctx);
        Addend mixed = mixer_->forward(xn, ctx, cache);
        if (!mixed.tensor.defined()) throw Error(kInvalidState, "pre_norm: the mixer added into the residual itself");
        mixed.transform.factor *= factor_;
        stream.add(std::move(mixed));
        if (!ff_) return;
        xn = ff_norm_->forward(stream, ctx);
        Addend fed = ff_->forward(xn, ctx);
        if (!fed.tensor.defined()) throw Error(kInvalidState, "pre_norm: the feed-forward added into the residual itself");
        fed.transform.factor *= factor_;
        stream.add(std::move(fed));
    }
    float factor_ = 1.0f;
    std::shared_ptr<Norm> mixer_norm_, ff_norm_;
    std::shared_ptr<Mixer> mixer_;
    std::shared_ptr<FeedForward> ff_;
};

class SandwichNormBlock : public Arrangement {
public:
    SandwichNormBlock(const LayerSpec& layer, BuildContext& build) {
        factor_ = (float)layer.params.get_double("residual_factor", 1.0);
        mixer_norm_ = make_part_as<Norm>("norm", layer.part("mixer_norm"), build);
        mixer_ = make_part_as<Mixer>("mixer", layer.part("mixer"), build);
        mixer_post_ = make_part_as<Norm>("norm", layer.part("mixer_post_norm"), build);
        if (layer.has("feed_forward")) {
            ff_norm_ = make_part_as<Norm>("norm", layer.part("feed_forward_norm"), build);
            ff_ = make_part_as<FeedForward>("feed_forward", layer.part("feed_forward"), build);
            ff_post_ = make_part_as<Norm>("norm", layer.part("feed_forward_post_norm"), build);
        }
    }
    std::vector<Part*> parts() override {
        std::vector<Part*> p = {mixer_norm_.get(), mixer_.get(), mixer_post_.get()};
        if (ff_) { p.push_back(ff_norm_.get()); p.push_back(ff_.get()); p.push_back(ff_post_.get()); }
        return p;
    }
    CacheNeed cache_need() const override { return mixer_->cache_need(); }
    void forward(ResidualStream& stream, StepContext& ctx, const CacheView& cache) override {
        // what a part gives is normed before it is added: no product adds into the residual behind this block's back,
        // and no norm's work is handed to a product
        ctx.residual = nullptr;
        ctx.residual_width = 0;
        ctx.row_scale = RowScale();
        ctx.norm_ahead = NormAhead();
        Tensor xn = mixer_norm_->forward(stream, ctx);
        Addend mixed = mixer_->forward(xn, ctx, cache);
        if (!mixed.tensor.defined()) throw Error(kInvalidState, "sandwich_norm: the mixer added into the residual itself");
        mixed.transform = mixer_post_->as_transform(factor_);
        stream.add(std::move(mixed));
        if (!ff_) return;
        xn = ff_norm_->forward(stream, ctx);
        Addend fed = ff_->forward(xn, ctx);
        if (!fed.tensor.defined()) throw Error(kInvalidState, "sandwich_norm: the feed-forward added into the residual itself");
        fed.transform = ff_post_->as_transform(factor_);
        stream.add(std::move(fed));
    }
private:
    float factor_ = 1.0f;
    std::shared_ptr<Norm> mixer_norm_, mixer_post_, ff_norm_, ff_post_;
    std::shared_ptr<Mixer> mixer_;
    std::shared_ptr<FeedForward> ff_;
};

class ParallelBlock : public Arrangement {
public:
    ParallelBlock(const LayerSpec& layer, BuildContext& build) {
        norm_ = make_part_as<Norm>("norm", layer.part("norm"), build);
        mixer_ = make_part_as<Mixer>("mixer", layer.part("mixer"), build);
        if (layer.has("feed_forward")) ff_ = make_part_as<FeedForward>("feed_forward", layer.part("feed_forward"), build);
    }
    std::vector<Part*> parts() override {
        std::vector<Part*> p = {norm_.get(), mixer_.get()};
        if (ff_) p.push_back(ff_.get());
        return p;
    }
    CacheNeed cache_need() const override { return mixer_->cache_need(); }
    void forward(ResidualStream& stream, StepContext& ctx, const CacheView& cache) override {
        // both parts read the same finished rows; a product may add into the residual itself (the rows are made by then),
        // but no norm's work is handed to it: the rows behind this layer are the sum of two addends
        ctx.row_scale = RowScale();
        ctx.norm_ahead = NormAhead();
        Tensor h = norm_->forward(stream, ctx);
        ctx.residual = stream.x.as<float>();
        ctx.residual_width = stream.x.shape[1];
        stream.add(mixer_->forward(h, ctx, cache));
        if (ff_) {
            Addend fed = ff_->forward(h, ctx);
            if (stream.has_pending) stream.add_also(std::move(fed));
            else stream.add(std::move(fed));
        }
    }
private:
    std::shared_ptr<Norm> norm_;
    std::shared_ptr<Mixer> mixer_;
    std::shared_ptr<FeedForward> ff_;
};

// The weights of a reinjection, as a part so that the loader, the folder check and random weights see them.
class ReinjectWeights : public Part {
public:
    ReinjectWeights(const Json& p, BuildContext& b)
        : Part(p, b), hidden_(p.at("hidden_size").as_int()), passes_(p.at("passes").as_int()), gemm_(b.options.get_string("gemm", "auto")) {
        if (hidden_ < 1 || passes_ < 1) throw ConfigError("reinject: hidden_size and passes must be positive");
    }
    std::vector<TensorSpec> tensor_specs() const override {
        return {{name_of("weight"), {hidden_, 2 * hidden_}, Role::Matrix, Init::Normal}, {name_of("step"), {passes_, hidden_}, Role::Vector, Init::Normal}};
    }
    void bind(WeightSource& src) override {
        proj = Linear(src.fetch(name_of("weight")), "reinject", gemm_);
        step = src.fetch(name_of("step"));
    }
    std::vector<std::string> required_libraries() const override { return proj.defined() ? proj.required_libraries() : std::vector<std::string>{"core"}; }
    int64_t hidden_, passes_;
    std::string gemm_;
    Linear proj;
    Tensor step;
};

class ReinjectBlock : public Arrangement {
public:
    ReinjectBlock(const LayerSpec& layer, BuildContext& build) : weights_(std::make_shared<ReinjectWeights>(layer.params, build)) {}
    std::vector<Part*> parts() override { return {weights_.get()}; }
    CacheNeed cache_need() const override { return CacheNeed(); }
    void forward(ResidualStream& stream, StepContext& ctx, const CacheView&) override {
        if (!ctx.embedding_output) throw Error(kInvalidState, "reinject: the model does not keep what the embedding gave");
        if (ctx.pass < 0 || ctx.pass >= weights_->passes_) throw Error(kInvalidState, "reinject: pass " + std::to_string(ctx.pass) + " of " + std::to_string(weights_->passes_));
        const int64_t E = weights_->hidden_;
        if (stream.has_pending && stream.pending.transform.defined()) fold_all_addends(stream, ctx);
        const DType dt = weights_->compute_dtype;
        Tensor cat = ctx.workspace->get("reinject_rows", {ctx.T, 2 * E}, dt);
        const CoreKernels& k = core_kernels();
        const Addend* a = stream.has_pending ? &stream.pending : nullptr;
        const Addend* b = stream.has_also ? &stream.also : nullptr;
        if (LaunchProfile::get().on()) {
            double bytes = (double)ctx.T * E * (12.0 + 2.0 * dtype_size(dt));
            if (a) bytes += (double)a->splits * ctx.T * E * dtype_size(a->tensor.dtype);
            if (b) bytes += (double)b->splits * ctx.T * E * dtype_size(b->tensor.dtype);
            LaunchProfile::get().note_cost(bytes, 0.0);
        }
        // cat = [x + what waits | e]; x restarts as the pass's step vector, and the product over cat is added to it
        QE_LAUNCH(k, k.concat_restart(stream.x.as<float>(), a ? a->tensor.data : nullptr, a ? a->tensor.code() : 0, a ? a->splits : 1,
                                      a ? (long long)ctx.T * E : 0, b ? b->tensor.data : nullptr, b ? b->tensor.code() : 0, b ? b->splits : 1,
                                      b ? (long long)ctx.T * E : 0, ctx.embedding_output, weights_->step.as<float>() + (size_t)ctx.pass * E,
                                      cat.data, cat.code(), ctx.T, (int)E, ctx.stream));
        stream.clear();
        ctx.residual = stream.x.as<float>();
        ctx.residual_width = E;
        ctx.row_scale = RowScale();
        ctx.norm_ahead = NormAhead();
        stream.add(weights_->proj(cat, ctx, "reinject_out", DType::F32, ctx.T, true, false, ctx.residual));
    }
private:
    std::shared_ptr<ReinjectWeights> weights_;
};

void register_norm_parts();
void register_routed_parts();
void register_state_space_parts();
void register_linear_attention_parts();
void register_recurrent_parts();
void register_latent_attention_parts();
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
    register_routed_parts();
    register_state_space_parts();
    register_linear_attention_parts();
    register_recurrent_parts();
    register_latent_attention_parts();
    register_arrangement("sandwich_norm", [](const LayerSpec& layer, BuildContext& build) {
        return std::unique_ptr<Arrangement>(new SandwichNormBlock(layer, build));
    });
    register_arrangement("parallel", [](const LayerSpec& layer, BuildContext& build) {
        return std::unique_ptr<Arrangement>(new ParallelBlock(layer, build));
    });
    register_arrangement("reinject", [](const LayerSpec& layer, BuildContext& build) {
        return std::unique_ptr<Arrangement>(new ReinjectBlock(layer, build));
    });
    register_arrangement("pre_norm", [](const LayerSpec& layer, BuildContext& build) {
        return std::unique_ptr<Arrangement>(new PreNormBlock(layer, build));
    });
}

}  // namespace qe
