// Gated linear attention, and two mixers that run side by side on the same input.
//
// gated_linear_attention: per head a matrix state S [dim, value_dim] in float32 that every token first lets decay,
// channel by channel, and then adds an outer product to:
//     q = Wq h * dim^(-1/2), k = Wk h, v = Wv h,  a = sigmoid(Wa2 (Wa1 h) + ba)^(1/tau)      (a per key channel)
//     S <- diag(a) S + k v^T,   o = S^T q
//     y = Wo (rmsnorm(o; per head, one weight for all heads) * silu(Wg h))
// The state lives in the request's state slot (zero at admission, carried from step to step, given back at release),
// so a prompt cut anywhere walks the same recurrence.  The decay (its logits, the logarithm of the sigmoid, the
// exponential), S, o, the head norm and the gate are float32 in every mode; the products follow the model's dtype,
// the decay's second product writes float32.  q, k, v and g come from one product over the stacked matrices.
//
// lightning_attention: the same matrix state with one constant decay per head and no logits:
//     q = silu(Wq h), k = silu(Wk h), v = silu(Wv h),   S <- decay[head] S + k v^T,   o = S^T q
//     y = Wo (rmsnorm(o; over all heads' values as one row, a weight per element) * sigmoid(Wg h))
// It shares the recurrence's kernel (the decay as a constant, the activations on the way in, o left raw) and the chunk
// lists with gated_linear_attention; the norm over the whole row and the gate are a kernel behind it.
//
// side_by_side: y = factor * (rmsnorm(left(h); w_left) + rmsnorm(right(h); w_right)), both norms over the model
// width; or, with "combine": "weighted_sum", y = left_factor * left(h) + right_factor * right(h) without norms (and
// without norm tensors).  "left" and "right" are mixers of any registered kind, given as {kind, params}; one of them may keep pages
// and one a state (CacheNeed::both), and each finds what it keeps in the layer's cache view.
#include <algorithm>
#include <cmath>

#include "linear.h"
#include "parts.h"

namespace qe {

// The chunk list of a step for the recurrence's kernel ("decayed.chunks", "decayed.seg_chunks"): every request's rows in
// chunks of `chunk` tokens when the longest portion has `from` tokens or more.  Shared by the mixers that use the kernel.
namespace {
void add_scan_chunks(StepPlan& plan, int chunk, int from) {
    if (plan.has("decayed.chunks")) return;
    int longest = 0;
    for (int n : plan.q_lens) longest = std::max(longest, n);
    if (longest < from) return;
    std::vector<int32_t> items, seg_items = {0};
    int row = 0;
    for (int s = 0; s < plan.S; s++) {
        const int n = plan.q_lens[s];
        for (int at = 0; at < n; at += chunk) {
            items.push_back(row + at); items.push_back(std::min(chunk, n - at)); items.push_back(s); items.push_back(at + chunk >= n);
        }
        row += n;
        seg_items.push_back((int32_t)(items.size() / 4));
    }
    plan.add("decayed.chunks", std::move(items));
    plan.add("decayed.seg_chunks", std::move(seg_items));
}
}  // namespace

// params: hidden_size, num_heads, head_dim, value_dim, decay_rank (null: the stored matrices' inner size), tau, norm_eps,
// names{q_proj, k_proj, v_proj, g_proj, o_proj, norm, decay_down, decay_up, decay_bias}.
class GatedLinearAttention : public Mixer {
public:
    GatedLinearAttention(const Json& p, BuildContext& b) : Mixer(p, b) {
        hidden_ = p.at("hidden_size").as_int();
        heads_ = (int)p.at("num_heads").as_int();
        dim_ = (int)p.at("head_dim").as_int();
        vdim_ = (int)p.at("value_dim").as_int();
        rank_ = p.get_int("decay_rank", -1);
        tau_ = p.at("tau").as_double();
        eps_ = p.at("norm_eps").as_double();
        if (heads_ < 1 || dim_ < 1 || vdim_ < 1 || rank_ == 0 || rank_ < -1) throw ConfigError("gated_linear_attention: heads, head_dim, value_dim and decay_rank must be positive");
        if (!(tau_ > 0)) throw ConfigError("gated_linear_attention: tau must be positive");
        gemm_ = b.options.get_string("gemm", "auto");
        key_width_ = (int64_t)heads_ * dim_;
        value_width_ = (int64_t)heads_ * vdim_;
    }

    std::vector<TensorSpec> tensor_specs() const override {
        return {{name_of("q_proj"), {key_width_, hidden_}, Role::Matrix, Init::Normal},
                {name_of("k_proj"), {key_width_, hidden_}, Role::Matrix, Init::Normal},
                {name_of("v_proj"), {value_width_, hidden_}, Role::Matrix, Init::Normal},
                {name_of("g_proj"), {value_width_, hidden_}, Role::Matrix, Init::Normal},
                {name_of("o_proj"), {hidden_, value_width_}, Role::Matrix, Init::Normal},
                {name_of("norm"), {vdim_}, Role::Vector, Init::Scale},
                {name_of("decay_down"), {rank_, hidden_}, Role::Matrix, Init::Normal},
                {name_of("decay_up"), {key_width_, rank_}, Role::Matrix, Init::Normal},
                {name_of("decay_bias"), {key_width_}, Role::Vector, Init::Normal}};
    }

    void bind(WeightSource& src) override {
        // one matrix [q | k | v | g]: the four projections of h are one product (a layout choice only)
        Tensor parts[4] = {src.fetch(name_of("q_proj")), src.fetch(name_of("k_proj")), src.fetch(name_of("v_proj")), src.fetch(name_of("g_proj"))};
        for (Tensor& t : parts)
            if (t.dtype != parts[0].dtype) throw WeightError("the projections of " + name_of("q_proj") + "'s mixer are stored in different precisions");
        Tensor all = src.arena().alloc(parts[0].dtype, {2 * key_width_ + 2 * value_width_, hidden_});
        size_t off = 0;
        for (Tensor& t : parts) {
            QE_CUDA(cudaMemcpyAsync(static_cast<char*>(all.data) + off, t.data, t.bytes(), cudaMemcpyDeviceToDevice, src.stream()));
            off += t.bytes();
        }
        QE_CUDA(cudaStreamSynchronize(src.stream()));
        for (Tensor& t : parts) src.release(t);
        qkvg_proj_ = Linear(all, "qkvg_proj", gemm_);
        decay_down_ = Linear(src.fetch(name_of("decay_down")), "decay_down", gemm_);
        decay_up_ = Linear(src.fetch(name_of("decay_up")), "decay_up", gemm_);
        if (decay_down_.out_features() != decay_up_.in_features())
            throw WeightError(name_of("decay_down") + " gives " + std::to_string(decay_down_.out_features()) + " values, " + name_of("decay_up") +
                              " takes " + std::to_string(decay_up_.in_features()));
        decay_bias_ = src.fetch(name_of("decay_bias"));
        norm_ = src.fetch(name_of("norm"));
        o_proj_ = Linear(src.fetch(name_of("o_proj")), "o_proj", gemm_);
    }

    std::vector<std::string> required_libraries() const override {
        const bool fast = qkvg_proj_.fast() || decay_down_.fast() || decay_up_.fast() || o_proj_.fast();
        return fast ? std::vector<std::string>{"core", "gemm100"} : std::vector<std::string>{"core"};
    }
    int preferred_row_multiple() const override { return (qkvg_proj_.fast() || o_proj_.fast()) ? 256 : 0; }

    // per head [value_dim][padded head_dim]: the kernel's threads own 16 key channels each, a power of two of them per column
    int64_t padded_dim() const {
        int64_t parts = 1;
        while (parts * 16 < dim_) parts *= 2;
        return parts * 16;
    }
    CacheNeed cache_need() const override { return CacheNeed::state({heads_, vdim_, padded_dim()}, DType::F32); }

    // A step with a long prompt portion cuts every request's rows into chunks for the recurrence (first row, rows, segment,
    // 1 on the request's last chunk) so that a prompt's tokens are spread over the device: the chunk list is this mixer's
    // own metadata, shared by all layers of its kind.
    void prepare_step(StepPlan& plan) override { add_scan_chunks(plan, kChunk, kChunkFrom); }

    Addend forward(const Tensor& x, StepContext& ctx, const CacheView& cache) override {
        const int64_t per_slot = (int64_t)heads_ * padded_dim() * vdim_;
        if (!cache.state.defined() || cache.state.dtype != DType::F32 || cache.state.numel() != (int64_t)cache.state.shape[0] * per_slot)
            throw Error(kInvalidState, "gated_linear_attention: the cache manager gave no state of this mixer's shape");
        const int T = ctx.T;
        const DType dt = compute_dtype;
        Workspace& ws = *ctx.workspace;
        const CoreKernels& k = core_kernels();
        const int64_t width = 2 * key_width_ + 2 * value_width_;
        Tensor qkvg = qkvg_proj_(x, ctx, "gla_qkvg", dt, T).tensor;                       // [T, q | k | v | g]
        Tensor low = decay_down_(x, ctx, "gla_decay_low", dt, T).tensor;                   // [T, rank]
        Tensor z = decay_up_(low, ctx, "gla_decay_logit", DType::F32, T).tensor;           // [T, heads * dim] float32
        Tensor raw = ws.get("gla_o_raw", {T, value_width_}, DType::F32);
        Tensor y = ws.get("gla_o", {T, value_width_}, dt);
        const size_t es = dtype_size(dt);
        char* base = static_cast<char*>(qkvg.data);
        const StepArray chunks = ctx.array("decayed.chunks"), seg_chunks = ctx.array("decayed.seg_chunks");
        const int n_chunks = chunks.count / 4;
        float *carry = nullptr, *decay = nullptr;
        if (n_chunks) {
            carry = ws.get("gla_carry", {n_chunks, heads_, vdim_, padded_dim()}, DType::F32).as<float>();
            decay = ws.get("gla_chunk_decay", {n_chunks, heads_, dim_}, DType::F32).as<float>();
        }
        if (LaunchProfile::get().on())      // q, k, v, g and the decay's logits in, o out twice (raw and gated), the state in and out
            LaunchProfile::get().note_cost((double)T * (width * es + key_width_ * 4.0 + value_width_ * (8.0 + es)) + 2.0 * ctx.S * per_slot * 4.0,
                                           (double)T * heads_ * dim_ * vdim_ * 5.0);
        QE_LAUNCH(k, k.decayed_scan(base, base + key_width_ * es, base + 2 * key_width_ * es, base + (2 * key_width_ + value_width_) * es,
                                    qkvg.code(), width, z.as<float>(), key_width_, decay_bias_.as<float>(), (float)tau_,
                                    (float)(1.0 / std::sqrt((double)dim_)), norm_.as<float>(), (float)eps_, cache.state.as<float>(), per_slot,
                                    ctx.seg_start, ctx.seg_slot, ctx.S, T, heads_, dim_, vdim_, n_chunks ? chunks.data : nullptr, n_chunks,
                                    n_chunks ? seg_chunks.data : nullptr, carry, decay, raw.as<float>(), y.data, nullptr, 0, 0, ctx.stream));
        return o_proj_(y, ctx, "gla_out", DType::F32, T, true, false, ctx.residual, nullptr, &ctx.norm_ahead);
    }

private:
    static constexpr int kChunk = 64;           // tokens of a chunk of the recurrence
    static constexpr int kChunkFrom = 128;      // the longest portion of a step from which the recurrence runs in chunks
    int64_t hidden_, key_width_, value_width_, rank_;
    int heads_, dim_, vdim_;
    double tau_, eps_;
    std::string gemm_;
    Linear qkvg_proj_, decay_down_, decay_up_, o_proj_;
    Tensor decay_bias_, norm_;
};

// params: hidden_size, num_heads, head_dim, value_dim, decay [num_heads] (each in (0, 1]), norm_eps,
// names{q_proj, k_proj, v_proj, g_proj, o_proj, norm}.
class LightningAttention : public Mixer {
public:
    LightningAttention(const Json& p, BuildContext& b) : Mixer(p, b) {
        hidden_ = p.at("hidden_size").as_int();
        heads_ = (int)p.at("num_heads").as_int();
        dim_ = (int)p.at("head_dim").as_int();
        vdim_ = (int)p.at("value_dim").as_int();
        eps_ = p.at("norm_eps").as_double();
        if (heads_ < 1 || dim_ < 1 || vdim_ < 1) throw ConfigError("lightning_attention: heads, head_dim and value_dim must be positive");
        const Json& d = p.at("decay");
        if (!d.is_array() || (int)d.size() != heads_) throw ConfigError("lightning_attention: decay must list one number per head");
        for (const Json& v : d.items()) {
            const double a = v.as_double();
            if (!(a > 0.0) || a > 1.0) throw ConfigError("lightning_attention: a decay must lie in (0, 1]");
            decay_host_.push_back((float)a);
        }
        gemm_ = b.options.get_string("gemm", "auto");
        key_width_ = (int64_t)heads_ * dim_;
        value_width_ = (int64_t)heads_ * vdim_;
    }
    std::vector<TensorSpec> tensor_specs() const override {
        return {{name_of("q_proj"), {key_width_, hidden_}, Role::Matrix, Init::Normal},
                {name_of("k_proj"), {key_width_, hidden_}, Role::Matrix, Init::Normal},
                {name_of("v_proj"), {value_width_, hidden_}, Role::Matrix, Init::Normal},
                {name_of("g_proj"), {value_width_, hidden_}, Role::Matrix, Init::Normal},
                {name_of("o_proj"), {hidden_, value_width_}, Role::Matrix, Init::Normal},
                {name_of("norm"), {value_width_}, Role::Vector, Init::Scale}};
    }
    void bind(WeightSource& src) override {
        // one matrix [q | k | v | g]: the four projections of h are one product (a layout choice only)
        Tensor parts[4] = {src.fetch(name_of("q_proj")), src.fetch(name_of("k_proj")), src.fetch(name_of("v_proj")), src.fetch(name_of("g_proj"))};
        for (Tensor& t : parts)
            if (t.dtype != parts[0].dtype) throw WeightError("the projections of " + name_of("q_proj") + "'s mixer are stored in different precisions");
        Tensor all = src.arena().alloc(parts[0].dtype, {2 * key_width_ + 2 * value_width_, hidden_});
        size_t off = 0;
        for (Tensor& t : parts) {
            QE_CUDA(cudaMemcpyAsync(static_cast<char*>(all.data) + off, t.data, t.bytes(), cudaMemcpyDeviceToDevice, src.stream()));
            off += t.bytes();
        }
        decay_ = src.arena().alloc(DType::F32, {heads_});
        QE_CUDA(cudaMemcpyAsync(decay_.data, decay_host_.data(), decay_host_.size() * sizeof(float), cudaMemcpyHostToDevice, src.stream()));
        QE_CUDA(cudaStreamSynchronize(src.stream()));
        for (Tensor& t : parts) src.release(t);
        qkvg_proj_ = Linear(all, "qkvg_proj", gemm_);
        norm_ = src.fetch(name_of("norm"));
        o_proj_ = Linear(src.fetch(name_of("o_proj")), "o_proj", gemm_);
    }
    std::vector<std::string> required_libraries() const override {
        return (qkvg_proj_.fast() || o_proj_.fast()) ? std::vector<std::string>{"core", "gemm100"} : std::vector<std::string>{"core"};
    }
    int preferred_row_multiple() const override { return (qkvg_proj_.fast() || o_proj_.fast()) ? 256 : 0; }
    int64_t padded_dim() const {
        int64_t parts = 1;
        while (parts * 16 < dim_) parts *= 2;
        return parts * 16;
    }
    CacheNeed cache_need() const override { return CacheNeed::state({heads_, vdim_, padded_dim()}, DType::F32); }
    void prepare_step(StepPlan& plan) override { add_scan_chunks(plan, kChunk, kChunkFrom); }

    Addend forward(const Tensor& x, StepContext& ctx, const CacheView& cache) override {
        const int64_t per_slot = (int64_t)heads_ * padded_dim() * vdim_;
        if (!cache.state.defined() || cache.state.dtype != DType::F32 || cache.state.numel() != (int64_t)cache.state.shape[0] * per_slot)
            throw Error(kInvalidState, "lightning_attention: the cache manager gave no state of this mixer's shape");
        const int T = ctx.T;
        const DType dt = compute_dtype;
        Workspace& ws = *ctx.workspace;
        const CoreKernels& k = core_kernels();
        const int64_t width = 2 * key_width_ + 2 * value_width_;
        Tensor qkvg = qkvg_proj_(x, ctx, "la_qkvg", dt, T).tensor;                         // [T, q | k | v | g]
        Tensor raw = ws.get("la_o_raw", {T, value_width_}, DType::F32);
        Tensor y = ws.get("la_o", {T, value_width_}, dt);
        const size_t es = dtype_size(dt);
        char* base = static_cast<char*>(qkvg.data);
        const StepArray chunks = ctx.array("decayed.chunks"), seg_chunks = ctx.array("decayed.seg_chunks");
        const int n_chunks = chunks.count / 4;
        float *carry = nullptr, *decay = nullptr;
        if (n_chunks) {
            carry = ws.get("la_carry", {n_chunks, heads_, vdim_, padded_dim()}, DType::F32).as<float>();
            decay = ws.get("la_chunk_decay", {n_chunks, heads_, dim_}, DType::F32).as<float>();
        }
        if (LaunchProfile::get().on())      // q, k and v in, o out, the state in and out
            LaunchProfile::get().note_cost((double)T * ((2 * key_width_ + value_width_) * es + value_width_ * 4.0) + 2.0 * ctx.S * per_slot * 4.0,
                                           (double)T * heads_ * dim_ * vdim_ * 5.0);
        QE_LAUNCH(k, k.decayed_scan(base, base + key_width_ * es, base + 2 * key_width_ * es, nullptr, qkvg.code(), width, nullptr, 0, nullptr,
                                    1.0f, 1.0f, nullptr, (float)eps_, cache.state.as<float>(), per_slot, ctx.seg_start, ctx.seg_slot, ctx.S, T,
                                    heads_, dim_, vdim_, n_chunks ? chunks.data : nullptr, n_chunks, n_chunks ? seg_chunks.data : nullptr,
                                    carry, decay, raw.as<float>(), nullptr, decay_.as<float>(), 1, 1, ctx.stream));
        if (LaunchProfile::get().on()) LaunchProfile::get().note_cost((double)T * value_width_ * (4.0 + 2.0 * es), 0.0);
        QE_LAUNCH(k, k.rms_gate(raw.as<float>(), norm_.as<float>(), (float)eps_, base + (2 * key_width_ + value_width_) * es, qkvg.code(), width,
                                1, y.data, y.code(), T, (int)value_width_, ctx.stream));
        return o_proj_(y, ctx, "la_out", DType::F32, T, true, false, ctx.residual, nullptr, &ctx.norm_ahead);
    }

private:
    static constexpr int kChunk = 64;           // tokens of a chunk of the recurrence
    static constexpr int kChunkFrom = 128;      // the longest portion of a step from which the recurrence runs in chunks
    int64_t hidden_, key_width_, value_width_;
    int heads_, dim_, vdim_;
    double eps_;
    std::string gemm_;
    std::vector<float> decay_host_;
    Linear qkvg_proj_, o_proj_;
    Tensor decay_, norm_;
};

// params: hidden_size, left {kind, params}, right {kind, params}, combine ("rms_mean", the default: eps, factor (default
// 0.5), names{left_norm, right_norm}; "weighted_sum": left_factor, right_factor).
class SideBySide : public Mixer {
public:
    SideBySide(const Json& p, BuildContext& b) : Mixer(p, b) {
        hidden_ = p.at("hidden_size").as_int();
        const std::string combine = p.get_string("combine", "rms_mean");
        if (combine != "rms_mean" && combine != "weighted_sum") throw ConfigError("side_by_side: combine is 'rms_mean' or 'weighted_sum', got '" + combine + "'");
        weighted_ = combine == "weighted_sum";
        if (weighted_) {
            left_factor_ = p.at("left_factor").as_double();
            right_factor_ = p.at("right_factor").as_double();
        } else {
            eps_ = p.at("eps").as_double();
            factor_ = p.get_double("factor", 0.5);
        }
        left_ = make_part_as<Mixer>("mixer", PartSpec::from_json(p.at("left")), b);
        right_ = make_part_as<Mixer>("mixer", PartSpec::from_json(p.at("right")), b);
        CacheNeed::both(left_->cache_need(), right_->cache_need());          // throws when the two cannot share a layer's cache
    }
    std::vector<TensorSpec> tensor_specs() const override {
        if (weighted_) return {};
        return {{name_of("left_norm"), {hidden_}, Role::Vector, Init::Scale}, {name_of("right_norm"), {hidden_}, Role::Vector, Init::Scale}};
    }
    void bind(WeightSource& src) override {
        if (!weighted_) {
            left_w_ = src.fetch(name_of("left_norm"));
            right_w_ = src.fetch(name_of("right_norm"));
        }
        left_->bind(src);
        right_->bind(src);
    }
    std::vector<Part*> children() override { return {left_.get(), right_.get()}; }
    std::vector<std::string> ignored_tensors() const override {
        std::vector<std::string> names = left_->ignored_tensors();
        for (const std::string& n : right_->ignored_tensors()) names.push_back(n);
        return names;
    }
    std::vector<std::string> required_libraries() const override {
        std::vector<std::string> libs = left_->required_libraries();
        for (const std::string& l : right_->required_libraries()) libs.push_back(l);
        return libs;
    }
    int preferred_row_multiple() const override { return std::max(left_->preferred_row_multiple(), right_->preferred_row_multiple()); }
    void prepare_step(StepPlan& plan) override {
        left_->prepare_step(plan);
        right_->prepare_step(plan);
    }
    CacheNeed cache_need() const override { return CacheNeed::both(left_->cache_need(), right_->cache_need()); }

    Addend forward(const Tensor& x, StepContext& ctx, const CacheView& cache) override {
        // each side's output is normed before anything is added: neither adds into the residual behind this part's back,
        // and neither gets rows without their factor or a norm to work ahead for
        float* residual = ctx.residual;
        const NormAhead ahead = ctx.norm_ahead;
        const RowScale row_scale = ctx.row_scale;
        if (row_scale.defined()) throw Error(kInvalidState, "side_by_side: its mixers take finished rows");
        ctx.residual = nullptr;
        ctx.norm_ahead = NormAhead();
        Addend a = left_->forward(x, ctx, cache);
        Addend b = right_->forward(x, ctx, cache);
        ctx.residual = residual;
        ctx.norm_ahead = ahead;
        if (!a.tensor.defined() || !b.tensor.defined()) throw Error(kInvalidState, "side_by_side: a mixer added into the residual itself");
        if (a.transform.defined() || b.transform.defined()) throw Error(kInvalidState, "side_by_side: a mixer's output carries a transform");
        const int T = ctx.T;
        Tensor out = ctx.workspace->get("side_by_side_out", {T, hidden_}, DType::F32);
        const CoreKernels& k = core_kernels();
        if (LaunchProfile::get().on())
            LaunchProfile::get().note_cost((double)T * hidden_ * (a.splits * dtype_size(a.tensor.dtype) + b.splits * dtype_size(b.tensor.dtype) + 4.0), 0.0);
        if (weighted_)
            QE_LAUNCH(k, k.pair_sum(a.tensor.data, a.tensor.code(), a.splits, (long long)T * hidden_, (float)left_factor_, b.tensor.data,
                                    b.tensor.code(), b.splits, (long long)T * hidden_, (float)right_factor_, out.as<float>(),
                                    (long long)T * hidden_, ctx.stream));
        else
            QE_LAUNCH(k, k.rms_pair_mean(a.tensor.data, a.tensor.code(), a.splits, (long long)T * hidden_, left_w_.as<float>(), b.tensor.data,
                                         b.tensor.code(), b.splits, (long long)T * hidden_, right_w_.as<float>(), (float)eps_, (float)factor_,
                                         out.as<float>(), T, (int)hidden_, ctx.stream));
        return Addend(out, 1);
    }

private:
    int64_t hidden_;
    bool weighted_ = false;
    double eps_ = 0.0, factor_ = 0.5, left_factor_ = 1.0, right_factor_ = 1.0;
    std::shared_ptr<Mixer> left_, right_;
    Tensor left_w_, right_w_;
};

void register_linear_attention_parts() {
    register_part("mixer", "lightning_attention", [](const Json& p, BuildContext& b) { return std::make_shared<LightningAttention>(p, b); });
    register_part("mixer", "gated_linear_attention", [](const Json& p, BuildContext& b) { return std::make_shared<GatedLinearAttention>(p, b); });
    register_part("mixer", "side_by_side", [](const Json& p, BuildContext& b) { return std::make_shared<SideBySide>(p, b); });
}

}  // namespace qe
