// The norms: RMSNorm, the layer norm with weight and (optional) bias, and "none" for a part that reads the residual
// itself, each with the residual add folded in.
//
// y = v * rsqrt(mean(v^2) + eps) * w, v = x + pending addend; the weight multiplies after normalising (plain w,
// not 1 + w).  Reference: src/gpu_ops.hip:24-56 (add + norm in one kernel), src/qwen_ops.cpp:8-13.
#include "parts.h"

namespace qe {

AddendTransform Norm::as_transform(float) const {
    throw ConfigError("this norm cannot be applied to an addend on its way into the residual");
}
void Norm::apply_in_place(Tensor&, StepContext&, int) {
    throw ConfigError("this norm cannot be applied to rows in place");
}

void fold_second_addend(ResidualStream& stream, StepContext& ctx) {
    if (!stream.has_also) return;
    const Addend& b = stream.also;
    const int64_t E = stream.x.shape[1];
    const CoreKernels& k = core_kernels();
    if (LaunchProfile::get().on()) LaunchProfile::get().note_cost((double)ctx.T * E * (8.0 + b.splits * dtype_size(b.tensor.dtype)), 0.0);
    QE_LAUNCH(k, k.add_dyntanh(stream.x.as<float>(), b.tensor.data, b.tensor.code(), b.splits, (long long)ctx.T * E, nullptr, 0, 1, 0, nullptr,
                               nullptr, nullptr, nullptr, ctx.T, (int)E, nullptr, 0, 1, ctx.stream));
    stream.has_also = false;
    stream.also = Addend();
}

namespace {
// what a norm's pass over the rows moves: the residual read (and written back when an addend is folded in), the
// addend's parts, the normed rows
void note_norm_cost(const ResidualStream& stream, int rows, int64_t width, DType out, bool write_back) {
    if (!LaunchProfile::get().on()) return;
    double bytes = 4.0 * rows * width + (double)rows * width * dtype_size(out);
    if (stream.has_pending) bytes += (double)stream.pending.splits * rows * width * dtype_size(stream.pending.tensor.dtype) + (write_back ? 4.0 * rows * width : 0.0);
    LaunchProfile::get().note_cost(bytes, 0.0);
}
// x += factor * norm(addend) for a pending addend with a transform, by the kernel that knows transforms; afterwards
// the stream has nothing pending.  For norms whose own kernel does not know them.
void fold_transformed(ResidualStream& stream, StepContext& ctx) {
    fold_second_addend(stream, ctx);
    if (!stream.has_pending || !stream.pending.transform.defined()) return;
    const Addend& a = stream.pending;
    const int64_t E = stream.x.shape[1];
    const CoreKernels& k = core_kernels();
    QE_LAUNCH(k, k.add_layernorm(stream.x.as<float>(), a.tensor.data, a.tensor.code(), a.splits, (long long)ctx.T * E,
                                 a.transform.weight, a.transform.bias, a.transform.eps, a.transform.factor, nullptr, nullptr, 0.0f,
                                 nullptr, ctx.T, (int)E, nullptr, 0, 1, ctx.stream));
    stream.clear();
}
}  // namespace

void fold_all_addends(ResidualStream& stream, StepContext& ctx) {
    fold_transformed(stream, ctx);            // the second addend, and a pending one that carries a transform
    if (!stream.has_pending) return;
    const Addend& a = stream.pending;
    const int64_t E = stream.x.shape[1];
    const CoreKernels& k = core_kernels();
    QE_LAUNCH(k, k.add_dyntanh(stream.x.as<float>(), a.tensor.data, a.tensor.code(), a.splits, (long long)ctx.T * E, nullptr, 0, 1, 0, nullptr,
                               nullptr, nullptr, nullptr, ctx.T, (int)E, nullptr, 0, 1, ctx.stream));
    stream.clear();
}

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
        // an addend whose transform is a factor alone is folded in by this norm's own kernel; a norm on the addend, or a
        // second addend, takes the kernel that knows those first
        const bool factor_only = stream.has_pending && !stream.has_also && stream.pending.transform.defined() && !stream.pending.transform.weight;
        if (!factor_only) fold_transformed(stream, ctx);
        Tensor out = ctx.workspace->get(rows ? "normed_rows" : "normed", {n, size_}, compute_dtype);
        const CoreKernels& k = core_kernels();
        const Addend* pend = stream.has_pending ? &stream.pending : nullptr;
        note_norm_cost(stream, n, size_, compute_dtype, !rows);
        if (factor_only)
            QE_LAUNCH(k, k.add_scaled_rmsnorm(stream.x.as<float>(), pend->tensor.data, pend->tensor.code(), pend->splits, (long long)ctx.T * size_,
                                              weight_.as<float>(), (float)eps_, rows, n, (int)size_, out.data, out.code(), rows ? 0 : 1,
                                              pend->transform.factor, ctx.stream));
        else
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
        if (stream.prepared.done() && stream.prepared.norm == this && !stream.has_pending && !stream.has_also) {
            // the product that added into the stream did this norm's pass in its epilogue
            Tensor rows = stream.prepared.rows;
            *scale = stream.prepared.scale;
            stream.clear();
            return rows;
        }
        if (compute_dtype != DType::BF16 || size_ % 4) return forward(stream, ctx, nullptr, 0);
        fold_transformed(stream, ctx);
        constexpr int kChunk = 512;                                   // columns per CTA of the kernel
        const int chunks = (int)((size_ + kChunk - 1) / kChunk);
        Tensor out = ctx.workspace->get("normed", {ctx.T, size_}, compute_dtype);
        Tensor sumsq = ctx.workspace->get("normed_sumsq", {ctx.T, chunks}, DType::F32);
        const CoreKernels& k = core_kernels();
        const Addend* pend = stream.has_pending ? &stream.pending : nullptr;
        note_norm_cost(stream, ctx.T, size_, compute_dtype, true);
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

// Layer norm with weight and bias: y = (v - mean(v)) / sqrt(var(v) + eps) * w + b, var the mean of the squared
// deviations, v = x + the pending addend.  A pending addend may carry a transform (a norm of this kind over the
// addend's own rows and a factor): the one kernel applies it, adds, and norms the sum, which is all a layer of the
// form x <- x + m * norm_b(f(norm_a(x))) needs between two parts.
// params: size, eps, names{weight, bias}; without a name for the bias the norm has none.
class LayerNorm : public Norm {
public:
    LayerNorm(const Json& p, BuildContext& b) : Norm(p, b), size_(p.at("size").as_int()), eps_(p.at("eps").as_double()) {
        if (size_ < 1 || !(eps_ >= 0)) throw ConfigError("layernorm: size must be positive and eps >= 0");
        has_bias_ = names_.count("bias") != 0;
    }
    std::vector<TensorSpec> tensor_specs() const override {
        std::vector<TensorSpec> s = {{name_of("weight"), {size_}, Role::Vector, Init::Scale}};
        if (has_bias_) s.push_back({name_of("bias"), {size_}, Role::Vector, Init::Normal});
        return s;
    }
    void bind(WeightSource& src) override {
        weight_ = src.fetch(name_of("weight"));
        if (has_bias_) bias_ = src.fetch(name_of("bias"));
    }
    Tensor forward(ResidualStream& stream, StepContext& ctx, const int32_t* rows, int n_rows) override {
        const int n = rows ? n_rows : ctx.T;
        fold_second_addend(stream, ctx);
        Tensor out = ctx.workspace->get(rows ? "normed_rows" : "normed", {n, size_}, compute_dtype);
        const CoreKernels& k = core_kernels();
        const Addend* a = stream.has_pending ? &stream.pending : nullptr;
        note_norm_cost(stream, n, size_, compute_dtype, !rows);
        QE_LAUNCH(k, k.add_layernorm(stream.x.as<float>(), a ? a->tensor.data : nullptr, a ? a->tensor.code() : 0, a ? a->splits : 1,
                                     a ? (long long)ctx.T * size_ : 0, a ? a->transform.weight : nullptr, a ? a->transform.bias : nullptr,
                                     a ? a->transform.eps : 0.0f, a ? a->transform.factor : 1.0f, weight_.as<float>(),
                                     has_bias_ ? bias_.as<float>() : nullptr, (float)eps_, rows, n, (int)size_, out.data, out.code(),
                                     rows ? 0 : 1, ctx.stream));
        if (!rows) stream.clear();
        return out;
    }
    AddendTransform as_transform(float factor) const override {
        AddendTransform t;
        t.weight = weight_.as<float>(); t.bias = has_bias_ ? bias_.as<float>() : nullptr; t.eps = (float)eps_; t.factor = factor;
        return t;
    }
private:
    int64_t size_;
    double eps_;
    bool has_bias_ = true;
    Tensor weight_, bias_;
};

// No norm at all, for a layer whose parts read the residual stream as it is (and norm what they give instead): the
// pending addend, with its transform, is folded in, and the rows come back in the compute dtype, in the same one pass.
// params: size.
class NoNorm : public Norm {
public:
    NoNorm(const Json& p, BuildContext& b) : Norm(p, b), size_(p.at("size").as_int()) {
        if (size_ < 1) throw ConfigError("norm 'none': size must be positive");
    }
    Tensor forward(ResidualStream& stream, StepContext& ctx, const int32_t* rows, int n_rows) override {
        const int n = rows ? n_rows : ctx.T;
        fold_second_addend(stream, ctx);
        Tensor out = ctx.workspace->get(rows ? "normed_rows" : "normed", {n, size_}, compute_dtype);
        const CoreKernels& k = core_kernels();
        const Addend* a = stream.has_pending ? &stream.pending : nullptr;
        note_norm_cost(stream, n, size_, compute_dtype, !rows);
        QE_LAUNCH(k, k.add_layernorm(stream.x.as<float>(), a ? a->tensor.data : nullptr, a ? a->tensor.code() : 0, a ? a->splits : 1,
                                     a ? (long long)ctx.T * size_ : 0, a ? a->transform.weight : nullptr, a ? a->transform.bias : nullptr,
                                     a ? a->transform.eps : 0.0f, a ? a->transform.factor : 1.0f, nullptr, nullptr, 0.0f, rows, n,
                                     (int)size_, out.data, out.code(), rows ? 0 : 1, ctx.stream));
        if (!rows) stream.clear();
        return out;
    }
private:
    int64_t size_;
};

// Dynamic tanh in the place of a norm: y = tanh(alpha * v) * w + b with a scalar alpha, v = x + what waits to be added.
// It takes no statistic of the row (and has no eps).  Both addends of a layer whose two parts read the same rows are
// folded in the same pass.  params: size, names{weight, bias, alpha}.
class DynamicTanh : public Norm {
public:
    DynamicTanh(const Json& p, BuildContext& b) : Norm(p, b), size_(p.at("size").as_int()) {
        if (size_ < 1) throw ConfigError("dyntanh: size must be positive");
    }
    std::vector<TensorSpec> tensor_specs() const override {
        return {{name_of("weight"), {size_}, Role::Vector, Init::Scale}, {name_of("bias"), {size_}, Role::Vector, Init::Normal},
                {name_of("alpha"), {}, Role::Vector, Init::Scale}};
    }
    void bind(WeightSource& src) override {
        weight_ = src.fetch(name_of("weight"));
        bias_ = src.fetch(name_of("bias"));
        alpha_ = src.fetch(name_of("alpha"));
    }
    Tensor forward(ResidualStream& stream, StepContext& ctx, const int32_t* rows, int n_rows) override {
        const int n = rows ? n_rows : ctx.T;
        if (stream.has_pending && stream.pending.transform.defined()) fold_all_addends(stream, ctx);
        Tensor out = ctx.workspace->get(rows ? "normed_rows" : "normed", {n, size_}, compute_dtype);
        const CoreKernels& k = core_kernels();
        const Addend* a = stream.has_pending ? &stream.pending : nullptr;
        const Addend* b = stream.has_also ? &stream.also : nullptr;
        if (LaunchProfile::get().on()) {
            double bytes = 4.0 * n * size_ + (double)n * size_ * dtype_size(compute_dtype);
            if (a) bytes += (double)a->splits * n * size_ * dtype_size(a->tensor.dtype);
            if (b) bytes += (double)b->splits * n * size_ * dtype_size(b->tensor.dtype);
            if ((a || b) && !rows) bytes += 4.0 * n * size_;
            LaunchProfile::get().note_cost(bytes, 0.0);
        }
        QE_LAUNCH(k, k.add_dyntanh(stream.x.as<float>(), a ? a->tensor.data : nullptr, a ? a->tensor.code() : 0, a ? a->splits : 1,
                                   a ? (long long)ctx.T * size_ : 0, b ? b->tensor.data : nullptr, b ? b->tensor.code() : 0,
                                   b ? b->splits : 1, b ? (long long)ctx.T * size_ : 0, alpha_.as<float>(), weight_.as<float>(),
                                   bias_.as<float>(), rows, n, (int)size_, out.data, out.code(), (!rows && (a || b)) ? 1 : 0, ctx.stream));
        if (!rows) stream.clear();
        return out;
    }
    void apply_in_place(Tensor& x, StepContext& ctx, int n) override {
        const CoreKernels& k = core_kernels();
        if (LaunchProfile::get().on()) LaunchProfile::get().note_cost(8.0 * n * size_, 0.0);
        QE_LAUNCH(k, k.add_dyntanh(x.as<float>(), nullptr, 0, 1, 0, nullptr, 0, 1, 0, alpha_.as<float>(), weight_.as<float>(), bias_.as<float>(),
                                   nullptr, n, (int)size_, x.data, x.code(), 0, ctx.stream));
    }
private:
    int64_t size_;
    Tensor weight_, bias_, alpha_;
};

void register_norm_parts() {
    register_part("norm", "dyntanh", [](const Json& p, BuildContext& b) { return std::make_shared<DynamicTanh>(p, b); });
    register_part("norm", "rmsnorm", [](const Json& p, BuildContext& b) { return std::make_shared<RMSNorm>(p, b); });
    register_part("norm", "layernorm", [](const Json& p, BuildContext& b) { return std::make_shared<LayerNorm>(p, b); });
    register_part("norm", "none", [](const Json& p, BuildContext& b) { return std::make_shared<NoNorm>(p, b); });
}

}  // namespace qe
