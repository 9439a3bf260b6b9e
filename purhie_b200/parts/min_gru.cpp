// A minimal gated recurrent unit as a mixer: gates that read the current token only, one float32 number of state per
// channel and request.
//
//     z = sigmoid(Wz h + bz),  u = Wx h + bx,  cand = u + 1/2 where u >= 0 and sigmoid(u) below
//     S <- (1 - z) S + z cand   (element by element, S = 0 at admission)
//     y = Wo (S * silu(Wg h))
// The state lives in the request's state slot (zeroed at admission, carried from step to step, given back at release), so
// a prompt cut anywhere walks the same recurrence.  The three projections of h are one product over the stacked matrices
// [z | x | g] that writes float32: the biases, both sigmoids, the candidate, S and the gate are float32 in every mode;
// only what enters the output product is rounded to the compute dtype.  A step with a long portion cuts every request's
// rows into chunks (the recurrence is linear in S, so chunks compose), listed as this mixer's own step metadata.
#include <algorithm>

#include "linear.h"
#include "parts.h"

namespace qe {

// params: hidden_size, width, names{z_proj, z_bias, x_proj, x_bias, g_proj, o_proj}.
class MinGRU : public Mixer {
public:
    MinGRU(const Json& p, BuildContext& b) : Mixer(p, b) {
        hidden_ = p.at("hidden_size").as_int();
        width_ = p.at("width").as_int();
        if (hidden_ < 1 || width_ < 1) throw ConfigError("min_gru: hidden_size and width must be positive");
        gemm_ = b.options.get_string("gemm", "auto");
    }
    std::vector<TensorSpec> tensor_specs() const override {
        return {{name_of("z_proj"), {width_, hidden_}, Role::Matrix, Init::Normal}, {name_of("z_bias"), {width_}, Role::Vector, Init::Normal},
                {name_of("x_proj"), {width_, hidden_}, Role::Matrix, Init::Normal}, {name_of("x_bias"), {width_}, Role::Vector, Init::Normal},
                {name_of("g_proj"), {width_, hidden_}, Role::Matrix, Init::Normal}, {name_of("o_proj"), {hidden_, width_}, Role::Matrix, Init::Normal}};
    }
    void bind(WeightSource& src) override {
        Tensor parts[3] = {src.fetch(name_of("z_proj")), src.fetch(name_of("x_proj")), src.fetch(name_of("g_proj"))};
        for (Tensor& t : parts)
            if (t.dtype != parts[0].dtype) throw WeightError("the projections of " + name_of("z_proj") + "'s mixer are stored in different precisions");
        Tensor all = src.arena().alloc(parts[0].dtype, {3 * width_, hidden_});
        size_t off = 0;
        for (Tensor& t : parts) {
            QE_CUDA(cudaMemcpyAsync(static_cast<char*>(all.data) + off, t.data, t.bytes(), cudaMemcpyDeviceToDevice, src.stream()));
            off += t.bytes();
        }
        QE_CUDA(cudaStreamSynchronize(src.stream()));
        for (Tensor& t : parts) src.release(t);
        in_proj_ = Linear(all, "zxg_proj", gemm_);
        z_bias_ = src.fetch(name_of("z_bias"));
        x_bias_ = src.fetch(name_of("x_bias"));
        o_proj_ = Linear(src.fetch(name_of("o_proj")), "o_proj", gemm_);
    }
    std::vector<std::string> required_libraries() const override {
        return (in_proj_.fast() || o_proj_.fast()) ? std::vector<std::string>{"core", "gemm100"} : std::vector<std::string>{"core"};
    }
    int preferred_row_multiple() const override { return (in_proj_.fast() || o_proj_.fast()) ? 256 : 0; }
    CacheNeed cache_need() const override { return CacheNeed::state({width_}, DType::F32); }

    // first row, rows, segment, 1 on the request's last chunk, for every request's rows, when the longest portion is long
    void prepare_step(StepPlan& plan) override {
        if (plan.has("min_gru.chunks")) return;
        int longest = 0;
        for (int n : plan.q_lens) longest = std::max(longest, n);
        if (longest < kChunkFrom) return;
        std::vector<int32_t> items, seg_items = {0};
        int row = 0;
        for (int s = 0; s < plan.S; s++) {
            const int n = plan.q_lens[s];
            for (int at = 0; at < n; at += kChunk) {
                items.push_back(row + at); items.push_back(std::min(kChunk, n - at)); items.push_back(s); items.push_back(at + kChunk >= n);
            }
            row += n;
            seg_items.push_back((int32_t)(items.size() / 4));
        }
        plan.add("min_gru.chunks", std::move(items));
        plan.add("min_gru.seg_chunks", std::move(seg_items));
    }

    Addend forward(const Tensor& x, StepContext& ctx, const CacheView& cache) override {
        if (!cache.state.defined() || cache.state.dtype != DType::F32 || cache.state.numel() != (int64_t)cache.state.shape[0] * width_)
            throw Error(kInvalidState, "min_gru: the cache manager gave no state of this mixer's shape");
        const int T = ctx.T;
        Workspace& ws = *ctx.workspace;
        const CoreKernels& k = core_kernels();
        Addend in = in_proj_(x, ctx, "gru_in", DType::F32, T, true);                 // [T, z | x | g] float32, maybe in parts
        Tensor y = ws.get("gru_y", {T, width_}, compute_dtype);
        const StepArray chunks = ctx.array("min_gru.chunks"), seg_chunks = ctx.array("min_gru.seg_chunks");
        const int n_chunks = chunks.count / 4;
        float* carry = n_chunks ? ws.get("gru_carry", {3, n_chunks, width_}, DType::F32).as<float>() : nullptr;
        if (LaunchProfile::get().on())      // the product's rows in (twice when chunked), y out, the state in and out
            LaunchProfile::get().note_cost((double)T * width_ * (3.0 * in.splits * dtype_size(in.tensor.dtype) * (n_chunks ? 5.0 / 3.0 : 1.0) +
                                                                 dtype_size(compute_dtype)) + 8.0 * ctx.S * width_, 12.0 * T * width_);
        QE_LAUNCH(k, k.min_gru_scan(in.tensor.data, in.tensor.code(), in.splits, (long long)T * 3 * width_, 3 * width_, z_bias_.as<float>(),
                                    x_bias_.as<float>(), cache.state.as<float>(), ctx.seg_start, ctx.seg_slot, ctx.S, T, (int)width_,
                                    n_chunks ? chunks.data : nullptr, n_chunks, n_chunks ? seg_chunks.data : nullptr, carry, y.data, y.code(),
                                    ctx.stream));
        return o_proj_(y, ctx, "gru_out", DType::F32, T, true, false, ctx.residual, nullptr, &ctx.norm_ahead);
    }

private:
    static constexpr int kChunk = 32;           // rows of a chunk of the recurrence
    static constexpr int kChunkFrom = 128;      // the longest portion of a step from which the recurrence runs in chunks
    int64_t hidden_, width_;
    std::string gemm_;
    Linear in_proj_, o_proj_;
    Tensor z_bias_, x_bias_;
};

void register_recurrent_parts() {
    register_part("mixer", "min_gru", [](const Json& p, BuildContext& b) { return std::make_shared<MinGRU>(p, b); });
}

}  // namespace qe
