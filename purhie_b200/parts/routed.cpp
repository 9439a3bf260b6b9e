// A mixture of gated feed-forward experts with a router.
//
// Router logits z = Wr x + b in float32 (the router's matrix is kept in float32 whatever the model's dtype; x is the
// normed row as the other products see it).  Each token takes the `top` experts with the largest logits (the lower
// index on a tie) with weights softmax(z over the chosen).  An expert is the gated unit of feed_forward.cpp without
// biases; the token's output is the weighted sum of its experts' outputs, added in the order of the choices.
//
// Other designs' options: "scoring": {"kind": "sigmoid", "groups", "keep"}: scores s = sigmoid(z); the choice goes by
// s + correction (a vector per expert, names.correction; without it by s), restricted to the `keep` runs of neighbouring
// experts (of `groups` equal runs) whose two largest choice values add up highest; the weights are the chosen
// experts' s as they are.  {"kind": "softmax", "groups", "keep", "scale"}: s = softmax(z) over all experts; the choice goes by
// s within the `keep` runs whose largest s is highest; the weights are the chosen s over their sum (+ 1e-20), times `scale`.
// names.shared_gate (a vector [hidden]): the shared part's sum is multiplied by sigmoid(gate . x), one number per token.
// "gated": false: an expert is Wd act(Wu x) with an activation of one argument ("relu2").
// "shared": {kind, params}: a feed-forward that runs for every token and is added to the chosen experts' sum.
//
// The (token, choice) pairs are sorted by expert on the device.  Which kernels then multiply:
//   * few pairs (decoding): one launch per matrix of a kernel that streams each chosen expert's weight rows once
//     (gemv_grouped); no count reaches the host, so the step is captured as a graph like any other;
//   * a step with prompt portions in bfloat16: the counts per expert are read back (one small copy and a wait per
//     layer; such steps are launched kernel by kernel anyway), the token rows are gathered in expert order, and every
//     expert's rows go through the tensor-core product as one contiguous slice;
//   * float32, or shapes the fast kernels refuse: gemm_grouped, the CUDA-core product over row tiles that never cross
//     from one expert to the next, all on the device.
// Whichever runs, a row's sum does not depend on what else is in the batch.
#include <algorithm>
#include <array>

#include "gate.h"
#include "linear.h"
#include "parts.h"

namespace qe {

// params: hidden_size, intermediate_size, experts, top, gated (default true), activation (as the gated feed-forward's;
// without a gate a name as the plain feed-forward's), scoring (null or as above), shared (null or {kind, params}),
// names{router, router_bias (optional), correction (optional), shared_gate (optional)}, expert_names [{gate_proj, up_proj, down_proj} per
// expert; without a gate {up_proj, down_proj}].
class RoutedGLU : public FeedForward {
public:
    RoutedGLU(const Json& p, BuildContext& b)
        : FeedForward(p, b), hidden_(p.at("hidden_size").as_int()), inter_(p.at("intermediate_size").as_int()),
          experts_((int)p.at("experts").as_int()), top_((int)p.at("top").as_int()) {
        if (experts_ < 1 || top_ < 1 || top_ > experts_)
            throw ConfigError("routed feed-forward: top " + std::to_string(top_) + " of " + std::to_string(experts_) + " experts");
        gated_ = p.get_bool("gated", true);
        if (gated_) gate_ = GateSpec::read(p);
        else unary_ = unary_activation(p.get_string("activation", "silu"));
        up_width_ = gated_ ? 2 * inter_ : inter_;
        const Json& names = p.at("expert_names");
        if (!names.is_array() || (int)names.size() != experts_) throw ConfigError("routed feed-forward: expert_names must list every expert");
        for (const Json& n : names.items())
            expert_names_.push_back({gated_ ? n.at("gate_proj").as_string() : std::string(), n.at("up_proj").as_string(), n.at("down_proj").as_string()});
        has_bias_ = names_.count("router_bias") != 0;
        has_correction_ = names_.count("correction") != 0;
        if (const Json* sc = p.find("scoring")) {
            if (!sc->is_null()) {
                const std::string kind = sc->get_string("kind", "");
                if (kind != "sigmoid" && kind != "softmax")
                    throw ConfigError("routed feed-forward: scoring of kind '" + kind + "' is not known (sigmoid, softmax)");
                scoring_ = kind == "sigmoid" ? 1 : 2;
                weight_scale_ = (float)sc->get_double("scale", 1.0);
                if (scoring_ != 2 && weight_scale_ != 1.0f) throw ConfigError("routed feed-forward: only softmax scoring scales its weights");
                groups_ = (int)sc->get_int("groups", 1);
                keep_ = (int)sc->get_int("keep", groups_);
                if (groups_ < 1 || experts_ % groups_ || keep_ < 1 || keep_ > groups_ || (long long)keep_ * (experts_ / groups_) < top_)
                    throw ConfigError("routed feed-forward: " + std::to_string(keep_) + " of " + std::to_string(groups_) + " runs of " +
                                      std::to_string(experts_) + " experts cannot give " + std::to_string(top_) + " choices");
            }
        }
        has_shared_gate_ = names_.count("shared_gate") != 0;
        if (has_correction_ && scoring_ != 1) throw ConfigError("routed feed-forward: a correction of the choice needs sigmoid scoring");
        if (const Json* sh = p.find("shared"))
            if (!sh->is_null()) shared_ = make_part_as<FeedForward>("feed_forward", PartSpec::from_json(*sh), b);
        if (has_shared_gate_ && !shared_) throw ConfigError("routed feed-forward: a gate of the shared part needs a shared part");
    }

    std::vector<TensorSpec> tensor_specs() const override {
        std::vector<TensorSpec> s = {{name_of("router"), {experts_, hidden_}, Role::Vector, Init::Normal}};
        if (has_bias_) s.push_back({name_of("router_bias"), {experts_}, Role::Vector, Init::Normal});
        if (has_correction_) s.push_back({name_of("correction"), {experts_}, Role::Vector, Init::Normal});
        if (has_shared_gate_) s.push_back({name_of("shared_gate"), {1, hidden_}, Role::Vector, Init::Normal});
        for (const auto& n : expert_names_) {
            if (gated_) s.push_back({n[0], {inter_, hidden_}, Role::Matrix, Init::Normal});
            s.push_back({n[1], {inter_, hidden_}, Role::Matrix, Init::Normal});
            s.push_back({n[2], {hidden_, inter_}, Role::Matrix, Init::Normal});
        }
        return s;
    }

    void bind(WeightSource& src) override {
        router_ = src.fetch(name_of("router"));
        if (has_bias_) router_bias_ = src.fetch(name_of("router_bias"));
        if (has_correction_) correction_ = src.fetch(name_of("correction"));
        if (has_shared_gate_) shared_gate_ = src.fetch(name_of("shared_gate"));
        if (shared_) shared_->bind(src);
        // the experts' matrices stacked: [experts, 2 ff, hidden] with gate and up rows interleaved (g0, u0, g1, u1, ...)
        // as the gated feed-forward lays them out (without a gate [experts, ff, hidden]), and [experts, hidden, ff]
        for (int e = 0; e < experts_; e++) {
            Tensor up = src.fetch(expert_names_[e][1]), down = src.fetch(expert_names_[e][2]);
            Tensor gate = gated_ ? src.fetch(expert_names_[e][0]) : up;
            if (e == 0) {
                gate_up_ = src.arena().alloc(up.dtype, {experts_, up_width_, hidden_});
                down_ = src.arena().alloc(down.dtype, {experts_, hidden_, inter_});
            }
            if (gate.dtype != gate_up_.dtype || up.dtype != gate_up_.dtype || down.dtype != down_.dtype)
                throw WeightError("the experts of a routed feed-forward are stored in different precisions");
            const size_t row = (size_t)hidden_ * dtype_size(up.dtype);
            char* gu = static_cast<char*>(gate_up_.data) + (size_t)e * up_width_ * row;
            if (gated_) {
                QE_CUDA(cudaMemcpy2DAsync(gu, 2 * row, gate.data, row, row, (size_t)inter_, cudaMemcpyDeviceToDevice, src.stream()));
                QE_CUDA(cudaMemcpy2DAsync(gu + row, 2 * row, up.data, row, row, (size_t)inter_, cudaMemcpyDeviceToDevice, src.stream()));
            } else {
                QE_CUDA(cudaMemcpyAsync(gu, up.data, up.bytes(), cudaMemcpyDeviceToDevice, src.stream()));
            }
            QE_CUDA(cudaMemcpyAsync(static_cast<char*>(down_.data) + (size_t)e * down.bytes(), down.data, down.bytes(),
                                    cudaMemcpyDeviceToDevice, src.stream()));
            QE_CUDA(cudaStreamSynchronize(src.stream()));
            if (gated_) src.release(gate);
            src.release(up);
            src.release(down);
        }
        // each expert's two matrices as products of their own, for the steps that run them slice by slice
        const std::string gemm = compute_dtype == DType::BF16 ? "auto" : "simple";
        for (int e = 0; e < experts_; e++) {
            Tensor gu(static_cast<char*>(gate_up_.data) + (size_t)e * up_width_ * hidden_ * dtype_size(gate_up_.dtype), gate_up_.dtype,
                      {up_width_, hidden_});
            Tensor dn(static_cast<char*>(down_.data) + (size_t)e * hidden_ * inter_ * dtype_size(down_.dtype), down_.dtype, {hidden_, inter_});
            expert_gate_up_.emplace_back(gu, "expert_gate_up", gemm);
            expert_down_.emplace_back(dn, "expert_down", gemm);
        }
        counts_host_.ensure((size_t)(experts_ + 1) * sizeof(int32_t));
    }

    std::vector<std::string> required_libraries() const override {
        std::vector<std::string> libs = {"core"};
        if (!expert_gate_up_.empty() && expert_gate_up_[0].fast()) libs.push_back("gemm100");
        if (shared_)
            for (const std::string& l : shared_->required_libraries()) libs.push_back(l);
        return libs;
    }
    std::vector<Part*> children() override { return shared_ ? std::vector<Part*>{shared_.get()} : std::vector<Part*>{}; }
    void prepare_step(StepPlan& plan) override { if (shared_) shared_->prepare_step(plan); }

    Addend forward(const Tensor& x, StepContext& ctx) override {
        const int T = ctx.T, R = T * top_;
        Workspace& ws = *ctx.workspace;
        const CoreKernels& k = core_kernels();
        Tensor choice = ws.get("moe_choice", {T, top_}, DType::I32), weight = ws.get("moe_weight", {T, top_}, DType::F32);
        if (LaunchProfile::get().on())
            LaunchProfile::get().note_cost((double)T * hidden_ * dtype_size(x.dtype) + 4.0 * experts_ * hidden_, 2.0 * T * experts_ * hidden_);
        // the part that runs for every token first: its result waits in the workspace (or is in the residual already)
        Addend always;
        if (shared_) {
            // its sum joins the experts' below: it neither adds into the residual itself nor works ahead for a norm
            float* residual = ctx.residual;
            const NormAhead ahead = ctx.norm_ahead;
            ctx.residual = nullptr;
            ctx.norm_ahead = NormAhead();
            always = shared_->forward(x, ctx);
            ctx.residual = residual;
            ctx.norm_ahead = ahead;
            if (always.tensor.defined() && (always.tensor.dtype != DType::F32 || always.transform.defined()))
                throw Error(kInvalidState, "routed feed-forward: the shared part must give float32 sums without a transform");
        }
        // sigmoid(gate . x) per token for the shared part's sum: one more row of the router's product
        float* shared_scale = shared_gate_.defined() ? ws.get("moe_shared_scale", {T}, DType::F32).as<float>() : nullptr;
        QE_LAUNCH(k, k.route(x.data, x.code(), router_.as<float>(), router_bias_.defined() ? router_bias_.as<float>() : nullptr, T, experts_,
                             (int)hidden_, top_, choice.as<int32_t>(), weight.as<float>(), scoring_,
                             correction_.defined() ? correction_.as<float>() : nullptr, groups_, keep_, weight_scale_,
                             shared_gate_.defined() ? shared_gate_.as<float>() : nullptr, shared_scale, ctx.stream));
        const int tiles = k.route_max_tiles(R, experts_);
        Tensor position = ws.get("moe_position", {R}, DType::I32), pair_at = ws.get("moe_pair_at", {R}, DType::I32);
        Tensor tile_list = ws.get("moe_tiles", {tiles, 3}, DType::I32), scratch = ws.get("moe_sort_scratch", {3 * experts_ + 1}, DType::I32);
        QE_LAUNCH(k, k.route_sort(choice.as<int32_t>(), R, experts_, position.as<int32_t>(), pair_at.as<int32_t>(),
                                  tile_list.as<int32_t>(), tiles, scratch.as<int32_t>(), ctx.stream));
        Tensor gu = ws.get("moe_gate_up", {R, up_width_}, compute_dtype);
        Tensor act = ws.get("moe_act", {R, inter_}, compute_dtype);
        Tensor y = ws.get("moe_down", {R, hidden_}, DType::F32);
        const bool slices = !ctx.decode_only && R > kFewPairs && compute_dtype == DType::BF16 && x.dtype == DType::BF16 &&
                            expert_gate_up_[0].fast() && expert_down_[0].fast() && hidden_ % 8 == 0 && inter_ % 8 == 0;
        const bool few = !slices && R <= kFewPairs && hidden_ % 8 == 0 && inter_ % 8 == 0;
        auto grouped = [&](const Tensor& in, const int32_t* pairs, int per_row, const Tensor& w, Tensor& out, int64_t N, int64_t K) {
            if (LaunchProfile::get().on()) {     // the matrices of the experts that can have been chosen, the rows in and out
                const double touched = std::min<double>(experts_, R);
                LaunchProfile::get().note_cost(touched * N * K * dtype_size(w.dtype) + (double)R * (K * dtype_size(in.dtype) + N * dtype_size(out.dtype)),
                                               2.0 * R * N * K);
            }
            if (few)
                QE_LAUNCH(k, k.gemv_grouped(in.data, in.code(), pairs, per_row, w.data, w.code(), tile_list.as<int32_t>(), tiles, out.data,
                                            out.code(), (int)N, (int)K, ctx.stream));
            else
                QE_LAUNCH(k, k.gemm_grouped(in.data, in.code(), pairs, per_row, w.data, w.code(), tile_list.as<int32_t>(), tiles, out.data,
                                            out.code(), (int)N, (int)K, ctx.stream));
        };
        std::vector<int32_t> first(experts_ + 1, 0);
        if (slices) {
            // where each expert's rows start, on the host (the sort left them behind its counts), and x in that order
            int32_t* host = static_cast<int32_t*>(counts_host_.data());
            QE_CUDA(cudaMemcpyAsync(host, scratch.as<int32_t>() + experts_, (size_t)(experts_ + 1) * sizeof(int32_t), cudaMemcpyDeviceToHost,
                                    ctx.stream));
            Tensor xs = ws.get("moe_x_sorted", {R, hidden_}, x.dtype);
            QE_LAUNCH(k, k.route_gather(x.data, x.code(), pair_at.as<int32_t>(), top_, xs.data, R, (int)hidden_, ctx.stream));
            QE_CUDA(cudaStreamSynchronize(ctx.stream));
            first.assign(host, host + experts_ + 1);
            for (int e = 0; e < experts_; e++) {
                const int at = first[e], n = first[e + 1] - first[e];
                if (n > 0) expert_gate_up_[e].into(xs.rows(at, n), ctx, gu.rows(at, n), n);
            }
        } else {
            grouped(x, pair_at.as<int32_t>(), top_, gate_up_, gu, up_width_, hidden_);
        }
        if (LaunchProfile::get().on()) LaunchProfile::get().note_cost((double)R * (up_width_ + inter_) * dtype_size(compute_dtype), 0.0);
        if (gated_)
            QE_LAUNCH(k, k.glu(gu.data, gu.code(), 1, 0, act.data, act.code(), R, (int)inter_, gate_.kind, gate_.alpha, gate_.limit,
                               gate_.shift, ctx.stream));
        else
            QE_LAUNCH(k, k.unary_act(gu.data, gu.code(), 1, 0, act.data, act.code(), (long long)R * inter_, unary_, ctx.stream));
        if (slices) {
            for (int e = 0; e < experts_; e++) {
                const int at = first[e], n = first[e + 1] - first[e];
                if (n > 0) expert_down_[e].into(act.rows(at, n), ctx, y.rows(at, n), n);
            }
        } else {
            grouped(act, nullptr, 1, down_, y, hidden_, inter_);
        }
        Tensor out = ws.get("moe_out", {T, hidden_}, DType::F32);
        QE_LAUNCH(k, k.route_combine(y.data, y.code(), position.as<int32_t>(), weight.as<float>(), T, top_, (int)hidden_, out.as<float>(),
                                     always.tensor.defined() ? always.tensor.as<float>() : nullptr, always.tensor.defined() ? always.splits : 0,
                                     (long long)T * hidden_, always.tensor.defined() ? shared_scale : nullptr, ctx.stream));
        return Addend(out, 1);
    }

private:
    static constexpr int kFewPairs = 256;       // up to this many (token, choice) pairs a step streams the experts' rows
    int64_t hidden_, inter_;
    int experts_, top_;
    GateSpec gate_;
    bool gated_ = true, has_bias_ = false, has_correction_ = false;
    bool has_shared_gate_ = false;
    int unary_ = 0, scoring_ = 0, groups_ = 1, keep_ = 1;
    float weight_scale_ = 1.0f;
    int64_t up_width_ = 0;
    std::shared_ptr<FeedForward> shared_;
    std::vector<std::array<std::string, 3>> expert_names_;
    std::vector<Linear> expert_gate_up_, expert_down_;
    PinnedBuffer counts_host_;
    Tensor router_, router_bias_, correction_, shared_gate_, gate_up_, down_;
};

void register_routed_parts() {
    register_part("feed_forward", "routed_glu", [](const Json& p, BuildContext& b) { return std::make_shared<RoutedGLU>(p, b); });
}

}  // namespace qe
