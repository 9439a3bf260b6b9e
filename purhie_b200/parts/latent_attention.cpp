// Attention whose keys and values are made from one small latent per token, and whose queries pass through a latent too.
//
//     c_q = rmsnorm(W_dq h; w_q),   q = W_uq c_q            per head [head_dim plain | rot_dim rotated]
//     [c' | r] = W_dkv h,  c = rmsnorm(c'; w_kv)            c: kv_rank wide, r: rot_dim wide, one rotated key part for all heads
//     head a:  k = [W_uk_a c | rot(r)],  v = W_uv_a c,  score = (q_plain . k_plain + rot(q_rot) . rot(r)) * scale
//     o_a = softmax over the visible positions (all earlier ones, or the last `window`) of the scores, times v
//     y = W_o concat_a(o_a * sigmoid(W_g h)_a)              "gate": true; without it the heads' outputs go to W_o as they are
//
// A token leaves only [c | rot(r)] in the cache: one row of kv_rank + rot_dim numbers and no value rows
// (CacheNeed::rows).  Keys and values are never made: q_plain . (W_uk_a c) = (W_uk_a^T q_plain) . c and
// sum_j p_j W_uv_a c_j = W_uv_a sum_j p_j c_j, so every head attends over the same cached rows with the query
// [W_uk_a^T q_plain | rot(q_rot)], takes the weighted sum of the rows' first kv_rank numbers, and W_uv_a expands that.
// The down projections W_dq, W_dkv and W_g are one product over the stacked matrices.  Norms, rotation, scores, softmax
// and the sums over the latent are float32 in every mode.
//
// In bfloat16 the attention runs on the tensor cores (latent_attention_mma.cu): the (token, head) pairs of a portion,
// heads side by side, are cut into tiles of 64 that prepare_step() lists, and when there are few tiles the keys of
// each are split over several CTAs.  Rows that kernel does not take, and float32, go through attention_generic.
#include <algorithm>
#include <cmath>

#include "linear.h"
#include "parts.h"

namespace qe {

// params: hidden_size, num_heads, head_dim (plain dimensions of a head), rot_dim (rotated ones), value_dim, q_rank, kv_rank,
// norm_eps, scale, window (null: all positions), gate (default false), position (a PartSpec as {kind, params} whose n_rot is
// at most rot_dim, or null), names{q_down, q_norm, q_up, kv_down, kv_norm, k_up, v_up, o_proj, gate (with "gate": true)}.
class LatentAttention : public Mixer {
public:
    LatentAttention(const Json& p, BuildContext& b) : Mixer(p, b) {
        hidden_ = p.at("hidden_size").as_int();
        heads_ = (int)p.at("num_heads").as_int();
        dim_ = (int)p.at("head_dim").as_int();
        rot_ = (int)p.at("rot_dim").as_int();
        vdim_ = (int)p.at("value_dim").as_int();
        q_rank_ = (int)p.at("q_rank").as_int();
        kv_rank_ = (int)p.at("kv_rank").as_int();
        eps_ = p.at("norm_eps").as_double();
        scale_ = p.at("scale").as_double();
        window_ = (int)p.get_int("window", 0);
        gated_ = p.get_bool("gate", false);
        if (heads_ < 1 || dim_ < 1 || rot_ < 0 || vdim_ < 1 || q_rank_ < 1 || kv_rank_ < 1 || window_ < 0)
            throw ConfigError("latent_attention: heads, head_dim, value_dim and the ranks must be positive");
        if (kv_rank_ + rot_ > kMaxRow)
            throw ConfigError("latent_attention: a cache row of " + std::to_string(kv_rank_ + rot_) + " numbers exceeds the supported " +
                              std::to_string(kMaxRow));
        if (const Json* pos = p.find("position")) {
            if (!pos->is_null()) {
                PartSpec spec = PartSpec::from_json(*pos);
                Json key_params = Json::object();
                for (const auto& m : spec.params.members()) if (m.first != "names") key_params.set(m.first, m.second);
                auto part = b.shared("position:" + spec.kind + ":" + key_params.dump(), [&] { return make_part("position", spec, b); });
                position_ = std::dynamic_pointer_cast<PositionEncoding>(part);
                if (!position_) throw ConfigError("part '" + spec.kind + "' is not a position encoding");
                if (position_->interleaved()) throw ConfigError("latent_attention: the rotated part turns in half pairs");
                if (position_->n_rot() > rot_) throw ConfigError("latent_attention: the encoding rotates more dimensions than rot_dim");
            }
        }
        gemm_ = b.options.get_string("gemm", "auto");
        attention_ = b.options.get_string("attention", "auto");
        down_width_ = (int64_t)q_rank_ + kv_rank_ + rot_ + (gated_ ? heads_ : 0);
    }

    std::vector<TensorSpec> tensor_specs() const override {
        std::vector<TensorSpec> s = {{name_of("q_down"), {q_rank_, hidden_}, Role::Matrix, Init::Normal},
                                     {name_of("q_norm"), {q_rank_}, Role::Vector, Init::Scale},
                                     {name_of("q_up"), {(int64_t)heads_ * (dim_ + rot_), q_rank_}, Role::Matrix, Init::Normal},
                                     {name_of("kv_down"), {(int64_t)kv_rank_ + rot_, hidden_}, Role::Matrix, Init::Normal},
                                     {name_of("kv_norm"), {kv_rank_}, Role::Vector, Init::Scale},
                                     {name_of("k_up"), {(int64_t)heads_ * dim_, kv_rank_}, Role::Matrix, Init::Normal},
                                     {name_of("v_up"), {(int64_t)heads_ * vdim_, kv_rank_}, Role::Matrix, Init::Normal},
                                     {name_of("o_proj"), {hidden_, (int64_t)heads_ * vdim_}, Role::Matrix, Init::Normal}};
        if (gated_) s.push_back({name_of("gate"), {heads_, hidden_}, Role::Matrix, Init::Normal});
        return s;
    }

    void bind(WeightSource& src) override {
        // one matrix [q_down | kv_down | gate]: the projections of h are one product (a layout choice only)
        std::vector<Tensor> parts = {src.fetch(name_of("q_down")), src.fetch(name_of("kv_down"))};
        if (gated_) parts.push_back(src.fetch(name_of("gate")));
        for (Tensor& t : parts)
            if (t.dtype != parts[0].dtype) throw WeightError("the down projections of " + name_of("q_down") + "'s mixer are stored in different precisions");
        Tensor all = src.arena().alloc(parts[0].dtype, {down_width_, hidden_});
        size_t off = 0;
        for (Tensor& t : parts) {
            QE_CUDA(cudaMemcpyAsync(static_cast<char*>(all.data) + off, t.data, t.bytes(), cudaMemcpyDeviceToDevice, src.stream()));
            off += t.bytes();
        }
        QE_CUDA(cudaStreamSynchronize(src.stream()));
        for (Tensor& t : parts) src.release(t);
        down_proj_ = Linear(all, "latent_down", gemm_);
        q_up_ = Linear(src.fetch(name_of("q_up")), "q_up", gemm_);
        q_norm_ = src.fetch(name_of("q_norm"));
        kv_norm_ = src.fetch(name_of("kv_norm"));
        k_up_ = src.fetch(name_of("k_up"));
        v_up_ = src.fetch(name_of("v_up"));
        o_proj_ = Linear(src.fetch(name_of("o_proj")), "o_proj", gemm_);
        if (position_) {
            position_->bind(src);
            table_ = position_->rotation_table();
        }
    }

    std::vector<std::string> required_libraries() const override {
        std::vector<std::string> libs = {"core"};
        if (down_proj_.fast() || q_up_.fast() || o_proj_.fast()) libs.push_back("gemm100");
        if (products_on_tensor_cores()) libs.push_back("latent");
        return libs;
    }

    // the products per head (any sizes) in bfloat16
    bool products_on_tensor_cores() const {
        return compute_dtype == DType::BF16 && attention_ != "generic" &&
               (!k_up_.defined() || (k_up_.dtype == DType::BF16 && v_up_.dtype == DType::BF16));
    }

    // the tensor-core kernel holds rows of at most 512 + 64 numbers, in 16-byte pieces
    bool on_tensor_cores() const {
        return compute_dtype == DType::BF16 && attention_ != "generic" && kv_rank_ % 8 == 0 && rot_ % 8 == 0 && kv_rank_ <= 512 && rot_ <= 64;
    }

    // tiles of kTileRows (token, head) pairs per segment: the segment and the first pair of each, the tiles that look
    // furthest back first
    void prepare_step(StepPlan& plan) override {
        if (!on_tensor_cores()) return;
        const std::string name = tiles_name();
        if (plan.has(name + ".seg")) return;
        struct Tile { int seg, first, reach; };
        std::vector<Tile> tiles;
        for (int s = 0; s < plan.S; s++) {
            const int n = plan.q_lens[s] * heads_, start = plan.ctx_lens[s] - plan.q_lens[s];
            for (int first = 0; first < n; first += kTileRows) {
                const int last_token = (std::min(first + kTileRows, n) - 1) / heads_;
                tiles.push_back({s, first, window_ ? std::min(window_ + last_token - first / heads_, start + last_token + 1) : start + last_token + 1});
            }
        }
        std::stable_sort(tiles.begin(), tiles.end(), [](const Tile& a, const Tile& b) { return a.reach > b.reach; });
        std::vector<int32_t> seg, first;
        for (const Tile& t : tiles) { seg.push_back(t.seg); first.push_back(t.first); }
        plan.add(name + ".seg", std::move(seg));
        plan.add(name + ".first", std::move(first));
    }
    std::vector<Part*> children() override { return position_ ? std::vector<Part*>{position_.get()} : std::vector<Part*>{}; }
    int preferred_row_multiple() const override { return (down_proj_.fast() || o_proj_.fast()) ? 256 : 0; }

    CacheNeed cache_need() const override { return CacheNeed::rows(kv_rank_ + rot_, window_); }

    Addend forward(const Tensor& x, StepContext& ctx, const CacheView& cache) override {
        if (!cache.writable) throw Error(kInvalidState, "latent_attention: a layer writes a cache of its own");
        if (cache.kv_heads != 1 || cache.key_dim != kv_rank_ + rot_)
            throw Error(kInvalidState, "latent_attention: the cache manager gave no rows of this mixer's width");
        const int T = ctx.T;
        const DType dt = compute_dtype;
        Workspace& ws = *ctx.workspace;
        const GroupStep& g = ctx.groups.at(cache.group);
        const CoreKernels& k = core_kernels();
        const int row = kv_rank_ + rot_, n_rot = position_ ? position_->n_rot() : 0;
        const int32_t* positions = ctx.position_column(position_ ? position_->position_column() : 0);
        const float* table = table_.defined() ? table_.as<float>() : nullptr;
        const int max_pos = table_.defined() ? (int)table_.shape[0] : 0;
        const size_t es = dtype_size(dt);

        Tensor down = down_proj_(x, ctx, "la_down", dt, T).tensor;                            // [T, c_q' | c' | r | gate logits]
        Tensor cq = ws.get("la_cq", {T, q_rank_}, dt);
        if (LaunchProfile::get().on()) LaunchProfile::get().note_cost((double)T * (down_width_ + q_rank_ + row) * es, 0.0);
        QE_LAUNCH(k, k.latent_prepare(down.data, down.code(), down_width_, q_rank_, kv_rank_, rot_, q_norm_.as<float>(), kv_norm_.as<float>(),
                                      (float)eps_, table, n_rot, max_pos, positions, g.slot_mapping, cq.data, cq.code(), cache.k_base,
                                      (int)cache.kv_dtype, cache.page_stride, cache.page_size, T, ctx.stream));
        Tensor q = q_up_(cq, ctx, "la_q", dt, T).tensor;                                      // [T, heads, plain | rotated]
        Tensor q_lat = ws.get("la_q_lat", {T, heads_, row}, dt);
        if (LaunchProfile::get().on())
            LaunchProfile::get().note_cost((double)T * heads_ * (dim_ + rot_ + row) * es + (double)k_up_.bytes(), 2.0 * T * heads_ * dim_ * kv_rank_);
        const bool tc_products = products_on_tensor_cores() && dt == DType::BF16;
        if (tc_products) {
            const LatentKernels& lk = latent_kernels();
            QE_LAUNCH(lk, lk.latent_absorb(q.data, k_up_.data, table, n_rot, max_pos, positions, q_lat.data, T, heads_, dim_, rot_, kv_rank_, ctx.stream));
        } else
        QE_LAUNCH(k, k.latent_absorb(q.data, q.code(), k_up_.data, k_up_.code(), table, n_rot, max_pos, positions, q_lat.data, q_lat.code(), T,
                                     heads_, dim_, rot_, kv_rank_, ctx.stream));
        // every head reads the one cached row per position: keys the whole row, values its first kv_rank numbers
        Tensor o_lat = ws.get("la_o_lat", {T, heads_, kv_rank_}, DType::F32);
        const int32_t* abs_positions = ctx.position_column(0);
        if (LaunchProfile::get().on()) {
            double seen = 0.0, read = 0.0;
            for (size_t i = 0; i < ctx.q_lens.size(); i++) {
                const double n = ctx.q_lens[i], len = ctx.ctx_lens[i];
                read += window_ ? std::min<double>(len, window_ + n) : len;
                seen += window_ ? n * std::min<double>(len, window_) : n * (len - n) + n * (n + 1) / 2.0;
            }
            LaunchProfile::get().note_cost(read * row * dtype_size(cache.kv_dtype) + (double)T * heads_ * (row * es + kv_rank_ * 4.0),
                                           2.0 * seen * heads_ * (row + kv_rank_));
        }
        // 16-byte copies: the rows of this entry start on such a boundary in every page (other entries of the group may not)
        const bool aligned = reinterpret_cast<uintptr_t>(cache.k_base) % 16 == 0 && cache.page_stride % 8 == 0;
        if (on_tensor_cores() && cache.kv_dtype == DType::BF16 && aligned) {
            const LatentKernels& lk = latent_kernels();
            const StepArray tiles = ctx.array(tiles_name() + ".seg"), firsts = ctx.array(tiles_name() + ".first");
            if (!tiles.count) throw Error(kInvalidState, "latent_attention: the step carries no tiles for this mixer");
            int splits = (int)ctx.option_int("latent_splits");           // a test's choice, else what fills the device
            if (splits < 1) splits = key_splits(tiles.count, std::max(ctx.decode_max_ctx, ctx.prefill_max_ctx), sm_count());
            float *part_o = nullptr, *part_ml = nullptr;
            if (splits > 1) {
                part_o = ws.get("la_part_o", {tiles.count, splits, kTileRows, kv_rank_}, DType::F32).as<float>();
                part_ml = ws.get("la_part_ml", {tiles.count, splits, kTileRows, 2}, DType::F32).as<float>();
            }
            QE_LAUNCH(lk, lk.attention(q_lat.data, cache.k_base, cache.page_stride, cache.page_size, g.block_table, g.table_width, ctx.seg_start,
                                       ctx.seg_ctx_len, tiles.data, firsts.data, tiles.count, o_lat.data, part_o, part_ml, heads_, kv_rank_,
                                       rot_, window_, (float)scale_, splits, ctx.stream));
        } else
        QE_LAUNCH(k, k.attention_generic(q_lat.data, q_lat.code(), cache.k_base, cache.k_base, (int)cache.kv_dtype, cache.page_stride,
                                         cache.page_size, g.block_table, g.table_width, ctx.row_seg, abs_positions, o_lat.data, o_lat.code(),
                                         T, heads_, 1, row, window_, (float)scale_, kv_rank_, 0, row, ctx.stream));
        Tensor out = ws.get("la_heads", {T, (int64_t)heads_ * vdim_}, dt);
        if (LaunchProfile::get().on())
            LaunchProfile::get().note_cost((double)T * heads_ * (kv_rank_ * 4.0 + vdim_ * es) + (double)v_up_.bytes(), 2.0 * T * heads_ * vdim_ * kv_rank_);
        const char* gate = gated_ ? static_cast<const char*>(down.data) + (size_t)(q_rank_ + row) * es : nullptr;
        if (tc_products && T > kFewRows) {               // few rows: more CTAs with a warp per value column
            const LatentKernels& lk = latent_kernels();
            QE_LAUNCH(lk, lk.latent_expand(o_lat.data, v_up_.data, gate, down_width_, out.data, T, heads_, kv_rank_, vdim_, ctx.stream));
        } else
        QE_LAUNCH(k, k.latent_expand(o_lat.data, o_lat.code(), v_up_.data, v_up_.code(), gate, down.code(), down_width_, out.data, out.code(), T,
                                     heads_, kv_rank_, vdim_, ctx.stream));
        return o_proj_(out, ctx, "la_out", DType::F32, T, true, false, ctx.residual, nullptr, &ctx.norm_ahead);
    }

private:
    // CTAs per tile: with fewer tiles than SMs the keys of a tile (blocks of 64) are cut so that the CTAs fill the
    // device about once; a split costs about a block more (its partial result goes through memory), and the merge grows with the parts it reads
    int key_splits(int n_tiles, int max_ctx, int sms) const {
        const int span = window_ ? std::min(max_ctx, window_ + kTileRows / heads_) : max_ctx;
        const int blocks = std::max(1, (span + 63) / 64);
        int best = 1;
        double best_cost = -1;
        for (int s = 1; s <= std::min(blocks, 32); s++) {
            const int per = (blocks + s - 1) / s;
            const double cost = (double)(((long long)n_tiles * s + sms - 1) / sms) * (per + (s > 1 ? 1.0 : 0.0)) + (s > 1 ? 2.0 + 0.25 * s : 0.0);
            if (best_cost < 0 || cost < best_cost - 1e-9) { best = s; best_cost = cost; }
        }
        return best;
    }
    std::string tiles_name() const { return "latent.tiles.h" + std::to_string(heads_) + (window_ ? ".w" + std::to_string(window_) : ""); }

    static constexpr int kFewRows = 16;
    static constexpr int kTileRows = 64;         // (token, head) pairs of a tile of the tensor-core kernel
    static constexpr int kMaxRow = 640;          // the widest cache row the attention kernel holds a query for
    int64_t hidden_, down_width_;
    int heads_, dim_, rot_, vdim_, q_rank_, kv_rank_, window_;
    bool gated_;
    double eps_, scale_;
    std::string gemm_, attention_;
    std::shared_ptr<PositionEncoding> position_;
    Linear down_proj_, q_up_, o_proj_;
    Tensor q_norm_, kv_norm_, k_up_, v_up_, table_;
};

void register_latent_attention_parts() {
    register_part("mixer", "latent_attention", [](const Json& p, BuildContext& b) { return std::make_shared<LatentAttention>(p, b); });
}

}  // namespace qe
