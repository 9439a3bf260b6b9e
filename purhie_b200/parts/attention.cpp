// Grouped-query attention over cache pages, with per-head RMSNorm on q and k and a position encoding.
//
// q = Wq x, k = Wk x, v = Wv x (+ optional biases, added before the norms); each q and k head is RMS-normalised
// over head_dim with a weight shared by all heads (same eps as the layer norms), then rotated; k and v go into
// the request's pages; query head h attends with kv head h / (HQ / HKV), scale 1 / sqrt(head_dim), causally,
// optionally only over the last `window` positions, or only over the positions of its own block of `chunk` positions
// (blocks counted from position 0 of the request, wherever a prompt was cut); then y = Wo o.
// Reference: src/qwen_model.cpp:940-975 (full_attention), src/attention.hip:273-313 (prep),
// src/attention.cpp:139-288 (host side; scale at :197), src/attention.h:73 (window),
// src/inference.cpp:623-646 (tensors and shapes).
//
// Options of other designs: values of another width than keys ("value_dim"; o_proj then reads num_heads * value_dim),
// and value mixing across layers ("value_mix": "first" | "blend"): the first such layer of a model leaves its v for
// every token of the step, the later ones cache and attend over v <- (1 - lambda) v + lambda v_first, with lambda a
// scalar tensor of their own ("value_mix_factor"); a sink (names.sink: one float32 number per query head that stands in
// the softmax's denominator as exp(sink), without a key or a value).
//
// K and V are written to pages before attention runs, and attention reads everything, the current step's keys
// included, from pages: a whole prompt, a portion and a decoded token are one algorithm per kernel.
//
// Which kernel: float32, or a head size the tensor-core kernels do not take -> attention_generic (any size, fixed
// order).  bfloat16 with head size 64 or 128 and groups up to 16: single-token segments go to the persistent
// TMA-fed split-key kernel (pages of 8..64 tokens; else the cp.async one), prompt portions to the tcgen05 kernel
// (head size 128, pages of 8 to 64) or the mma.sync tiled kernel.  The tile lists those two want are this
// part's own metadata: prepare_step() adds them to the step.
#include <algorithm>
#include <cmath>

#include "linear.h"
#include "parts.h"

namespace qe {

namespace {
constexpr int kBlockKeys = 64, kMaxSplits = 32;
constexpr int kTile = 64;          // rows of a query tile of the mma.sync prefill kernel
constexpr int kTileLarge = 128;    // rows of a query tile of the tcgen05 prefill kernel
constexpr int kTileAll = 16;       // rows of a tile of the kernel that takes all heads of a tile at once
constexpr int kCtasPerSm = 3;      // cp.async decode CTAs that fit one SM (68 KB of shared memory each at head_dim 128)
inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Splits of the key range for the cp.async decode kernel.  CTAs run in waves of kCtasPerSm per SM; the number of
// splits is the one that minimises waves x (fixed cost + blocks per split).
int decode_splits(int n_rows, int kv_heads, int max_ctx, int sms, int window) {
    const int span = window ? std::min(max_ctx, window) : max_ctx;
    const int blocks = std::max(1, ceil_div(span, kBlockKeys)), pairs = std::max(1, n_rows * kv_heads), slots = kCtasPerSm * sms;
    int best = 1;
    double best_cost = -1;
    for (int s = 1; s <= std::min(blocks, kMaxSplits); s++) {
        const int per = ceil_div(blocks, s);
        if (s > 1 && ceil_div(blocks, per) != s) continue;        // the same blocks per split as a smaller s
        const double cost = (double)ceil_div((long long)pairs * s, slots) * (4.0 + per);
        if (best_cost < 0 || cost < best_cost - 1e-9) { best = s; best_cost = cost; }
    }
    return best;
}

// Splits for the persistent kernel: two CTAs per SM take items in turn, so the time is (items per CTA, rounded
// up) x (blocks of 64 keys per item + what an item costs beside its blocks), plus the merge kernel when the keys
// are split.  A split item costs about a block and a half more (its partial result goes to memory), a whole one
// next to nothing, and the merge grows with the number of parts it reads: measured at 1 to 128 rows of 1,024 to
// 8,192 keys.
int bulk_splits(int n_rows, int kv_heads, int max_ctx, int sms, int window) {
    const int span = window ? std::min(max_ctx, window) : max_ctx;
    const int blocks = std::max(1, ceil_div(span, kBlockKeys)), pairs = std::max(1, n_rows * kv_heads);
    int best = 1;
    double best_cost = -1;
    for (int s = 1; s <= std::min(blocks, kMaxSplits); s++) {
        const int per = ceil_div(blocks, s);
        if (s > 1 && ceil_div(blocks, per) != s) continue;
        const double cost = (double)ceil_div((long long)pairs * s, 2 * sms) * (per + (s > 1 ? 1.5 : 0.25)) + (s > 1 ? 2.0 + 0.15 * s : 0.0);
        if (best_cost < 0 || cost < best_cost - 1e-9) { best = s; best_cost = cost; }
    }
    return best;
}

// CTAs per tile of the tcgen05 prefill kernel.  The time is about (rounds of the CTAs over two slots per SM) x
// (blocks of 64 keys per CTA + a few for its start) plus, when tiles are shared, what writing and merging the
// partial results costs.  Many tiles, or tiles that look back over few keys, stay whole; a short portion late
// in a long context is cut so that its CTAs fill the device once.
int tc5_splits(int n_tiles, int heads, int max_ctx, int sms, int window) {
    const int span = window ? std::min(max_ctx, window + 128) : max_ctx;
    const int blocks = std::max(1, ceil_div(span, 64)), ctas = std::max(1, n_tiles * heads);
    int best = 1;
    double best_cost = -1;
    for (int s = 1; s <= std::min(16, blocks); s++) {
        double cost = (double)ceil_div((long long)ctas * s, 2 * sms) * (ceil_div(blocks, s) + 4);
        if (s > 1) cost += 8 + 0.5 * s + 0.024 * ctas * s;
        if (best_cost < 0 || cost < best_cost - 1e-9) { best = s; best_cost = cost; }
    }
    return best;
}

// CTAs per tile of the kernel that takes all heads of a 16-row tile at once: with fewer tiles than the device holds CTAs
// (decoding, a short portion, few heads) the keys of a tile are shared so that every place is filled about once; a CTA
// keeps at least two blocks of 32 keys.  It depends on the step's bucketed reach only, so a decode graph replays.
int tile16_splits(int n_tiles, int max_ctx, int window, int places) {
    const int span = window ? std::min(max_ctx, window + 16) : max_ctx;
    const int blocks = std::max(1, ceil_div(span, 32));
    if (2 * n_tiles > places || blocks < 4) return 1;
    return std::max(1, std::min({places / std::max(n_tiles, 1), blocks / 2, 32}));
}

// The prompt portions of a step cut into tiles of `rows` rows: segment and first row (within the portion) of
// each tile (single_rows: a decode row is a tile too, so that every row of the step is in one).  The tiles that look
// furthest back come first: the grid starts them first and the short ones fill the tail.
void add_tiles(StepPlan& plan, int rows, const std::string& name, bool single_rows = false) {
    if (plan.has(name + ".seg")) return;
    struct Tile { int seg, first, reach; };
    std::vector<Tile> tiles;
    for (int s = 0; s < plan.S; s++) {
        const int n = plan.q_lens[s];
        if (n == 1 && !single_rows) continue;
        for (int first = 0; first < n; first += rows)
            tiles.push_back({s, first, plan.ctx_lens[s] - n + std::min(first + rows, n)});
    }
    std::stable_sort(tiles.begin(), tiles.end(), [](const Tile& a, const Tile& b) { return a.reach > b.reach; });
    std::vector<int32_t> seg, first;
    for (const Tile& t : tiles) { seg.push_back(t.seg); first.push_back(t.first); }
    plan.add(name + ".seg", std::move(seg));
    plan.add(name + ".first", std::move(first));
}
}  // namespace

// params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim (null: head_dim), qk_norm_eps (null: no q/k norm),
// bias, position (a PartSpec as {kind, params}, or null), window (null: all positions), chunk (null: no block mask),
// scale (null: 1/sqrt(head_dim)), value_mix (null | "first" | "blend"),
// names{q_proj, k_proj, v_proj, o_proj, q_norm, k_norm, q_bias, k_bias, v_bias, value_mix_factor}.
class Attention : public Mixer {
public:
    Attention(const Json& p, BuildContext& b) : Mixer(p, b) {
        hidden_ = p.at("hidden_size").as_int();
        heads_ = (int)p.at("num_heads").as_int();
        kv_heads_ = (int)p.at("num_kv_heads").as_int();
        head_dim_ = (int)p.at("head_dim").as_int();
        value_dim_ = (int)p.get_int("value_dim", head_dim_);
        if (value_dim_ < 1) throw ConfigError("attention: value_dim must be positive");
        const std::string mix = p.get_string("value_mix", "");
        if (!mix.empty() && mix != "first" && mix != "blend") throw ConfigError("attention: value_mix is 'first' or 'blend', got '" + mix + "'");
        value_mix_ = mix == "first" ? 1 : mix == "blend" ? 2 : 0;
        if (heads_ < 1 || kv_heads_ < 1 || heads_ % kv_heads_)
            throw ConfigError(std::to_string(heads_) + " query heads are not a multiple of " + std::to_string(kv_heads_) + " kv heads");
        const Json* eps = p.find("qk_norm_eps");
        has_norm_ = eps && !eps->is_null();
        eps_ = has_norm_ ? eps->as_double() : 0.0;
        has_bias_ = p.get_bool("bias", false);
        has_sink_ = names_.count("sink") != 0;
        window_ = (int)p.get_int("window", 0);
        chunk_ = (int)p.get_int("chunk", 0);
        if (chunk_ < 0) throw ConfigError("attention: a block mask holds at least one position");
        const Json* sc = p.find("scale");
        scale_ = (sc && !sc->is_null()) ? sc->as_double() : 1.0 / std::sqrt((double)head_dim_);
        if (const Json* pos = p.find("position")) {
            if (!pos->is_null()) {
                PartSpec spec = PartSpec::from_json(*pos);
                Json key_params = Json::object();
                for (const auto& m : spec.params.members()) if (m.first != "names") key_params.set(m.first, m.second);
                auto part = b.shared("position:" + spec.kind + ":" + key_params.dump(), [&] { return make_part("position", spec, b); });
                position_ = std::dynamic_pointer_cast<PositionEncoding>(part);
                if (!position_) throw ConfigError("part '" + spec.kind + "' is not a position encoding");
            }
        }
        gemm_ = b.options.get_string("gemm", "auto");
        attention_ = b.options.get_string("attention", "auto");
        q_width_ = (int64_t)heads_ * head_dim_;
        kv_width_ = (int64_t)kv_heads_ * head_dim_;
        v_width_ = (int64_t)kv_heads_ * value_dim_;
        o_width_ = (int64_t)heads_ * value_dim_;
    }

    // ---- weights ----------------------------------------------------------------------------------------------
    std::vector<TensorSpec> tensor_specs() const override {
        std::vector<TensorSpec> s = {{name_of("q_proj"), {q_width_, hidden_}, Role::Matrix, Init::Normal},
                                     {name_of("k_proj"), {kv_width_, hidden_}, Role::Matrix, Init::Normal},
                                     {name_of("v_proj"), {v_width_, hidden_}, Role::Matrix, Init::Normal},
                                     {name_of("o_proj"), {hidden_, o_width_}, Role::Matrix, Init::Normal}};
        if (value_mix_ == 2) s.push_back({name_of("value_mix_factor"), {}, Role::Vector, Init::Normal});
        if (has_sink_) s.push_back({name_of("sink"), {heads_}, Role::Vector, Init::Normal});
        if (has_norm_) {
            s.push_back({name_of("q_norm"), {head_dim_}, Role::Vector, Init::Scale});
            s.push_back({name_of("k_norm"), {head_dim_}, Role::Vector, Init::Scale});
        }
        if (has_bias_) {
            s.push_back({name_of("q_bias"), {q_width_}, Role::Vector, Init::Normal});
            s.push_back({name_of("k_bias"), {kv_width_}, Role::Vector, Init::Normal});
            s.push_back({name_of("v_bias"), {v_width_}, Role::Vector, Init::Normal});
        }
        return s;
    }

    void bind(WeightSource& src) override {
        // one matrix [q | k | v] so that the three projections are one product (a layout choice only)
        Tensor parts[3] = {src.fetch(name_of("q_proj")), src.fetch(name_of("k_proj")), src.fetch(name_of("v_proj"))};
        if (parts[0].dtype != parts[1].dtype || parts[0].dtype != parts[2].dtype)
            throw WeightError(name_of("q_proj") + ", " + name_of("k_proj") + " and " + name_of("v_proj") + " are stored in different precisions");
        Tensor qkv = src.arena().alloc(parts[0].dtype, {q_width_ + kv_width_ + v_width_, hidden_});
        size_t off = 0;
        for (Tensor& t : parts) {
            QE_CUDA(cudaMemcpyAsync(static_cast<char*>(qkv.data) + off, t.data, t.bytes(), cudaMemcpyDeviceToDevice, src.stream()));
            off += t.bytes();
        }
        if (has_bias_) {
            Tensor b[3] = {src.fetch(name_of("q_bias")), src.fetch(name_of("k_bias")), src.fetch(name_of("v_bias"))};
            bias_ = src.arena().alloc(DType::F32, {q_width_ + kv_width_ + v_width_});
            off = 0;
            for (Tensor& t : b) {
                QE_CUDA(cudaMemcpyAsync(static_cast<char*>(bias_.data) + off, t.data, t.bytes(), cudaMemcpyDeviceToDevice, src.stream()));
                off += t.bytes();
            }
            QE_CUDA(cudaStreamSynchronize(src.stream()));
            for (Tensor& t : b) src.release(t);
        }
        QE_CUDA(cudaStreamSynchronize(src.stream()));
        for (Tensor& t : parts) src.release(t);
        qkv_proj_ = Linear(qkv, "qkv_proj", gemm_);
        q_only_proj_ = Linear(qkv.rows(0, q_width_), "q_proj", gemm_);
        o_proj_ = Linear(src.fetch(name_of("o_proj")), "o_proj", gemm_);
        if (has_norm_) {
            q_norm_ = src.fetch(name_of("q_norm"));
            k_norm_ = src.fetch(name_of("k_norm"));
        }
        if (value_mix_ == 2) mix_factor_ = src.fetch(name_of("value_mix_factor"));
        if (has_sink_) sink_ = src.fetch(name_of("sink"));
        if (position_) {
            position_->bind(src);
            table_ = position_->rotation_table();
        }
    }

    std::vector<std::string> required_libraries() const override {
        std::vector<std::string> libs = {"core"};
        if (qkv_proj_.fast() || o_proj_.fast()) libs.push_back("gemm100");
        if (use_flash()) libs.push_back("flash");
        return libs;
    }
    std::vector<std::string> ignored_tensors() const override {
        // the first mixing layer has nothing to blend with; a factor stored for it is not read
        if (value_mix_ == 1 && names_.count("value_mix_factor")) return {name_of("value_mix_factor")};
        return {};
    }
    std::vector<Part*> children() override { return position_ ? std::vector<Part*>{position_.get()} : std::vector<Part*>{}; }
    // rows per tile of the products for many tokens (the tcgen05 pair kernel): a scheduler may end a step there
    int preferred_row_multiple() const override { return (qkv_proj_.fast() || o_proj_.fast()) ? 256 : 0; }

    // how far back a row can look at most: the window, the mask's block, the smaller of the two (0: all the way)
    int reach() const { return window_ && chunk_ ? std::min(window_, chunk_) : window_ ? window_ : chunk_; }

    bool use_flash() const {
        if (compute_dtype != DType::BF16 || attention_ == "generic") return false;
        const int group = heads_ / kv_heads_;
        // (of the tensor-core kernels the tcgen05 prompt kernel and the TMA decode kernel know sinks: heads of 128)
        const bool ok = (head_dim_ == 64 || head_dim_ == 128) && value_dim_ == head_dim_ && group >= 1 && group <= 16 &&
                        (!has_sink_ || head_dim_ == 128);
        if (!ok && attention_ == "flash")
            throw KernelError("the flash attention kernels do not take head_dim " + std::to_string(head_dim_) + " with " +
                              std::to_string(group) + " query heads per kv head");
        return ok;
    }

    // ---- cache and step metadata ------------------------------------------------------------------------------
    CacheNeed cache_need() const override { return CacheNeed::pages(kv_heads_, head_dim_, window_, value_dim_, chunk_); }

    // attention with a sink in bfloat16 runs on the tensor-core kernel that knows sinks (a tile of 16 rows, all heads)
    bool use_sink_kernel() const {
        return has_sink_ && compute_dtype == DType::BF16 && attention_ != "generic" && !chunk_ &&
               core_kernels().attention_talking_mma_supports(heads_, kv_heads_, head_dim_, value_dim_);
    }

    void prepare_step(StepPlan& plan) override {
        if (use_sink_kernel()) add_tiles(plan, kTileAll, "attention.tiles16", true);
        if (!use_flash()) return;
        bool portions = false;
        for (int n : plan.q_lens) portions |= n > 1;
        if (!portions) return;
        add_tiles(plan, kTile, "attention.tiles64");
        add_tiles(plan, kTileLarge, "attention.tiles128");
    }

    // Few rows in bfloat16: the qkv product's float32 sums are linear in the rows, and the kernel that adds them up
    // (per-head norm, rotation, cache write) multiplies by the factor the norm in front left out.
    // Many rows: either the qkv product's epilogue applies the factor (K whole), or K is cut and the same kernel as
    // above adds up the parts.
    bool takes_unscaled_rows(const StepContext& ctx) const override {
        auto takes = [&](const Linear& proj) {
            return proj.swapped_for(ctx.T, true, false) || proj.applies_row_scale(ctx.T, compute_dtype, false, true) ||
                   proj.gives_partial_sums(ctx.T, true);
        };
        return compute_dtype == DType::BF16 && takes(qkv_proj_) && (!q_only_proj_.defined() || takes(q_only_proj_));
    }

    // ---- step ----------------------------------------------------------------------------------------------------
    Addend forward(const Tensor& x, StepContext& ctx, const CacheView& cache) override {
        const int T = ctx.T;
        Workspace& ws = *ctx.workspace;
        const DType dt = compute_dtype;
        const GroupStep& g = ctx.groups.at(cache.group);
        const CoreKernels& core = core_kernels();
        const Linear& proj = cache.writable ? qkv_proj_ : q_only_proj_;
        // rows without their factor (RowScale): the product's epilogue applies it where it can, else the kernel behind it
        const bool scale_in_product = ctx.row_scale.defined() && proj.applies_row_scale(T, dt, false, true);
        if (!cache.writable && value_mix_) throw Error(kInvalidState, "a layer that mixes values writes a cache of its own");
        Addend qkv = proj(x, ctx, "qkv", dt, T, true, false, nullptr, scale_in_product ? &ctx.row_scale : nullptr);
        // the values of the first mixing layer, per token of the step: written by that layer, read by the later ones
        float* v_first = value_mix_ ? ws.get("attention.v_first", {T, v_width_}, DType::F32).as<float>() : nullptr;
        const RowScale later = scale_in_product ? RowScale() : ctx.row_scale;
        const int kv_heads_written = cache.writable ? kv_heads_ : 0;
        Tensor q = ws.get("q", {T, heads_, head_dim_}, dt);
        const int column = position_ ? position_->position_column() : 0;
        const int32_t* positions = ctx.position_column(column);
        if (LaunchProfile::get().on()) {       // reads the product's rows (every split), writes q and the cache rows
            const double row = (double)(q_width_ + (int64_t)kv_heads_written * (head_dim_ + value_dim_));
            LaunchProfile::get().note_cost((double)T * row * (qkv.splits * dtype_size(qkv.tensor.dtype) + dtype_size(dt)), 0.0);
        }
        QE_LAUNCH(core, core.qk_norm_rope_kv_write(
            qkv.tensor.data, qkv.tensor.code(), qkv.splits, (long long)T * (q_width_ + (int64_t)kv_heads_written * (head_dim_ + value_dim_)),
            bias_.defined() ? bias_.as<float>() : nullptr, has_norm_ ? q_norm_.as<float>() : nullptr,
            has_norm_ ? k_norm_.as<float>() : nullptr, (float)eps_, table_.defined() ? table_.as<float>() : nullptr,
            position_ ? position_->n_rot() : 0, table_.defined() ? (int)table_.shape[0] : 0, positions,
            cache.writable ? g.slot_mapping : nullptr, q.data, q.code(), cache.k_base, cache.v_base, (int)cache.kv_dtype,
            cache.page_stride, cache.page_size, T, heads_, kv_heads_written, head_dim_,
            position_ && position_->interleaved() ? 1 : 0, later.sumsq, later.chunks, later.width, later.eps, value_dim_, v_first,
            mix_factor_.defined() ? mix_factor_.as<float>() : nullptr, value_mix_, ctx.stream));
        Tensor out = ws.get("attn_out", {T, o_width_}, dt);
        const int32_t* abs_positions = ctx.position_column(0);       // the mask always follows the index in the request
        if (LaunchProfile::get().on()) {
            // keys and values each row looks back over (read once per request and kv head at best), q in, the output out;
            // two products of a row with every key it sees
            double seen = 0.0, read = 0.0;
            for (size_t i = 0; i < ctx.q_lens.size(); i++) {
                const double n = ctx.q_lens[i], len = ctx.ctx_lens[i];
                const int reach = this->reach();
                const double span = reach ? std::min<double>(len, reach + n) : len;
                read += span;
                seen += reach ? n * std::min<double>(len, chunk_ ? reach / 2.0 : reach) : n * (len - n) + n * (n + 1) / 2.0;
            }
            const double kv = dtype_size(cache.kv_dtype);
            LaunchProfile::get().note_cost(read * kv_heads_ * (head_dim_ + value_dim_) * kv + (double)T * (q_width_ + o_width_) * dtype_size(dt),
                                           2.0 * seen * heads_ * (head_dim_ + value_dim_));
        }
        const StepArray t16 = ctx.array("attention.tiles16.seg"), t16f = ctx.array("attention.tiles16.first");
        // a sink rides in the tcgen05 prompt kernel and the TMA decode kernel only: pages they take, and no other choice by option
        const bool pages_ok = (cache.page_size == 8 || cache.page_size == 16 || cache.page_size == 32 || cache.page_size == 64) && cache.num_pages > 0;
        const bool sink_ok = !has_sink_ || (pages_ok && ctx.option("prefill_kernel") != "mma_sync" && ctx.option("decode_kernel") != "cp_async" &&
                                            ctx.option("sink_kernel") != "tile");
        if (use_flash() && sink_ok) {
            if (cache.kv_dtype != DType::BF16) throw KernelError("attention_flash: the cache must be bfloat16");
            flash(q, cache, g, ctx, out, abs_positions);
        } else if (use_sink_kernel() && cache.kv_dtype == DType::BF16 && t16.count) {
            int splits = (int)ctx.option_int("tile16_splits");
            if (splits < 1)
                splits = tile16_splits(t16.count, std::max(ctx.decode_max_ctx, ctx.prefill_max_ctx), window_,
                                       sm_count() * core.attention_talking_mma_ctas_per_sm(heads_, kv_heads_, head_dim_, value_dim_) /
                                           (heads_ > 16 ? 2 : 1));      // above 16 heads a tile takes a pair of CTAs
            float *part_o = nullptr, *part_ml = nullptr;
            if (splits > 1) {
                part_o = ws.get("attn16_part_o", {T, heads_, splits, value_dim_}, DType::F32).as<float>();
                part_ml = ws.get("attn16_part_ml", {T, heads_, splits, 2}, DType::F32).as<float>();
            }
            QE_LAUNCH(core, core.attention_talking_mma(q.data, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, g.block_table,
                                                       g.table_width, ctx.seg_start, ctx.seg_ctx_len, t16.data, t16f.data, t16.count, out.data,
                                                       heads_, kv_heads_, head_dim_, value_dim_, window_, 0, (float)scale_, 0.0f, nullptr,
                                                       nullptr, nullptr, sink_.as<float>(), nullptr, 0, splits, T, part_o, part_ml, ctx.stream));
        } else if (has_sink_) {
            QE_LAUNCH(core, core.attention_generic_sink(q.data, q.code(), cache.k_base, cache.v_base, (int)cache.kv_dtype, cache.page_stride,
                                                        cache.page_size, g.block_table, g.table_width, ctx.row_seg, abs_positions, out.data,
                                                        out.code(), T, heads_, kv_heads_, head_dim_, window_, (float)scale_, value_dim_, chunk_, 0,
                                                        sink_.as<float>(), ctx.stream));
        } else {
            QE_LAUNCH(core, core.attention_generic(q.data, q.code(), cache.k_base, cache.v_base, (int)cache.kv_dtype, cache.page_stride,
                                                   cache.page_size, g.block_table, g.table_width, ctx.row_seg, abs_positions, out.data,
                                                   out.code(), T, heads_, kv_heads_, head_dim_, window_, (float)scale_, value_dim_, chunk_, 0,
                                                   ctx.stream));
        }
        return o_proj_(out, ctx, "o_out", DType::F32, T, true, false, ctx.residual, nullptr, &ctx.norm_ahead);
    }

private:
    // All rows of the step: q [T, HQ, D] bfloat16 -> out [T, HQ * D] bfloat16.
    void flash(const Tensor& q, const CacheView& cache, const GroupStep& g, StepContext& ctx, Tensor& out, const int32_t* positions) {
        const FlashKernels& f = flash_kernels();
        Workspace& ws = *ctx.workspace;
        const int sms = sm_count();
        StepArray t64 = ctx.array("attention.tiles64.seg"), t64f = ctx.array("attention.tiles64.first");
        StepArray t128 = ctx.array("attention.tiles128.seg"), t128f = ctx.array("attention.tiles128.first");
        const bool tc5_ok = head_dim_ == 128 && (cache.page_size == 8 || cache.page_size == 16 || cache.page_size == 32 || cache.page_size == 64) && cache.num_pages > 0;
        if (t64.count && t128.count && tc5_ok && ctx.option("prefill_kernel") != "mma_sync") {
            int splits = (int)ctx.option_int("prefill_splits");
            if (!splits) splits = tc5_splits(t128.count, heads_, ctx.prefill_max_ctx, sms, reach());
            float *part_o = nullptr, *part_ml = nullptr;
            if (splits > 1) {
                part_o = ws.get("attn_tile_part_o", {ctx.T, heads_, splits, head_dim_}, DType::F32).as<float>();
                part_ml = ws.get("attn_tile_part_ml", {ctx.T, heads_, splits, 2}, DType::F32).as<float>();
            }
            if (has_sink_)
                QE_LAUNCH(f, f.prefill_tc5_sink(q.data, ctx.T, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, cache.num_pages,
                                                g.block_table, g.table_width, ctx.seg_start, ctx.seg_ctx_len, t128.data, t128f.data, t128.count,
                                                out.data, heads_, kv_heads_, head_dim_, window_, chunk_, (float)scale_, splits, part_o, part_ml,
                                                ctx.attention_error, sink_.as<float>(), ctx.stream));
            else
                QE_LAUNCH(f, f.prefill_tc5(q.data, ctx.T, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, cache.num_pages,
                                           g.block_table, g.table_width, ctx.seg_start, ctx.seg_ctx_len, t128.data, t128f.data, t128.count,
                                           out.data, heads_, kv_heads_, head_dim_, window_, chunk_, (float)scale_, splits, part_o, part_ml,
                                           ctx.attention_error, ctx.stream));
        } else if (t64.count) {
            if (has_sink_) throw Error(kInvalidState, "attention: the tiled prompt kernel knows no sink");
            QE_LAUNCH(f, f.prefill(q.data, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, g.block_table, g.table_width,
                                   ctx.seg_start, ctx.seg_ctx_len, t64.data, t64f.data, t64.count, out.data, heads_, kv_heads_,
                                   head_dim_, window_, chunk_, (float)scale_, ctx.stream));
        }
        if (!ctx.n_decode_rows) return;
        const int n = ctx.n_decode_rows;
        const bool bulk_ok = cache.page_size % 8 == 0 && kBlockKeys % cache.page_size == 0 && cache.num_pages > 0;
        const bool bulk = bulk_ok && ctx.option("decode_kernel") != "cp_async";
        int splits = (int)ctx.option_int("decode_splits");            // a test's choice, else what the cost model picks
        if (splits < 1 || splits > kMaxSplits)
            splits = bulk ? bulk_splits(n, kv_heads_, ctx.decode_max_ctx, sms, reach())
                          : decode_splits(n, kv_heads_, ctx.decode_max_ctx, sms, reach());
        float *part_o = nullptr, *part_ml = nullptr;
        if (splits > 1) {
            part_o = ws.get("attn_part_o", {n, heads_, splits, head_dim_}, DType::F32).as<float>();
            part_ml = ws.get("attn_part_ml", {n, heads_, splits, 2}, DType::F32).as<float>();
        }
        if (bulk && has_sink_)
            QE_LAUNCH(f, f.decode_bulk_sink(q.data, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, cache.num_pages, g.block_table,
                                            g.table_width, ctx.decode_rows, n, ctx.row_seg, positions, part_o, part_ml, out.data, heads_,
                                            kv_heads_, head_dim_, splits, window_, chunk_, (float)scale_, 0, ctx.attention_error,
                                            sink_.as<float>(), ctx.stream));
        else if (bulk)
            QE_LAUNCH(f, f.decode_bulk(q.data, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, cache.num_pages, g.block_table,
                                       g.table_width, ctx.decode_rows, n, ctx.row_seg, positions, part_o, part_ml, out.data, heads_,
                                       kv_heads_, head_dim_, splits, window_, chunk_, (float)scale_, 0, ctx.attention_error, ctx.stream));
        else if (has_sink_)
            throw Error(kInvalidState, "attention: the cp.async decode kernel knows no sink");
        else
            QE_LAUNCH(f, f.decode(q.data, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, g.block_table, g.table_width,
                                  ctx.decode_rows, n, ctx.row_seg, positions, part_o, part_ml, out.data, heads_, kv_heads_, head_dim_,
                                  splits, window_, chunk_, (float)scale_, ctx.stream));
    }

    int64_t hidden_, q_width_, kv_width_, v_width_, o_width_;
    int heads_, kv_heads_, head_dim_, value_dim_, window_, chunk_ = 0, value_mix_ = 0;
    bool has_norm_, has_bias_, has_sink_ = false;
    double eps_, scale_;
    std::string gemm_, attention_;
    std::shared_ptr<PositionEncoding> position_;
    Linear qkv_proj_, q_only_proj_, o_proj_;
    Tensor q_norm_, k_norm_, bias_, table_, mix_factor_, sink_;
};

// Grouped-query attention whose heads talk to each other before the softmax.
//
//   q = Wq h, k = Wk h; q and k are RMS-normed over their whole width (all heads as one row, a weight per element;
//   "joint_norm_eps" null: no norm); v = Wv h, or, with "values": "keys", the keys as projected, before their norm (the
//   mixer then has no Wv).  No rotation.  For the row at position z and a key at p:
//       s_g = (q_g . k_kv(g)) * scale;   s_g <- cap * tanh(s_g / cap)   ("softcap" null: no cap);
//       s_g <- s_g - r1_g ln(1 + r2_g (z - p))   (names.distance_slope and names.distance_rate, both or none);
//       s_h <- sum_g talk[h, g] s_g              (names.head_mix, [heads, heads]; absent: the heads stay apart);
//   softmax over the last `window` positions (null: all), with exp(sink_h) in the denominator when names.sink is given;
//   the heads side by side times sigmoid(Wg h) (names.gate_proj; absent: no gate); y = Wo o.
// The projections of h are one product over the stacked matrices [q | k | (v) | (g)].  The normed keys and the values go
// into the request's pages before attention runs, and attention reads everything from pages, so a whole prompt, a
// portion and a decoded token are one algorithm.  Scores, the cap, the bias, the mix and the softmax are float32 in
// every mode.
// params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim (null: head_dim), values ("projection" | "keys"),
// joint_norm_eps, window, scale (null: 1/sqrt(head_dim)), softcap,
// names{q_proj, k_proj, v_proj, o_proj, q_norm, k_norm, distance_slope, distance_rate, head_mix, sink, gate_proj}.
class TalkingAttention : public Mixer {
public:
    TalkingAttention(const Json& p, BuildContext& b) : Mixer(p, b) {
        hidden_ = p.at("hidden_size").as_int();
        heads_ = (int)p.at("num_heads").as_int();
        kv_heads_ = (int)p.at("num_kv_heads").as_int();
        head_dim_ = (int)p.at("head_dim").as_int();
        value_dim_ = (int)p.get_int("value_dim", head_dim_);
        if (heads_ < 1 || kv_heads_ < 1 || heads_ % kv_heads_)
            throw ConfigError(std::to_string(heads_) + " query heads are not a multiple of " + std::to_string(kv_heads_) + " kv heads");
        if (head_dim_ < 1 || value_dim_ < 1) throw ConfigError("talking_attention: head_dim and value_dim must be positive");
        const std::string values = p.get_string("values", "projection");
        if (values != "projection" && values != "keys") throw ConfigError("talking_attention: values is 'projection' or 'keys', got '" + values + "'");
        values_are_keys_ = values == "keys";
        if (values_are_keys_ && value_dim_ != head_dim_)
            throw ConfigError("talking_attention: values that are the keys are " + std::to_string(head_dim_) + " wide, not " + std::to_string(value_dim_));
        const Json* eps = p.find("joint_norm_eps");
        has_norm_ = eps && !eps->is_null();
        eps_ = has_norm_ ? eps->as_double() : 0.0;
        window_ = (int)p.get_int("window", 0);
        const Json* sc = p.find("scale");
        scale_ = (sc && !sc->is_null()) ? sc->as_double() : 1.0 / std::sqrt((double)head_dim_);
        const Json* cap = p.find("softcap");
        softcap_ = (cap && !cap->is_null()) ? cap->as_double() : 0.0;
        if (softcap_ < 0.0) throw ConfigError("talking_attention: softcap must be positive");
        has_distance_ = names_.count("distance_slope") != 0;
        if (has_distance_ != (names_.count("distance_rate") != 0)) throw ConfigError("talking_attention: the distance bias needs both distance_slope and distance_rate");
        has_mix_ = names_.count("head_mix") != 0;
        has_sink_ = names_.count("sink") != 0;
        has_gate_ = names_.count("gate_proj") != 0;
        gemm_ = b.options.get_string("gemm", "auto");
        attention_ = b.options.get_string("attention", "auto");
        q_width_ = (int64_t)heads_ * head_dim_;
        kv_width_ = (int64_t)kv_heads_ * head_dim_;
        v_width_ = values_are_keys_ ? 0 : (int64_t)kv_heads_ * value_dim_;
        o_width_ = (int64_t)heads_ * value_dim_;
        g_width_ = has_gate_ ? o_width_ : 0;
    }

    std::vector<TensorSpec> tensor_specs() const override {
        std::vector<TensorSpec> s = {{name_of("q_proj"), {q_width_, hidden_}, Role::Matrix, Init::Normal},
                                     {name_of("k_proj"), {kv_width_, hidden_}, Role::Matrix, Init::Normal},
                                     {name_of("o_proj"), {hidden_, o_width_}, Role::Matrix, Init::Normal}};
        if (!values_are_keys_) s.push_back({name_of("v_proj"), {v_width_, hidden_}, Role::Matrix, Init::Normal});
        if (has_gate_) s.push_back({name_of("gate_proj"), {g_width_, hidden_}, Role::Matrix, Init::Normal});
        if (has_norm_) {
            s.push_back({name_of("q_norm"), {q_width_}, Role::Vector, Init::Scale});
            s.push_back({name_of("k_norm"), {kv_width_}, Role::Vector, Init::Scale});
        }
        if (has_distance_) {
            s.push_back({name_of("distance_slope"), {heads_}, Role::Vector, Init::Normal});
            s.push_back({name_of("distance_rate"), {heads_}, Role::Vector, Init::Scale});
        }
        if (has_mix_) s.push_back({name_of("head_mix"), {heads_, heads_}, Role::Vector, Init::Normal});
        if (has_sink_) s.push_back({name_of("sink"), {heads_}, Role::Vector, Init::Normal});
        return s;
    }

    void bind(WeightSource& src) override {
        // one matrix [q | k | (v) | (g)] so that the projections of h are one product (a layout choice only)
        std::vector<Tensor> parts = {src.fetch(name_of("q_proj")), src.fetch(name_of("k_proj"))};
        if (!values_are_keys_) parts.push_back(src.fetch(name_of("v_proj")));
        if (has_gate_) parts.push_back(src.fetch(name_of("gate_proj")));
        for (Tensor& t : parts)
            if (t.dtype != parts[0].dtype) throw WeightError("the projections of " + name_of("q_proj") + "'s mixer are stored in different precisions");
        Tensor all = src.arena().alloc(parts[0].dtype, {q_width_ + kv_width_ + v_width_ + g_width_, hidden_});
        size_t off = 0;
        for (Tensor& t : parts) {
            QE_CUDA(cudaMemcpyAsync(static_cast<char*>(all.data) + off, t.data, t.bytes(), cudaMemcpyDeviceToDevice, src.stream()));
            off += t.bytes();
        }
        QE_CUDA(cudaStreamSynchronize(src.stream()));
        for (Tensor& t : parts) src.release(t);
        in_proj_ = Linear(all, "qkvg_proj", gemm_);
        o_proj_ = Linear(src.fetch(name_of("o_proj")), "o_proj", gemm_);
        if (has_norm_) {
            q_norm_ = src.fetch(name_of("q_norm"));
            k_norm_ = src.fetch(name_of("k_norm"));
        }
        if (has_distance_) {
            slope_ = src.fetch(name_of("distance_slope"));
            rate_ = src.fetch(name_of("distance_rate"));
        }
        if (has_mix_) mix_ = src.fetch(name_of("head_mix"));
        if (has_sink_) sink_ = src.fetch(name_of("sink"));
    }

    std::vector<std::string> required_libraries() const override {
        return (in_proj_.fast() || o_proj_.fast()) ? std::vector<std::string>{"core", "gemm100"} : std::vector<std::string>{"core"};
    }
    int preferred_row_multiple() const override { return (in_proj_.fast() || o_proj_.fast()) ? 256 : 0; }
    CacheNeed cache_need() const override { return CacheNeed::pages(kv_heads_, head_dim_, window_, value_dim_); }

    // bfloat16 with sizes the tensor-core kernel takes: a tile of 16 rows and all heads per CTA; else the plain kernel
    bool use_mma() const {
        return compute_dtype == DType::BF16 && attention_ != "generic" &&
               core_kernels().attention_talking_mma_supports(heads_, kv_heads_, head_dim_, value_dim_);
    }
    void prepare_step(StepPlan& plan) override {
        if (use_mma()) add_tiles(plan, kTileAll, "attention.tiles16", true);
    }

    Addend forward(const Tensor& x, StepContext& ctx, const CacheView& cache) override {
        if (!cache.writable) throw Error(kInvalidState, "talking_attention writes a cache of its own");
        const int T = ctx.T;
        Workspace& ws = *ctx.workspace;
        const DType dt = compute_dtype;
        const GroupStep& g = ctx.groups.at(cache.group);
        const CoreKernels& core = core_kernels();
        const int64_t width = q_width_ + kv_width_ + v_width_ + g_width_;
        Addend in = in_proj_(x, ctx, "talk_in", dt, T, !has_gate_);
        Tensor q = ws.get("talk_q", {T, heads_, head_dim_}, dt);
        const size_t in_size = dtype_size(in.tensor.dtype);
        if (LaunchProfile::get().on())
            LaunchProfile::get().note_cost((double)T * ((q_width_ + kv_width_ + v_width_) * (double)in.splits * in_size +
                                                        (q_width_ + kv_width_ + (double)kv_heads_ * value_dim_) * dtype_size(dt)), 0.0);
        QE_LAUNCH(core, core.joint_norm_kv_write(in.tensor.data, in.tensor.code(), in.splits, (long long)T * width, width,
                                                 has_norm_ ? q_norm_.as<float>() : nullptr, has_norm_ ? k_norm_.as<float>() : nullptr, (float)eps_,
                                                 g.slot_mapping, q.data, q.code(), cache.k_base, cache.v_base, (int)cache.kv_dtype, cache.page_stride,
                                                 cache.page_size, T, heads_, kv_heads_, head_dim_, value_dim_, values_are_keys_ ? 0 : 1, ctx.stream));
        // the gate's logits stay where the product left them (a product that feeds a gate keeps K whole)
        const void* gate = nullptr;
        if (has_gate_) {
            if (in.splits != 1) throw Error(kInvalidState, "talking_attention: the gate's logits came as partial sums");
            gate = static_cast<const char*>(in.tensor.data) + (q_width_ + kv_width_ + v_width_) * in_size;
        }
        const int gate_code = in.tensor.code();
        const long long gate_stride = width;
        Tensor out = ws.get("talk_out", {T, o_width_}, dt);
        if (LaunchProfile::get().on()) {
            double seen = 0.0, read = 0.0;
            for (size_t i = 0; i < ctx.q_lens.size(); i++) {
                const double n = ctx.q_lens[i], len = ctx.ctx_lens[i];
                read += window_ ? std::min<double>(len, window_ + n) : len;
                seen += window_ ? n * std::min<double>(len, window_) : n * (len - n) + n * (n + 1) / 2.0;
            }
            LaunchProfile::get().note_cost(read * kv_heads_ * (head_dim_ + value_dim_) * dtype_size(cache.kv_dtype) +
                                               (double)T * (q_width_ + o_width_ + g_width_) * dtype_size(dt),
                                           2.0 * seen * heads_ * (head_dim_ + value_dim_ + (has_mix_ ? heads_ : 0)));
        }
        const StepArray t16 = ctx.array("attention.tiles16.seg"), t16f = ctx.array("attention.tiles16.first");
        if (use_mma() && cache.kv_dtype == DType::BF16 && t16.count && (!gate || in.tensor.dtype == DType::BF16)) {
            int splits = (int)ctx.option_int("tile16_splits");
            if (splits < 1)
                splits = tile16_splits(t16.count, std::max(ctx.decode_max_ctx, ctx.prefill_max_ctx), window_,
                                       sm_count() * core.attention_talking_mma_ctas_per_sm(heads_, kv_heads_, head_dim_, value_dim_) /
                                           (heads_ > 16 ? 2 : 1));      // above 16 heads a tile takes a pair of CTAs
            float *part_o = nullptr, *part_ml = nullptr;
            if (splits > 1) {
                part_o = ws.get("attn16_part_o", {T, heads_, splits, value_dim_}, DType::F32).as<float>();
                part_ml = ws.get("attn16_part_ml", {T, heads_, splits, 2}, DType::F32).as<float>();
            }
            QE_LAUNCH(core, core.attention_talking_mma(q.data, cache.k_base, cache.v_base, cache.page_stride, cache.page_size, g.block_table,
                                                       g.table_width, ctx.seg_start, ctx.seg_ctx_len, t16.data, t16f.data, t16.count, out.data,
                                                       heads_, kv_heads_, head_dim_, value_dim_, window_, 0, (float)scale_, (float)softcap_,
                                                       has_distance_ ? slope_.as<float>() : nullptr, has_distance_ ? rate_.as<float>() : nullptr,
                                                       has_mix_ ? mix_.as<float>() : nullptr, has_sink_ ? sink_.as<float>() : nullptr, gate,
                                                       gate_stride, splits, T, part_o, part_ml, ctx.stream));
        } else {
            QE_LAUNCH(core, core.attention_talking(q.data, q.code(), cache.k_base, cache.v_base, (int)cache.kv_dtype, cache.page_stride, cache.page_size,
                                                   g.block_table, g.table_width, ctx.row_seg, ctx.position_column(0), out.data, out.code(), T, heads_,
                                                   kv_heads_, head_dim_, value_dim_, window_, 0, (float)scale_, (float)softcap_,
                                                   has_distance_ ? slope_.as<float>() : nullptr, has_distance_ ? rate_.as<float>() : nullptr,
                                                   has_mix_ ? mix_.as<float>() : nullptr, has_sink_ ? sink_.as<float>() : nullptr, gate, gate_code,
                                                   gate_stride, ctx.stream));
        }
        return o_proj_(out, ctx, "talk_o", DType::F32, T, true, false, ctx.residual, nullptr, &ctx.norm_ahead);
    }

private:
    int64_t hidden_, q_width_, kv_width_, v_width_, o_width_, g_width_;
    int heads_, kv_heads_, head_dim_, value_dim_, window_;
    bool values_are_keys_, has_norm_, has_distance_, has_mix_, has_sink_, has_gate_;
    double eps_, scale_, softcap_;
    std::string gemm_, attention_;
    Linear in_proj_, o_proj_;
    Tensor q_norm_, k_norm_, slope_, rate_, mix_, sink_;
};

void register_mixer_parts() {
    register_part("mixer", "attention", [](const Json& p, BuildContext& b) { return std::make_shared<Attention>(p, b); });
    register_part("mixer", "talking_attention", [](const Json& p, BuildContext& b) { return std::make_shared<TalkingAttention>(p, b); });
}

}  // namespace qe
