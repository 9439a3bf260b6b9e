// Attention whose heads talk to each other before the softmax, over cache pages, and the kernel that prepares its
// queries, keys and values.
//
//   joint_norm_kv_write   from the rows [q | k | ...] of one product (partial sums added up): q and k are RMS-normed over
//                         their whole width (all heads as one row, one weight per element; a null weight: no norm), q
//                         goes out in the compute dtype, the normed k goes to the key rows of the token's cache slot, and
//                         the value rows receive k as it was projected, before the norm (values that are the keys), or
//                         the v part of the row when the product has one.
//   attention_talking     for the row at position z and every key p that it sees (first_seen(z) <= p <= z):
//                             s_g = (q_g . k_kv(g)) * scale
//                             s_g = cap * tanh(s_g / cap)                          (cap > 0)
//                             s_g = s_g - r1_g * ln(1 + r2_g * (z - p))            (r1, r2 given)
//                             s'_h = sum_g talk[h][g] * s_g                        (talk given: [HQ, HQ])
//                         then a softmax over the seen keys per head h (with exp(sink_h) in the denominator when a sink
//                         is given), o_h = sum_p w_hp v_kv(h)p, and o_h * sigmoid(gate_h) when a gate row is given.
//                         Because every head's score enters every head's softmax, one block handles all heads of a row:
//                         warp g scores head g for 32 keys at a time (a key per lane), the block exchanges the scores
//                         through shared memory, and warp h mixes, runs the online softmax and sums the values of head h
//                         (above 32 heads a warp takes two or four heads in turn).
// All arithmetic is float32 in an order that depends on (z, window) only, never on how a request was cut into steps or
// on what else is in the batch.  Cache addressing as in qk_norm_rope.cu.
#include "common.cuh"

#include <math.h>

namespace {

using namespace ph;

constexpr int MAX_DV = 512;      // widest value row
constexpr int MAX_HEADS = 64;    // a block per row: a warp per head up to 32 heads, two or four heads per warp above

// HPW: heads per warp.  A block has ceil(HQ / HPW) warps; warp w takes the heads w, w + warps, ... (at most HPW of them).
template <typename TQ, typename TKV, typename TG, typename TO, int HPW>
__global__ void attention_talking_kernel(const TQ* __restrict__ q, const TKV* __restrict__ k_base, const TKV* __restrict__ v_base,
                                         long long page_stride, int page_size, const int32_t* __restrict__ block_table, int table_stride,
                                         const int32_t* __restrict__ row_seg, const int32_t* __restrict__ positions,
                                         TO* __restrict__ out, int HQ, int HKV, int D, int DV, int window, int chunk, float scale,
                                         float cap, const float* __restrict__ r1, const float* __restrict__ r2,
                                         const float* __restrict__ talk, const float* __restrict__ sink, const TG* __restrict__ gate,
                                         long long gate_stride) {
    extern __shared__ float smem[];
    float* qs = smem;                          // [HQ][D]
    float* sc = qs + (size_t)HQ * D;           // [HQ][32]: the heads' own scores of the current 32 keys
    float* tk = sc + (size_t)HQ * 32;          // [HQ][HQ]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int t = blockIdx.x;
    const int group = HQ / HKV;
    const int z = positions[t];
    const int lo = first_seen(z, window, chunk);
    const int32_t* table = block_table + (size_t)row_seg[t] * table_stride;
    const TQ* qr = q + (size_t)t * HQ * D;
    for (int i = threadIdx.x; i < HQ * D; i += blockDim.x) qs[i] = to_float<TQ>(qr[i]);
    if (talk)
        for (int i = threadIdx.x; i < HQ * HQ; i += blockDim.x) tk[i] = talk[i];
    __syncthreads();

    float m[HPW], l[HPW];
    float acc[HPW][MAX_DV / 32];
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
        m[u] = -INFINITY; l[u] = 0.0f;
#pragma unroll
        for (int i = 0; i < MAX_DV / 32; ++i) acc[u][i] = 0.0f;
    }

    for (int base = lo; base <= z; base += 32) {
        const int p = base + lane;
        const bool seen = p <= z;
        int page = 0, off = 0;
        if (seen) { page = table[p / page_size]; off = p % page_size; }
        float s[HPW];
#pragma unroll
        for (int u = 0; u < HPW; ++u) {
            const int h = warp + u * warps;
            s[u] = 0.0f;
            if (h < HQ && seen) {
                const TKV* krow = k_base + (size_t)page * page_stride + ((size_t)(h / group) * page_size + off) * D;
                const float* qh = qs + (size_t)h * D;
                float dot = 0.0f;
                for (int d = 0; d < D; ++d) dot += qh[d] * to_float<TKV>(krow[d]);
                float v = dot * scale;
                if (cap > 0.0f) v = cap * tanhf(v / cap);
                if (r1) v -= r1[h] * log1pf(r2[h] * (float)(z - p));
                s[u] = v;
            }
        }
        if (talk) {
#pragma unroll
            for (int u = 0; u < HPW; ++u) {
                const int h = warp + u * warps;
                if (h < HQ) sc[h * 32 + lane] = s[u];
            }
            __syncthreads();
#pragma unroll
            for (int u = 0; u < HPW; ++u) {
                const int h = warp + u * warps;
                if (h >= HQ) continue;
                float mixed = 0.0f;
                for (int j = 0; j < HQ; ++j) mixed += tk[h * HQ + j] * sc[j * 32 + lane];
                s[u] = mixed;
            }
        }
        const int n = (z - base + 1) < 32 ? (z - base + 1) : 32;
#pragma unroll
        for (int u = 0; u < HPW; ++u) {
            const int h = warp + u * warps;
            if (h >= HQ) continue;                         // the whole warp: h depends on the warp alone
            const float sv = seen ? s[u] : -INFINITY;
            const float m_new = fmaxf(m[u], warp_max(sv));
            const float pexp = seen ? expf(sv - m_new) : 0.0f;
            const float corr = expf(m[u] - m_new);         // m = -inf on the first block: corr = 0, l and acc are 0
            l[u] = l[u] * corr + warp_sum(pexp);
#pragma unroll
            for (int i = 0; i < MAX_DV / 32; ++i) acc[u][i] *= corr;
            const TKV* vrow = seen ? v_base + (size_t)page * page_stride + ((size_t)(h / group) * page_size + off) * DV : nullptr;
            for (int j = 0; j < n; ++j) {
                const float pj = __shfl_sync(0xffffffffu, pexp, j);
                const unsigned long long vp = __shfl_sync(0xffffffffu, (unsigned long long)vrow, j);
                const TKV* vj = (const TKV*)vp;
#pragma unroll
                for (int i = 0; i < MAX_DV / 32; ++i) {
                    const int d = lane + 32 * i;
                    if (d < DV) acc[u][i] += pj * to_float<TKV>(vj[d]);
                }
            }
            m[u] = m_new;
        }
        if (talk) __syncthreads();                     // the scores are read before the next block overwrites them
    }
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
        const int h = warp + u * warps;
        if (h >= HQ) continue;
        if (sink) {
            const float sk = sink[h], top = fmaxf(m[u], sk), corr = expf(m[u] - top);
            l[u] = l[u] * corr + expf(sk - top);
#pragma unroll
            for (int i = 0; i < MAX_DV / 32; ++i) acc[u][i] *= corr;
        }
        TO* o = out + ((size_t)t * HQ + h) * DV;
        const TG* gr = gate ? gate + (size_t)t * gate_stride + (size_t)h * DV : nullptr;
        const float inv = 1.0f / l[u];
#pragma unroll
        for (int i = 0; i < MAX_DV / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < DV) {
                float v = acc[u][i] * inv;
                if (gr) v *= 1.0f / (1.0f + expf(-to_float<TG>(gr[d])));
                o[d] = from_float<TO>(v);
            }
        }
    }
}

// One block per token.  The row holds [q (QW) | k (KW) | v (VW, or nothing when the keys are the values) | ...].
template <typename TI, typename TQ, typename TKV>
__global__ void joint_norm_kv_write_kernel(const TI* __restrict__ rows, int splits, long long split_stride, long long row_width,
                                           const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                           const int32_t* __restrict__ slot_mapping, TQ* __restrict__ q_out, TKV* __restrict__ k_base,
                                           TKV* __restrict__ v_base, long long page_stride, int page_size, int HQ, int HKV, int D, int DV,
                                           int v_from_row) {
    extern __shared__ float buf[];             // [QW + KW]
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int QW = HQ * D, KW = HKV * D;
    const TI* src = rows + (size_t)t * row_width;
    float sq = 0.0f, sk = 0.0f;
    for (int i = threadIdx.x; i < QW + KW; i += blockDim.x) {
        float v = 0.0f;
        for (int s = 0; s < splits; ++s) v += to_float<TI>(src[(size_t)s * split_stride + i]);
        buf[i] = v;
        if (i < QW) sq += v * v; else sk += v * v;
    }
    const float iq = q_w ? rsqrtf(block_sum_any(sq, scratch) / (float)QW + eps) : 1.0f;
    const float ik = k_w ? rsqrtf(block_sum_any(sk, scratch) / (float)KW + eps) : 1.0f;
    __syncthreads();
    TQ* qo = q_out + (size_t)t * QW;
    for (int i = threadIdx.x; i < QW; i += blockDim.x) qo[i] = from_float<TQ>(q_w ? buf[i] * iq * q_w[i] : buf[i]);
    if (!slot_mapping) return;
    const int slot = slot_mapping[t];
    if (slot < 0) return;
    const size_t page_at = (size_t)(slot / page_size) * page_stride;
    const int off = slot % page_size;
    for (int i = threadIdx.x; i < KW; i += blockDim.x) {
        const int h = i / D, d = i % D;
        const float raw = buf[QW + i];
        k_base[page_at + ((size_t)h * page_size + off) * D + d] = from_float<TKV>(k_w ? raw * ik * k_w[i] : raw);
        if (!v_from_row) v_base[page_at + ((size_t)h * page_size + off) * DV + d] = from_float<TKV>(raw);
    }
    if (v_from_row) {
        for (int i = threadIdx.x; i < HKV * DV; i += blockDim.x) {
            const int h = i / DV, d = i % DV;
            float v = 0.0f;
            for (int s = 0; s < splits; ++s) v += to_float<TI>(src[(size_t)s * split_stride + QW + KW + i]);
            v_base[page_at + ((size_t)h * page_size + off) * DV + d] = from_float<TKV>(v);
        }
    }
}

// The same with eight consecutive elements per access (every width a multiple of 8, rows 16-byte aligned): a thread's
// elements never straddle a head.  The sums of squares are taken per thread over its own elements, then over the block:
// their order depends on the widths alone.
template <typename TI, typename TQ, typename TKV>
__global__ void joint_norm_kv_write_vec_kernel(const TI* __restrict__ rows, int splits, long long split_stride, long long row_width,
                                               const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                               const int32_t* __restrict__ slot_mapping, TQ* __restrict__ q_out, TKV* __restrict__ k_base,
                                               TKV* __restrict__ v_base, long long page_stride, int page_size, int HQ, int HKV, int D, int DV,
                                               int v_from_row) {
    extern __shared__ float buf[];             // [QW + KW]
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int QW = HQ * D, KW = HKV * D;
    const TI* src = rows + (size_t)t * row_width;
    float sq = 0.0f, sk = 0.0f;
    for (int i = threadIdx.x * 8; i < QW + KW; i += blockDim.x * 8) {
        float v[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        for (int s = 0; s < splits; ++s) {
            float u[8];
            load8(src + (size_t)s * split_stride + i, u);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] += u[j];
        }
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { buf[i + j] = v[j]; ss += v[j] * v[j]; }
        if (i < QW) sq += ss; else sk += ss;
    }
    const float iq = q_w ? rsqrtf(block_sum_any(sq, scratch) / (float)QW + eps) : 1.0f;
    const float ik = k_w ? rsqrtf(block_sum_any(sk, scratch) / (float)KW + eps) : 1.0f;
    __syncthreads();
    TQ* qo = q_out + (size_t)t * QW;
    for (int i = threadIdx.x * 8; i < QW; i += blockDim.x * 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = q_w ? buf[i + j] * iq * q_w[i + j] : buf[i + j];
        store8(qo + i, v);
    }
    if (!slot_mapping) return;
    const int slot = slot_mapping[t];
    if (slot < 0) return;
    const size_t page_at = (size_t)(slot / page_size) * page_stride;
    const int off = slot % page_size;
    for (int i = threadIdx.x * 8; i < KW; i += blockDim.x * 8) {
        const int h = i / D, d = i % D;
        float raw[8], v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { raw[j] = buf[QW + i + j]; v[j] = k_w ? raw[j] * ik * k_w[i + j] : raw[j]; }
        store8(k_base + page_at + ((size_t)h * page_size + off) * D + d, v);
        if (!v_from_row) store8(v_base + page_at + ((size_t)h * page_size + off) * DV + d, raw);
    }
    if (v_from_row) {
        for (int i = threadIdx.x * 8; i < HKV * DV; i += blockDim.x * 8) {
            const int h = i / DV, d = i % DV;
            float v[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            for (int s = 0; s < splits; ++s) {
                float u[8];
                load8(src + (size_t)s * split_stride + QW + KW + i, u);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += u[j];
            }
            store8(v_base + page_at + ((size_t)h * page_size + off) * DV + d, v);
        }
    }
}

}  // namespace

// gate: rows of HQ * DV logits, gate_stride elements apart, in gate_dtype (null: no gate).  cap 0: no cap.  r1, r2, talk,
// sink: float32 per head ([HQ], [HQ], [HQ, HQ], [HQ]) or null.
PH_EXPORT int ph_attention_talking(const void* q, int q_dtype, const void* k_base, const void* v_base, int kv_dtype, long long page_stride,
                                   int page_size, const int32_t* block_table, int table_stride, const int32_t* row_seg,
                                   const int32_t* positions, void* out, int out_dtype, int T, int HQ, int HKV, int D, int DV, int window,
                                   int chunk, float scale, float cap, const float* r1, const float* r2, const float* talk,
                                   const float* sink, const void* gate, int gate_dtype, long long gate_stride, cudaStream_t stream) {
    if (!q || !k_base || !v_base || !block_table || !row_seg || !positions || !out || T < 0 || HQ < 1 || HKV < 1 || D < 1 || DV < 1 ||
        page_size < 1 || window < 0 || chunk < 0 || !valid_dtype(q_dtype) || !valid_dtype(kv_dtype) || !valid_dtype(out_dtype) ||
        (gate && !valid_dtype(gate_dtype)) || (r1 == nullptr) != (r2 == nullptr) || cap < 0.0f)
        return fail(PH_ERR_ARG, "attention_talking: bad arguments (T %d, HQ %d, HKV %d, D %d, DV %d)", T, HQ, HKV, D, DV);
    if (HQ % HKV) return fail(PH_ERR_ARG, "attention_talking: %d query heads are not a multiple of %d kv heads", HQ, HKV);
    if (HQ > MAX_HEADS) return fail(PH_ERR_UNSUPPORTED, "attention_talking: %d heads exceed the supported %d", HQ, MAX_HEADS);
    if (DV > MAX_DV) return fail(PH_ERR_UNSUPPORTED, "attention_talking: value rows of %d exceed the supported %d", DV, MAX_DV);
    const size_t smem = ((size_t)HQ * D + (size_t)HQ * 32 + (size_t)HQ * HQ) * sizeof(float);
    if (smem > 200 * 1024) return fail(PH_ERR_UNSUPPORTED, "attention_talking: %d heads of %d do not fit shared memory", HQ, D);
    if (T == 0) return PH_OK;
    if (!gate) gate_dtype = q_dtype;
    // (two heads per warp take 94 registers a thread and four take 127: 20 and 16 warps are what an SM's registers hold)
    const int hpw = HQ <= 32 ? 1 : HQ <= 40 ? 2 : 4, warps = (HQ + hpw - 1) / hpw;
#define LAUNCH_N(TQ, TKV, TG, TO, N)                                                                                              \
    do {                                                                                                                          \
        auto kern = attention_talking_kernel<TQ, TKV, TG, TO, N>;                                                                 \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                 \
        kern<<<T, warps * 32, smem, stream>>>((const TQ*)q, (const TKV*)k_base, (const TKV*)v_base, page_stride, page_size, block_table, \
                                              table_stride, row_seg, positions, (TO*)out, HQ, HKV, D, DV, window, chunk, scale, cap, \
                                              r1, r2, talk, sink, (const TG*)gate, gate_stride);                                  \
    } while (0)
#define LAUNCH(TQ, TKV, TG, TO)                                                                                                   \
    do {                                                                                                                          \
        if (hpw == 1) LAUNCH_N(TQ, TKV, TG, TO, 1); else if (hpw == 2) LAUNCH_N(TQ, TKV, TG, TO, 2); else LAUNCH_N(TQ, TKV, TG, TO, 4); \
    } while (0)
    PH_DISPATCH(q_dtype, TQ, PH_DISPATCH(kv_dtype, TKV, PH_DISPATCH(gate_dtype, TG, PH_DISPATCH(out_dtype, TO, LAUNCH(TQ, TKV, TG, TO)))));
#undef LAUNCH
#undef LAUNCH_N
    return check_launch("attention_talking");
}

// rows: [splits][T][row_width] in rows_dtype.  q_w [HQ * D] and k_w [HKV * D] float32 or null.  slot_mapping null: no
// cache write (q only).  v_from_row 0: the values are the keys as projected; 1: the row's third part [HKV * DV].
PH_EXPORT int ph_joint_norm_kv_write(const void* rows, int rows_dtype, int splits, long long split_stride, long long row_width,
                                     const float* q_w, const float* k_w, float eps, const int32_t* slot_mapping, void* q_out, int q_dtype,
                                     void* k_base, void* v_base, int kv_dtype, long long page_stride, int page_size, int T, int HQ,
                                     int HKV, int D, int DV, int v_from_row, cudaStream_t stream) {
    if (!rows || !q_out || T < 0 || HQ < 1 || HKV < 1 || D < 1 || DV < 1 || splits < 1 || page_size < 1 || !valid_dtype(rows_dtype) ||
        !valid_dtype(q_dtype) || !valid_dtype(kv_dtype) || (slot_mapping && (!k_base || !v_base)))
        return fail(PH_ERR_ARG, "joint_norm_kv_write: bad arguments (T %d, HQ %d, HKV %d, D %d)", T, HQ, HKV, D);
    if (!v_from_row && DV != D) return fail(PH_ERR_ARG, "joint_norm_kv_write: values that are the keys are as wide as the keys (%d, not %d)", D, DV);
    const long long need = (long long)(HQ + HKV) * D + (v_from_row ? (long long)HKV * DV : 0);
    if (row_width < need) return fail(PH_ERR_ARG, "joint_norm_kv_write: rows of %lld elements hold no %lld", row_width, need);
    const size_t smem = (size_t)(HQ + HKV) * D * sizeof(float);
    if (smem > 200 * 1024) return fail(PH_ERR_UNSUPPORTED, "joint_norm_kv_write: rows of %d elements do not fit shared memory", (HQ + HKV) * D);
    if (T == 0) return PH_OK;
    const int threads = (HQ + HKV) * D >= 2048 ? 512 : 256;
    const bool vec = D % 8 == 0 && DV % 8 == 0 && row_width % 8 == 0 && split_stride % 8 == 0 && page_stride % 8 == 0 &&
                     (((uintptr_t)rows | (uintptr_t)q_out | (uintptr_t)k_base | (uintptr_t)v_base) % 32) == 0;
    if (vec) {
        const int vthreads = (HQ + HKV) * D / 8 >= 256 ? 256 : 128;
#define LAUNCH_VEC(TI, TQ, TKV)                                                                                                    \
    do {                                                                                                                           \
        auto kern = joint_norm_kv_write_vec_kernel<TI, TQ, TKV>;                                                                   \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
        kern<<<T, vthreads, smem, stream>>>((const TI*)rows, splits, split_stride, row_width, q_w, k_w, eps, slot_mapping, (TQ*)q_out, \
                                            (TKV*)k_base, (TKV*)v_base, page_stride, page_size, HQ, HKV, D, DV, v_from_row);       \
    } while (0)
        PH_DISPATCH(rows_dtype, TI, PH_DISPATCH(q_dtype, TQ, PH_DISPATCH(kv_dtype, TKV, LAUNCH_VEC(TI, TQ, TKV))));
#undef LAUNCH_VEC
        return check_launch("joint_norm_kv_write");
    }
#define LAUNCH(TI, TQ, TKV)                                                                                                        \
    do {                                                                                                                           \
        auto kern = joint_norm_kv_write_kernel<TI, TQ, TKV>;                                                                       \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
        kern<<<T, threads, smem, stream>>>((const TI*)rows, splits, split_stride, row_width, q_w, k_w, eps, slot_mapping, (TQ*)q_out, \
                                           (TKV*)k_base, (TKV*)v_base, page_stride, page_size, HQ, HKV, D, DV, v_from_row);        \
    } while (0)
    PH_DISPATCH(rows_dtype, TI, PH_DISPATCH(q_dtype, TQ, PH_DISPATCH(kv_dtype, TKV, LAUNCH(TI, TQ, TKV))));
#undef LAUNCH
    return check_launch("joint_norm_kv_write");
}
