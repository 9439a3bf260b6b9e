// Attention whose keys and values are made from one small latent per token, computed without ever making them.
//
// A token leaves [c | r] in the cache: c its normed latent (C wide), r one rotated key part (R wide) that all heads share.
// Head h's key is [Wuk_h c | r] and its value Wuv_h c.  Since q_plain . (Wuk_h c) = (Wuk_h^T q_plain) . c and
// sum_j p_j Wuv_h c_j = Wuv_h (sum_j p_j c_j), every head attends over the same rows [c | r] with the query
// [Wuk_h^T q_plain | q_rot] and takes sum_j p_j c_j, which Wuv_h expands afterwards: attention with one key/value head,
// keys C + R wide, values the first C of a key row.
//
//   latent_prepare   per token from the stacked down product [q latent | kv latent | r | ...]: the RMS norm of the query
//                    latent (for the up product), the RMS norm of the kv latent and the rotation of r into the token's
//                    cache row.
//   latent_absorb    q_lat[t, h] = [Wuk_h^T q_plain[t, h] | rotate(q_rot[t, h])]
//   latent_expand    out[t, h] = (Wuv_h o_lat[t, h]) * sigmoid(gate[t, h])
// The attention itself is attention_generic (values read out of the key rows) or the tensor-core kernels of
// latent_attention_mma.cu.  Sums here are float32 with the contraction index ascending, whatever else is in the batch.
#include "common.cuh"

#include <math.h>

namespace {

using namespace ph;

// (u, v) turned by the angle whose cosine and sine are c and s
__device__ __forceinline__ float turn_u(float u, float v, float c, float s) { return u * c - v * s; }
__device__ __forceinline__ float turn_v(float u, float v, float c, float s) { return v * c + u * s; }

constexpr int PREP_THREADS = 128;      // a block per token: its threads walk the latents 128 apart

template <typename TD, typename TQ, typename TKV>
__global__ void latent_prepare_kernel(const TD* __restrict__ down, long long down_stride, int Q, int C, int R,
                                      const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                                      const float* __restrict__ cos_sin, int n_rot, int max_pos, const int32_t* __restrict__ positions,
                                      const int32_t* __restrict__ slot_mapping, TQ* __restrict__ cq, TKV* __restrict__ k_base,
                                      long long page_stride, int page_size, int T) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x;
    const int t = blockIdx.x;
    const TD* row = down + (size_t)t * down_stride;
    // the query latent
    float ss = 0.0f;
    for (int i = lane; i < Q; i += PREP_THREADS) { const float v = to_float<TD>(row[i]); ss += v * v; }
    float inv = rsqrtf(block_sum<PREP_THREADS>(ss, scratch) / (float)Q + eps);
    for (int i = lane; i < Q; i += PREP_THREADS) cq[(size_t)t * Q + i] = from_float<TQ>(to_float<TD>(row[i]) * inv * wq[i]);
    if (!slot_mapping) return;
    // the kv latent and the shared rotated key part, into the token's cache row
    const int slot = slot_mapping[t];
    TKV* dst = k_base + (size_t)(slot / page_size) * page_stride + (size_t)(slot % page_size) * (C + R);
    ss = 0.0f;
    for (int i = lane; i < C; i += PREP_THREADS) { const float v = to_float<TD>(row[Q + i]); ss += v * v; }
    inv = rsqrtf(block_sum<PREP_THREADS>(ss, scratch) / (float)C + eps);
    for (int i = lane; i < C; i += PREP_THREADS) dst[i] = from_float<TKV>(to_float<TD>(row[Q + i]) * inv * wkv[i]);
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);     // positions are validated on the host
    const float* cs = cos_sin + (size_t)pos * n_rot;
    const int half = n_rot / 2;
    const TD* r = row + Q + C;
    for (int i = lane; i < R; i += PREP_THREADS) {
        float v = to_float<TD>(r[i]);
        if (i < half) v = turn_u(v, to_float<TD>(r[i + half]), cs[i], cs[half + i]);
        else if (i < n_rot) v = turn_v(to_float<TD>(r[i - half]), v, cs[i - half], cs[i]);
        dst[C + i] = from_float<TKV>(v);
    }
}

constexpr int AB_TOK = 8, AB_THREADS = 128;

// q [T, H, D + R] -> q_lat [T, H, C + R]; grid (column tiles of C, H, token tiles).  Thread c of a tile sums over d
// ascending for AB_TOK tokens at once; the first column tile also rotates the R last dimensions.
template <typename TQ, typename TW, typename TO>
__global__ void latent_absorb_kernel(const TQ* __restrict__ q, const TW* __restrict__ wuk, const float* __restrict__ cos_sin, int n_rot,
                                     int max_pos, const int32_t* __restrict__ positions, TO* __restrict__ q_lat, int T, int H, int D,
                                     int R, int C) {
    extern __shared__ float qs[];      // [AB_TOK][D + R]
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y, t0 = blockIdx.z * AB_TOK, DR = D + R;
    for (int i = threadIdx.x; i < AB_TOK * DR; i += blockDim.x) {
        const int tt = i / DR, d = i % DR;
        qs[i] = t0 + tt < T ? to_float<TQ>(q[((size_t)(t0 + tt) * H + h) * DR + d]) : 0.0f;
    }
    __syncthreads();
    const int c = blockIdx.x * AB_THREADS + threadIdx.x;
    if (c < C) {
        float acc[AB_TOK];
#pragma unroll
        for (int i = 0; i < AB_TOK; ++i) acc[i] = 0.0f;
        const TW* w = wuk + (size_t)h * D * C + c;
        for (int d = 0; d < D; ++d) {
            const float wv = to_float<TW>(w[(size_t)d * C]);
#pragma unroll
            for (int i = 0; i < AB_TOK; ++i) acc[i] = fmaf(qs[i * DR + d], wv, acc[i]);
        }
#pragma unroll
        for (int i = 0; i < AB_TOK; ++i)
            if (t0 + i < T) q_lat[((size_t)(t0 + i) * H + h) * (C + R) + c] = from_float<TO>(acc[i]);
    }
    if (blockIdx.x != 0) return;
    const int half = n_rot / 2;
    for (int i = threadIdx.x; i < AB_TOK * R; i += blockDim.x) {
        const int tt = i / R, d = i % R;
        if (t0 + tt >= T) continue;
        int pos = positions[t0 + tt];
        pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
        const float* cs = cos_sin + (size_t)pos * n_rot;
        const float* r = qs + tt * DR + D;
        float v = r[d];
        if (d < half) v = turn_u(v, r[d + half], cs[d], cs[half + d]);
        else if (d < n_rot) v = turn_v(r[d - half], v, cs[d - half], cs[d]);
        q_lat[((size_t)(t0 + tt) * H + h) * (C + R) + C + d] = from_float<TO>(v);
    }
}

constexpr int EX_TOK = 8, EX_WARPS = 8;

// o_lat [T, H, C] -> out [T, H * DV]; grid (value tiles of EX_WARPS, H, token tiles).  A warp owns one value column: its
// lanes walk c, 32 apart, for EX_TOK tokens at once, and add up with a butterfly.
template <typename TI, typename TW, typename TG, typename TO>
__global__ void latent_expand_kernel(const TI* __restrict__ o_lat, const TW* __restrict__ wuv, const TG* __restrict__ gate,
                                     long long gate_stride, TO* __restrict__ out, int T, int H, int C, int DV) {
    extern __shared__ float os[];      // [EX_TOK][C]
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.y, t0 = blockIdx.z * EX_TOK;
    for (int i = threadIdx.x; i < EX_TOK * C; i += blockDim.x) {
        const int tt = i / C, c = i % C;
        os[i] = t0 + tt < T ? to_float<TI>(o_lat[((size_t)(t0 + tt) * H + h) * C + c]) : 0.0f;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int v = blockIdx.x * EX_WARPS + warp;
    if (v >= DV) return;
    const TW* w = wuv + ((size_t)h * DV + v) * C;
    float acc[EX_TOK];
#pragma unroll
    for (int i = 0; i < EX_TOK; ++i) acc[i] = 0.0f;
    for (int c = lane; c < C; c += 32) {
        const float wv = to_float<TW>(w[c]);
#pragma unroll
        for (int i = 0; i < EX_TOK; ++i) acc[i] = fmaf(os[i * C + c], wv, acc[i]);
    }
#pragma unroll
    for (int i = 0; i < EX_TOK; ++i) {
        const float total = warp_sum(acc[i]);
        if (lane == 0 && t0 + i < T) {
            const float g = gate ? 1.0f / (1.0f + expf(-to_float<TG>(gate[(size_t)(t0 + i) * gate_stride + h]))) : 1.0f;
            out[((size_t)(t0 + i) * H + h) * DV + v] = from_float<TO>(total * g);
        }
    }
}

}  // namespace

// down [T, down_stride]: columns [0, Q) the query latent, [Q, Q + C) the kv latent, [Q + C, Q + C + R) the shared key part.
// cq [T, Q] <- RMS(query latent) * wq.  With slot_mapping: the token's cache row (one key head, C + R wide, no value rows)
// <- [RMS(kv latent) * wkv | r rotated over its first n_rot dimensions in half pairs].  cos_sin [max_pos, n_rot].
PH_EXPORT int ph_latent_prepare(const void* down, int down_dtype, long long down_stride, int Q, int C, int R, const float* wq,
                                const float* wkv, float eps, const float* cos_sin, int n_rot, int max_pos, const int32_t* positions,
                                const int32_t* slot_mapping, void* cq, int cq_dtype, void* k_base, int kv_dtype, long long page_stride,
                                int page_size, int T, cudaStream_t stream) {
    if (!down || !wq || !cq || Q < 1 || C < 1 || R < 0 || T < 0 || n_rot < 0 || n_rot > R || n_rot % 2 || (n_rot && (!cos_sin || !positions)) ||
        (slot_mapping && (!k_base || !wkv || page_size < 1)) || !valid_dtype(down_dtype) || !valid_dtype(cq_dtype) || !valid_dtype(kv_dtype))
        return fail(PH_ERR_ARG, "latent_prepare: bad arguments (T %d, latents %d and %d, rotated %d of %d)", T, Q, C, n_rot, R);
    if (T == 0) return PH_OK;
    const unsigned blocks = (unsigned)T;
#define LAUNCH(TD, TQ, TKV)                                                                                                       \
    launch_overlapped(latent_prepare_kernel<TD, TQ, TKV>, dim3(blocks), dim3(PREP_THREADS), 0, stream, (const TD*)down, down_stride, Q, \
                      C, R, wq, wkv, eps, cos_sin, n_rot, max_pos, positions, slot_mapping, (TQ*)cq, (TKV*)k_base, page_stride, page_size, T)
    PH_DISPATCH(down_dtype, TD, PH_DISPATCH(cq_dtype, TQ, PH_DISPATCH(kv_dtype, TKV, LAUNCH(TD, TQ, TKV))));
#undef LAUNCH
    return check_launch("latent_prepare");
}

// q [T, H, D + R], wuk [H * D, C] -> q_lat [T, H, C + R].
PH_EXPORT int ph_latent_absorb(const void* q, int q_dtype, const void* wuk, int w_dtype, const float* cos_sin, int n_rot, int max_pos,
                               const int32_t* positions, void* q_lat, int out_dtype, int T, int H, int D, int R, int C,
                               cudaStream_t stream) {
    if (!q || !wuk || !q_lat || T < 0 || H < 1 || D < 1 || R < 0 || C < 1 || n_rot < 0 || n_rot > R || n_rot % 2 ||
        (n_rot && (!cos_sin || !positions)) || !valid_dtype(q_dtype) || !valid_dtype(w_dtype) || !valid_dtype(out_dtype))
        return fail(PH_ERR_ARG, "latent_absorb: bad arguments (T %d, H %d, D %d + %d, C %d)", T, H, D, R, C);
    if (T == 0) return PH_OK;
    const size_t smem = (size_t)AB_TOK * (D + R) * sizeof(float);
    if (smem > 48 * 1024) return fail(PH_ERR_UNSUPPORTED, "latent_absorb: a head of %d + %d dimensions does not fit", D, R);
    const dim3 grid((unsigned)((C + AB_THREADS - 1) / AB_THREADS), (unsigned)H, (unsigned)((T + AB_TOK - 1) / AB_TOK));
#define LAUNCH(TQ, TW, TO)                                                                                                       \
    launch_overlapped(latent_absorb_kernel<TQ, TW, TO>, grid, dim3(AB_THREADS), smem, stream, (const TQ*)q, (const TW*)wuk, cos_sin, n_rot, \
                      max_pos, positions, (TO*)q_lat, T, H, D, R, C)
    PH_DISPATCH(q_dtype, TQ, PH_DISPATCH(w_dtype, TW, PH_DISPATCH(out_dtype, TO, LAUNCH(TQ, TW, TO))));
#undef LAUNCH
    return check_launch("latent_absorb");
}

// o_lat [T, H, C], wuv [H * DV, C], gate [T, gate_stride] (logit of head h at column h; null: no gate) -> out [T, H * DV].
PH_EXPORT int ph_latent_expand(const void* o_lat, int in_dtype, const void* wuv, int w_dtype, const void* gate, int gate_dtype,
                               long long gate_stride, void* out, int out_dtype, int T, int H, int C, int DV, cudaStream_t stream) {
    if (!o_lat || !wuv || !out || T < 0 || H < 1 || C < 1 || DV < 1 || !valid_dtype(in_dtype) || !valid_dtype(w_dtype) ||
        !valid_dtype(gate_dtype) || !valid_dtype(out_dtype))
        return fail(PH_ERR_ARG, "latent_expand: bad arguments (T %d, H %d, C %d, DV %d)", T, H, C, DV);
    if (T == 0) return PH_OK;
    const size_t smem = (size_t)EX_TOK * C * sizeof(float);
    if (smem > 48 * 1024) return fail(PH_ERR_UNSUPPORTED, "latent_expand: a latent of %d does not fit", C);
    const dim3 grid((unsigned)((DV + EX_WARPS - 1) / EX_WARPS), (unsigned)H, (unsigned)((T + EX_TOK - 1) / EX_TOK));
#define LAUNCH(TI, TW, TG, TO)                                                                                                   \
    launch_overlapped(latent_expand_kernel<TI, TW, TG, TO>, grid, dim3(EX_WARPS * 32), smem, stream, (const TI*)o_lat, (const TW*)wuv, \
                      (const TG*)gate, gate_stride, (TO*)out, T, H, C, DV)
    PH_DISPATCH(in_dtype, TI, PH_DISPATCH(w_dtype, TW, PH_DISPATCH(gate_dtype, TG, PH_DISPATCH(out_dtype, TO, LAUNCH(TI, TW, TG, TO)))));
#undef LAUNCH
    return check_launch("latent_expand");
}
