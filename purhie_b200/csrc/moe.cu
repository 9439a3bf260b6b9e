// Routing of a mixture of experts and the products of the chosen experts, all on the device (no count ever goes
// to the host, so a step with routing can be captured as a graph).
//
//   route          per token: the router's logits w x + b in float32 (the router's matrix is float32 whatever the
//                  model's dtype), the `top` largest of them (the lower index wins a tie), and the softmax over the
//                  chosen logits alone (scoring 0).  Scoring 1: scores s = sigmoid(logit); the choice goes by s + correction
//                  (a vector per expert), the weights are the chosen experts' s as they are; with groups > 1 the experts
//                  form `groups` equal runs of neighbours, a run's rank is the sum of its two largest choice values, and
//                  only experts of the `keep` best runs (the lower index on a tie) can be chosen.
//   route_sort     the (token, choice) pairs sorted by expert: position of each pair, pair at each position, and a
//                  list of row tiles (expert, first position, rows) that never cross from one expert to the next.
//   gemm_grouped   y[i] = W[expert of i] x[source row of i] for the sorted positions i, tile by tile; float32
//                  multiply-add on the CUDA cores with k ascending inside one thread (the order of gemm_simple),
//                  so a row's result depends on neither its place in the batch nor its place among the expert's rows.
//   gemv_grouped   the same product for a handful of rows per expert (decoding): a warp per output feature streams
//                  that feature's weight row once, 16 bytes per lane and load, for up to eight rows of the tile at a
//                  time; a row's sum is taken in one order (lane by lane over k, then a butterfly), whatever else
//                  the tile holds.  This is weight streaming: its bound is the bytes of the chosen experts.
//   route_combine  out[t] = base[t] (optional: float32 partial sums of a part that runs for every token, times base_scale[t]
//                  where a factor per token is given) + the sum over the
//                  token's choices, in the order of the choices, of weight * y[position of (t, j)].
#include "common.cuh"

namespace {

using namespace ph;

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int MAX_TOP = 32;

// One block per token.  The warps share the experts: a warp's lanes walk k four elements at a time and add their parts
// with a butterfly, so a logit's sum is taken in one order whatever the batch.  Then the first warp picks: `top` times
// the largest logit not yet taken (the lower index on a tie), and the softmax over the picked ones.
constexpr int RT_WARPS = 16, MAX_EXPERTS = 1024;

// TOK tokens per block share every load of the router's rows (many tokens: the matrix is read TOK times less often).
template <typename TX, int TOK>
__global__ void __launch_bounds__(RT_WARPS * 32) route_kernel(const TX* __restrict__ x, const float* __restrict__ w,
                                                              const float* __restrict__ bias, int T, int E, int K, int top,
                                                              int32_t* __restrict__ choice, float* __restrict__ weight, int scoring,
                                                              const float* __restrict__ correction, int groups, int keep,
                                                              float weight_scale, const float* __restrict__ gate_w,
                                                              float* __restrict__ gate_out) {
    __shared__ float logit[TOK][MAX_EXPERTS / TOK];             // what the choice goes by
    __shared__ float score[TOK][MAX_EXPERTS / TOK];             // scoring 1: sigmoid(logit), what the weights are
    __shared__ float run_rank[TOK][MAX_EXPERTS / TOK];
    __shared__ unsigned char taken[TOK][MAX_EXPERTS / TOK];
    __shared__ float picked_value[TOK][MAX_TOP];
    __shared__ int picked_index[TOK][MAX_TOP];
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * TOK, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TX* xr[TOK];
#pragma unroll
    for (int i = 0; i < TOK; ++i) xr[i] = x + (size_t)(t0 + i < T ? t0 + i : t0) * K;
    // one more row when a gate per token is asked for: gate_out[t] = sigmoid(gate_w . x[t])
    for (int e = warp; e < E + (gate_w ? 1 : 0); e += RT_WARPS) {
        const float* wr = e < E ? w + (size_t)e * K : gate_w;
        float acc[TOK];
#pragma unroll
        for (int i = 0; i < TOK; ++i) acc[i] = 0.0f;
        if ((K & 3) == 0) {
            for (int k0 = lane * 4; k0 < K; k0 += 512) {          // four strides of 128 elements in flight
                float4 wv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    wv[u] = k0 + 128 * u < K ? *reinterpret_cast<const float4*>(wr + k0 + 128 * u) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int i = 0; i < TOK; ++i) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (k0 + 128 * u >= K) continue;
                        const float4 xv = load4(xr[i] + k0 + 128 * u);
                        acc[i] = fmaf(xv.x, wv[u].x, acc[i]);
                        acc[i] = fmaf(xv.y, wv[u].y, acc[i]);
                        acc[i] = fmaf(xv.z, wv[u].z, acc[i]);
                        acc[i] = fmaf(xv.w, wv[u].w, acc[i]);
                    }
                }
            }
        } else {
            for (int k = lane; k < K; k += 32)
#pragma unroll
                for (int i = 0; i < TOK; ++i) acc[i] = fmaf(to_float<TX>(xr[i][k]), wr[k], acc[i]);
        }
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
            const float total = warp_sum(acc[i]);
            if (lane == 0 && e == E) {
                if (t0 + i < T) gate_out[t0 + i] = 1.0f / (1.0f + expf(-total));
            } else if (lane == 0) {
                float z = total + (bias ? bias[e] : 0.0f);
                if (scoring == 1) {
                    z = 1.0f / (1.0f + expf(-z));
                    score[i][e] = z;
                    if (correction) z += correction[e];
                }
                logit[i][e] = z;
                taken[i][e] = 0;
            }
        }
    }
    __syncthreads();
    if (warp >= TOK || t0 + warp >= T) return;                 // one warp per token picks
    const int t = t0 + warp;
    if (scoring == 2) {
        // the softmax over all experts: what the choice goes by and what the weights are made of
        float largest = -INFINITY;
        for (int e = lane; e < E; e += 32) largest = fmaxf(largest, logit[warp][e]);
        largest = warp_max(largest);
        float sum = 0.0f;
        for (int e = lane; e < E; e += 32) { const float x = expf(logit[warp][e] - largest); logit[warp][e] = x; sum += x; }
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) logit[warp][e] = logit[warp][e] / sum;
        __syncwarp();
    }
    if (groups > 1 && keep < groups) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float first = -INFINITY, second = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = logit[warp][e];
                if (v > first) { second = first; first = v; }
                else if (v > second) second = v;
            }
            run_rank[warp][g] = (per > 1 && scoring != 2) ? first + second : first;      // scoring 2: a run counts as its best
        }
        __syncwarp();
        for (int g = lane; g < groups; g += 32) {
            const float mine = run_rank[warp][g];
            int ahead = 0;
            for (int o = 0; o < groups; ++o) {
                const float other = run_rank[warp][o];
                ahead += (other > mine || (other == mine && o < g)) ? 1 : 0;
            }
            if (ahead >= keep)
                for (int e = g * per; e < (g + 1) * per; ++e) taken[warp][e] = 1;
        }
        __syncwarp();
    }
    for (int j = 0; j < top; ++j) {
        int best = -1;
        float best_v = 0.0f;
        for (int e = lane; e < E; e += 32) {
            if (taken[warp][e]) continue;
            const float v = logit[warp][e];
            if (best < 0 || v > best_v) { best = e; best_v = v; }      // ascending e: the lower index keeps a tie
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const int other = __shfl_xor_sync(0xffffffffu, best, o);
            const float other_v = __shfl_xor_sync(0xffffffffu, best_v, o);
            if (other >= 0 && (best < 0 || other_v > best_v || (other_v == best_v && other < best))) { best = other; best_v = other_v; }
        }
        if (lane == 0) {
            taken[warp][best] = 1;
            picked_value[warp][j] = best_v;
            picked_index[warp][j] = best;
            choice[(size_t)t * top + j] = best;
        }
        __syncwarp();
    }
    if (scoring == 1) {
        if (lane < top) weight[(size_t)t * top + lane] = score[warp][picked_index[warp][lane]];
        return;
    }
    if (scoring == 2) {
        // the chosen scores over their sum (added in the order of the choices), times the scale
        float sum = 0.0f;
        for (int j = 0; j < top; ++j) sum += picked_value[warp][j];
        for (int j = lane; j < top; j += 32) weight[(size_t)t * top + j] = picked_value[warp][j] / (sum + 1e-20f) * weight_scale;
        return;
    }
    const float largest = picked_value[warp][0];
    const float mine = lane < top ? expf(picked_value[warp][lane] - largest) : 0.0f;
    const float sum = warp_sum(mine);
    if (lane < top) weight[(size_t)t * top + lane] = mine / sum;
}

// One block.  counts -> offsets -> a position for every pair; tiles[3 * i] = (expert, first position, rows), rows 0
// for the tiles that are left over.
__global__ void route_sort_kernel(const int32_t* __restrict__ choice, int R, int E, int32_t* __restrict__ position,
                                  int32_t* __restrict__ pair_at, int32_t* __restrict__ tiles, int max_tiles,
                                  int32_t* __restrict__ cursor /* [3 * E + 1] scratch */) {
    pdl_launch_dependents();
    pdl_wait();
    int32_t* count = cursor;            // [E]
    int32_t* offset = cursor + E;       // [E + 1]
    int32_t* fill = cursor + 2 * E + 1; // [E]
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = fill[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < R; i += blockDim.x) atomicAdd(&count[choice[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tile = 0;
        for (int e = 0; e < E; ++e) {
            offset[e] = at;
            for (int r0 = 0; r0 < count[e] && tile < max_tiles; r0 += BM, ++tile) {
                tiles[3 * tile] = e;
                tiles[3 * tile + 1] = at + r0;
                tiles[3 * tile + 2] = min(BM, count[e] - r0);
            }
            at += count[e];
        }
        offset[E] = at;
        for (; tile < max_tiles; ++tile) { tiles[3 * tile] = 0; tiles[3 * tile + 1] = 0; tiles[3 * tile + 2] = 0; }
    }
    __syncthreads();
    // which of an expert's places a pair gets is left to chance: a row's result does not depend on its place
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const int e = choice[i];
        const int at = offset[e] + atomicAdd(&fill[e], 1);
        position[i] = at;
        pair_at[at] = i;
    }
}

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256) gemm_grouped_kernel(const TX* __restrict__ x, const int32_t* __restrict__ pair_at,
                                                           int pairs_per_row, const TW* __restrict__ w,
                                                           const int32_t* __restrict__ tiles, TY* __restrict__ y, int N, int K) {
    __shared__ float xs[BK][BM + 1];
    __shared__ float ws[BK][BN + 1];
    __shared__ int src_row[BM];
    pdl_launch_dependents();
    pdl_wait();
    const int expert = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    if (rows == 0) return;
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * BN;
    const TW* we = w + (size_t)expert * N * K;
    // the source row of x for each row of the tile: the pair's token (pairs_per_row pairs per token), or the position itself
    if (tid < BM) src_row[tid] = tid < rows ? (pair_at ? pair_at[row0 + tid] / pairs_per_row : row0 + tid) : -1;
    __syncthreads();
    const int tr = tid / (BN / TN), tc = tid % (BN / TN);
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx / BK, kk = idx % BK;
            const int k = k0 + kk;
            float xv = 0.0f, wv = 0.0f;
            if (k < K) {
                if (src_row[r] >= 0) xv = to_float<TX>(x[(size_t)src_row[r] * K + k]);
                if (n0 + r < N) wv = to_float<TW>(we[(size_t)(n0 + r) * K + k]);
            }
            xs[kk][r] = xv;
            ws[kk][r] = wv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[kk][tr * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[kk][tc * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = tr * TM + i;
        if (m >= rows) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tc * TN + j;
            if (n < N) y[(size_t)(row0 + m) * N + n] = from_float<TY>(acc[i][j]);
        }
    }
}

constexpr int GV_ROWS = 8, GV_WARPS = 8, GV_FEATURES = 4;

// grid (ceil(N / (GV_WARPS * GV_FEATURES)), tiles); K % 8 == 0 and 16-byte aligned rows (checked by the launcher).  A warp
// streams GV_FEATURES weight rows side by side (as many 16-byte loads in flight per lane, and every load of x used that
// many times); the sum of one (row, feature) is taken lane by lane over k ascending, then by a butterfly.
template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(GV_WARPS * 32) gemv_grouped_kernel(const TX* __restrict__ x, const int32_t* __restrict__ pair_at,
                                                                     int pairs_per_row, const TW* __restrict__ w,
                                                                     const int32_t* __restrict__ tiles, TY* __restrict__ y, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int expert = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    if (rows == 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * GV_WARPS + warp) * GV_FEATURES;
    if (n0 >= N) return;
    const TW* wr[GV_FEATURES];
#pragma unroll
    for (int f = 0; f < GV_FEATURES; ++f) wr[f] = w + ((size_t)expert * N + (n0 + f < N ? n0 + f : n0)) * K;
    for (int r0 = 0; r0 < rows; r0 += GV_ROWS) {
        const TX* xr[GV_ROWS];
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r) {
            const int i = row0 + r0 + (r0 + r < rows ? r : 0);             // rows past the end repeat the first (never used)
            xr[r] = x + (size_t)(pair_at ? pair_at[i] / pairs_per_row : i) * K;
        }
        float acc[GV_ROWS][GV_FEATURES];
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r)
#pragma unroll
            for (int f = 0; f < GV_FEATURES; ++f) acc[r][f] = 0.0f;
        for (int k = lane * 8; k < K; k += 32 * 8) {
            float wv[GV_FEATURES][8];
#pragma unroll
            for (int f = 0; f < GV_FEATURES; ++f) load8(wr[f] + k, wv[f]);
#pragma unroll
            for (int r = 0; r < GV_ROWS; ++r) {
                if (r0 + r >= rows) continue;                              // the same for the whole block
                float xv[8];
                load8(xr[r] + k, xv);
#pragma unroll
                for (int f = 0; f < GV_FEATURES; ++f)
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[r][f] = fmaf(xv[j], wv[f][j], acc[r][f]);
            }
        }
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r) {
            if (r0 + r >= rows) continue;
#pragma unroll
            for (int f = 0; f < GV_FEATURES; ++f) {
                const float total = warp_sum(acc[r][f]);
                if (lane == 0 && n0 + f < N) y[(size_t)(row0 + r0 + r) * N + n0 + f] = from_float<TY>(total);
            }
        }
    }
}

// out[i] = x[token of the pair at sorted position i]: the rows of x in the order of the experts
template <typename TX>
__global__ void route_gather_kernel(const TX* __restrict__ x, const int32_t* __restrict__ pair_at, int pairs_per_row,
                                    TX* __restrict__ out, int K, long long total) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long i = idx / K;
    const int k = (int)(idx % K);
    out[idx] = x[(size_t)(pair_at[i] / pairs_per_row) * K + k];
}
// the same, 16 bytes per thread (vec = elements of 16 bytes; K a multiple of it)
template <typename TX>
__global__ void route_gather_vec_kernel(const TX* __restrict__ x, const int32_t* __restrict__ pair_at, int pairs_per_row,
                                        TX* __restrict__ out, int K, int vec, long long total) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int per_row = K / vec;
    const long long i = idx / per_row;
    const int k = (int)(idx % per_row) * vec;
    *reinterpret_cast<uint4*>(out + (size_t)i * K + k) =
        *reinterpret_cast<const uint4*>(x + (size_t)(pair_at[i] / pairs_per_row) * K + k);
}

template <typename TY>
__global__ void route_combine_kernel(const TY* __restrict__ y, const int32_t* __restrict__ position, const float* __restrict__ weight,
                                     int top, float* __restrict__ out, int E_out, long long total, const float* __restrict__ base,
                                     int base_splits, long long base_stride, const float* __restrict__ base_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int t = (int)(idx / E_out), c = (int)(idx % E_out);
    float acc = 0.0f;
    if (base) {
        for (int s = 0; s < base_splits; ++s) acc += base[(size_t)s * base_stride + idx];
        if (base_scale) acc *= base_scale[t];
    }
    for (int j = 0; j < top; ++j)
        acc += weight[(size_t)t * top + j] * to_float<TY>(y[(size_t)position[(size_t)t * top + j] * E_out + c]);
    out[idx] = acc;
}

// float32 y, four columns per thread
__global__ void route_combine_vec_kernel(const float* __restrict__ y, const int32_t* __restrict__ position, const float* __restrict__ weight,
                                         int top, float* __restrict__ out, int E_out, long long total4, const float* __restrict__ base,
                                         int base_splits, long long base_stride, const float* __restrict__ base_scale) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total4) return;
    const int per_row = E_out / 4;
    const int t = (int)(idx / per_row), c = (int)(idx % per_row) * 4;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (base)
        for (int s = 0; s < base_splits; ++s) {
            const float4 v = *reinterpret_cast<const float4*>(base + (size_t)s * base_stride + (size_t)t * E_out + c);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    if (base && base_scale) { const float f = base_scale[t]; acc.x *= f; acc.y *= f; acc.z *= f; acc.w *= f; }
    for (int j = 0; j < top; ++j) {
        const float wj = weight[(size_t)t * top + j];
        const float4 v = *reinterpret_cast<const float4*>(y + (size_t)position[(size_t)t * top + j] * E_out + c);
        acc.x += wj * v.x; acc.y += wj * v.y; acc.z += wj * v.z; acc.w += wj * v.w;
    }
    *reinterpret_cast<float4*>(out + (size_t)t * E_out + c) = acc;
}

}  // namespace

// x [T, K] (the model's dtype), w [E, K] float32, bias [E] or null -> choice [T, top], weight [T, top].
// scoring 0: softmax over the chosen logits; 1: sigmoid scores, the choice by score + correction (null: none), within the
// `keep` best of `groups` runs of neighbouring experts (groups 1: no runs).
// scoring 2: scores are the softmax over all experts; a run counts as its largest score; the weights are the chosen scores over
// their sum (+ 1e-20), times weight_scale.  gate_w ([K] float32, or null) with gate_out [T]: sigmoid(gate_w . x) per token.
PH_EXPORT int ph_route(const void* x, int x_dtype, const float* w, const float* bias, int T, int E, int K, int top, int32_t* choice,
                       float* weight, int scoring, const float* correction, int groups, int keep, float weight_scale,
                       const float* gate_w, float* gate_out, cudaStream_t stream) {
    if (!x || !w || !choice || !weight || T < 0 || E < 1 || K < 1 || top < 1 || top > E || !valid_dtype(x_dtype))
        return fail(PH_ERR_ARG, "route: bad arguments (T %d, experts %d, K %d, top %d)", T, E, K, top);
    if (scoring < 0 || scoring > 2 || (gate_w && !gate_out) || groups < 1 || E % groups || keep < 1 || keep > groups || (long long)keep * (E / groups) < top)
        return fail(PH_ERR_ARG, "route: scoring %d with %d of %d runs of %d experts cannot give %d choices", scoring, keep, groups,
                    E / (groups > 0 ? groups : 1), top);
    if (top > MAX_TOP || E > MAX_EXPERTS)
        return fail(PH_ERR_UNSUPPORTED, "route: top %d of %d experts exceeds the supported %d of %d", top, E, MAX_TOP, MAX_EXPERTS);
    if (T == 0) return PH_OK;
    const bool aligned = (((uintptr_t)x | (uintptr_t)w) & 15) == 0 || (K & 3) != 0;
    if (!aligned) return fail(PH_ERR_ARG, "route: the rows must be 16-byte aligned");
    if (T >= 64 && E <= MAX_EXPERTS / 4)
        PH_DISPATCH(x_dtype, TX, launch_overlapped(route_kernel<TX, 4>, dim3((T + 3) / 4), dim3(RT_WARPS * 32), 0, stream, (const TX*)x, w,
                                                   bias, T, E, K, top, choice, weight, scoring, correction, groups, keep, weight_scale, gate_w,
                                                   gate_out));
    else
        PH_DISPATCH(x_dtype, TX, launch_overlapped(route_kernel<TX, 1>, dim3(T), dim3(RT_WARPS * 32), 0, stream, (const TX*)x, w, bias, T,
                                                   E, K, top, choice, weight, scoring, correction, groups, keep, weight_scale, gate_w, gate_out));
    return check_launch("route");
}

PH_EXPORT int ph_route_max_tiles(int R, int E) { return (R + BM - 1) / BM + E; }

// choice [R] (R = tokens x top) -> position [R], pair_at [R], tiles [3 * max_tiles]; scratch: 3 * E + 1 int32.
PH_EXPORT int ph_route_sort(const int32_t* choice, int R, int E, int32_t* position, int32_t* pair_at, int32_t* tiles,
                            int max_tiles, int32_t* scratch, cudaStream_t stream) {
    if (!choice || !position || !pair_at || !tiles || !scratch || R < 0 || E < 1 || max_tiles < ph_route_max_tiles(R, E))
        return fail(PH_ERR_ARG, "route_sort: bad arguments (pairs %d, experts %d, tiles %d)", R, E, max_tiles);
    if (R == 0) return PH_OK;
    launch_overlapped(route_sort_kernel, dim3(1), dim3(E < 256 ? 256 : 1024), 0, stream, choice, R, E, position, pair_at, tiles,
                      max_tiles, scratch);
    return check_launch("route_sort");
}

// y [R, N] at the sorted positions; x rows are looked up through pair_at / pairs_per_row (null: x is already sorted);
// w [experts, N, K].
PH_EXPORT int ph_gemm_grouped(const void* x, int x_dtype, const int32_t* pair_at, int pairs_per_row, const void* w, int w_dtype,
                              const int32_t* tiles, int max_tiles, void* y, int y_dtype, int N, int K, cudaStream_t stream) {
    if (!x || !w || !tiles || !y || max_tiles < 1 || N < 1 || K < 1 || pairs_per_row < 1 || !valid_dtype(x_dtype) ||
        !valid_dtype(w_dtype) || !valid_dtype(y_dtype))
        return fail(PH_ERR_ARG, "gemm_grouped: bad arguments (tiles %d, N %d, K %d)", max_tiles, N, K);
    if (max_tiles > 65535) return fail(PH_ERR_UNSUPPORTED, "gemm_grouped: %d row tiles exceed the supported 65535", max_tiles);
    dim3 grid((N + BN - 1) / BN, max_tiles);
#define LAUNCH(TX, TW, TY)                                                                                                \
    launch_overlapped(gemm_grouped_kernel<TX, TW, TY>, grid, dim3(256), 0, stream, (const TX*)x, pair_at, pairs_per_row, \
                      (const TW*)w, tiles, (TY*)y, N, K)
    PH_DISPATCH(x_dtype, TX, PH_DISPATCH(w_dtype, TW, PH_DISPATCH(y_dtype, TY, LAUNCH(TX, TW, TY))));
#undef LAUNCH
    return check_launch("gemm_grouped");
}

PH_EXPORT int ph_route_gather(const void* x, int dtype, const int32_t* pair_at, int pairs_per_row, void* out, int R, int K,
                              cudaStream_t stream) {
    if (!x || !pair_at || !out || R < 0 || K < 1 || pairs_per_row < 1 || !valid_dtype(dtype))
        return fail(PH_ERR_ARG, "route_gather: bad arguments (rows %d, K %d)", R, K);
    const long long total = (long long)R * K;
    if (total == 0) return PH_OK;
    const int vec = dtype == PH_F32 ? 4 : 8;
    if (K % vec == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
        const long long n = total / vec;
        PH_DISPATCH(dtype, TX, launch_overlapped(route_gather_vec_kernel<TX>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
                                                 (const TX*)x, pair_at, pairs_per_row, (TX*)out, K, vec, n));
        return check_launch("route_gather");
    }
    PH_DISPATCH(dtype, TX, launch_overlapped(route_gather_kernel<TX>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                                             (const TX*)x, pair_at, pairs_per_row, (TX*)out, K, total));
    return check_launch("route_gather");
}

// As gemm_grouped, for few rows per expert.  PH_ERR_UNSUPPORTED when K is not a multiple of 8 or a row is not
// 16-byte aligned (the caller then takes gemm_grouped).
PH_EXPORT int ph_gemv_grouped(const void* x, int x_dtype, const int32_t* pair_at, int pairs_per_row, const void* w, int w_dtype,
                              const int32_t* tiles, int max_tiles, void* y, int y_dtype, int N, int K, cudaStream_t stream) {
    if (!x || !w || !tiles || !y || max_tiles < 1 || N < 1 || K < 1 || pairs_per_row < 1 || !valid_dtype(x_dtype) ||
        !valid_dtype(w_dtype) || !valid_dtype(y_dtype))
        return fail(PH_ERR_ARG, "gemv_grouped: bad arguments (tiles %d, N %d, K %d)", max_tiles, N, K);
    if (K % 8 || (((uintptr_t)x | (uintptr_t)w) & 15))
        return fail(PH_ERR_UNSUPPORTED, "gemv_grouped: K %d must be a multiple of 8 and the operands 16-byte aligned", K);
    if (max_tiles > 65535) return fail(PH_ERR_UNSUPPORTED, "gemv_grouped: %d row tiles exceed the supported 65535", max_tiles);
    dim3 grid((N + GV_WARPS * GV_FEATURES - 1) / (GV_WARPS * GV_FEATURES), max_tiles);
#define LAUNCH(TX, TW, TY)                                                                                                    \
    launch_overlapped(gemv_grouped_kernel<TX, TW, TY>, grid, dim3(GV_WARPS * 32), 0, stream, (const TX*)x, pair_at, pairs_per_row, \
                      (const TW*)w, tiles, (TY*)y, N, K)
    PH_DISPATCH(x_dtype, TX, PH_DISPATCH(w_dtype, TW, PH_DISPATCH(y_dtype, TY, LAUNCH(TX, TW, TY))));
#undef LAUNCH
    return check_launch("gemv_grouped");
}

PH_EXPORT int ph_route_combine(const void* y, int y_dtype, const int32_t* position, const float* weight, int T, int top, int E_out,
                               float* out, const float* base, int base_splits, long long base_stride, const float* base_scale,
                               cudaStream_t stream) {
    if (!y || !position || !weight || !out || T < 0 || top < 1 || E_out < 1 || !valid_dtype(y_dtype) || (base && base_splits < 1))
        return fail(PH_ERR_ARG, "route_combine: bad arguments (T %d, top %d, width %d)", T, top, E_out);
    const long long total = (long long)T * E_out;
    if (total == 0) return PH_OK;
    if (y_dtype == PH_F32 && E_out % 4 == 0 && (((uintptr_t)y | (uintptr_t)out | (uintptr_t)base) & 15) == 0 && base_stride % 4 == 0) {
        launch_overlapped(route_combine_vec_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, stream, (const float*)y, position,
                          weight, top, out, E_out, total / 4, base, base_splits, base_stride, base_scale);
        return check_launch("route_combine");
    }
    PH_DISPATCH(y_dtype, TY, launch_overlapped(route_combine_kernel<TY>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                                               (const TY*)y, position, weight, top, out, E_out, total, base, base_splits, base_stride, base_scale));
    return check_launch("route_combine");
}
