// Gated linear attention: a matrix-valued state per head that decays channel by channel, and what surrounds it.
//
//   decayed_scan   per request and head, token by token in the order of the rows:
//                      a_t = sigmoid(z_t + b)^(1/tau)            per key channel, as exp(-softplus(-(z_t + b)) / tau)
//                      S   <- diag(a_t) S + k_t v_t^T            S is [D, DV] float32 and lives in the request's state slot
//                      o_t  = S^T (q_t * q_scale)
//                  followed, for the rows the block has just written, by the per-head RMS norm over DV with a weight
//                  shared by the heads and the gate silu(g_t): y_t = o_t * rsqrt(mean(o_t^2) + eps) * w * silu(g_t)
//                  (head_norm_gate as a launch of its own where a head's columns are spread over several blocks).
//                  A block owns one (request, head): thread (column, part) keeps 16 state values of its column in
//                  registers, q, k and the decay of a tile of tokens are staged in shared memory while the next tile is
//                  on its way, and the parts of a column add up with a butterfly, in a fixed order.  A step with a long
//                  portion cuts every request's rows into chunks of 64 tokens: the chunks' own sums from a zero state
//                  side by side, a carry pass S <- (product of the chunk's decays) S + (the chunk's sum) over each
//                  request's chunks, then the outputs chunk by chunk from the state at each chunk's start.  Either way a
//                  prompt cut anywhere walks the same recurrence, up to the rounding of the association.
//   rms_pair_mean  out = (a * rsqrt(mean(a^2) + eps) * wa + b * rsqrt(mean(b^2) + eps) * wb) * factor per row: the
//                  outputs of two mixers that read the same input, each RMS-normed over the model width, combined.
// Everything here is float32 arithmetic; q, k, v and g may be stored in bfloat16.
#include "common.cuh"

#include <math.h>

namespace {

using namespace ph;

// log(sigmoid(x)) without overflow: -(max(-x, 0) + log1p(exp(-|x|)))
__device__ __forceinline__ float log_sigmoid(float x) { return -(fmaxf(-x, 0.0f) + log1pf(expf(-fabsf(x)))); }

// what q, k and v pass through on their way into the recurrence: nothing, or silu
__device__ __forceinline__ float act_in(float x, int kind) { return kind ? x / (1.0f + expf(-x)) : x; }

struct ScanParams {
    const void* q; const void* k; const void* v; const void* g;     // rows of the compute dtype, `stride` elements apart
    long long stride;
    const float* z; long long z_stride;                              // [T, H * D] float32: the decay's logits without their bias
    const float* z_bias;                                             // [H * D] or null
    float inv_tau, q_scale, eps;
    const float* norm_w;                                             // [DV]
    float* state; long long slot_stride;                             // [slots][H][DV][padded D]
    const int32_t* seg_start; const int32_t* seg_slot;
    const int32_t* chunks;                                           // [n][4]: first row, rows, segment, 1 on a request's last chunk
    const int32_t* seg_chunks;                                       // [S + 1]: the chunks of each segment
    float* carry;                                                    // [chunks][H][DV][padded D]: a chunk's own sum, then the state at its start
    float* decay;                                                    // [chunks][H][D]: the product of the chunk's decays
    float* raw;                                                      // [T, H * DV] float32 scratch: o before the norm
    void* out;                                                       // [T, H * DV] in the compute dtype
    int H, D, DV;
    int parts;                                                       // threads that share a column (a power of two), DPT key channels each
    int cols;                                                        // columns of a head per block
    int tile;                                                        // tokens staged at a time
    int fused_norm;                                                  // the block holds all of a head's columns and norms its rows
    const float* head_decay;                                         // [H] or null: one constant decay per head instead of the logits
    int in_act;                                                      // 1: q, k and v pass through silu on their way in
};

constexpr int DPT = 16;          // key channels per thread
constexpr int CPT = 4;           // columns per thread: 64 state values in registers, and every staged q, k and decay read serves four columns
constexpr int SLICE = DPT + 4;   // a thread's slice of q, k or the decay in shared memory, padded so that the parts' 16-byte reads miss each other's banks
constexpr int LOADS = 8;         // values a thread fetches per staged tile
constexpr int MAX_THREADS = 256;

// y = o * rsqrt(mean over the head's DV values of o^2 + eps) * w * silu(g) for the rows [row0, row0 + n) of head h, a warp per row
template <typename TX>
__device__ __forceinline__ void norm_gate_rows(const ScanParams& p, int h, int row0, int n, int warp, int warps, int lane) {
    const int H = p.H, DV = p.DV;
    const TX* gb = static_cast<const TX*>(p.g) + (size_t)h * DV;
    TX* out = static_cast<TX*>(p.out);
    for (int t = warp; t < n; t += warps) {
        const size_t at = (size_t)(row0 + t) * H * DV + (size_t)h * DV;
        float ss = 0.0f;
        for (int c = lane; c < DV; c += 32) { const float o = p.raw[at + c]; ss += o * o; }
        const float inv = rsqrtf(warp_sum(ss) / (float)DV + p.eps);
        for (int c = lane; c < DV; c += 32) {
            const float gate = to_float<TX>(gb[(size_t)(row0 + t) * p.stride + c]);
            out[at + c] = from_float<TX>(p.raw[at + c] * inv * p.norm_w[c] * (gate / (1.0f + expf(-gate))));
        }
    }
}

// Two float32 operations in one instruction (each half rounded as the single operation would be).
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n.reg .b64 ra, rb, rc, rd;\n"
        "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\nmov.b64 rc, {%6, %7};\n"
        "fma.rn.f32x2 rd, ra, rb, rc;\n"
        "mov.b64 {%0, %1}, rd;\n}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("{\n.reg .b64 ra, rb, rd;\n"
        "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\n"
        "mul.rn.f32x2 rd, ra, rb;\n"
        "mov.b64 {%0, %1}, rd;\n}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

template <typename TX> __device__ __forceinline__ uint32_t raw_bits(const TX* p);
template <> __device__ __forceinline__ uint32_t raw_bits<float>(const float* p) { return __float_as_uint(*p); }
template <> __device__ __forceinline__ uint32_t raw_bits<__nv_bfloat16>(const __nv_bfloat16* p) { return *reinterpret_cast<const unsigned short*>(p); }
template <typename TX> __device__ __forceinline__ float from_bits(uint32_t b);
template <> __device__ __forceinline__ float from_bits<float>(uint32_t b) { return __uint_as_float(b); }
template <> __device__ __forceinline__ float from_bits<__nv_bfloat16>(uint32_t b) { return __uint_as_float(b << 16); }

// The recurrence over a run of rows of one request and head.  Thread (column group, part) keeps the state of CPT columns x
// DPT key channels in registers; the `parts` threads of a column group are neighbouring lanes and add their partial sums
// with a butterfly, so a token costs no barrier.  q (scaled), k and the decay of `tile` tokens at a time wait in shared
// memory; the next tile is fetched into registers while this one is computed.  A head's state is stored [column][padded
// D], so that a thread's values are 64 contiguous bytes per column.
// MODE 0: a whole portion: the state comes from the request's slot and goes back there.
// MODE 1: a chunk from a zero state: no output, the chunk's own sum goes to p.carry.
// MODE 2: a chunk from the state at its start (p.carry after the carry pass): output only.
template <typename TX, int MODE>
__global__ void __launch_bounds__(MAX_THREADS, 2) decayed_scan_kernel(ScanParams p) {
    extern __shared__ float smem[];
    const int D = p.D, DV = p.DV, H = p.H, parts = p.parts, cols = p.cols, TT = p.tile;
    const int SL = parts * SLICE;                      // a staged row of q, k or the decay
    const int Dpad = parts * DPT;
    float* stage = smem;                               // [2][TT][3][SL]
    float* vs = smem + 2 * TT * 3 * SL;                // [2][TT][cols]
    const int item = blockIdx.x, h = blockIdx.y;
    const int part = threadIdx.x & (parts - 1), lcol = (threadIdx.x / parts) * CPT;
    const int col = blockIdx.z * cols + lcol;          // the first of this thread's columns
    pdl_launch_dependents();
    pdl_wait();
    int row0, n, seg;
    if (MODE == 0) { seg = item; row0 = p.seg_start[seg]; n = p.seg_start[seg + 1] - row0; }
    else { row0 = p.chunks[4 * item]; n = p.chunks[4 * item + 1]; seg = p.chunks[4 * item + 2]; }
    if (n <= 0) return;
    float* S = (MODE == 0 ? p.state + (size_t)p.seg_slot[seg] * p.slot_stride + (size_t)h * Dpad * DV
                          : p.carry + ((size_t)item * H + h) * Dpad * DV) + (size_t)part * DPT;
    float2 s[CPT / 2][DPT];                            // columns in pairs: two float32 operations per instruction
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
            float4 v4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (MODE != 1 && col + c < DV) v4 = *reinterpret_cast<const float4*>(S + (size_t)(col + c) * Dpad + i);
            if (c & 1) { s[c / 2][i].y = v4.x; s[c / 2][i + 1].y = v4.y; s[c / 2][i + 2].y = v4.z; s[c / 2][i + 3].y = v4.w; }
            else { s[c / 2][i].x = v4.x; s[c / 2][i + 1].x = v4.y; s[c / 2][i + 2].x = v4.z; s[c / 2][i + 3].x = v4.w; }
        }

    const TX* qb = static_cast<const TX*>(p.q) + (size_t)h * D;
    const TX* kb = static_cast<const TX*>(p.k) + (size_t)h * D;
    const TX* vb = static_cast<const TX*>(p.v) + (size_t)h * DV + (size_t)blockIdx.z * cols;
    const float* zb = p.z + (size_t)h * D;
    const int per_token = 3 * D + cols, per_tile = TT * per_token;
    // quotients of small integers by a float reciprocal (exact far beyond a tile's few thousand elements)
    const float inv_per_token = 1.0f / (float)per_token, inv_D = 1.0f / (float)D;
    auto token_of = [&](int e) { return (int)(((float)e + 0.5f) * inv_per_token); };
    auto which_of = [&](int r) { return (int)(((float)r + 0.5f) * inv_D); };
    uint32_t fetched[LOADS];
    // element e of a tile: token e / per_token, then q[D], k[D], decay logit[D], v[cols]
    auto fetch = [&](int t0) {
#pragma unroll
        for (int u = 0; u < LOADS; ++u) {
            const int e = threadIdx.x + u * blockDim.x;
            fetched[u] = 0;
            if (e >= per_tile) continue;
            const int tt = token_of(e), r = e - tt * per_token;
            if (t0 + tt >= n) continue;
            const size_t row = (size_t)(row0 + t0 + tt);
            if (r < D) fetched[u] = raw_bits<TX>(qb + row * p.stride + r);
            else if (r < 2 * D) fetched[u] = raw_bits<TX>(kb + row * p.stride + (r - D));
            else if (r < 3 * D) fetched[u] = p.head_decay ? 0u : __float_as_uint(zb[row * p.z_stride + (r - 2 * D)]);
            else if ((int)(blockIdx.z * cols) + r - 3 * D < DV) fetched[u] = raw_bits<TX>(vb + row * p.stride + (r - 3 * D));
        }
    };
    auto put = [&](int buf) {
#pragma unroll
        for (int u = 0; u < LOADS; ++u) {
            const int e = threadIdx.x + u * blockDim.x;
            if (e >= per_tile) continue;
            const int tt = token_of(e), r = e - tt * per_token;
            if (r < 3 * D) {
                const int which = which_of(r), d = r - which * D;
                float val;
                if (which == 0) val = act_in(from_bits<TX>(fetched[u]), p.in_act) * p.q_scale;
                else if (which == 1) val = act_in(from_bits<TX>(fetched[u]), p.in_act);
                else if (p.head_decay) val = p.head_decay[h];
                else val = expf(log_sigmoid(__uint_as_float(fetched[u]) + (p.z_bias ? p.z_bias[(size_t)h * D + d] : 0.0f)) * p.inv_tau);
                stage[((size_t)(buf * TT + tt) * 3 + which) * SL + (d / DPT) * SLICE + (d % DPT)] = val;
            } else {
                vs[(size_t)(buf * TT + tt) * cols + (r - 3 * D)] = act_in(from_bits<TX>(fetched[u]), p.in_act);
            }
        }
    };
    // slices past D stay zero: a decay of 0 on a state of 0 with a key of 0
    if (Dpad != D) {
        for (int i = threadIdx.x; i < 2 * TT * 3 * SL; i += blockDim.x) stage[i] = 0.0f;
        __syncthreads();
    }
    fetch(0);
    put(0);
    __syncthreads();
    for (int t0 = 0, buf = 0; t0 < n; t0 += TT, buf ^= 1) {
        const bool more = t0 + TT < n;
        if (more) fetch(t0 + TT);
        const int count = min(TT, n - t0);
        for (int tt = 0; tt < count; ++tt) {
            const float* qs = stage + (size_t)(buf * TT + tt) * 3 * SL + part * SLICE;
            const float* ks = qs + SL;
            const float* as = ks + SL;
            const float4 v4 = *reinterpret_cast<const float4*>(vs + (size_t)(buf * TT + tt) * cols + lcol);
            const float2 vt[CPT / 2] = {make_float2(v4.x, v4.y), make_float2(v4.z, v4.w)};
            float2 acc2[CPT / 2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
            for (int i = 0; i < DPT; i += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(qs + i), k4 = *reinterpret_cast<const float4*>(ks + i),
                             a4 = *reinterpret_cast<const float4*>(as + i);
                const float qv[4] = {q4.x, q4.y, q4.z, q4.w}, kv[4] = {k4.x, k4.y, k4.z, k4.w}, av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 qq = make_float2(qv[j], qv[j]), kk = make_float2(kv[j], kv[j]), aa = make_float2(av[j], av[j]);
#pragma unroll
                    for (int c = 0; c < CPT / 2; ++c) {
                        s[c][i + j] = fma2(aa, s[c][i + j], mul2(kk, vt[c]));       // a s + k v, the product rounded first
                        if (MODE != 1) acc2[c] = fma2(s[c][i + j], qq, acc2[c]);
                    }
                }
            }
            float acc[CPT] = {acc2[0].x, acc2[0].y, acc2[1].x, acc2[1].y};
            if (MODE != 1) {
#pragma unroll
                for (int c = 0; c < CPT; ++c)
                    for (int o = 1; o < parts; o <<= 1) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], o);
                if (part == 0) {
                    float* dst = p.raw + (size_t)(row0 + t0 + tt) * H * DV + (size_t)h * DV + col;
#pragma unroll
                    for (int c = 0; c < CPT; ++c)
                        if (col + c < DV) dst[c] = acc[c];
                }
            }
        }
        if (more) put(buf ^ 1);
        __syncthreads();
    }
    if (MODE != 2)
#pragma unroll
        for (int c = 0; c < CPT; ++c)
#pragma unroll
            for (int i = 0; i < DPT; i += 4)
                if (col + c < DV)
                    *reinterpret_cast<float4*>(S + (size_t)(col + c) * Dpad + i) =
                        (c & 1) ? make_float4(s[c / 2][i].y, s[c / 2][i + 1].y, s[c / 2][i + 2].y, s[c / 2][i + 3].y)
                                : make_float4(s[c / 2][i].x, s[c / 2][i + 1].x, s[c / 2][i + 2].x, s[c / 2][i + 3].x);
    if (MODE == 1 || !p.fused_norm) return;
    // the rows this block wrote: norm over the head's DV values, the weight, the gate
    __syncthreads();
    norm_gate_rows<TX>(p, h, row0, n, threadIdx.x >> 5, blockDim.x >> 5, threadIdx.x & 31);
}

template <typename TX>
__global__ void head_norm_gate_kernel(ScanParams p, int T) {
    pdl_launch_dependents();
    pdl_wait();
    const int warps = blockDim.x >> 5;
    const long long item = (long long)blockIdx.x * warps + (threadIdx.x >> 5);
    if (item >= (long long)T * p.H) return;
    norm_gate_rows<TX>(p, (int)(item % p.H), (int)(item / p.H), 1, 0, 1, threadIdx.x & 31);
}

// decay[chunk][h][d] = the product over the chunk's tokens of their decay of channel d, in the order of the tokens
__global__ void chunk_decay_kernel(ScanParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int item = blockIdx.x, h = blockIdx.y;
    const int row0 = p.chunks[4 * item], n = p.chunks[4 * item + 1];
    for (int d = threadIdx.x; d < p.D; d += blockDim.x) {
        const float bias = p.z_bias ? p.z_bias[(size_t)h * p.D + d] : 0.0f;
        float prod = 1.0f;
        if (p.head_decay) {                        // the constant, token by token as the recurrence multiplies it
            const float a = p.head_decay[h];
            for (int t = 0; t < n; ++t) prod *= a;
            p.decay[((size_t)item * p.H + h) * p.D + d] = prod;
            continue;
        }
        const float* zz = p.z + (size_t)row0 * p.z_stride + (size_t)h * p.D + d;
        for (int t = 0; t < n; t += 8) {
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = t + j < n ? zz[(size_t)(t + j) * p.z_stride] : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (t + j < n) prod *= expf(log_sigmoid(x[j] + bias) * p.inv_tau);
        }
        p.decay[((size_t)item * p.H + h) * p.D + d] = prod;
    }
}

// The carry over a request's chunks: S enters from the slot; for every chunk in turn carry[chunk] becomes the state at its
// start and S <- decay[chunk] * S + (the chunk's own sum); the last S goes back to the slot.  One thread per state element.
__global__ void chunk_carry_kernel(ScanParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int seg = blockIdx.y, Dpad = p.parts * DPT;
    const long long per_head = (long long)Dpad * p.DV, e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per_head * p.H) return;
    const int h = (int)(e / per_head), d = (int)(e % Dpad);              // a head's state is [column][padded D]
    if (d >= p.D) return;                                               // the padding stays zero
    float* slot = p.state + (size_t)p.seg_slot[seg] * p.slot_stride + e;
    float S = *slot;
    const int first = p.seg_chunks[seg], last = p.seg_chunks[seg + 1];
    const size_t step = (size_t)per_head * p.H, dstep = (size_t)p.H * p.D;
    float* at = p.carry + (size_t)first * step + e;
    const float* dec = p.decay + (size_t)first * dstep + (size_t)h * p.D + d;
    constexpr int B = 8;                                   // eight chunks' values on their way at a time
    for (int c = first; c < last; c += B) {
        float own[B], a[B];
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const bool in = c + j < last;
            own[j] = in ? at[(size_t)j * step] : 0.0f;
            a[j] = in ? dec[(size_t)j * dstep] : 1.0f;
        }
#pragma unroll
        for (int j = 0; j < B; ++j) {
            if (c + j < last) at[(size_t)j * step] = S;
            S = c + j < last ? fmaf(a[j], S, own[j]) : S;
        }
        at += (size_t)B * step;
        dec += (size_t)B * dstep;
    }
    *slot = S;
}

template <typename TA, typename TB>
__global__ void rms_pair_mean_kernel(const TA* __restrict__ a, int a_splits, long long a_stride, const float* __restrict__ wa,
                                     const TB* __restrict__ b, int b_splits, long long b_stride, const float* __restrict__ wb,
                                     float eps, float factor, float* __restrict__ out, int E) {
    extern __shared__ float buf[];            // [2][E]
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * E;
    float sa = 0.0f, sb = 0.0f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float x = 0.0f, y = 0.0f;
        for (int s = 0; s < a_splits; ++s) x += to_float<TA>(a[(size_t)s * a_stride + row + i]);
        for (int s = 0; s < b_splits; ++s) y += to_float<TB>(b[(size_t)s * b_stride + row + i]);
        buf[i] = x; buf[E + i] = y;
        sa += x * x; sb += y * y;
    }
    const float ia = rsqrtf(block_sum_any(sa, scratch) / (float)E + eps);
    const float ib = rsqrtf(block_sum_any(sb, scratch) / (float)E + eps);
    for (int i = threadIdx.x; i < E; i += blockDim.x) out[row + i] = (buf[i] * ia * wa[i] + buf[E + i] * ib * wb[i]) * factor;
}

// The same for float32 addends with rows of a multiple of four columns: 16-byte loads, the sums of a thread's columns kept
// in registers between the two passes (at most ROUNDS x 4 columns a thread).
template <int ROUNDS>
__global__ void rms_pair_mean_vec_kernel(const float* __restrict__ a, int a_splits, long long a_stride, const float* __restrict__ wa,
                                         const float* __restrict__ b, int b_splits, long long b_stride, const float* __restrict__ wb,
                                         float eps, float factor, float* __restrict__ out, int E) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * E;
    float4 x[ROUNDS], y[ROUNDS];
    float sa = 0.0f, sb = 0.0f;
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {
        const int i = (threadIdx.x + r * blockDim.x) * 4;
        x[r] = y[r] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i >= E) continue;
        for (int s = 0; s < a_splits; ++s) {
            const float4 u = *reinterpret_cast<const float4*>(a + (size_t)s * a_stride + row + i);
            x[r].x += u.x; x[r].y += u.y; x[r].z += u.z; x[r].w += u.w;
        }
        for (int s = 0; s < b_splits; ++s) {
            const float4 u = *reinterpret_cast<const float4*>(b + (size_t)s * b_stride + row + i);
            y[r].x += u.x; y[r].y += u.y; y[r].z += u.z; y[r].w += u.w;
        }
        sa += (x[r].x * x[r].x + x[r].y * x[r].y) + (x[r].z * x[r].z + x[r].w * x[r].w);
        sb += (y[r].x * y[r].x + y[r].y * y[r].y) + (y[r].z * y[r].z + y[r].w * y[r].w);
    }
    const float ia = rsqrtf(block_sum_any(sa, scratch) / (float)E + eps);
    const float ib = rsqrtf(block_sum_any(sb, scratch) / (float)E + eps);
#pragma unroll
    for (int r = 0; r < ROUNDS; ++r) {
        const int i = (threadIdx.x + r * blockDim.x) * 4;
        if (i >= E) continue;
        const float4 u = *reinterpret_cast<const float4*>(wa + i), v = *reinterpret_cast<const float4*>(wb + i);
        *reinterpret_cast<float4*>(out + row + i) =
            make_float4((x[r].x * ia * u.x + y[r].x * ib * v.x) * factor, (x[r].y * ia * u.y + y[r].y * ib * v.y) * factor,
                        (x[r].z * ia * u.z + y[r].z * ib * v.z) * factor, (x[r].w * ia * u.w + y[r].w * ib * v.w) * factor);
    }
}

// y = o * rsqrt(mean over the whole row of o^2 + eps) * w * gate(g), gate 0: silu, 1: sigmoid; a block per row
template <typename TG, typename TO>
__global__ void rms_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps, const TG* __restrict__ g,
                                long long g_stride, int gate, TO* __restrict__ out, int W) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * W;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) { const float x = o[row + i]; ss += x * x; }
    const float inv = rsqrtf(block_sum_any(ss, scratch) / (float)W + eps);
    const TG* gr = g + (size_t)blockIdx.x * g_stride;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float z = to_float<TG>(gr[i]), s = 1.0f / (1.0f + expf(-z));
        out[row + i] = from_float<TO>(o[row + i] * inv * w[i] * (gate ? s : z * s));
    }
}

}  // namespace

// o [T, W] float32 -> out [T, W]: the RMS norm over the whole row with the weight w, times silu (gate 0) or sigmoid (gate 1)
// of g, whose rows are g_stride elements apart.
PH_EXPORT int ph_rms_gate(const float* o, const float* w, float eps, const void* g, int g_dtype, long long g_stride, int gate, void* out,
                          int out_dtype, int T, int W, cudaStream_t stream) {
    if (!o || !w || !g || !out || T < 0 || W < 1 || gate < 0 || gate > 1 || !valid_dtype(g_dtype) || !valid_dtype(out_dtype))
        return fail(PH_ERR_ARG, "rms_gate: bad arguments (T %d, W %d)", T, W);
    if (T == 0) return PH_OK;
    int threads = (W / 4 + 31) / 32 * 32;
    threads = threads < 64 ? 64 : threads > 512 ? 512 : threads;
    PH_DISPATCH(g_dtype, TG, PH_DISPATCH(out_dtype, TO,
        launch_overlapped(rms_gate_kernel<TG, TO>, dim3(T), dim3(threads), 0, stream, o, w, eps, (const TG*)g, g_stride, gate, (TO*)out, W)));
    return check_launch("rms_gate");
}

// A request's state is [H][DV][padded D] float32, padded D = 16 times the power of two that holds D / 16 (the kernel's
// threads own 16 key channels each); slot_stride is its size.
// head_decay ([H], or null): every key channel of head h decays by head_decay[h] at every token, and z is not read.
// in_act 1: q, k and v pass through silu first.  raw_only 1: o is left in `raw` (float32) and neither normed nor gated.
// chunks (n_chunks > 0): the step's rows cut into chunks per request ([n][4]: first row, rows, segment, last flag) with
// seg_chunks [S + 1], carry [n_chunks, H, DV, padded D] and decay [n_chunks, H, D] as scratch: the chunks' own sums side by side,
// a carry pass over each request's chunks, then the outputs chunk by chunk.  Without chunks a block walks a whole portion.
PH_EXPORT int ph_decayed_scan(const void* q, const void* k, const void* v, const void* g, int dtype, long long stride, const float* z,
                              long long z_stride, const float* z_bias, float tau, float q_scale, const float* norm_w, float eps,
                              float* state, long long slot_stride, const int32_t* seg_start, const int32_t* seg_slot, int S, int T, int H,
                              int D, int DV, const int32_t* chunks, int n_chunks, const int32_t* seg_chunks, float* carry, float* decay,
                              float* raw, void* out, const float* head_decay, int in_act, int raw_only, cudaStream_t stream) {
    if (!q || !k || !v || !state || !seg_start || !seg_slot || !raw || S < 0 || T < 0 || H < 1 || D < 1 ||
        DV < 1 || !(tau > 0.0f) || !valid_dtype(dtype) || n_chunks < 0 || (n_chunks && (!chunks || !seg_chunks || !carry || !decay)) ||
        (!z && !head_decay) || (!raw_only && (!g || !norm_w || !out)))
        return fail(PH_ERR_ARG, "decayed_scan: bad arguments (S %d, H %d, D %d, DV %d)", S, H, D, DV);
    if (S == 0 || T == 0) return PH_OK;
    int parts = 1;
    while (parts * DPT < D) parts *= 2;
    if (parts > 32) return fail(PH_ERR_UNSUPPORTED, "decayed_scan: %d key channels per head exceed the supported %d", D, 32 * DPT);
    if (slot_stride != (long long)H * parts * DPT * DV)
        return fail(PH_ERR_ARG, "decayed_scan: a request's state holds %d heads of %d columns of %d (padded) key channels", H, DV, parts * DPT);
    const int unit = CPT * 32 / parts;                             // columns of one warp
    int cols = (DV + unit - 1) / unit * unit;
    if (cols / CPT * parts > MAX_THREADS) cols = MAX_THREADS / parts * CPT;
    // a narrow head with many key channels: idle columns, so that the block has the threads to fetch a token's values
    while (3 * D + cols > LOADS * (cols / CPT * parts) && (cols + unit) / CPT * parts <= MAX_THREADS) cols += unit;
    const int threads = cols / CPT * parts;
    int tile = 16;
    while (tile > 1 && tile * (3 * D + cols) > LOADS * threads) tile /= 2;
    if (tile * (3 * D + cols) > LOADS * threads) return fail(PH_ERR_UNSUPPORTED, "decayed_scan: a token of %d + %d values does not fit a tile", 3 * D, cols);
    ScanParams p;
    p.q = q; p.k = k; p.v = v; p.g = g; p.stride = stride; p.z = z; p.z_stride = z_stride; p.z_bias = z_bias;
    p.inv_tau = 1.0f / tau; p.q_scale = q_scale; p.eps = eps; p.norm_w = norm_w; p.state = state; p.slot_stride = slot_stride;
    p.seg_start = seg_start; p.seg_slot = seg_slot; p.chunks = chunks; p.seg_chunks = seg_chunks; p.carry = carry; p.decay = decay;
    p.raw = raw; p.out = out; p.H = H; p.D = D; p.DV = DV; p.parts = parts; p.cols = cols; p.tile = tile;
    p.head_decay = head_decay; p.in_act = in_act ? 1 : 0;
    const int col_tiles = (DV + cols - 1) / cols;
    p.fused_norm = col_tiles == 1 && !raw_only;
    const size_t smem = (size_t)(2 * tile * 3 * parts * SLICE + 2 * tile * cols) * sizeof(float);
#define LAUNCH_SCAN(TX, MODE, ITEMS)                                                                                             \
    do {                                                                                                                         \
        if (smem > 48 * 1024) cudaFuncSetAttribute(decayed_scan_kernel<TX, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_overlapped(decayed_scan_kernel<TX, MODE>, dim3(ITEMS, H, col_tiles), dim3(threads), smem, stream, p);            \
    } while (0)
    if (n_chunks == 0) {
        PH_DISPATCH(dtype, TX, LAUNCH_SCAN(TX, 0, S));
    } else {
        launch_overlapped(chunk_decay_kernel, dim3(n_chunks, H), dim3(D >= 128 ? 128 : 64), 0, stream, p);
        PH_DISPATCH(dtype, TX, LAUNCH_SCAN(TX, 1, n_chunks));
        const long long elements = (long long)H * parts * DPT * DV;
        launch_overlapped(chunk_carry_kernel, dim3((unsigned)((elements + 255) / 256), S), dim3(256), 0, stream, p);
        PH_DISPATCH(dtype, TX, LAUNCH_SCAN(TX, 2, n_chunks));
    }
#undef LAUNCH_SCAN
    if (!p.fused_norm && !raw_only) {
        const long long items = (long long)T * H;
        PH_DISPATCH(dtype, TX, launch_overlapped(head_norm_gate_kernel<TX>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, p, T));
    }
    return check_launch("decayed_scan");
}

PH_EXPORT int ph_rms_pair_mean(const void* a, int a_dtype, int a_splits, long long a_stride, const float* wa, const void* b, int b_dtype,
                               int b_splits, long long b_stride, const float* wb, float eps, float factor, float* out, int T, int E,
                               cudaStream_t stream) {
    if (!a || !b || !wa || !wb || !out || T < 0 || E < 1 || a_splits < 1 || b_splits < 1 || !valid_dtype(a_dtype) || !valid_dtype(b_dtype))
        return fail(PH_ERR_ARG, "rms_pair_mean: bad arguments (T %d, E %d)", T, E);
    if (T == 0) return PH_OK;
    const uintptr_t all = (uintptr_t)a | (uintptr_t)b | (uintptr_t)wa | (uintptr_t)wb | (uintptr_t)out;
    if (a_dtype == PH_F32 && b_dtype == PH_F32 && E % 4 == 0 && E <= 16384 && (all & 15) == 0 && a_stride % 4 == 0 && b_stride % 4 == 0) {
        const int quads = E / 4;
        // few rows: a thread per quad (latency); many rows: up to four quads a thread (the rows fill the device)
        const int rounds = T >= 256 ? (quads <= 128 ? 1 : quads <= 256 ? 2 : 4) : (quads <= 1024 ? 1 : quads <= 2048 ? 2 : 4);
        const int vthreads = ((quads + rounds - 1) / rounds + 31) / 32 * 32;
        const float* fa = (const float*)a;
        const float* fb = (const float*)b;
        if (rounds == 1) launch_overlapped(rms_pair_mean_vec_kernel<1>, dim3(T), dim3(vthreads), 0, stream, fa, a_splits, a_stride, wa, fb, b_splits, b_stride, wb, eps, factor, out, E);
        else if (rounds == 2) launch_overlapped(rms_pair_mean_vec_kernel<2>, dim3(T), dim3(vthreads), 0, stream, fa, a_splits, a_stride, wa, fb, b_splits, b_stride, wb, eps, factor, out, E);
        else launch_overlapped(rms_pair_mean_vec_kernel<4>, dim3(T), dim3(vthreads), 0, stream, fa, a_splits, a_stride, wa, fb, b_splits, b_stride, wb, eps, factor, out, E);
        return check_launch("rms_pair_mean");
    }
    const size_t smem = (size_t)2 * E * sizeof(float);
    if (smem > 200 * 1024) return fail(PH_ERR_UNSUPPORTED, "rms_pair_mean: two rows of %d do not fit shared memory", E);
    // few rows: a thread per two columns (latency); many rows: a quarter of that (the rows fill the device)
    int threads = (T >= 256 ? E / 8 : E / 2 + 31) / 32 * 32;
    threads = threads < 64 ? 64 : threads > 1024 ? 1024 : threads;
#define LAUNCH_PAIR(TA, TB)                                                                                                      \
    do {                                                                                                                         \
        if (smem > 48 * 1024) cudaFuncSetAttribute(rms_pair_mean_kernel<TA, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_overlapped(rms_pair_mean_kernel<TA, TB>, dim3(T), dim3(threads), smem, stream, (const TA*)a, a_splits, a_stride, wa, \
                          (const TB*)b, b_splits, b_stride, wb, eps, factor, out, E);                                           \
    } while (0)
    PH_DISPATCH(a_dtype, TA, PH_DISPATCH(b_dtype, TB, LAUNCH_PAIR(TA, TB)));
#undef LAUNCH_PAIR
    return check_launch("rms_pair_mean");
}
