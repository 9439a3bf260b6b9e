// A minimal gated recurrent unit, element by element, and the weighted sum of two mixers' outputs.
//
//   min_gru_scan   per request and channel c, over the request's rows in order:
//                      z = sigmoid(a_z + b_z),  u = a_x + b_x,  cand = u + 1/2 where u >= 0, sigmoid(u) below
//                      S <- (1 - z) S + z cand,   y = S * silu(a_g)
//                  with [a_z | a_x | a_g] the rows of one product (partial sums added up), S the float32 state of the
//                  request's slot (read at the first row, written back after the last).  The gates read the current
//                  token only, so the recurrence is linear in S: S_t = A_t S_(t-1) + B_t with A = 1 - z, B = z cand.
//                  Short portions: a thread per (request, channel) walks the rows.  A step with a long portion cuts every
//                  request's rows into chunks (the list the step carries): a first launch composes each chunk's (A, B)
//                  from S = 0, a second walks each request's chunks in order and leaves the state at every chunk's start,
//                  a third walks the chunks side by side and writes y.
//   pair_sum       out = fa * a + fb * b per element, a and b the outputs of two mixers (partial sums added up), float32 out.
// Everything is float32; the product rows may be stored in bfloat16.
#include "common.cuh"

#include <math.h>

namespace {

using namespace ph;

__device__ __forceinline__ float sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename TI>
__device__ __forceinline__ float sum_parts(const TI* p, int splits, long long split_stride) {
    float v = 0.0f;
    for (int s = 0; s < splits; ++s) v += to_float<TI>(p[(size_t)s * split_stride]);
    return v;
}

// One step of the recurrence from the three product values of a token and channel.
__device__ __forceinline__ void gru_terms(float az, float ax, float bz, float bx, float& keep, float& put) {
    const float z = sigmoidf(az + bz), u = ax + bx;
    const float cand = u >= 0.0f ? u + 0.5f : sigmoidf(u);
    keep = 1.0f - z;
    put = z * cand;
}

// mode 0: walk the rows [row0, row0 + n) from the state in `start`, write y and leave the last state in `finish` (if given).
// mode 1: compose the rows' (A, B) from S = 0 and store them (no y).
template <typename TI, typename TO>
__device__ __forceinline__ void walk(const TI* __restrict__ rows, int splits, long long split_stride, long long row_width, int W,
                                     const float* __restrict__ bz, const float* __restrict__ bx, int row0, int n, int c, float s,
                                     TO* __restrict__ y, float* __restrict__ finish, float* __restrict__ a_out, float* __restrict__ b_out) {
    float a = 1.0f;
    const float zb = bz ? bz[c] : 0.0f, xb = bx ? bx[c] : 0.0f;
    for (int i = 0; i < n; ++i) {
        const TI* r = rows + (size_t)(row0 + i) * row_width + c;
        float keep, put;
        gru_terms(sum_parts(r, splits, split_stride), sum_parts(r + W, splits, split_stride), zb, xb, keep, put);
        s = __fmaf_rn(keep, s, put);
        if (a_out) a *= keep;
        if (y) {
            const float g = sum_parts(r + 2 * W, splits, split_stride);
            y[(size_t)(row0 + i) * W + c] = from_float<TO>(s * (g * sigmoidf(g)));
        }
    }
    if (finish) *finish = s;
    if (a_out) { *a_out = a; *b_out = s; }
}

// whole requests: a thread per (request, channel)
template <typename TI, typename TO>
__global__ void min_gru_rows_kernel(const TI* __restrict__ rows, int splits, long long split_stride, long long row_width, int W,
                                    const float* __restrict__ bz, const float* __restrict__ bx, float* __restrict__ state,
                                    const int32_t* __restrict__ seg_start, const int32_t* __restrict__ seg_slot, TO* __restrict__ y) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, seg = blockIdx.y;
    if (c >= W) return;
    const int row0 = seg_start[seg], n = seg_start[seg + 1] - row0;
    if (n <= 0) return;
    float* st = state + (size_t)seg_slot[seg] * W + c;
    walk<TI, TO>(rows, splits, split_stride, row_width, W, bz, bx, row0, n, c, *st, y, st, nullptr, nullptr);
}

// chunks [n][4]: first row, rows, segment, 1 on a request's last chunk
template <typename TI, typename TO>
__global__ void min_gru_chunk_kernel(const TI* __restrict__ rows, int splits, long long split_stride, long long row_width, int W,
                                     const float* __restrict__ bz, const float* __restrict__ bx, const int32_t* __restrict__ chunks,
                                     float* __restrict__ ca, float* __restrict__ cb, const float* __restrict__ cs, TO* __restrict__ y) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, k = blockIdx.y;
    if (c >= W) return;
    const int row0 = chunks[4 * k], n = chunks[4 * k + 1];
    if (y) walk<TI, TO>(rows, splits, split_stride, row_width, W, bz, bx, row0, n, c, cs[(size_t)k * W + c], y, nullptr, nullptr, nullptr);
    else walk<TI, TO>(rows, splits, split_stride, row_width, W, bz, bx, row0, n, c, 0.0f, nullptr, nullptr, ca + (size_t)k * W + c, cb + (size_t)k * W + c);
}

// a thread per (request, channel) walks the request's chunks: cs[k] = the state at the start of chunk k
__global__ void min_gru_carry_kernel(const float* __restrict__ ca, const float* __restrict__ cb, float* __restrict__ cs,
                                     const int32_t* __restrict__ seg_chunks, const int32_t* __restrict__ seg_slot, float* __restrict__ state, int W) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, seg = blockIdx.y;
    if (c >= W) return;
    const int k0 = seg_chunks[seg], k1 = seg_chunks[seg + 1];
    if (k1 <= k0) return;
    float* st = state + (size_t)seg_slot[seg] * W + c;
    float s = *st;
    for (int k = k0; k < k1; ++k) {
        cs[(size_t)k * W + c] = s;
        s = __fmaf_rn(ca[(size_t)k * W + c], s, cb[(size_t)k * W + c]);
    }
    *st = s;
}

template <typename TA, typename TB>
__global__ void pair_sum_kernel(const TA* __restrict__ a, int a_splits, long long a_stride, float fa, const TB* __restrict__ b,
                                int b_splits, long long b_stride, float fb, float* __restrict__ out, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = fa * sum_parts(a + i, a_splits, a_stride) + fb * sum_parts(b + i, b_splits, b_stride);
}

}  // namespace

// rows: [splits][T][row_width] in rows_dtype, a row [a_z (W) | a_x (W) | a_g (W) | ...].  state: [slots][W] float32.
// chunks / seg_chunks (device, may be null with n_chunks 0): the step's chunk list; carry: 3 * n_chunks * W floats of scratch.
PH_EXPORT int ph_min_gru_scan(const void* rows, int rows_dtype, int splits, long long split_stride, long long row_width,
                              const float* z_bias, const float* x_bias, float* state, const int32_t* seg_start, const int32_t* seg_slot,
                              int S, int T, int W, const int32_t* chunks, int n_chunks, const int32_t* seg_chunks, float* carry, void* out,
                              int out_dtype, cudaStream_t stream) {
    if (!rows || !state || !seg_start || !seg_slot || !out || S < 0 || T < 0 || W < 1 || splits < 1 || row_width < 3LL * W ||
        !valid_dtype(rows_dtype) || !valid_dtype(out_dtype) || (n_chunks > 0 && (!chunks || !seg_chunks || !carry)))
        return fail(PH_ERR_ARG, "min_gru_scan: bad arguments (S %d, T %d, W %d)", S, T, W);
    if (S == 0 || T == 0) return PH_OK;
    const int threads = 128;
    const unsigned bx = (unsigned)((W + threads - 1) / threads);
    if (n_chunks > 0) {
        float *ca = carry, *cb = carry + (size_t)n_chunks * W, *cs = carry + 2 * (size_t)n_chunks * W;
#define LAUNCH(TI, TO)                                                                                                                 \
        do {                                                                                                                           \
            min_gru_chunk_kernel<TI, TO><<<dim3(bx, n_chunks), threads, 0, stream>>>((const TI*)rows, splits, split_stride, row_width, W, \
                                                                                     z_bias, x_bias, chunks, ca, cb, nullptr, nullptr); \
            min_gru_carry_kernel<<<dim3(bx, S), threads, 0, stream>>>(ca, cb, cs, seg_chunks, seg_slot, state, W);                    \
            min_gru_chunk_kernel<TI, TO><<<dim3(bx, n_chunks), threads, 0, stream>>>((const TI*)rows, splits, split_stride, row_width, W, \
                                                                                     z_bias, x_bias, chunks, ca, cb, cs, (TO*)out);    \
        } while (0)
        PH_DISPATCH(rows_dtype, TI, PH_DISPATCH(out_dtype, TO, LAUNCH(TI, TO)));
#undef LAUNCH
        return check_launch("min_gru_scan (chunks)");
    }
#define LAUNCH(TI, TO)                                                                                                                 \
    min_gru_rows_kernel<TI, TO><<<dim3(bx, S), threads, 0, stream>>>((const TI*)rows, splits, split_stride, row_width, W, z_bias, x_bias, \
                                                                     state, seg_start, seg_slot, (TO*)out)
    PH_DISPATCH(rows_dtype, TI, PH_DISPATCH(out_dtype, TO, LAUNCH(TI, TO)));
#undef LAUNCH
    return check_launch("min_gru_scan");
}

PH_EXPORT int ph_pair_sum(const void* a, int a_dtype, int a_splits, long long a_stride, float fa, const void* b, int b_dtype, int b_splits,
                          long long b_stride, float fb, float* out, long long n, cudaStream_t stream) {
    if (!a || !b || !out || n < 0 || a_splits < 1 || b_splits < 1 || !valid_dtype(a_dtype) || !valid_dtype(b_dtype))
        return fail(PH_ERR_ARG, "pair_sum: bad arguments");
    if (n == 0) return PH_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
#define LAUNCH(TA, TB) pair_sum_kernel<TA, TB><<<blocks, 256, 0, stream>>>((const TA*)a, a_splits, a_stride, fa, (const TB*)b, b_splits, b_stride, fb, out, n)
    PH_DISPATCH(a_dtype, TA, PH_DISPATCH(b_dtype, TB, LAUNCH(TA, TB)));
#undef LAUNCH
    return check_launch("pair_sum");
}
