// Dynamic tanh as a norm, with the residual add folded in, and the re-start of the residual stream from itself and
// from what the embedding gave.
//
//   add_dyntanh     v = x + (addend a) + (addend b), both optional and each possibly split-K partial sums; x <- v when
//                   asked; y = tanh(alpha * v) * w + bias.  No statistic of the row is taken, so the elements are
//                   independent and a row needs no block of its own.  `rows` gathers (y only); out may be x itself.
//   concat_restart  cat[t] = [x[t] + addends | x0[t]] in the product's dtype, and x[t] <- start (a row that every token
//                   gets): what a product over cat is then added to.
// Everything is float32 arithmetic; tanh is tanhf.
#include "common.cuh"

#include <math.h>

namespace {

using namespace ph;

template <typename T> __device__ __forceinline__ float4 sum_splits(const T* a, int splits, long long stride, size_t at) {
    float4 s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int i = 0; i < splits; ++i) {
        const float4 v = load4(a + (size_t)i * stride + at);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    return s;
}

template <typename TA, typename TB, typename TO>
__global__ void add_dyntanh_kernel(float* x, const TA* __restrict__ a, int a_splits, long long a_stride,
                                   const TB* __restrict__ b, int b_splits, long long b_stride, const float* __restrict__ alpha,
                                   const float* __restrict__ w, const float* __restrict__ bias, const int32_t* __restrict__ rows,
                                   long long quads, int E, TO* out, int write_back) {
    pdl_launch_dependents();
    pdl_wait();
    const long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= quads) return;
    const int per_row = E / 4;
    const long long r = q / per_row;
    const int c = (int)(q % per_row) * 4;
    const size_t at = (size_t)(rows ? rows[r] : r) * E + c;
    float4 v = *reinterpret_cast<const float4*>(x + at);
    if (a) { const float4 s = sum_splits<TA>(a, a_splits, a_stride, at); v.x += s.x; v.y += s.y; v.z += s.z; v.w += s.w; }
    if (b) { const float4 s = sum_splits<TB>(b, b_splits, b_stride, at); v.x += s.x; v.y += s.y; v.z += s.z; v.w += s.w; }
    if (write_back) *reinterpret_cast<float4*>(x + at) = v;
    if (!out) return;
    const float al = alpha[0];
    const float4 wv = *reinterpret_cast<const float4*>(w + c), bv = *reinterpret_cast<const float4*>(bias + c);
    const float y[4] = {tanhf(al * v.x) * wv.x + bv.x, tanhf(al * v.y) * wv.y + bv.y, tanhf(al * v.z) * wv.z + bv.z,
                        tanhf(al * v.w) * wv.w + bv.w};
    store4(out + (size_t)r * E + c, y);
}

// the same, element by element, for widths that are no multiple of four
template <typename TA, typename TB, typename TO>
__global__ void add_dyntanh_scalar_kernel(float* __restrict__ x, const TA* __restrict__ a, int a_splits, long long a_stride,
                                          const TB* __restrict__ b, int b_splits, long long b_stride, const float* __restrict__ alpha,
                                          const float* __restrict__ w, const float* __restrict__ bias, const int32_t* __restrict__ rows,
                                          long long total, int E, TO* out, int write_back) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / E;
    const int c = (int)(i % E);
    const size_t at = (size_t)(rows ? rows[r] : r) * E + c;
    float v = x[at];
    if (a) for (int s = 0; s < a_splits; ++s) v += to_float<TA>(a[(size_t)s * a_stride + at]);
    if (b) for (int s = 0; s < b_splits; ++s) v += to_float<TB>(b[(size_t)s * b_stride + at]);
    if (write_back) x[at] = v;
    if (out) out[(size_t)r * E + c] = from_float<TO>(tanhf(alpha[0] * v) * w[c] + bias[c]);
}

template <typename TA, typename TB, typename TO>
__global__ void concat_restart_kernel(float* __restrict__ x, const TA* __restrict__ a, int a_splits, long long a_stride,
                                      const TB* __restrict__ b, int b_splits, long long b_stride, const float* __restrict__ x0,
                                      const float* __restrict__ start, TO* __restrict__ cat, long long total, int E) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / E;
    const int c = (int)(i % E);
    float v = x[i];
    if (a) for (int s = 0; s < a_splits; ++s) v += to_float<TA>(a[(size_t)s * a_stride + i]);
    if (b) for (int s = 0; s < b_splits; ++s) v += to_float<TB>(b[(size_t)s * b_stride + i]);
    cat[(size_t)r * 2 * E + c] = from_float<TO>(v);
    cat[(size_t)r * 2 * E + E + c] = from_float<TO>(x0[i]);
    x[i] = start ? start[c] : 0.0f;
}

}  // namespace

// x [T, E] float32; addends a and b (null: none) of [splits][T, E]; alpha a scalar on the device; w, bias [E].
// rows (null: all n rows in place): the rows of x that out's n rows come from; then nothing is written back.
// out (null: only the sum is wanted) [n, E] in out_dtype; it may be x itself when out_dtype is float32 and rows is null.
PH_EXPORT int ph_add_dyntanh(float* x, const void* a, int a_dtype, int a_splits, long long a_stride, const void* b, int b_dtype, int b_splits,
                             long long b_stride, const float* alpha, const float* w, const float* bias, const int32_t* rows, int n, int E,
                             void* out, int out_dtype, int write_back, cudaStream_t stream) {
    if (!x || n < 0 || E < 1 || (a && a_splits < 1) || (b && b_splits < 1) || !valid_dtype(a_dtype) || !valid_dtype(b_dtype) ||
        !valid_dtype(out_dtype) || (out && (!alpha || !w || !bias)) || (rows && write_back))
        return fail(PH_ERR_ARG, "add_dyntanh: bad arguments (rows %d, width %d)", n, E);
    if (n == 0) return PH_OK;
    const long long total = (long long)n * E;
    const uintptr_t all = (uintptr_t)x | (uintptr_t)a | (uintptr_t)b | (uintptr_t)w | (uintptr_t)bias | (uintptr_t)out;
    if (E % 4 == 0 && (all & 15) == 0 && a_stride % 4 == 0 && b_stride % 4 == 0) {
        const long long quads = total / 4;
        PH_DISPATCH(a_dtype, TA, PH_DISPATCH(b_dtype, TB, PH_DISPATCH(out_dtype, TO,
            launch_overlapped(add_dyntanh_kernel<TA, TB, TO>, dim3((unsigned)((quads + 255) / 256)), dim3(256), 0, stream, x, (const TA*)a,
                              a_splits, a_stride, (const TB*)b, b_splits, b_stride, alpha, w, bias, rows, quads, E, (TO*)out, write_back))));
        return check_launch("add_dyntanh");
    }
    PH_DISPATCH(a_dtype, TA, PH_DISPATCH(b_dtype, TB, PH_DISPATCH(out_dtype, TO,
        launch_overlapped(add_dyntanh_scalar_kernel<TA, TB, TO>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x,
                          (const TA*)a, a_splits, a_stride, (const TB*)b, b_splits, b_stride, alpha, w, bias, rows, total, E, (TO*)out,
                          write_back))));
    return check_launch("add_dyntanh");
}

// cat [T, 2E] in cat_dtype <- [x + addends | x0]; x <- start (a row [E], null: zeros).
PH_EXPORT int ph_concat_restart(float* x, const void* a, int a_dtype, int a_splits, long long a_stride, const void* b, int b_dtype,
                                int b_splits, long long b_stride, const float* x0, const float* start, void* cat, int cat_dtype, int T, int E,
                                cudaStream_t stream) {
    if (!x || !x0 || !cat || T < 0 || E < 1 || (a && a_splits < 1) || (b && b_splits < 1) || !valid_dtype(a_dtype) || !valid_dtype(b_dtype) ||
        !valid_dtype(cat_dtype))
        return fail(PH_ERR_ARG, "concat_restart: bad arguments (T %d, width %d)", T, E);
    const long long total = (long long)T * E;
    if (total == 0) return PH_OK;
    PH_DISPATCH(a_dtype, TA, PH_DISPATCH(b_dtype, TB, PH_DISPATCH(cat_dtype, TO,
        launch_overlapped(concat_restart_kernel<TA, TB, TO>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, (const TA*)a,
                          a_splits, a_stride, (const TB*)b, b_splits, b_stride, x0, start, (TO*)cat, total, E))));
    return check_launch("concat_restart");
}
