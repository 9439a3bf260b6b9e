// Gated activations over rows laid out [g0, u0, g1, u1, ...] (gate and up rows of the weight interleaved, as the
// SwiGLU kernel reads them), with the gate's family as a parameter:
//   kind 0 (silu):           out = g / (1 + exp(-g)) * u
//   kind 1 (clamped swish):  g' = min(g, limit), u' = clamp(u, -limit, limit), out = g' * sigmoid(alpha * g') * (u' + shift)
//   kind 2 (gelu, tanh form): out = 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) * u
// and activations of one argument over plain rows (unary_act): kind 0 silu, kind 1 the square of relu.
// The sums over split-K partial results and the activation are float32.
#include "common.cuh"

namespace {

using namespace ph;

__device__ __forceinline__ float gated(float g, float u, int kind, float alpha, float limit, float shift) {
    if (kind == 0) return g / (1.0f + expf(-g)) * u;
    if (kind == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + shift);
}

template <typename TI, typename TO>
__global__ void glu_kernel(const TI* __restrict__ gu, int splits, long long split_stride, TO* __restrict__ out, int FF,
                           long long total, int kind, float alpha, float limit, float shift) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const TI* g = gu + idx * 2;
    float gv = 0.0f, uv = 0.0f;
    for (int s = 0; s < splits; ++s) {
        gv += to_float<TI>(g[(size_t)s * split_stride]);
        uv += to_float<TI>(g[(size_t)s * split_stride + 1]);
    }
    out[idx] = from_float<TO>(gated(gv, uv, kind, alpha, limit, shift));
}

// four outputs per thread: eight inputs in one or two 16-byte loads per split
template <typename TI, typename TO>
__global__ void glu_vec_kernel(const TI* __restrict__ gu, int splits, long long split_stride, TO* __restrict__ out, long long total4,
                               int kind, float alpha, float limit, float shift) {
    pdl_launch_dependents();
    pdl_wait();
    const long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= total4) return;
    float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    for (int s = 0; s < splits; ++s) {
        float v[8];
        load8(gu + (size_t)s * split_stride + q * 8, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += v[i];
    }
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = gated(acc[2 * i], acc[2 * i + 1], kind, alpha, limit, shift);
    store4(out + q * 4, o);
}

__device__ __forceinline__ float unary(float x, int kind) {
    if (kind == 0) return x / (1.0f + expf(-x));
    x = fmaxf(x, 0.0f);
    return x * x;
}

template <typename TI, typename TO>
__global__ void unary_act_kernel(const TI* __restrict__ in, int splits, long long split_stride, TO* __restrict__ out, long long total,
                                 int kind) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    float x = 0.0f;
    for (int s = 0; s < splits; ++s) x += to_float<TI>(in[(size_t)s * split_stride + idx]);
    out[idx] = from_float<TO>(unary(x, kind));
}

template <typename TI, typename TO>
__global__ void unary_act_vec_kernel(const TI* __restrict__ in, int splits, long long split_stride, TO* __restrict__ out, long long total4,
                                     int kind) {
    pdl_launch_dependents();
    pdl_wait();
    const long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= total4) return;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int s = 0; s < splits; ++s) {
        const float4 v = load4(in + (size_t)s * split_stride + q * 4);
        acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = unary(acc[i], kind);
    store4(out + q * 4, acc);
}

}  // namespace

PH_EXPORT int ph_unary_act(const void* in, int in_dtype, int splits, long long split_stride, void* out, int out_dtype, long long n,
                           int kind, cudaStream_t stream) {
    if (!in || !out || n < 0 || splits < 1 || kind < 0 || kind > 1 || !valid_dtype(in_dtype) || !valid_dtype(out_dtype))
        return fail(PH_ERR_ARG, "unary_act: bad arguments (n %lld, kind %d)", n, kind);
    if (n == 0) return PH_OK;
    if (n % 4 == 0 && split_stride % 4 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
        const long long total4 = n / 4;
        PH_DISPATCH(in_dtype, TI, PH_DISPATCH(out_dtype, TO,
            launch_overlapped(unary_act_vec_kernel<TI, TO>, dim3((unsigned)((total4 + 255) / 256)), dim3(256), 0, stream, (const TI*)in,
                              splits, split_stride, (TO*)out, total4, kind)));
        return check_launch("unary_act");
    }
    PH_DISPATCH(in_dtype, TI, PH_DISPATCH(out_dtype, TO,
        launch_overlapped(unary_act_kernel<TI, TO>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const TI*)in, splits,
                          split_stride, (TO*)out, n, kind)));
    return check_launch("unary_act");
}

PH_EXPORT int ph_glu(const void* gate_up, int in_dtype, int splits, long long split_stride, void* out, int out_dtype, int T,
                     int FF, int kind, float alpha, float limit, float shift, cudaStream_t stream) {
    if (!gate_up || !out || T < 0 || FF < 1 || splits < 1 || kind < 0 || kind > 2 || !valid_dtype(in_dtype) || !valid_dtype(out_dtype))
        return fail(PH_ERR_ARG, "glu: bad arguments (T %d, FF %d, kind %d)", T, FF, kind);
    const long long total = (long long)T * FF;
    if (total == 0) return PH_OK;
    if (FF % 4 == 0 && split_stride % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
        const long long total4 = total / 4;
        PH_DISPATCH(in_dtype, TI, PH_DISPATCH(out_dtype, TO,
            launch_overlapped(glu_vec_kernel<TI, TO>, dim3((unsigned)((total4 + 255) / 256)), dim3(256), 0, stream, (const TI*)gate_up,
                              splits, split_stride, (TO*)out, total4, kind, alpha, limit, shift)));
        return check_launch("glu");
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    PH_DISPATCH(in_dtype, TI, PH_DISPATCH(out_dtype, TO,
        launch_overlapped(glu_kernel<TI, TO>, dim3(blocks), dim3(256), 0, stream, (const TI*)gate_up, splits, split_stride,
                          (TO*)out, FF, total, kind, alpha, limit, shift)));
    return check_launch("glu");
}
