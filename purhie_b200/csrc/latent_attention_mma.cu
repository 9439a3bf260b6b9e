// Attention over cached latent rows on the tensor cores (bfloat16 in, float32 scores, softmax and accumulation).
//
// A cache row is [c | r]: C numbers of latent, R of the rotated key part.  Every head attends over the same rows:
// its key is the whole row, its value the row's first C numbers (latent_attention.cu says why).  So the rows of
// a query tile are (token, head) pairs, heads of one token side by side, and the keys are read once for all heads.
//
//   * latent_attention: one CTA of 8 warps per (64 query rows of one request, split of the keys).  Warp w owns
//     the 16 rows (w & 3) * 16 .. + 15.  For every block of BK keys the two warps of a row group score half of
//     the keys each (Q K^T over C + R, Q read from shared memory), leave the raw scores in shared memory (a barrier of
//     the pair), read back all BK, and run the same online softmax; then each adds P V for its half of the C output columns, which
//     keeps the float32 accumulators at C / 2 columns per warp.
//   * latent_attention_combine merges the splits of a tile in a fixed order.
// Rows are held in shared memory padded to CP and RP columns (zeros), row pitch (CP + RP) * 2 + 16 bytes so that the
// eight rows of an ldmatrix fall into different banks.  Keys outside the visible range of the tile are zero-filled:
// whatever a reused page holds never reaches a product.  The row at position z sees max(0, z - window + 1) .. z.
#include "attention_mma.cuh"

namespace {

using namespace ph;
using namespace ph_attn;

constexpr int LA_ROWS = 64;        // query rows of a tile
constexpr int LA_THREADS = 256;

template <int CP, int RP> struct LatentShape {
    static constexpr int DK = CP + RP;
    static constexpr int PITCH = DK * 2 + 16;                       // bytes from a row to the next
    static constexpr int BK = CP >= 512 ? 32 : 64;                  // keys per block
    static constexpr int S_PITCH = BK + 8;                          // floats
    static constexpr int Q_BYTES = LA_ROWS * PITCH, K_BYTES = BK * PITCH;
    static constexpr int SMEM = Q_BYTES + 2 * K_BYTES + LA_ROWS * S_PITCH * 4;
};

// rows [first, first + n) x (C + R) of `src` (row_stride elements apart, or gathered from pages) into a padded tile
template <int CP, int RP>
__device__ __forceinline__ void fill_row(uint32_t dst, const __nv_bfloat16* src, bool valid, int C, int R, int part, int parts) {
    // chunks of 8 columns: [0, CP / 8) the latent, [CP / 8, (CP + RP) / 8) the rotated part
    constexpr int CH = (CP + RP) / 8;
    for (int ch = part; ch < CH; ch += parts) {
        const bool lat = ch < CP / 8;
        const int col = lat ? ch * 8 : C + (ch - CP / 8) * 8;
        const bool there = valid && (lat ? col < C : col < C + R);
        cp_async16(dst + ch * 16, src + (there ? col : 0), there);
    }
}

template <int CP, int RP>
__global__ void __launch_bounds__(LA_THREADS, 1) latent_attention_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_base, long long page_stride, int page_size,
    const int32_t* __restrict__ block_table, int table_stride, const int32_t* __restrict__ seg_start,
    const int32_t* __restrict__ seg_ctx_len, const int32_t* __restrict__ tile_seg, const int32_t* __restrict__ tile_first,
    float* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int H, int C, int R, int window,
    float scale_log2, int splits) {
    using L = LatentShape<CP, RP>;
    constexpr int BK = L::BK, PITCH = L::PITCH, HALF = CP / 2, NKW = BK / 2;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t q_tile = smem_u32(smem);
    const uint32_t k_tiles = q_tile + L::Q_BYTES;
    float* s_buf = (float*)(smem + L::Q_BYTES + 2 * L::K_BYTES);

    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.y, split = blockIdx.x;
    const int seg = tile_seg[tile], first = tile_first[tile];       // first: the tile's first (token, head) pair of its portion
    const int row0 = seg_start[seg], q_len = seg_start[seg + 1] - row0;
    const int ctx_len = seg_ctx_len[seg];
    const int n_rows = min(LA_ROWS, q_len * H - first);
    const int z_base = ctx_len - q_len;                              // position of the portion's first token
    const int z_first = z_base + first / H, z_last = z_base + (first + n_rows - 1) / H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rg = warp & 3, half = warp >> 2;
    const int DKg = C + R;
    const int32_t* table = block_table + (size_t)seg * table_stride;

    const int lo_tile = first_seen(z_first, window, 0);
    const int kb_first = lo_tile / BK, kb_last = z_last / BK;
    const int per = (kb_last - kb_first + splits) / splits;         // blocks per split, rounded up
    const int kb0 = kb_first + split * per, kb1 = min(kb_last, kb0 + per - 1);

    // this thread's two rows
    const int r0 = rg * 16 + (lane >> 2), r1 = r0 + 8;
    const int z0 = z_base + (first + min(r0, n_rows - 1)) / H, z1 = z_base + (first + min(r1, n_rows - 1)) / H;
    const int lo0 = first_seen(z0, window, 0), lo1 = first_seen(z1, window, 0);
    const int lo_max = first_seen(z_last, window, 0);

    float o[HALF / 8][4];
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
#pragma unroll
    for (int dt = 0; dt < HALF / 8; ++dt)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[dt][i] = 0.0f;

    // four threads fill a row
    auto load_keys = [&](int kb, uint32_t dst) {
        for (int r = threadIdx.x >> 2; r < BK; r += LA_THREADS / 4) {
            const int p = kb * BK + r;
            const bool valid = p >= lo_tile && p <= z_last;
            const __nv_bfloat16* src = k_base;
            if (valid) src += (size_t)table[p / page_size] * page_stride + (size_t)(p % page_size) * DKg;
            fill_row<CP, RP>(dst + r * PITCH, src, valid, C, R, threadIdx.x & 3, 4);
        }
    };

    if (kb0 <= kb1) {
        for (int r = threadIdx.x >> 2; r < LA_ROWS; r += LA_THREADS / 4) {
            const bool valid = r < n_rows;
            fill_row<CP, RP>(q_tile + r * PITCH, q + ((size_t)row0 * H + first + (valid ? r : 0)) * DKg, valid, C, R, threadIdx.x & 3, 4);
        }
        load_keys(kb0, k_tiles);
        cp_async_commit();
    }
    for (int kb = kb0; kb <= kb1; ++kb) {
        const uint32_t k_tile = k_tiles + ((kb - kb0) & 1) * L::K_BYTES;
        cp_async_wait<0>();
        __syncthreads();                                             // block kb is there; everyone is done with block kb - 1
        if (kb < kb1) {
            load_keys(kb + 1, k_tiles + ((kb - kb0 + 1) & 1) * L::K_BYTES);
            cp_async_commit();
        }
        const int key0 = kb * BK;
        const bool rows_here = rg * 16 < n_rows;                     // a row group beyond the tile's rows only helps to load
        if (rows_here) {   // scores of this warp's half of the keys
            // even and odd steps of the contraction add into sums of their own: twice as many independent chains of mma
            float s[NKW / 8][4], s2[NKW / 8][4];
#pragma unroll
            for (int nt = 0; nt < NKW / 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) s[nt][i] = s2[nt][i] = 0.0f;
#pragma unroll 4
            for (int ks = 0; ks < L::DK / 16; ++ks) {
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4(q_tile + (rg * 16 + (lane & 15)) * PITCH + (ks * 2 + (lane >> 4)) * 16, a0, a1, a2, a3);
#pragma unroll
                for (int nt = 0; nt < NKW / 8; nt += 2) {
                    uint32_t b0, b1, b2, b3;
                    const int row = half * NKW + nt * 8 + (lane & 7) + ((lane >> 4) << 3);
                    ldmatrix_x4(k_tile + row * PITCH + (ks * 2 + ((lane >> 3) & 1)) * 16, b0, b1, b2, b3);
                    if (ks & 1) {
                        mma_bf16(s2[nt], a0, a1, a2, a3, b0, b1);
                        mma_bf16(s2[nt + 1], a0, a1, a2, a3, b2, b3);
                    } else {
                        mma_bf16(s[nt], a0, a1, a2, a3, b0, b1);
                        mma_bf16(s[nt + 1], a0, a1, a2, a3, b2, b3);
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < NKW / 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) s[nt][i] += s2[nt][i];
#pragma unroll
            for (int nt = 0; nt < NKW / 8; ++nt) {
                const int col = half * NKW + nt * 8 + (lane & 3) * 2;
                *(float2*)(s_buf + r0 * L::S_PITCH + col) = make_float2(s[nt][0], s[nt][1]);
                *(float2*)(s_buf + r1 * L::S_PITCH + col) = make_float2(s[nt][2], s[nt][3]);
            }
        }
        if (!rows_here) continue;
        // only the two warps of a row group exchange scores: a barrier of their 64 threads (ids 1 .. 4; 0 is the CTA's)
        asm volatile("bar.sync %0, 64;" ::"r"(1 + rg) : "memory");
        float p[BK / 8][4];
#pragma unroll
        for (int nt = 0; nt < BK / 8; ++nt) {
            const int col = nt * 8 + (lane & 3) * 2;
            const float2 u = *(const float2*)(s_buf + r0 * L::S_PITCH + col), v = *(const float2*)(s_buf + r1 * L::S_PITCH + col);
            p[nt][0] = u.x; p[nt][1] = u.y; p[nt][2] = v.x; p[nt][3] = v.y;
        }
        const bool need_mask = key0 + BK - 1 > z_first || key0 < lo_max;
        softmax_update<HALF, BK>(p, key0, z0, z1, lo0, lo1, need_mask, scale_log2, m, l, o);
        // O[16 x HALF] += P[16 x BK] V[BK x HALF], V the columns half * HALF .. of the key rows
#pragma unroll
        for (int j = 0; j < BK / 16; ++j) {
            const uint32_t a0 = pack_bf16(p[2 * j][0], p[2 * j][1]), a1 = pack_bf16(p[2 * j][2], p[2 * j][3]);
            const uint32_t a2 = pack_bf16(p[2 * j + 1][0], p[2 * j + 1][1]), a3 = pack_bf16(p[2 * j + 1][2], p[2 * j + 1][3]);
            const int row = j * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
            for (int dt = 0; dt < HALF / 8; dt += 2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(k_tile + row * PITCH + (half * (HALF / 8) + dt + (lane >> 4)) * 16, b0, b1, b2, b3);
                mma_bf16(o[dt], a0, a1, a2, a3, b0, b1);
                mma_bf16(o[dt + 1], a0, a1, a2, a3, b2, b3);
            }
        }
    }
    const size_t out_row0 = (size_t)row0 * H + first;
    if (splits == 1) {
        const float inv0 = l[0] == 0.0f ? 0.0f : 1.0f / l[0], inv1 = l[1] == 0.0f ? 0.0f : 1.0f / l[1];
#pragma unroll
        for (int dt = 0; dt < HALF / 8; ++dt) {
            const int d = half * HALF + dt * 8 + (lane & 3) * 2;
            if (d >= C) continue;
            if (r0 < n_rows) *(float2*)(out + (out_row0 + r0) * C + d) = make_float2(o[dt][0] * inv0, o[dt][1] * inv0);
            if (r1 < n_rows) *(float2*)(out + (out_row0 + r1) * C + d) = make_float2(o[dt][2] * inv1, o[dt][3] * inv1);
        }
        return;
    }
    // a split leaves (maximum, sum) and the unnormalised sums per row
    const size_t part = ((size_t)tile * splits + split) * LA_ROWS;
    if (half == 0 && (lane & 3) == 0) {
        if (r0 < n_rows) *(float2*)(part_ml + (part + r0) * 2) = make_float2(m[0], l[0]);
        if (r1 < n_rows) *(float2*)(part_ml + (part + r1) * 2) = make_float2(m[1], l[1]);
    }
#pragma unroll
    for (int dt = 0; dt < HALF / 8; ++dt) {
        const int d = half * HALF + dt * 8 + (lane & 3) * 2;
        if (d >= C) continue;
        if (r0 < n_rows) *(float2*)(part_o + (part + r0) * C + d) = make_float2(o[dt][0], o[dt][1]);
        if (r1 < n_rows) *(float2*)(part_o + (part + r1) * C + d) = make_float2(o[dt][2], o[dt][3]);
    }
}

// out[row] = sum over the splits s, in order, of 2^(m_s - M) o_s, over sum_s 2^(m_s - M) l_s, M the largest m_s.
__global__ void latent_attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                const int32_t* __restrict__ seg_start, const int32_t* __restrict__ tile_seg,
                                                const int32_t* __restrict__ tile_first, float* __restrict__ out, int H, int C, int splits) {
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.y, r = blockIdx.x;
    const int seg = tile_seg[tile], first = tile_first[tile];
    const int row0 = seg_start[seg], q_len = seg_start[seg + 1] - row0;
    if (r >= q_len * H - first) return;
    const size_t part = (size_t)tile * splits * LA_ROWS + r;
    float top = -INFINITY;
    for (int s = 0; s < splits; ++s) top = fmaxf(top, part_ml[(part + (size_t)s * LA_ROWS) * 2]);
    float sum = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float* ml = part_ml + (part + (size_t)s * LA_ROWS) * 2;
        if (ml[1] > 0.0f) sum += exp2f(ml[0] - top) * ml[1];
    }
    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
    float* dst = out + ((size_t)row0 * H + first + r) * C;
    for (int d = threadIdx.x; d < C; d += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float* ml = part_ml + (part + (size_t)s * LA_ROWS) * 2;
            if (ml[1] > 0.0f) acc += exp2f(ml[0] - top) * part_o[(part + (size_t)s * LA_ROWS) * C + d];
        }
        dst[d] = acc * inv;
    }
}

template <int CP, int RP>
cudaError_t launch_latent(dim3 grid, cudaStream_t stream, const __nv_bfloat16* q, const __nv_bfloat16* k_base, long long page_stride,
                          int page_size, const int32_t* block_table, int table_stride, const int32_t* seg_start,
                          const int32_t* seg_ctx_len, const int32_t* tile_seg, const int32_t* tile_first, float* out, float* part_o,
                          float* part_ml, int H, int C, int R, int window, float scale_log2, int splits) {
    constexpr int SMEM = LatentShape<CP, RP>::SMEM;
    static_assert(SMEM <= 227 * 1024, "the tiles do not fit in shared memory");
    static bool set = false;        // per instantiation
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<CP, RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return e;
        set = true;
    }
    return launch_overlapped(latent_attention_kernel<CP, RP>, grid, dim3(LA_THREADS), (size_t)SMEM, stream, q, k_base, page_stride, page_size,
                             block_table, table_stride, seg_start, seg_ctx_len, tile_seg, tile_first, out, part_o, part_ml, H, C, R, window,
                             scale_log2, splits);
}

// ---- the products per head around the attention ---------------------------------------------------------------------
// out[t, h, n] = sum_k a[t, h, k] * B_h[k, n] for every head h, on the tensor cores with float32 sums:
//   absorb (KN = true):   a = q [T, H, lda] (the first K = D of each head's row), B_h = wuk[h * K + k, n] (n contiguous),
//                         out = q_lat [T, H, ldo] bfloat16; the CTAs of the first column tile also rotate the R numbers
//                         behind the first K into the R numbers behind the first N of the output row;
//   expand (KN = false):  a = o_lat [T, H, K] float32, B_h = wuv[h * N + n, k] (k contiguous), out [T, H * N] bfloat16,
//                         times sigmoid(gate[t, h]).
// One CTA of four warps per (64 columns, head, 64 tokens); K in steps of 32 through shared memory.
constexpr int HG_BM = 64, HG_BN = 64, HG_BK = 32, HG_THREADS = 128;
constexpr int HG_PITCH_K = HG_BK * 2 + 16;      // bytes of a row of 32 k (A tiles, and B tiles stored n by k)
constexpr int HG_PITCH_N = HG_BN * 2 + 16;      // bytes of a row of 64 n (B tiles stored k by n)

// Eight elements from src, of which the first `left` exist (the rest are zero), as bfloat16 to shared memory; `vec`: src is
// 16-byte aligned (32 for float32) whenever all eight exist.
template <typename T> __device__ __forceinline__ void stage8(uint8_t* dst, const T* src, int left, bool vec) {
    float v[8];
    if (left >= 8 && vec) {
        load8(src, v);
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = j < left ? to_float<T>(src[j]) : 0.0f;
    }
    store8((__nv_bfloat16*)dst, v);
}

template <bool KN, typename TA>
__global__ void __launch_bounds__(HG_THREADS) head_product_kernel(
    const TA* __restrict__ a, long long lda, const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ out, long long ldo, int T,
    int H, int K, int N, const __nv_bfloat16* __restrict__ gate, long long gate_stride, int R, const float* __restrict__ cos_sin,
    int n_rot, int max_pos, const int32_t* __restrict__ positions) {
    __shared__ __align__(16) uint8_t a_s[HG_BM * HG_PITCH_K];
    __shared__ __align__(16) uint8_t b_s[KN ? HG_BK * HG_PITCH_N : HG_BN * HG_PITCH_K];
    pdl_launch_dependents();
    pdl_wait();
    const int n0 = blockIdx.x * HG_BN, h = blockIdx.y, t0 = blockIdx.z * HG_BM;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t a_tile = smem_u32(a_s), b_tile = smem_u32(b_s);
    const bool vec_a = lda % 8 == 0 && reinterpret_cast<uintptr_t>(a) % 32 == 0;
    const bool vec_b = (KN ? N : K) % 8 == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0;
    float acc[HG_BN / 8][4];
#pragma unroll
    for (int nt = 0; nt < HG_BN / 8; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += HG_BK) {
        // A: 64 tokens x 32 k, eight k at a time
        for (int i = threadIdx.x; i < HG_BM * (HG_BK / 8); i += HG_THREADS) {
            const int r = i / (HG_BK / 8), k = (i % (HG_BK / 8)) * 8;
            const TA* src = a + ((size_t)(t0 + r) * H + h) * lda + k0 + k;
            stage8<TA>(a_s + r * HG_PITCH_K + k * 2, src, t0 + r < T ? K - k0 - k : 0, vec_a);
        }
        if (KN) {       // B: 32 k x 64 n, n contiguous in memory
            for (int i = threadIdx.x; i < HG_BK * (HG_BN / 8); i += HG_THREADS) {
                const int k = i / (HG_BN / 8), n = (i % (HG_BN / 8)) * 8;
                stage8<__nv_bfloat16>(b_s + k * HG_PITCH_N + n * 2, b + ((size_t)h * K + k0 + k) * N + n0 + n, k0 + k < K ? N - n0 - n : 0, vec_b);
            }
        } else {        // B: 64 n x 32 k, k contiguous in memory
            for (int i = threadIdx.x; i < HG_BN * (HG_BK / 8); i += HG_THREADS) {
                const int n = i / (HG_BK / 8), k = (i % (HG_BK / 8)) * 8;
                stage8<__nv_bfloat16>(b_s + n * HG_PITCH_K + k * 2, b + ((size_t)h * N + n0 + n) * K + k0 + k, n0 + n < N ? K - k0 - k : 0, vec_b);
            }
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < HG_BK / 16; ++ks) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(a_tile + (warp * 16 + (lane & 15)) * HG_PITCH_K + (ks * 2 + (lane >> 4)) * 16, a0, a1, a2, a3);
#pragma unroll
            for (int nt = 0; nt < HG_BN / 8; nt += 2) {
                uint32_t b0, b1, b2, b3;
                if (KN) {
                    const int row = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                    ldmatrix_x4_trans(b_tile + row * HG_PITCH_N + (nt + (lane >> 4)) * 16, b0, b1, b2, b3);
                } else {
                    const int row = nt * 8 + (lane & 7) + ((lane >> 4) << 3);
                    ldmatrix_x4(b_tile + row * HG_PITCH_K + (ks * 2 + ((lane >> 3) & 1)) * 16, b0, b1, b2, b3);
                }
                mma_bf16(acc[nt], a0, a1, a2, a3, b0, b1);
                mma_bf16(acc[nt + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();
    }
    const int r0 = t0 + warp * 16 + (lane >> 2), r1 = r0 + 8;
    float g0 = 1.0f, g1 = 1.0f;
    if (gate) {
        if (r0 < T) g0 = 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)r0 * gate_stride + h])));
        if (r1 < T) g1 = 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)r1 * gate_stride + h])));
    }
    const bool pairs = N % 2 == 0 && ldo % 2 == 0;      // two neighbours are one 4-byte store
#pragma unroll
    for (int nt = 0; nt < HG_BN / 8; ++nt) {
        const int n = n0 + nt * 8 + (lane & 3) * 2;
#pragma unroll
        for (int half_row = 0; half_row < 2; ++half_row) {
            const int r = half_row ? r1 : r0;
            const float g = half_row ? g1 : g0, u = acc[nt][half_row * 2] * g, v = acc[nt][half_row * 2 + 1] * g;
            if (r >= T || n >= N) continue;
            __nv_bfloat16* dst = out + ((size_t)r * H + h) * ldo + n;
            if (pairs) *(uint32_t*)dst = pack_bf16(u, v);
            else {
                dst[0] = __float2bfloat16_rn(u);
                if (n + 1 < N) dst[1] = __float2bfloat16_rn(v);
            }
        }
    }
    if (!KN || R == 0 || blockIdx.x != 0) return;
    // the rotated part of the query: the R numbers behind the K plain ones, turned over their first n_rot in half pairs
    const int half = n_rot / 2;
    for (int i = threadIdx.x; i < HG_BM * R; i += HG_THREADS) {
        const int t = t0 + i / R, d = i % R;
        if (t >= T) continue;
        const TA* r = a + ((size_t)t * H + h) * lda + K;
        float v = to_float<TA>(r[d]);
        if (d < n_rot) {
            int pos = positions[t];
            pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
            const float* cs = cos_sin + (size_t)pos * n_rot;
            if (d < half) v = v * cs[d] - to_float<TA>(r[d + half]) * cs[half + d];
            else v = v * cs[d - half] + to_float<TA>(r[d - half]) * cs[d];
        }
        out[((size_t)t * H + h) * ldo + N + d] = __float2bfloat16_rn(v);
    }
}

}  // namespace

PH_DEFINE_LAST_ERROR(ph_latent)

// q [T, H, D + R] bfloat16, wuk [H * D, C] bfloat16 -> q_lat [T, H, C + R] bfloat16 = [Wuk_h^T q_plain | rotate(q_rot)]
// (latent_absorb of latent_attention.cu on the tensor cores).
PH_EXPORT int ph_latent_absorb_mma(const void* q, const void* wuk, const float* cos_sin, int n_rot, int max_pos, const int32_t* positions,
                                   void* q_lat, int T, int H, int D, int R, int C, cudaStream_t stream) {
    if (!q || !wuk || !q_lat || T < 0 || H < 1 || D < 1 || R < 0 || C < 1 || n_rot < 0 || n_rot > R || n_rot % 2 ||
        (n_rot && (!cos_sin || !positions)))
        return fail(PH_ERR_ARG, "latent_absorb_mma: bad arguments (T %d, H %d, D %d + %d, C %d)", T, H, D, R, C);
    if (T == 0) return PH_OK;
    const dim3 grid((unsigned)((C + HG_BN - 1) / HG_BN), (unsigned)H, (unsigned)((T + HG_BM - 1) / HG_BM));
    cudaError_t e = launch_overlapped(head_product_kernel<true, __nv_bfloat16>, grid, dim3(HG_THREADS), 0, stream, (const __nv_bfloat16*)q,
                                      (long long)(D + R), (const __nv_bfloat16*)wuk, (__nv_bfloat16*)q_lat, (long long)(C + R), T, H, D, C,
                                      (const __nv_bfloat16*)nullptr, 0LL, R, cos_sin, n_rot, max_pos, positions);
    if (e != cudaSuccess) return fail(PH_ERR_LAUNCH, "latent_absorb_mma: %s", cudaGetErrorString(e));
    return check_launch("latent_absorb_mma");
}

// o_lat [T, H, C] float32, wuv [H * DV, C] bfloat16, gate [T, gate_stride] bfloat16 (head h's logit at column h; null: none)
// -> out [T, H * DV] bfloat16 = (Wuv_h o_lat[t, h]) * sigmoid(gate[t, h]) (latent_expand on the tensor cores).
PH_EXPORT int ph_latent_expand_mma(const void* o_lat, const void* wuv, const void* gate, long long gate_stride, void* out, int T, int H,
                                   int C, int DV, cudaStream_t stream) {
    if (!o_lat || !wuv || !out || T < 0 || H < 1 || C < 1 || DV < 1)
        return fail(PH_ERR_ARG, "latent_expand_mma: bad arguments (T %d, H %d, C %d, DV %d)", T, H, C, DV);
    if (T == 0) return PH_OK;
    const dim3 grid((unsigned)((DV + HG_BN - 1) / HG_BN), (unsigned)H, (unsigned)((T + HG_BM - 1) / HG_BM));
    cudaError_t e = launch_overlapped(head_product_kernel<false, float>, grid, dim3(HG_THREADS), 0, stream, (const float*)o_lat, (long long)C,
                                      (const __nv_bfloat16*)wuv, (__nv_bfloat16*)out, (long long)DV, T, H, C, DV,
                                      (const __nv_bfloat16*)gate, gate_stride, 0, (const float*)nullptr, 0, 0, (const int32_t*)nullptr);
    if (e != cudaSuccess) return fail(PH_ERR_LAUNCH, "latent_expand_mma: %s", cudaGetErrorString(e));
    return check_launch("latent_expand_mma");
}


// 1 when the kernel takes a cache row of C + R numbers, else 0
PH_EXPORT int ph_latent_attention_supports(int C, int R) {
    return C >= 8 && C <= 512 && R >= 0 && R <= 64 && C % 8 == 0 && R % 8 == 0;
}

// q [T, H, C + R] bfloat16 (the queries in latent form), cache rows [C + R] bfloat16 in pages -> out [T, H, C] float32, the
// softmax-weighted sums of the rows' first C numbers.  tile_seg / tile_first [n_tiles]: segment and first (token, head) pair
// (counted within the segment's portion, heads fastest) of each tile of 64 pairs.  splits > 1: part_o [n_tiles, splits, 64, C]
// and part_ml [n_tiles, splits, 64, 2] float32 hold the partial results, merged by a second kernel.
PH_EXPORT int ph_latent_attention(const void* q, const void* k_base, long long page_stride, int page_size, const int32_t* block_table,
                                  int table_stride, const int32_t* seg_start, const int32_t* seg_ctx_len, const int32_t* tile_seg,
                                  const int32_t* tile_first, int n_tiles, void* out, float* part_o, float* part_ml, int H, int C, int R,
                                  int window, float scale, int splits, cudaStream_t stream) {
    if (!q || !k_base || !block_table || !seg_start || !seg_ctx_len || !tile_seg || !tile_first || !out || n_tiles < 0 || H < 1 ||
        page_size < 1 || window < 0 || splits < 1 || (splits > 1 && (!part_o || !part_ml)))
        return fail(PH_ERR_ARG, "latent_attention: bad arguments (tiles %d, H %d, splits %d)", n_tiles, H, splits);
    if (!ph_latent_attention_supports(C, R))
        return fail(PH_ERR_UNSUPPORTED, "latent_attention: rows of %d + %d numbers are not taken (multiples of 8, at most 512 + 64)", C, R);
    if (n_tiles > 65535) return fail(PH_ERR_UNSUPPORTED, "latent_attention: %d tiles exceed the grid", n_tiles);
    if (n_tiles == 0) return PH_OK;
    const float scale_log2 = scale * LOG2E;
    const dim3 grid((unsigned)splits, (unsigned)n_tiles);
    cudaError_t e;
#define LAUNCH(CP, RP)                                                                                                                   \
    e = launch_latent<CP, RP>(grid, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_base, page_stride, page_size, block_table,   \
                              table_stride, seg_start, seg_ctx_len, tile_seg, tile_first, (float*)out, part_o, part_ml, H, C, R, window, \
                              scale_log2, splits)
    if (C <= 128) { if (R <= 16) LAUNCH(128, 16); else LAUNCH(128, 64); }
    else if (C <= 256) { if (R <= 16) LAUNCH(256, 16); else LAUNCH(256, 64); }
    else { if (R <= 16) LAUNCH(512, 16); else LAUNCH(512, 64); }
#undef LAUNCH
    if (e != cudaSuccess) return fail(PH_ERR_LAUNCH, "latent_attention: %s", cudaGetErrorString(e));
    if (splits > 1) {
        e = launch_overlapped(latent_attention_combine_kernel, dim3(LA_ROWS, (unsigned)n_tiles), dim3(128), 0, stream, (const float*)part_o,
                              (const float*)part_ml, seg_start, tile_seg, tile_first, (float*)out, H, C, splits);
        if (e != cudaSuccess) return fail(PH_ERR_LAUNCH, "latent_attention_combine: %s", cudaGetErrorString(e));
    }
    return check_launch("latent_attention");
}
