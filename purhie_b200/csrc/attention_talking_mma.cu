// Attention whose heads talk to each other before the softmax, on the tensor cores (bfloat16 in, float32 scores, cap,
// bias, mix, softmax and sums): the many-row and the few-row form of attention_talking (attention_talking.cu states the
// equations).  It also serves attention that only has a sink, or only a gate: every extra is optional.
//
// One CTA per tile of 16 query rows of one request (a decode row is a tile of one row) and ALL heads, a warp per head:
// every head's score at a (row, key) pair enters every head's softmax, so the heads of a tile must meet.  Keys are walked
// in blocks of 32 from the first one the tile sees to its last row's position.  Per block the CTA gathers the keys and
// values of all kv heads from the pages into shared memory (16-byte cp.async, rows outside the visible range zero-filled,
// so whatever an unwritten or reused page holds never reaches a product); warp h computes S_h = Q_h K_kv(h)^T with
// mma.sync.m16n8k16, scales, caps and biases it in float32 and leaves it in shared memory; after a barrier it reads all
// heads' scores at its own (row, key) places and mixes them with its row of the talk matrix; then the online softmax
// (running maximum and sum per row) and O_h += P_h V_kv(h) on the tensor cores with P rounded to bfloat16, as in the
// other tensor-core attention kernels.  The sink joins the denominator at the end; the gate multiplies the output.
// Q tiles of all heads pass through the shared memory that the keys use afterwards.
// More than 16 heads (up to 32): a cluster of two CTAs takes a tile, each CTA half of the heads with their kv heads; a
// warp writes its head's scores into its own CTA's shared memory and into the partner's (distributed shared memory: 2 KB
// cross per warp and block, where reading the partner's half from there would be 32 KB), and the two barriers of a block
// become barriers of the cluster.  Both CTAs walk the same key blocks, so they meet the same barriers.
#include "attention_mma.cuh"

#include <cooperative_groups.h>

namespace {

using namespace ph;
using namespace ph_attn;

constexpr int BM = 16;            // query rows of a tile
constexpr int BK = 32;            // keys of a block
constexpr int SP = 40;            // floats between two rows of the exchanged scores (8-byte accesses miss each other's banks)
constexpr int BIAS_N = 48;        // distances row - key + 31 of a block: 0 .. 46
constexpr int MAX_HEADS = 16;      // a warp per head, and a thread keeps its head's Q and O in registers

struct TalkParams {
    const __nv_bfloat16* q; const __nv_bfloat16* k_base; const __nv_bfloat16* v_base;
    long long page_stride; int page_size;
    int page_shift;               // log2(page_size) when it is a power of two, else -1
    const int32_t* block_table; int table_stride;
    const int32_t* seg_start; const int32_t* seg_ctx_len; const int32_t* tile_seg; const int32_t* tile_first;
    __nv_bfloat16* out;
    int HQ, HKV, window, chunk;
    float scale, cap;
    const float* r1; const float* r2; const float* talk; const float* sink;
    const __nv_bfloat16* gate; long long gate_stride;
    int kv_bytes;                 // bytes of the region that holds Q first and the blocks of K and V afterwards
    int pair;                     // 1: a cluster of two CTAs per tile, each with half of the heads
    int stages;                   // 1 or 2 blocks of keys and values in shared memory
    int splits;                   // CTAs that share a tile's keys (blockIdx.y); above 1 they leave partial results
    float* part_o;                // [T][HQ][splits][DV] float32, unnormalised
    float* part_ml;               // [T][HQ][splits][2]: the exponent's reference (log2 domain) and the sum
};

// tanh from the hardware's exponential: a few float32 operations with an error near 1e-6, far below what the bfloat16
// weights of the softmax keep
__device__ __forceinline__ float fast_tanh(float x) {
    const float e = __expf(-2.0f * fabsf(x));
    return copysignf(__fdividef(1.0f - e, 1.0f + e), x);
}

template <int D, int DV>
__global__ void __launch_bounds__(MAX_HEADS * 32) attention_talking_mma_kernel(const TalkParams p) {
    constexpr int KP = D * 2 + 16, VP = DV * 2 + 16;          // bytes between two rows of a K (Q) and of a V tile
    extern __shared__ __align__(128) uint8_t smem[];
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = p.pair ? (int)cluster.block_rank() : 0;
    const int HA = p.HQ;                                      // all heads: what a score is mixed over, and the output's stride
    const int HQ = p.pair ? p.HQ / 2 : p.HQ, HKV = p.pair ? p.HKV / 2 : p.HKV;      // this CTA's heads and kv heads
    const int h0 = rank * HQ, kv0 = rank * HKV;               // the first of them
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, threads = blockDim.x;
    const int h = warp, g = h / (HQ / HKV);                   // within this CTA
    const uint32_t region = smem_u32(smem);
    float* sc = reinterpret_cast<float*>(smem + p.kv_bytes);  // [HA][BM][SP]: all heads' scores, the partner's half written by the partner
    float* tk = sc + (size_t)HA * BM * SP;                    // [HQ][HA]: this CTA's rows of the mix
    float* bias = tk + (size_t)HQ * HA + (size_t)h * BIAS_N;  // this head's distance bias for the block's 47 distances
    float* sc_other = p.pair ? cluster.map_shared_rank(sc, rank ^ 1) : nullptr;      // the same array in the partner's shared memory

    const int tile = p.pair ? blockIdx.x / 2 : blockIdx.x;
    const int seg = p.tile_seg[tile], first = p.tile_first[tile];
    const int row0 = p.seg_start[seg], q_len = p.seg_start[seg + 1] - row0;
    const int ctx_len = p.seg_ctx_len[seg];
    const int n_rows = min(BM, q_len - first);
    const int z_first = ctx_len - q_len + first, z_last = z_first + n_rows - 1;
    const int32_t* table = p.block_table + (size_t)seg * p.table_stride;

    // Q of all heads: [HQ][BM] rows of D; rows beyond the portion are zero
    {
        constexpr int CPR = D / 8;
        for (int i = threadIdx.x; i < HQ * BM * CPR; i += threads) {
            const int c = i % CPR, r = (i / CPR) % BM, hh = i / (CPR * BM);
            const bool valid = r < n_rows;
            const __nv_bfloat16* src = p.q + ((size_t)(row0 + first + (valid ? r : 0)) * HA + h0 + hh) * D + c * 8;
            cp_async16(region + (uint32_t)((hh * BM + r) * KP + c * 16), src, valid);
        }
        cp_async_commit();
    }
    if (p.talk)
        for (int i = threadIdx.x; i < HQ * HA; i += threads) tk[i] = p.talk[(size_t)h0 * HA + i];
    cp_async_wait<0>();
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
        ldmatrix_x4(region + (uint32_t)((h * BM + (lane & 15)) * KP + (ks * 2 + (lane >> 4)) * 16), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    __syncthreads();                                          // everybody holds its Q: the region is free for keys

    const int r0 = lane >> 2, r1 = r0 + 8;
    const int z0 = z_first + min(r0, n_rows - 1), z1 = z_first + min(r1, n_rows - 1);
    const int lo0 = first_seen(z0, p.window, p.chunk), lo1 = first_seen(z1, p.window, p.chunk);
    const int lo_tile = first_seen(z_first, p.window, p.chunk), lo_last = first_seen(z_last, p.window, p.chunk);
    const float b1 = p.r1 ? p.r1[h0 + h] : 0.0f, b2 = p.r2 ? p.r2[h0 + h] : 0.0f;

    float o[DV / 8][4];
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
#pragma unroll
    for (int dt = 0; dt < DV / 8; ++dt)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[dt][i] = 0.0f;

    // this CTA's share of the tile's key blocks
    int kb_first = lo_tile / BK, kb_last = z_last / BK;
    if (p.splits > 1) {
        const int per = (kb_last - kb_first + p.splits) / p.splits;
        kb_first += (int)blockIdx.y * per;
        kb_last = min(kb_last, kb_first + per - 1);
    }
    const bool upper = n_rows > 8;                            // rows 8 .. 15 of the tile exist
    // the keys and values of every kv head for the block that starts at key0, into one of the stages
    const uint32_t stage_bytes = (uint32_t)(HKV * BK * (KP + VP));
    auto load_block = [&](int key0, int stage) {
        constexpr int KC = D / 8, VC = DV / 8;
        const uint32_t kt = region + stage * stage_bytes, vt = kt + (uint32_t)(HKV * BK * KP);
        for (int i = threadIdx.x; i < HKV * BK * (KC + VC); i += threads) {
            const int c = i % (KC + VC), r = (i / (KC + VC)) % BK, gg = i / ((KC + VC) * BK);
            const int pos = key0 + r;
            const bool valid = pos >= lo_tile && pos <= z_last;
            size_t page_at = 0, slot = 0;
            if (valid) {
                const int page = p.page_shift >= 0 ? pos >> p.page_shift : pos / p.page_size;
                page_at = (size_t)table[page] * p.page_stride;
                slot = (size_t)(kv0 + gg) * p.page_size + (pos - page * p.page_size);
            }
            if (c < KC) cp_async16(kt + (uint32_t)((gg * BK + r) * KP + c * 16), p.k_base + page_at + slot * D + c * 8, valid);
            else cp_async16(vt + (uint32_t)((gg * BK + r) * VP + (c - KC) * 16), p.v_base + page_at + slot * DV + (c - KC) * 8, valid);
        }
        cp_async_commit();
    };
    // two stages: the next block is on its way while this one is worked on; one stage where shared memory has no room for two
    if (p.stages == 2 && kb_first <= kb_last) load_block(kb_first * BK, 0);
    for (int kb = kb_first; kb <= kb_last; ++kb) {
        const int key0 = kb * BK;
        int stage = 0;
        if (p.stages == 2) {
            stage = (kb - kb_first) & 1;
            if (kb < kb_last) { load_block(key0 + BK, stage ^ 1); cp_async_wait<1>(); }
            else cp_async_wait<0>();
        } else {
            load_block(key0, 0);
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t k_tiles = region + stage * stage_bytes, v_tiles = k_tiles + (uint32_t)(HKV * BK * KP);
        if (p.r1) {
            // the bias depends on the distance alone: row - key takes 47 values in a block, a lane makes two of them
            __syncwarp();
            for (int idx = lane; idx < BIAS_N - 1; idx += 32) bias[idx] = b1 * log1pf(b2 * (float)max(z_first - key0 + idx - (BK - 1), 0));
            __syncwarp();
        }
        float s[BK / 8][4];
        warp_qk<D, BK, true>(qf, k_tiles + (uint32_t)(g * BK * KP), 0, s);
        const float inv_cap = p.cap > 0.0f ? 1.0f / p.cap : 0.0f;
#pragma unroll
        for (int nt = 0; nt < BK / 8; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (i >= 2 && !upper) continue;              // a tile of few rows (a decode row) skips the copies of its last row
                float v = s[nt][i] * p.scale;
                if (p.cap > 0.0f) v = p.cap * fast_tanh(v * inv_cap);
                if (p.r1) v -= bias[(i < 2 ? r0 : r1) - (nt * 8 + (lane & 3) * 2 + (i & 1)) + (BK - 1)];
                s[nt][i] = v;
            }
        if (p.talk) {
#pragma unroll
            for (int nt = 0; nt < BK / 8; ++nt) {
                const int c = nt * 8 + (lane & 3) * 2;
                *reinterpret_cast<float2*>(sc + ((size_t)(h0 + h) * BM + r0) * SP + c) = make_float2(s[nt][0], s[nt][1]);
                *reinterpret_cast<float2*>(sc + ((size_t)(h0 + h) * BM + r1) * SP + c) = make_float2(s[nt][2], s[nt][3]);
                if (sc_other) {
                    *reinterpret_cast<float2*>(sc_other + ((size_t)(h0 + h) * BM + r0) * SP + c) = make_float2(s[nt][0], s[nt][1]);
                    if (upper) *reinterpret_cast<float2*>(sc_other + ((size_t)(h0 + h) * BM + r1) * SP + c) = make_float2(s[nt][2], s[nt][3]);
                }
            }
            if (p.pair) cluster.sync(); else __syncthreads();
            // the mix in packed pairs: a thread's two neighbouring columns are one 64-bit accumulator
            unsigned long long acc[BK / 8][2];
#pragma unroll
            for (int nt = 0; nt < BK / 8; ++nt) acc[nt][0] = acc[nt][1] = 0ull;
#pragma unroll 4
            for (int j = 0; j < HA; ++j) {                    // over all heads, in the order of the heads whichever CTA holds them
                unsigned long long ww;
                asm("mov.b64 %0, {%1, %1};" : "=l"(ww) : "f"(tk[h * HA + j]));
                const float* from = sc + (size_t)j * BM * SP;
#pragma unroll
                for (int nt = 0; nt < BK / 8; ++nt) {
                    const int c = nt * 8 + (lane & 3) * 2;
                    const unsigned long long a = *reinterpret_cast<const unsigned long long*>(from + (size_t)r0 * SP + c);
                    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc[nt][0]) : "l"(ww), "l"(a));
                    if (upper) {
                        const unsigned long long b = *reinterpret_cast<const unsigned long long*>(from + (size_t)r1 * SP + c);
                        asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc[nt][1]) : "l"(ww), "l"(b));
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < BK / 8; ++nt) {
                asm("mov.b64 {%0, %1}, %2;" : "=f"(s[nt][0]), "=f"(s[nt][1]) : "l"(acc[nt][0]));
                asm("mov.b64 {%0, %1}, %2;" : "=f"(s[nt][2]), "=f"(s[nt][3]) : "l"(acc[nt][1]));
            }
        }
        // masks only where the block touches the diagonal or the window's edge of one of the tile's rows
        const bool need_mask = key0 + BK - 1 > z_first || key0 < lo_last;
        softmax_update<DV, BK>(s, key0, z0, z1, lo0, lo1, need_mask, LOG2E, m, l, o);
        warp_pv<DV, BK, true>(s, v_tiles + (uint32_t)(g * BK * VP), 0, o);
        // scores and tiles are read (the scores by the partner too) before the next block overwrites them
        if (p.pair && p.talk) cluster.sync(); else __syncthreads();
    }
    if (p.splits > 1) {
        // (reference, sum, unnormalised output) of this CTA's keys; the merge adds the sink and the gate
        const int T_HQ = HA;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int r = k ? r1 : r0;
            if (r >= n_rows) continue;
            const size_t slot = ((size_t)(row0 + first + r) * T_HQ + h0 + h) * p.splits + blockIdx.y;
            if ((lane & 3) == 0) { p.part_ml[slot * 2] = m[k]; p.part_ml[slot * 2 + 1] = l[k]; }
#pragma unroll
            for (int dt = 0; dt < DV / 8; ++dt) {
                const int d = dt * 8 + (lane & 3) * 2;
                *reinterpret_cast<float2*>(p.part_o + slot * DV + d) = make_float2(o[dt][2 * k], o[dt][2 * k + 1]);
            }
        }
        return;
    }
    if (p.sink) {
        const float sk = p.sink[h0 + h] * LOG2E;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float top = fmaxf(m[k], sk), corr = exp2f(m[k] - top);      // m = -inf cannot happen: a row sees itself
            l[k] = l[k] * corr + exp2f(sk - top);
#pragma unroll
            for (int dt = 0; dt < DV / 8; ++dt) { o[dt][2 * k] *= corr; o[dt][2 * k + 1] *= corr; }
        }
    }
    const float inv0 = l[0] == 0.0f ? 0.0f : 1.0f / l[0], inv1 = l[1] == 0.0f ? 0.0f : 1.0f / l[1];
    const size_t width = (size_t)HA * DV;
#pragma unroll
    for (int dt = 0; dt < DV / 8; ++dt) {
        const int d = dt * 8 + (lane & 3) * 2;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int r = k ? r1 : r0;
            if (r >= n_rows) continue;
            const size_t row = (size_t)(row0 + first + r);
            float a = o[dt][2 * k] * (k ? inv1 : inv0), b = o[dt][2 * k + 1] * (k ? inv1 : inv0);
            if (p.gate) {
                const __nv_bfloat162 gg = *reinterpret_cast<const __nv_bfloat162*>(p.gate + row * p.gate_stride + (size_t)(h0 + h) * DV + d);
                a *= 1.0f / (1.0f + expf(-__low2float(gg)));
                b *= 1.0f / (1.0f + expf(-__high2float(gg)));
            }
            *(uint32_t*)(p.out + row * width + (size_t)(h0 + h) * DV + d) = pack_bf16(a, b);
        }
    }
}

// One block per (row, head): the partial results of the key splits merged in ascending order, then the sink and the gate.
__global__ void attention_talking_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits,
                                               const float* __restrict__ sink, const __nv_bfloat16* __restrict__ gate, long long gate_stride,
                                               __nv_bfloat16* __restrict__ out, int HQ, int DV) {
    const int t = blockIdx.x, h = blockIdx.y;
    const size_t slot0 = ((size_t)t * HQ + h) * splits;
    float top = sink ? sink[h] * LOG2E : -INFINITY;
    for (int s = 0; s < splits; ++s) top = fmaxf(top, part_ml[(slot0 + s) * 2]);
    float l = sink ? exp2f(sink[h] * LOG2E - top) : 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float ms = part_ml[(slot0 + s) * 2];
        if (ms != -INFINITY) l += exp2f(ms - top) * part_ml[(slot0 + s) * 2 + 1];
    }
    const float inv = l == 0.0f ? 0.0f : 1.0f / l;
    for (int d = threadIdx.x; d < DV; d += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float ms = part_ml[(slot0 + s) * 2];
            if (ms != -INFINITY) acc += exp2f(ms - top) * part_o[(slot0 + s) * DV + d];
        }
        float v = acc * inv;
        if (gate) v *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)t * gate_stride + (size_t)h * DV + d])));
        out[((size_t)t * HQ + h) * DV + d] = __float2bfloat16_rn(v);
    }
}

// (of one CTA: with more than MAX_HEADS heads a CTA holds half of the heads and kv heads)
bool paired(int HQ) { return HQ > MAX_HEADS; }
size_t region_bytes(int HQ, int HKV, int D, int DV, int stages) {
    if (paired(HQ)) { HQ /= 2; HKV /= 2; }
    const size_t qb = (size_t)HQ * BM * (D * 2 + 16), kvb = (size_t)stages * HKV * BK * ((D * 2 + 16) + (DV * 2 + 16));
    return ((qb > kvb ? qb : kvb) + 127) / 128 * 128;
}
size_t smem_need(int HQ, int HKV, int D, int DV, int stages) {
    const int HL = paired(HQ) ? HQ / 2 : HQ;
    return region_bytes(HQ, HKV, D, DV, stages) + ((size_t)HQ * BM * SP + (size_t)HL * HQ + (size_t)HL * BIAS_N) * sizeof(float);
}
constexpr size_t SMEM_LIMIT = 227 * 1024;
bool instantiated(int D, int DV) {
    return (D == DV && (D == 16 || D == 32 || D == 48 || D == 64 || D == 96 || D == 128)) || (D == 64 && DV == 32) || (D == 32 && DV == 64);
}

}  // namespace

// 1 when the kernel takes these sizes (head sizes it is built for, a warp per head, everything in shared memory).
PH_EXPORT int ph_attention_talking_mma_supports(int HQ, int HKV, int D, int DV) {
    if (HQ < 1 || HKV < 1 || HQ % HKV || HQ > 2 * MAX_HEADS || !instantiated(D, DV)) return 0;
    if (paired(HQ) && (HQ % 2 || HKV % 2)) return 0;          // two CTAs halve the heads and the kv heads
    return smem_need(HQ, HKV, D, DV, 1) <= SMEM_LIMIT ? 1 : 0;
}

// CTAs of the kernel that one SM holds at these sizes (registers: 128 a thread; shared memory), 0 when it does not take them.
PH_EXPORT int ph_attention_talking_mma_ctas_per_sm(int HQ, int HKV, int D, int DV) {
    if (!ph_attention_talking_mma_supports(HQ, HKV, D, DV)) return 0;
    const int stages = smem_need(HQ, HKV, D, DV, 2) <= SMEM_LIMIT ? 2 : 1;
    const int by_regs = 65536 / (128 * (paired(HQ) ? HQ / 2 : HQ) * 32), by_smem = (int)(SMEM_LIMIT / (smem_need(HQ, HKV, D, DV, stages) + 1024));
    const int n = by_regs < by_smem ? by_regs : by_smem;
    return n < 1 ? 1 : n;
}

// q [T, HQ, D], out [T, HQ * DV] and the cache in bfloat16; the gate's rows (null: none) in bfloat16, gate_stride elements
// apart.  tile_seg / tile_first [n_tiles]: the request and the first row (within its portion) of each tile of 16 rows;
// every row of the step belongs to one tile.  splits > 1: that many CTAs share each tile's keys and leave partial results
// in part_o [T][HQ][splits][DV] and part_ml [T][HQ][splits][2] (float32), which a second kernel merges over all T rows.
PH_EXPORT int ph_attention_talking_mma(const void* q, const void* k_base, const void* v_base, long long page_stride, int page_size,
                                       const int32_t* block_table, int table_stride, const int32_t* seg_start, const int32_t* seg_ctx_len,
                                       const int32_t* tile_seg, const int32_t* tile_first, int n_tiles, void* out, int HQ, int HKV, int D,
                                       int DV, int window, int chunk, float scale, float cap, const float* r1, const float* r2,
                                       const float* talk, const float* sink, const void* gate, long long gate_stride, int splits, int T,
                                       float* part_o, float* part_ml, cudaStream_t stream) {
    if (!q || !k_base || !v_base || !block_table || !seg_start || !seg_ctx_len || !tile_seg || !tile_first || !out || n_tiles < 0 ||
        page_size < 1 || window < 0 || chunk < 0 || (r1 == nullptr) != (r2 == nullptr) || cap < 0.0f || splits < 1 || splits > 64 ||
        (splits > 1 && (!part_o || !part_ml || T < 1 || ((uintptr_t)part_o % 8))))
        return fail(PH_ERR_ARG, "attention_talking_mma: bad arguments");
    if (!ph_attention_talking_mma_supports(HQ, HKV, D, DV))
        return fail(PH_ERR_UNSUPPORTED, "attention_talking_mma: %d / %d heads of %d / %d are not taken", HQ, HKV, D, DV);
    if ((page_stride * 2) % 16 || ((uintptr_t)k_base | (uintptr_t)v_base | (uintptr_t)q) % 16 || (gate && (gate_stride % 2 || (uintptr_t)gate % 4)))
        return fail(PH_ERR_ARG, "attention_talking_mma: rows must be 16-byte aligned");
    if (n_tiles == 0) return PH_OK;
    TalkParams p;
    p.q = (const __nv_bfloat16*)q; p.k_base = (const __nv_bfloat16*)k_base; p.v_base = (const __nv_bfloat16*)v_base;
    p.page_stride = page_stride; p.page_size = page_size;
    p.page_shift = -1;
    for (int b = 0; b < 30; ++b) if ((1 << b) == page_size) p.page_shift = b;
 p.block_table = block_table; p.table_stride = table_stride;
    p.seg_start = seg_start; p.seg_ctx_len = seg_ctx_len; p.tile_seg = tile_seg; p.tile_first = tile_first;
    p.out = (__nv_bfloat16*)out; p.HQ = HQ; p.HKV = HKV; p.window = window; p.chunk = chunk; p.scale = scale; p.cap = cap;
    p.r1 = r1; p.r2 = r2; p.talk = talk; p.sink = sink; p.gate = (const __nv_bfloat16*)gate; p.gate_stride = gate_stride;
    p.pair = paired(HQ) ? 1 : 0;
    p.stages = smem_need(HQ, HKV, D, DV, 2) <= SMEM_LIMIT ? 2 : 1;
    p.kv_bytes = (int)region_bytes(HQ, HKV, D, DV, p.stages);
    p.splits = splits; p.part_o = part_o; p.part_ml = part_ml;
    const size_t smem = smem_need(HQ, HKV, D, DV, p.stages);
#define CASE(DD, VV)                                                                                                      \
    if (D == DD && DV == VV) {                                                                                            \
        auto kern = attention_talking_mma_kernel<DD, VV>;                                                                 \
        if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
            return fail(PH_ERR_LAUNCH, "attention_talking_mma: %zu bytes of shared memory were refused", smem);           \
        if (p.pair) {                                                                                                     \
            cudaLaunchConfig_t cfg = {};                                                                                  \
            cfg.gridDim = dim3(2 * n_tiles, splits); cfg.blockDim = dim3(HQ / 2 * 32); cfg.dynamicSmemBytes = smem; cfg.stream = stream; \
            cudaLaunchAttribute attr[1];                                                                                  \
            attr[0].id = cudaLaunchAttributeClusterDimension;                                                             \
            attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;                     \
            cfg.attrs = attr; cfg.numAttrs = 1;                                                                           \
            if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) return check_launch("attention_talking_mma (cluster)"); \
        } else {                                                                                                          \
            kern<<<dim3(n_tiles, splits), HQ * 32, smem, stream>>>(p);                                                    \
        }                                                                                                                 \
        if (splits > 1)                                                                                                   \
            attention_talking_merge_kernel<<<dim3(T, HQ), DV >= 64 ? 64 : 32, 0, stream>>>(part_o, part_ml, splits, sink, p.gate, gate_stride, \
                                                                                             p.out, HQ, DV);               \
        return check_launch("attention_talking_mma");                                                                     \
    }
    CASE(16, 16) CASE(32, 32) CASE(48, 48) CASE(64, 64) CASE(96, 96) CASE(128, 128) CASE(64, 32) CASE(32, 64)
#undef CASE
    return fail(PH_ERR_UNSUPPORTED, "attention_talking_mma: head sizes %d / %d", D, DV);
}
