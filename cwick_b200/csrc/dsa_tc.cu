// dsa_tc.cu -- the DSA lightning indexer on tensor cores, with exact selection (cwk_dsa_select).
//
// The reference's score is an f32 sum in a fixed order (src/attention.c:573-582); a tensor-core
// contraction accumulates in another order, so its scores can differ in the last bits and flip
// candidates that sit on the selection threshold. The selection here is still exact:
//
//   1. indexer_scores_tc_kernel: approximate scores a[c] for every key with tcgen05 MMAs.
//      Keys are E4M3 codes with a positive per-key scale, so
//        sum_h w_h ReLU(q_h . (code_c * s_c)) = s_c * sum_h sign(w_h) ReLU(|w_h| q_h . code_c):
//      the codes are widened to f16 (exact) on their way through shared memory; the f32 query,
//      times |w_h| and a power of two, is split into an f16 high part and an f16 low part (128 MMA
//      columns), so the MMA D[128 keys][hi|lo] = codes . q^T has exact products and f32
//      accumulation, and the epilogue adds the two halves, applies ReLU, the signs and the key's scale.
//   2. band_classify_kernel: a radix select on a[] gives the approximate want-th largest score tau.
//      The want-th largest value moves by at most delta when every score moves by at most delta, so
//      keys with a > tau + 2*delta are certainly selected (refined = +inf), keys with
//      a < tau - 2*delta certainly are not (-inf), and the band in between is listed. (delta is
//      taken as 2^-9 of the row's largest score, far above the contraction's and the query
//      split's worst case.)
//   3. the same kernel then re-scores the listed keys in the reference's exact order on CUDA cores (the
//      cluster's blocks share the list).
//   4. the selection kernel (csrc/dsa.cu) takes the exact threshold from the re-scored keys and
//      writes the reference's list in the reference's order.
//
// Pipeline of step 1 per 128-key tile: TMA (raw E4M3 tile, 16 KB, 8 stages) -> 8 converter warps
// (cvt.rn.f16x2.e4m3x2; a thread owns a key row and stores its f16 pairs into tensor memory, where
// they are the MMA's A operand: shared-memory bandwidth bounds this kernel, and so the MMAs read only
// the query from it) -> MMA issuer (8 MMAs, M 128, N 128) -> 4 epilogue warps (TMEM -> a[c]).
// Blocks are persistent over the tiles of one sequence.
// Every mbarrier wait is bounded and records a code in the context's error word when it gives up.
#include <algorithm>

#include <cuda_fp16.h>

#include "tc_common.cuh"
#include "topk_radix.cuh"

namespace {

constexpr int IT_KEYS = 128, IT_HD = 128, IT_IH = 64;
constexpr int RAW_STAGES = 8;
constexpr int RAW_BYTES = IT_KEYS * IT_HD;              // 16384
constexpr int IT_QROWS = 2 * IT_IH;                      // q split into f16 hi and lo parts: 128 MMA columns
constexpr int Q_BYTES_I = IT_QROWS * IT_HD * 2;         // 32768: two [128][64] f16 blocks
constexpr int I_OFF_Q = 0;
constexpr int I_OFF_RAW = Q_BYTES_I;                    // 8 stages of raw E4M3 tiles (128-byte swizzle)
constexpr uint32_t I_COL_D = 0, I_COL_A = 256;          // TMEM: two 128-column accumulators, two 64-column A operands (f16 pairs)
constexpr int I_OFF_BAR = I_OFF_RAW + RAW_STAGES * RAW_BYTES;
constexpr int I_OFF_W = I_OFF_BAR + 256;                // 19 words: warp maxima of the query split, 1 / scale, sign masks of the head weights
constexpr int I_SMEM = I_OFF_W + 256 + 1024;
constexpr int IT_THREADS = 512;                          // TMA, MMA, 2 idle | 8 converter warps | 4 epilogue warps
constexpr int IT_CONV = 256;
enum { IB_RAW_FULL = 0, IB_RAW_EMPTY = 8, IB_A_FULL = 16, IB_A_EMPTY = 18, IB_D_FULL = 20, IB_D_EMPTY = 22, IB_COUNT = 24 };

// M x N f16 x f16 -> f32, both operands K-major
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N) {
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Four E4M3 codes -> four f16, exactly (every E4M3 value is an f16 value): the hardware's paired
// conversion, two codes per instruction.
__device__ __forceinline__ uint2 e4m3x4_f16x4(uint32_t w) {
    uint2 r;
    asm("{\n.reg .b16 lo, hi;\nmov.b32 {lo, hi}, %2;\ncvt.rn.f16x2.e4m3x2 %0, lo;\ncvt.rn.f16x2.e4m3x2 %1, hi;\n}\n" : "=r"(r.x), "=r"(r.y) : "r"(w));
    return r;
}

struct IdxParams {
    const float *kscale;      // [B][key_stride]
    const float *q;           // f32 [B][64][128]
    const float *wt;          // f32 [B][64] head weights
    const int32_t *n;         // [B]
    float *sc;                // [B][key_stride]
    int32_t *band;            // [B][2] counters of the classification that follows: zeroed here
    int64_t key_stride;
    int *err;
};

__global__ void __launch_bounds__(IT_THREADS, 1)
indexer_scores_tc_kernel(const __grid_constant__ CUtensorMap tm_keys, const IdxParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const uint32_t bar0 = base + I_OFF_BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(sm + I_OFF_BAR + 8 * IB_COUNT + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // this block's tiles: a contiguous range of ONE sequence (so q and the weights are loaded once)
    const int blocks_per_seq = gridDim.x;
    const int b = blockIdx.y;
    const int nb = p.n[b];
    const int ntile = (nb + IT_KEYS - 1) / IT_KEYS;
    const int t_begin = (int)((int64_t)ntile * blockIdx.x / blocks_per_seq);
    const int t_end = (int)((int64_t)ntile * (blockIdx.x + 1) / blocks_per_seq);
    const int nt = t_end - t_begin;
    if (blockIdx.x == 0 && tid < 2) p.band[2 * b + tid] = 0;
    if (nt <= 0) return;

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_keys) : "memory");
        for (int i = 0; i < IB_COUNT; i++) {
            uint32_t cnt = 1u;
            if (i >= IB_RAW_EMPTY && i < IB_A_EMPTY) cnt = IT_CONV;   // raw_empty, a_full: every converter thread
            if (i >= IB_D_EMPTY) cnt = 128u;                          // d_empty: every epilogue thread
            mbar_init(bar(i), cnt);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // The B operand, built once per block from the f32 query of this sequence: every element is multiplied by
    // the magnitude of its head's weight (w ReLU(x) = sign(w) ReLU(|w| x)) and by a power of two that brings the
    // sequence's largest product into [2^13, 2^14); rows 0-63 of the operand hold the f16 roundings, rows 64-127
    // the f16 roundings of the remainders (22 bits of every product survive). Two swizzled [128][64] blocks.
    float *s_red = reinterpret_cast<float *>(sm + I_OFF_W);           // [16] warp maxima, then [16] = 1 / scale, [17..18] sign masks
    {
        const int h = tid >> 3, d0 = (tid & 7) * 16;
        const float w = fabsf(p.wt[(int64_t)b * IT_IH + h]);
        float x[16];
        float m = 0.f;
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
            const float4 v = *reinterpret_cast<const float4 *>(p.q + ((int64_t)b * IT_IH + h) * IT_HD + d0 + j);
            x[j] = v.x * w; x[j + 1] = v.y * w; x[j + 2] = v.z * w; x[j + 3] = v.w * w;
            m = fmaxf(m, fmaxf(fmaxf(fabsf(x[j]), fabsf(x[j + 1])), fmaxf(fabsf(x[j + 2]), fabsf(x[j + 3]))));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) s_red[warp] = m;
        if (tid < IT_IH) {
            const uint32_t neg = __ballot_sync(0xffffffffu, p.wt[(int64_t)b * IT_IH + tid] < 0.f);
            if (lane == 0) reinterpret_cast<uint32_t *>(s_red)[17 + warp] = neg;
        }
        __syncthreads();
        m = 0.f;
#pragma unroll
        for (int i = 0; i < IT_THREADS / 32; i++) m = fmaxf(m, s_red[i]);
        float scale = 1.f, inv = 1.f;
        if (m > 0.f && m < INFINITY) {
            const int e = (int)((__float_as_uint(m) >> 23) & 255u) - 127;     // floor(log2 m) for normal m
            const int sh = max(-100, min(100, 13 - e));
            scale = __uint_as_float((uint32_t)(127 + sh) << 23);
            inv = __uint_as_float((uint32_t)(127 - sh) << 23);
        }
        if (tid == 0) s_red[16] = inv;
        uint32_t hi[8], lo[8];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            const float a0 = x[j] * scale, a1 = x[j + 1] * scale;
            const __half h0 = __float2half_rn(a0), h1 = __float2half_rn(a1);
            const __half l0 = __float2half_rn(a0 - __half2float(h0)), l1 = __float2half_rn(a1 - __half2float(h1));
            hi[j >> 1] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
            lo[j >> 1] = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
        }
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const int c16 = (tid & 7) * 2 + c;                                 // 16-byte chunk of the 256-byte row
            uint8_t *blk = sm + I_OFF_Q + (c16 >> 3) * (IT_QROWS * 128);
            const int cc = c16 & 7;
            *reinterpret_cast<uint4 *>(blk + h * 128 + ((cc ^ (h & 7)) << 4)) = make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
            *reinterpret_cast<uint4 *>(blk + (IT_IH + h) * 128 + ((cc ^ ((IT_IH + h) & 7)) << 4)) =
                make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            for (int i = 0; i < nt && ok; i++) {
                const int r = i % RAW_STAGES, use = i / RAW_STAGES;
                ok = mbar_wait(bar(IB_RAW_EMPTY + r), (uint32_t)((use & 1) ^ 1), p.err, 801);
                if (!ok) break;
                mbar_expect_tx(bar(IB_RAW_FULL + r), RAW_BYTES);
                tma_load_2d(base + I_OFF_RAW + r * RAW_BYTES, &tm_keys, 0,
                            (int)((int64_t)b * p.key_stride + (int64_t)(t_begin + i) * IT_KEYS), bar(IB_RAW_FULL + r));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t ID = idesc_f16(128, IT_QROWS);
            bool ok = true;
            for (int i = 0; i < nt && ok; i++) {
                const int ab = i & 1, use = i >> 1;
                ok = mbar_wait(bar(IB_A_FULL + ab), (uint32_t)(use & 1), p.err, 803);
                if (ok) ok = mbar_wait(bar(IB_D_EMPTY + ab), (uint32_t)((use & 1) ^ 1), p.err, 804);
                if (!ok) break;
                tc_fence_after();
                const uint64_t db = smem_desc(base + I_OFF_Q, 16, 1024);
#pragma unroll
                for (int ks = 0; ks < 8; ks++)          // A: the converted keys in tensor memory, 16 f16 of every row = 8 columns per step
                    umma_bf16_ts(tmem + I_COL_D + ab * 128, tmem + I_COL_A + ab * 64 + ks * 8,
                                 db + (uint64_t)(((ks >> 2) * (IT_QROWS * 128) + (ks & 3) * 32) >> 4), ID, ks != 0);
                umma_commit(bar(IB_A_EMPTY + ab));
                umma_commit(bar(IB_D_FULL + ab));
            }
        }
    } else if (warp >= 4 && warp < 12) {
        // ---------------- converters: raw E4M3 tile -> f16 pairs in tensor memory, the MMA's A operand
        // A thread owns one key row (= its TMEM lane) and half of its 128 codes; the MMAs then read only the query
        // from shared memory.
        const int q4 = warp & 3, hv = (warp - 4) >> 2;
        const int row = q4 * 32 + lane;
        const uint32_t tl = tmem + ((uint32_t)(q4 * 32) << 16);
        bool ok = true;
        for (int i = 0; i < nt; i++) {
            const int r = i % RAW_STAGES, ruse = i / RAW_STAGES, ab = i & 1, ause = i >> 1;
            ok = mbar_wait(bar(IB_RAW_FULL + r), (uint32_t)(ruse & 1), p.err, 805);
            if (ok) ok = mbar_wait(bar(IB_A_EMPTY + ab), (uint32_t)((ause & 1) ^ 1), p.err, 806);
            ok = __all_sync(0xffffffffu, ok);            // the TMEM stores below are warp-wide
            if (!ok) break;
            tc_fence_after();
            const uint8_t *src = sm + I_OFF_RAW + r * RAW_BYTES + row * 128;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t w[16];
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int ch = hv * 4 + half * 2 + j;                    // 16 codes = dims ch*16 .. +15
                    const uint4 v = *reinterpret_cast<const uint4 *>(src + ((ch ^ (row & 7)) << 4));
                    const uint2 c0 = e4m3x4_f16x4(v.x), c1 = e4m3x4_f16x4(v.y), c2 = e4m3x4_f16x4(v.z), c3 = e4m3x4_f16x4(v.w);
                    w[8 * j] = c0.x; w[8 * j + 1] = c0.y; w[8 * j + 2] = c1.x; w[8 * j + 3] = c1.y;
                    w[8 * j + 4] = c2.x; w[8 * j + 5] = c2.y; w[8 * j + 6] = c3.x; w[8 * j + 7] = c3.y;
                }
                TMEM_ST16(w, 0, tl + I_COL_A + ab * 64 + hv * 32 + half * 16);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            mbar_arrive(bar(IB_A_FULL + ab));
            mbar_arrive(bar(IB_RAW_EMPTY + r));
        }
    } else if (warp >= 12) {
        // ---------------- epilogue: hi + lo, ReLU, signed head sum, key scale
        const int q4 = warp & 3;
        const int row = q4 * 32 + lane;
        const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
        const float unscale = s_red[16];
        const uint32_t neg[2] = {reinterpret_cast<const uint32_t *>(s_red)[17], reinterpret_cast<const uint32_t *>(s_red)[18]};
        const bool any_neg = (neg[0] | neg[1]) != 0;
        bool ok = true;
        for (int i = 0; i < nt; i++) {
            const int ab = i & 1, use = i >> 1;
            ok = mbar_wait(bar(IB_D_FULL + ab), (uint32_t)(use & 1), p.err, 807);
            if (!ok) break;
            tc_fence_after();
            const int64_t key = (int64_t)(t_begin + i) * IT_KEYS + row;
            const float ksc = key < nb ? p.kscale[(int64_t)b * p.key_stride + key] : 0.f;
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t v[32], u[32];
                TMEM_LD16(v, 0, tlane + ab * 128 + c * 32);             // codes . q_hi
                TMEM_LD16(v, 16, tlane + ab * 128 + c * 32 + 16);
                TMEM_LD16(u, 0, tlane + ab * 128 + 64 + c * 32);        // codes . q_lo
                TMEM_LD16(u, 16, tlane + ab * 128 + 64 + c * 32 + 16);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (!any_neg) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        acc0 += fmaxf(__uint_as_float(v[j]) + __uint_as_float(u[j]), 0.f);
                        acc1 += fmaxf(__uint_as_float(v[j + 1]) + __uint_as_float(u[j + 1]), 0.f);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float r0 = fmaxf(__uint_as_float(v[j]) + __uint_as_float(u[j]), 0.f);
                        const float r1 = fmaxf(__uint_as_float(v[j + 1]) + __uint_as_float(u[j + 1]), 0.f);
                        acc0 += __uint_as_float(__float_as_uint(r0) ^ (((neg[c] >> j) & 1u) << 31));
                        acc1 += __uint_as_float(__float_as_uint(r1) ^ (((neg[c] >> (j + 1)) & 1u) << 31));
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar(IB_D_EMPTY + ab));
            if (key < nb) p.sc[(int64_t)b * p.key_stride + key] = (acc0 + acc1) * unscale * ksc;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

__device__ __forceinline__ float e4m3_to_f32_i(uint32_t b) {
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    float mag;
    if (e == 0) mag = (float)m * 0.001953125f;
    else if (e == 15 && m == 7) mag = __int_as_float(0x7fc00000);
    else mag = __uint_as_float(((e + 120u) << 23) | (m << 20));
    return (b & 0x80u) ? -mag : mag;
}

constexpr int BC_KEYS = 64;                                   // band keys re-scored per pass and block
constexpr int BC_QLD = IT_HD + 4;                             // padded q rows in shared memory
constexpr int BC_SMEM = (IT_IH * BC_QLD + IT_IH + BC_KEYS * IT_HD + BC_KEYS * (IT_IH + 1)) * 4;

// One cluster per sequence: the row's largest approximate score, the exact want-th largest
// approximate score tau, then the classification of every key: certainly selected (refined =
// +inf), certainly not (refined = -inf), or in the band |a - tau| <= eps, whose indices are appended
// to band_list. band_count[2b] counts the band's entries, band_count[2b + 1] the keys above the band
// (both zeroed by the scoring kernel before it). The same launch then re-scores the band exactly and
// writes the selection.
__global__ void __cluster_dims__(TK_CL, 1, 1) __launch_bounds__(TK_THREADS, 1)
band_classify_kernel(const float *approx, int64_t stride, const int32_t *n, int want, float *refined, int32_t *band_list,
                     int32_t *band_count, const uint8_t *keys, const float *kscale, const float *q, const float *wt,
                     int keep_self, int32_t *sel, int64_t sel_ld, int32_t *nsel, long long *trace) {
#ifdef CWK_TRACE
#define BTRACE(i) do { if (trace && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) trace[i] = clock64(); } while (0)
#else
#define BTRACE(i) do { } while (0)
#endif
    (void)trace;
    BTRACE(0);
    extern __shared__ __align__(16) float bc_sm[];
    float *sq = bc_sm, *sw = sq + IT_IH * BC_QLD, *skey = sw + IT_IH, *sprod = skey + BC_KEYS * IT_HD;
    cg::cluster_group cl = cg::this_cluster();
    const unsigned rank = cl.block_rank();
    const int b = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    const int nb = n[b];
    const float *s = approx + (int64_t)b * stride;
    float *f = refined + (int64_t)b * stride;
    const TkSlice sl = tk_slice(nb, rank);
    int32_t *out = sel + (int64_t)b * sel_ld;
    if (nb <= want) {                         // everything is selected: any finite value will do
        for (int i = sl.begin + tid; i < sl.end; i += TK_THREADS) { f[i] = s[i]; out[i] = i; }
        if (rank == 0 && tid == 0) nsel[b] = nb;
        return;
    }
    __shared__ TkShared sh;
    __shared__ float red[32];
    uint32_t kc[TK_PT];
    if (sl.cached) tk_load(s, sl.begin, sl.end, kc);
    // the query and the head weights of this sequence, for the exact re-scoring at the end (padded rows: the heads of a
    // key's 16 threads then read different banks)
    for (int i = tid; i < IT_IH * (IT_HD / 4); i += TK_THREADS) {
        const int h = i / (IT_HD / 4), c = i % (IT_HD / 4);
        *reinterpret_cast<float4 *>(sq + h * BC_QLD + c * 4) = __ldg(reinterpret_cast<const float4 *>(q + ((int64_t)b * IT_IH + h) * IT_HD) + c);
    }
    if (tid < IT_IH) sw[tid] = wt[(int64_t)b * IT_IH + tid];
    // largest score of this block's slice (scores are sums of non-negative terms)
    float m = 0.f;
    for (int c0 = sl.begin; c0 < sl.end; c0 += TK_CHUNK) {
        if (!sl.cached) tk_load(s, c0, sl.end, kc);
        const int i0 = c0 + tid * TK_PT;
#pragma unroll
        for (int j = 0; j < TK_PT; j++)
            if (i0 + j < sl.end) m = fmaxf(m, fabsf(order_key_inverse(kc[j])));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[tid >> 5] = m;
    __syncthreads();
    if (tid < 32) {
        m = red[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) sh.fmax = m;
    }
    uint32_t prefix;
    int remaining;
    BTRACE(1);
    tk_radix_select(s, sl, kc, want, sh, prefix, remaining);       // its cluster barriers also publish fmax
    BTRACE(2);
    m = 0.f;
#pragma unroll
    for (unsigned r = 0; r < TK_CL; r++) m = fmaxf(m, *cl.map_shared_rank(&sh.fmax, r));
    const float tau = order_key_inverse(prefix);
    const float eps = 2.0f * 0.001953125f * m;              // 2 * delta, delta = 2^-9 of the row's largest score
    const float hi = tau + eps, lo = tau - eps;
    int32_t *list = band_list + (int64_t)b * stride;
    for (int c0 = sl.begin; c0 < sl.end; c0 += TK_CHUNK) {
        if (!sl.cached) tk_load(s, c0, sl.end, kc);
        const int i0 = c0 + tid * TK_PT;
        uint32_t inb = 0;
        float v[TK_PT];
#pragma unroll
        for (int j = 0; j < TK_PT; j++) {
            const float a = order_key_inverse(kc[j]);
            v[j] = a > hi ? INFINITY : -INFINITY;
            if (i0 + j < sl.end && !(a > hi) && !(a < lo)) inb |= 1u << j;     // NaN lands here too and is re-scored exactly
        }
        if (i0 + TK_PT <= sl.end && (reinterpret_cast<uintptr_t>(f + i0) & 15u) == 0) {
            *reinterpret_cast<float4 *>(f + i0) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4 *>(f + i0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
        } else {
#pragma unroll
            for (int j = 0; j < TK_PT; j++)
                if (i0 + j < sl.end) f[i0 + j] = v[j];
        }
        {
            int nab = 0;
#pragma unroll
            for (int j = 0; j < TK_PT; j++) nab += (i0 + j < sl.end && v[j] > 0.f) ? 1 : 0;
            nab = __reduce_add_sync(0xffffffffu, nab);
            if (lane == 0 && nab) atomicAdd(band_count + 2 * b + 1, nab);
        }
        // band entries: one global atomic per warp (the list's order does not matter; the rescoring
        // kernel overwrites refined[] at these indices)
        const int mine = __popc(inb);
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        const int wtot = __shfl_sync(0xffffffffu, incl, 31);
        int at = 0;
        if (lane == 31 && wtot) at = atomicAdd(band_count + 2 * b, wtot);
        at = __shfl_sync(0xffffffffu, at, 31) + incl - mine;
#pragma unroll
        for (int j = 0; j < TK_PT; j++)
            if (inb & (1u << j)) list[at++] = i0 + j;
    }
    BTRACE(3);
    cl.sync();                              // every block's part of the band list is written (and fmax has been read everywhere)
    BTRACE(4);
    // ---- exact scores of the band (the reference's order: src/attention.c:573-582 with dot_f32's grouping, :249-258).
    // The cluster's blocks share the list evenly; 64 keys per pass: dequantise into shared memory (16 threads per key),
    // 2 x 2 (key, head) dots per thread, then one thread per key adds the 64 weighted terms in head order.
    const int total = *reinterpret_cast<volatile int32_t *>(band_count + 2 * b);
    const int per = (total + TK_CL - 1) / TK_CL;
    const int k_begin = min(total, (int)rank * per), k_end = min(total, k_begin + per);
    for (int k0 = k_begin; k0 < k_end; k0 += BC_KEYS) {
        {
            const int kk = tid >> 4, part = tid & 15;
            if (k0 + kk < k_end) {
                const int c = list[k0 + kk];
                const float sc = kscale[(int64_t)b * stride + c];
                const uint2 v = *reinterpret_cast<const uint2 *>(keys + ((int64_t)b * stride + c) * IT_HD + part * 8);
                float *dst = skey + kk * IT_HD + part * 8;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    dst[j] = __fmul_rn(e4m3_to_f32_i((v.x >> (8 * j)) & 0xffu), sc);
                    dst[4 + j] = __fmul_rn(e4m3_to_f32_i((v.y >> (8 * j)) & 0xffu), sc);
                }
            }
        }
        __syncthreads();
        {
            // a thread owns 2 keys x 2 heads (a warp: one key pair, broadcast, against all 64 heads): half the shared-memory
            // reads of one (key, head) pair per thread. Every dot keeps the reference's order: four strided accumulators
            // with separate multiply and add, then (s0 + s1) + (s2 + s3).
            const int ka = (tid >> 5) * 2, ha = lane, hb2 = lane + 32;
            const float4 *kp0 = reinterpret_cast<const float4 *>(skey + ka * IT_HD), *kp1 = kp0 + IT_HD / 4;
            const float4 *qp0 = reinterpret_cast<const float4 *>(sq + ha * BC_QLD), *qp1 = reinterpret_cast<const float4 *>(sq + hb2 * BC_QLD);
            float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f}, b0[4] = {0.f, 0.f, 0.f, 0.f}, b1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
            for (int i = 0; i < IT_HD / 4; i++) {
                const float4 k0v = kp0[i], k1v = kp1[i], q0v = qp0[i], q1v = qp1[i];
                a0[0] = __fadd_rn(a0[0], __fmul_rn(k0v.x, q0v.x)); a0[1] = __fadd_rn(a0[1], __fmul_rn(k0v.y, q0v.y));
                a0[2] = __fadd_rn(a0[2], __fmul_rn(k0v.z, q0v.z)); a0[3] = __fadd_rn(a0[3], __fmul_rn(k0v.w, q0v.w));
                a1[0] = __fadd_rn(a1[0], __fmul_rn(k0v.x, q1v.x)); a1[1] = __fadd_rn(a1[1], __fmul_rn(k0v.y, q1v.y));
                a1[2] = __fadd_rn(a1[2], __fmul_rn(k0v.z, q1v.z)); a1[3] = __fadd_rn(a1[3], __fmul_rn(k0v.w, q1v.w));
                b0[0] = __fadd_rn(b0[0], __fmul_rn(k1v.x, q0v.x)); b0[1] = __fadd_rn(b0[1], __fmul_rn(k1v.y, q0v.y));
                b0[2] = __fadd_rn(b0[2], __fmul_rn(k1v.z, q0v.z)); b0[3] = __fadd_rn(b0[3], __fmul_rn(k1v.w, q0v.w));
                b1[0] = __fadd_rn(b1[0], __fmul_rn(k1v.x, q1v.x)); b1[1] = __fadd_rn(b1[1], __fmul_rn(k1v.y, q1v.y));
                b1[2] = __fadd_rn(b1[2], __fmul_rn(k1v.z, q1v.z)); b1[3] = __fadd_rn(b1[3], __fmul_rn(k1v.w, q1v.w));
            }
            auto fin = [&](const float (&s4)[4], int kk, int h) {
                float d = __fadd_rn(__fadd_rn(s4[0], s4[1]), __fadd_rn(s4[2], s4[3]));
                if (d < 0.f) d = 0.f;
                sprod[kk * (IT_IH + 1) + h] = __fmul_rn(d, sw[h]);
            };
            fin(a0, ka, ha); fin(a1, ka, hb2); fin(b0, ka + 1, ha); fin(b1, ka + 1, hb2);
        }
        __syncthreads();
        if (tid < BC_KEYS && k0 + tid < k_end) {
            float tot = 0.f;
#pragma unroll 8
            for (int h = 0; h < IT_IH; h++) tot = __fadd_rn(tot, sprod[tid * (IT_IH + 1) + h]);
            f[list[k0 + tid]] = tot;
        }
        __syncthreads();
    }
    // ---- the selection itself, on the refined row: the exact threshold is the (want - certainly selected)-th largest of the
    // re-scored keys; then the reference's list in the reference's order
    BTRACE(5);
    cl.sync();                              // every block's re-scored keys are in refined[]
    BTRACE(6);
    if (sl.cached) tk_load(f, sl.begin, sl.end, kc);
    tk_threshold_and_compact(f, sl, kc, nb, want, keep_self, 0, out, nsel + b, list, total,
                             *reinterpret_cast<volatile int32_t *>(band_count + 2 * b + 1), sh);
    BTRACE(7);
}

}  // namespace

extern "C" int cwk_topk_select(cwk_ctx *ctx, const float *sc, int64_t sc_stride, const int32_t *n, int max_n, int B, int want,
                               int keep_self, int32_t *sel, int64_t sel_ld, int32_t *nsel);
extern "C" int cwk_indexer_scores_fp8(cwk_ctx *ctx, const void *keys, const float *kscale, int64_t key_stride, const float *q,
                                      const float *wt, const int32_t *n, int max_n, int B, int ih, int hd, float *sc);

// The fused DSA selection: approximate scores on tensor cores, exact top-`want`.
extern "C" int cwk_dsa_select(cwk_ctx *ctx, const void *keys, const float *kscale, int64_t key_stride, const float *q,
                              const float *wt, const int32_t *n, int max_n, int B, int ih, int hd, int want, int keep_self,
                              int32_t *sel, int64_t sel_ld, int32_t *nsel, float *scores_out) {
    if (!ctx || !keys || !kscale || !q || !wt || !n || !sel || !nsel || B <= 0 || want <= 0 || max_n < 0 || sel_ld < want + 1)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "dsa_select: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (max_n == 0) {
        CWK_CUDA(ctx, cudaMemsetAsync(nsel, 0, (size_t)B * sizeof(int32_t), ctx->stream));
        return CWK_OK;
    }
    const bool tc_ok = ih == IT_IH && hd == IT_HD && ((uintptr_t)keys % 16) == 0 && cwk_encode_tiled_fn() != nullptr &&
                       ctx->force_mla_path != 0 && ctx->force_mla_path != 1;
    // workspace: approx f32 [B][stride], refined f32 [B][stride], band list int32 [B][stride], band counts [B][2]
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const size_t b_sc = up((size_t)B * key_stride * 4);
    int s = cwk_reserve_work(ctx, 3 * b_sc + up((size_t)B * 8));
    if (s != CWK_OK) return s;
    uint8_t *w = (uint8_t *)ctx->work;
    float *approx = (float *)w, *refined = (float *)(w + b_sc);
    int32_t *band_list = (int32_t *)(w + 2 * b_sc);
    int32_t *band = (int32_t *)(w + 3 * b_sc);
    if (!tc_ok) {
        // shapes the tensor-core path is not built for: exact scores for every key
        s = cwk_indexer_scores_fp8(ctx, keys, kscale, key_stride, q, wt, n, max_n, B, ih, hd, scores_out ? scores_out : approx);
        if (s != CWK_OK) return s;
        return cwk_topk_select(ctx, scores_out ? scores_out : approx, key_stride, n, max_n, B, want, keep_self, sel, sel_ld, nsel);
    }
    s = cwk_ensure_err_word(ctx);
    if (s != CWK_OK) return s;
    CUtensorMap tm_keys;
    {
        CwkEncodeTiledFn enc = cwk_encode_tiled_fn();
        cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)B * (cuuint64_t)key_stride};
        cuuint64_t strides[1] = {(cuuint64_t)hd};
        cuuint32_t box[2] = {(cuuint32_t)hd, IT_KEYS};
        cuuint32_t es[2] = {1, 1};
        if (enc(&tm_keys, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(keys), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled(keys) failed");
    }
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(indexer_scores_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, I_SMEM));
        CWK_CUDA(ctx, cudaFuncSetAttribute(band_classify_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BC_SMEM));
        attr_set[ctx->device & 15] = true;
    }
    IdxParams p;
    p.kscale = kscale; p.q = q; p.wt = wt; p.n = n; p.sc = approx; p.band = band; p.key_stride = key_stride; p.err = ctx->dev_err;
    const int tiles = (max_n + IT_KEYS - 1) / IT_KEYS;
    const int bps = std::max(1, std::min(tiles, ctx->sm_count / B));
    {
        CwkKernelTimer timer(ctx);
        indexer_scores_tc_kernel<<<dim3(bps, B), IT_THREADS, I_SMEM, ctx->stream>>>(tm_keys, p);
        CWK_LAUNCH_CHECK(ctx, "indexer_scores_tc_kernel");
    }
    {
        CwkKernelTimer timer(ctx);
        band_classify_kernel<<<dim3(TK_CL, B), TK_THREADS, BC_SMEM, ctx->stream>>>(approx, key_stride, n, want, refined, band_list, band,
                                                                                  (const uint8_t *)keys, kscale, q, wt, keep_self, sel, sel_ld, nsel,
                                                                                  (long long *)ctx->tc_trace);
        CWK_LAUNCH_CHECK(ctx, "band_classify_kernel");
    }
    if (scores_out) CWK_CUDA(ctx, cudaMemcpyAsync(scores_out, refined, (size_t)B * key_stride * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    return CWK_OK;
}
