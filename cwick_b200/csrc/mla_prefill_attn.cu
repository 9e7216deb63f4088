// mla_prefill_attn.cu -- causal MLA prefill attention with the queries as the MMA's rows.
//
// The decode kernel (mla_decode_tc.cu) treats a query token as 64 rows (its heads) of a 576-wide
// product against the latent cache; run once per token of a prompt, its MMAs are 64 columns wide,
// bound by shared-memory bandwidth, and every 128-key tile is a serial chain. A prompt has a better
// shape: per HEAD, 128 consecutive tokens are the 128 rows of an MMA. Scores are taken against the
// head's expanded key, not against the latent:
//
//   s[t][h][c] = q_nope[t][h] . (W_uk[h] lat[c])  +  q_rope[t][h] . k_rope[c]        (192-wide)
//   out[t][h]  = sum_c softmax_c(s) lat[c]                                            (512-wide)
//
// which is the absorbed attention of src/attention.c:741-782 with the product W_uk^T q_nope . lat
// re-associated: the same scores, 192 instead of 576 multiply-adds each, and the values are still the
// shared latent, so the output is the absorbed [tokens][heads][512] result. Two kernels:
//
//   kexp_tc_kernel: Kx[h][c][0:128] = W_uk[h] lat[c] (tcgen05, W_uk[h] resident per block as the
//     K-major B operand, latent tiles streamed), Kx[h][c][128:192] = k_rope[c]. Head-major: a head's 64-key tile is
//     24 KB of consecutive memory (token-major rows would lie 24 KB apart and crowd a few L2 slices).
//   prefill_attn_kernel: one block = 128 queries x one head x one half of the 512 value columns
//     (the accumulator of a half, 128 x 256 f32, is half of tensor memory; both halves recompute
//     the 192-wide scores, which is cheaper than any exchange). Keys stream in tiles of 64 through a
//     3-deep ring (24 KB each), latent halves through a 3-deep ring (32 KB each), one TMA box each. The query tile
//     itself sits in tensor memory (96 columns of bf16 pairs) as the A operand of the score MMAs: shared-memory
//     bandwidth is what bounds this kernel, and this way the score MMAs read only the keys from it.
//     Per tile: S = Q Kx^T (12 MMAs, M 128 x N 64) into one of two TMEM score buffers; the softmax
//     warps own one query row per thread (TMEM lane = row, so row maxima and sums need no shuffles),
//     write P (bf16) to shared memory; O += P lat (4 MMAs, M 128 x N 256). The two products have
//     issuer threads of their own and three score buffers, so the scores run up to two tiles ahead of the values and
//     the tensor pipe works under the softmax.
//     The kernel has two forms. The fast one splits the 64 keys of a row between two softmax warp groups
//     (two threads per row) and never rescales: a row's reference exponent is its largest score of the first
//     tile, later scores may outrun it by up to 2^64 (bf16 P and the f32 accumulators have the range), and a
//     block that sees more raises a flag. The exact one (one thread per row, lazy rescale of its own TMEM lane
//     when a score outruns the reference by 2^8) runs right after it and recomputes the flagged blocks only.
//
// Every mbarrier wait is bounded and records a code in the context's error word when it gives up.
#include <algorithm>

#include "tc_common.cuh"

namespace {

constexpr int PA_QT = 128, PA_KT = 64, PA_DV = 256, PA_L = 512, PA_ROW = 576;
constexpr int PA_C_BYTES = PA_KT * PA_DV * 2;         // 32768: four [64][64] blocks
constexpr int PA_P_BYTES = PA_QT * PA_KT * 2;         // 16384: one [128][64] block
constexpr int PA_KST = 3;
constexpr int PA_OFF_K = 0;                            // (the query tile lives in tensor memory, not here)
// The kernel serves two shapes. MLA prefill: 192-wide expanded keys, the 512 value columns in two halves, three value
// stages. GQA prefill (Qwen3.5 layers): 256-wide keys and values of one KV head, two value stages (the key tiles are
// 32 KB instead of 24 KB). Shared-memory layout and the query tile's width in tensor memory follow from DQK and CST.
template <int DQK_, int CST_>
struct PaCfg {
    static constexpr int DQK = DQK_, CST = CST_;
    static constexpr int K_BYTES = PA_KT * DQK * 2;    // 24576 / 32768: DQK / 64 blocks of [64][64]
    static constexpr int OFF_C = PA_OFF_K + PA_KST * K_BYTES;
    static constexpr int OFF_P = OFF_C + CST * PA_C_BYTES;
    static constexpr int OFF_BAR = OFF_P + 2 * PA_P_BYTES;
    static constexpr int OFF_X = OFF_BAR + 512;        // [4][128] f32 maxima, [4][128] f32 sums exchanged between the softmax groups; 8 item numbers
    static constexpr int SMEM = OFF_X + 4096 + 64 + 1024;
    static_assert(SMEM <= 232448, "shared-memory budget");
    static_assert(384 + DQK / 2 <= 512, "tensor-memory budget");
};
using PaMla = PaCfg<192, 3>;
using PaGqa = PaCfg<256, 2>;
static_assert(PaMla::OFF_BAR == 204800, "shared-memory budget");
constexpr uint32_t PA_COL_O = 0, PA_COL_S = 256, PA_COL_Q = 384;   // S buffers at 256 and 320; Q: DQK / 2 columns of bf16 pairs
constexpr float PA_LAZY = 8.f;                         // exact form: rescale when a score outruns the reference by 2^8
constexpr float PA_RANGE = 64.f;                       // fast form: flag the block when a score outruns it by 2^64
constexpr int PA_SBUF = 2;                             // score buffers in tensor memory
enum { PB_QFULL = 0, PB_KFULL = 1, PB_KEMPTY = 4, PB_CFULL = 7, PB_CEMPTY = 10, PB_SFULL = 13, PB_SEMPTY = 15, PB_PFULL = 17, PB_PEMPTY = 19,
       PB_ODONE = 21, PB_QEMPTY = 22, PB_OFREE = 23, PB_XM = 24, PB_XL = 25, PB_ITEM = 26, PB_COUNT = 34 };

struct AttnParams {
    const uint16_t *q;  // bf16 [n][nh][DQK] (MLA: rope part rotated)
    uint16_t *out;      // bf16 [n][nh][512] (MLA) / [n][nh][256] (GQA)
    int n, nh, T;       // T = pos0 + n cached rows
    int group;          // GQA: query heads per KV head (MLA: unused)
    int64_t pos0;
    float scale_log2;
    int *flags;         // one word per item: fast form sets it, exact form runs only where it is set
    int *counter;       // [3]: item counters of the fast and the exact form, number of flags raised; zero at launch
    int *err;
};

struct AttnItem {
    int q0, h, half, nt;
};

// Work item w of the attention grid: query tiles from the longest to the shortest inside one (head, half), then the next
// (head, half): blocks that run at the same time work on the same few heads, whose keys stay in L2.
__device__ __forceinline__ AttnItem attn_item(int w, const AttnParams &p, int nq) {
    AttnItem it;
    const int qtile = nq - 1 - (w % nq), hh = w / nq;
    it.q0 = qtile * PA_QT;
    it.h = hh % p.nh;
    it.half = hh / p.nh;                                                   // GQA: the grid has one "half", always 0
    const int64_t last_q = p.pos0 + min(it.q0 + PA_QT - 1, p.n - 1);     // keys 0 .. pos0 + (last query of the item): tiles of 64
    it.nt = (int)(last_q / PA_KT) + 1;
    return it;
}

// Persistent: one block per SM takes items from a global counter until none is left. The first TMA operation of a
// block waits several thousand cycles for its tensor map, tensor memory is allocated once, and the loads of the next
// item run under the epilogue of this one.
template <int NWG, class CFG, bool GQA>      // NWG softmax warp groups: 2 or 4 = fast form (a row's 64 keys shared by 2 or 4 threads), 1 = exact form
__global__ void __launch_bounds__(128 + 128 * NWG, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_c, const AttnParams p) {
    constexpr int PA_DQK = CFG::DQK, PA_K_BYTES = CFG::K_BYTES, PA_CST = CFG::CST, PA_OFF_C = CFG::OFF_C, PA_OFF_P = CFG::OFF_P,
                  PA_OFF_BAR = CFG::OFF_BAR, PA_OFF_X = CFG::OFF_X;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const uint32_t bar0 = base + PA_OFF_BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(sm + PA_OFF_BAR + 8 * PB_COUNT + 8);
    volatile int *s_item = reinterpret_cast<volatile int *>(sm + PA_OFF_X + 4096);      // ring of 8 item numbers
    float *s_m = reinterpret_cast<float *>(sm + PA_OFF_X), *s_l = s_m + 512;              // [4][128] each

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (NWG == 1 && p.counter[2] == 0) return;                   // the repair pass: the fast form raised no flag
    const int nq = (p.n + PA_QT - 1) / PA_QT;
    const int total = nq * p.nh * (GQA ? 1 : 2);

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_c) : "memory");
        for (int i = 0; i < PB_COUNT; i++) {
            const bool by_soft = (i >= PB_SEMPTY && i < PB_PEMPTY) || i == PB_QFULL || i == PB_OFREE || i == PB_XM || i == PB_XL;
            mbar_init(bar(i), by_soft ? (uint32_t)(128 * NWG) : 1u);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;

    // item k of this block, as published by the key producer (-1: no more)
    auto next_item = [&](int k, int &w) -> bool {
        if (!mbar_wait(bar(PB_ITEM + (k & 7)), (uint32_t)((k >> 3) & 1), p.err, 1031)) return false;
        w = s_item[k & 7];
        return true;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ item fetcher and TMA producer of the key ring
        if (lane == 0) {
            bool ok = true;
            int kc = 0;                              // key tiles issued so far (ring position and phase run across items)
            for (int k = 0; ok; k++) {
                int w = atomicAdd(p.counter + (NWG == 1 ? 1 : 0), 1);
                if (NWG == 1)                         // the repair pass takes flagged items only
                    while (w < total && p.flags[w] == 0) w = atomicAdd(p.counter + 1, 1);
                if (w >= total) w = -1;
                s_item[k & 7] = w;                    // the roles of a block stay within a few tiles of each other: 8 slots cannot wrap
                mbar_arrive(bar(PB_ITEM + (k & 7)));
                if (w < 0) break;
                const AttnItem it = attn_item(w, p, nq);
                for (int i = 0; i < it.nt && ok; i++, kc++) {
                    const int ks = kc % PA_KST, ku = kc / PA_KST;
                    ok = mbar_wait(bar(PB_KEMPTY + ks), (uint32_t)((ku & 1) ^ 1), p.err, 1001);
                    if (!ok) break;
                    mbar_expect_tx(bar(PB_KFULL + ks), PA_K_BYTES);
                    if (GQA) tma_load_3d(base + PA_OFF_K + ks * PA_K_BYTES, &tm_k, 0, i * PA_KT, (it.h / p.group) * (PA_DQK / 64), bar(PB_KFULL + ks));
                    else tma_load_3d(base + PA_OFF_K + ks * PA_K_BYTES, &tm_k, 0, it.h * p.T + i * PA_KT, 0, bar(PB_KFULL + ks));
                }
            }
            if (!ok)        // drain the copies still in flight before leaving
                for (int j = (kc > PA_KST ? kc - PA_KST : 0); j < kc; j++)
                    mbar_wait(bar(PB_KFULL + j % PA_KST), (uint32_t)((j / PA_KST) & 1), p.err, 1004);
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------ TMA producer of the latent ring (its slots come free much
        // later than the key slots: a thread of its own, so that the keys run ahead)
        if (lane == 0) {
            bool ok = true;
            int cc = 0;
            for (int k = 0; ok; k++) {
                int w;
                ok = next_item(k, w);
                if (!ok || w < 0) break;
                const AttnItem it = attn_item(w, p, nq);
                for (int i = 0; i < it.nt && ok; i++, cc++) {
                    const int cs = cc % PA_CST, cu = cc / PA_CST;
                    ok = mbar_wait(bar(PB_CEMPTY + cs), (uint32_t)((cu & 1) ^ 1), p.err, 1002);
                    if (!ok) break;
                    mbar_expect_tx(bar(PB_CFULL + cs), PA_C_BYTES);
                    tma_load_3d(base + PA_OFF_C + cs * PA_C_BYTES, &tm_c, 0, i * PA_KT, (GQA ? it.h / p.group : it.half) * 4, bar(PB_CFULL + cs));
                }
            }
            if (!ok)
                for (int j = (cc > PA_CST ? cc - PA_CST : 0); j < cc; j++)
                    mbar_wait(bar(PB_CFULL + j % PA_CST), (uint32_t)((j / PA_CST) & 1), p.err, 1005);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer of the scores
        // The two products have issuers of their own (this warp and warp 3): a wait on an mbarrier costs a
        // lone thread some 300 cycles even when the phase is long complete, and one thread doing all four
        // waits of a tile in turn was the longest chain of the kernel.
        if (lane == 0) {
            constexpr uint32_t ID_QK = idesc_bf16(128, PA_KT, 0, 0);
            bool ok = true;
            int kc = 0;                              // score tiles issued so far
            for (int k = 0; ok; k++) {
                int w;
                ok = next_item(k, w);
                if (!ok || w < 0) break;
                const AttnItem it = attn_item(w, p, nq);
                ok = mbar_wait(bar(PB_QFULL), (uint32_t)(k & 1), p.err, 1011);     // the softmax threads have written the item's query tile into tensor memory
                if (!ok) break;
                tc_fence_after();
                // scores of a tile: S[kc % 2] = Q Kx^T, three 64-wide blocks of the 192 dims, four 16-wide steps each
                for (int i = 0; i < it.nt && ok; i++, kc++) {
                    const int ks = kc % PA_KST, ku = kc / PA_KST, sb = kc % PA_SBUF, su = kc / PA_SBUF;
                    ok = mbar_wait(bar(PB_KFULL + ks), (uint32_t)(ku & 1), p.err, 1012);
                    if (ok) ok = mbar_wait(bar(PB_SEMPTY + sb), (uint32_t)((su & 1) ^ 1), p.err, 1013);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t dK = smem_desc(base + PA_OFF_K + ks * PA_K_BYTES, 16, 1024);
#pragma unroll
                    for (int s = 0; s < PA_DQK / 16; s++)
                        umma_bf16_ts(tmem + PA_COL_S + sb * PA_KT, tmem + PA_COL_Q + s * 8,       // A: 16 bf16 of every row = 8 TMEM columns per step
                                     dK + (uint64_t)(((s >> 2) * (PA_KT * 128) + (s & 3) * 32) >> 4), ID_QK, s != 0);
                    umma_commit(bar(PB_KEMPTY + ks));
                    umma_commit(bar(PB_SFULL + sb));
                }
                if (ok) umma_commit(bar(PB_QEMPTY));       // the query tile may be replaced once these MMAs are done
            }
        }
    } else if (warp == 3) {
        // ------------------------------------------------------------ MMA issuer of the values
        if (lane == 0) {
            constexpr uint32_t ID_PV = idesc_bf16(128, PA_DV, 0, 1);
            bool ok = true;
            int cc = 0;                              // value tiles issued so far
            for (int k = 0; ok; k++) {
                int w;
                ok = next_item(k, w);
                if (!ok || w < 0) break;
                const AttnItem it = attn_item(w, p, nq);
                if (k > 0) {                         // the accumulator of the previous item has been read out
                    ok = mbar_wait(bar(PB_OFREE), (uint32_t)((k - 1) & 1), p.err, 1016);
                    if (!ok) break;
                }
                for (int i = 0; i < it.nt && ok; i++, cc++) {
                    const int cs = cc % PA_CST, cu = cc / PA_CST, pb = cc & 1, pu = cc >> 1;
                    ok = mbar_wait(bar(PB_CFULL + cs), (uint32_t)(cu & 1), p.err, 1014);
                    if (ok) ok = mbar_wait(bar(PB_PFULL + pb), (uint32_t)(pu & 1), p.err, 1015);
                    if (!ok) break;
                    tc_fence_after();
                    // values: O += P lat, P [128 q][64 keys] K-major, lat half [64 keys][256] with the 256 contiguous (MN-major, four 64-wide blocks)
                    const uint64_t dP = smem_desc(base + PA_OFF_P + pb * PA_P_BYTES, 16, 1024);
                    const uint64_t dC = smem_desc(base + PA_OFF_C + cs * PA_C_BYTES, PA_KT * 128, 1024);
#pragma unroll
                    for (int s = 0; s < 4; s++)
                        umma_bf16(tmem + PA_COL_O, dP + (uint64_t)((s * 32) >> 4), dC + (uint64_t)((s * 2048) >> 4), ID_PV, (s != 0) ? 1u : (uint32_t)(i != 0));
                    umma_commit(bar(PB_CEMPTY + cs));
                    umma_commit(bar(PB_PEMPTY + pb));
                }
                if (ok) umma_commit(bar(PB_ODONE));
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------ softmax, (correction,) epilogue
        // A thread owns query row `row` (= its TMEM lane) and NC of a tile's 64 key columns.
        constexpr int NC = PA_KT / NWG;
        const int q4 = warp & 3, wg = (warp - 4) >> 2;
        const int row = q4 * 32 + lane;
        const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
        bool ok = true;
        int tc = 0;                                  // tiles done so far (score buffer, P buffer and their phases run across items)
        for (int k = 0; ok; k++) {
            int w;
            ok = next_item(k, w);
            if (!ok || w < 0) break;
            const AttnItem it = attn_item(w, p, nq);
            const int q0 = it.q0, h = it.h, half = it.half, nt = it.nt;
            const int64_t tq = p.pos0 + q0 + row;                    // this row's position: keys 0..tq are visible
            // The query tile is the A operand of every score MMA of the item; it is kept in tensor memory (row = lane, two
            // consecutive bf16 per 32-bit column), so that those MMAs read only the keys from shared memory. A thread
            // copies its row's share: DQK / 2 columns split between the copying groups. The tile of item k + 1 is copied
            // BEFORE the epilogue of item k (below), so that the next item's first scores are computed under that epilogue.
            auto load_query = [&](int q0_, int h_) {
                constexpr int QG = (NWG == 4 && ((PA_DQK / 2) / 4) % 16 != 0) ? 2 : NWG;      // groups that copy (16-word stores)
                constexpr int QW = (PA_DQK / 2) / QG;                // 32-bit words per copying thread
                const int t = q0_ + row;
                const uint4 *src = reinterpret_cast<const uint4 *>(p.q + ((int64_t)t * p.nh + h_) * PA_DQK) + wg * (QW / 4);
#pragma unroll
                for (int c = 0; c < (wg < QG ? QW / 16 : 0); c++) {
                    uint32_t wv[16];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const uint4 v = (t < p.n) ? src[c * 4 + j] : make_uint4(0, 0, 0, 0);
                        wv[4 * j] = v.x; wv[4 * j + 1] = v.y; wv[4 * j + 2] = v.z; wv[4 * j + 3] = v.w;
                    }
                    TMEM_ST16(wv, 0, tlane + PA_COL_Q + wg * QW + c * 16);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                mbar_arrive(bar(PB_QFULL));
            };
            if (k == 0) load_query(q0, h);
            float m = 0.f, l = 0.f;
            for (int i = 0; i < nt && ok; i++, tc++) {
                const int sb = tc & 1, su = tc >> 1;             // P buffer of this tile
                const int s3 = tc % PA_SBUF;                      // its score buffer
                ok = __all_sync(0xffffffffu, mbar_wait(bar(PB_SFULL + s3), (uint32_t)((tc / PA_SBUF) & 1), p.err, 1021));   // warp-uniform: the TMEM loads below are warp-wide
                if (!ok) break;
                tc_fence_after();
                uint32_t v[NC];
#pragma unroll
                for (int c = 0; c < NC / 16; c++) TMEM_LD16(v, c * 16, tlane + PA_COL_S + s3 * PA_KT + wg * NC + c * 16);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                tc_fence_before();
                mbar_arrive(bar(PB_SEMPTY + s3));
                float s[NC];
                float mt = -INFINITY;
                const int64_t k0 = (int64_t)i * PA_KT + wg * NC;
                if ((int64_t)i * PA_KT + PA_KT - 1 <= p.pos0 + q0) {   // every key of the tile is visible to every row of the item
#pragma unroll
                    for (int j = 0; j < NC; j++) { s[j] = __uint_as_float(v[j]) * p.scale_log2; mt = fmaxf(mt, s[j]); }
                } else {
#pragma unroll
                    for (int j = 0; j < NC; j++) {
                        s[j] = (k0 + j <= tq) ? __uint_as_float(v[j]) * p.scale_log2 : -INFINITY;
                        mt = fmaxf(mt, s[j]);
                    }
                }
                if (NWG >= 2) {
                    if (i == 0) {                                    // reference exponent of the row: its largest score of the first tile
                        s_m[wg * 128 + row] = mt;
                        mbar_arrive(bar(PB_XM));
                        ok = mbar_wait(bar(PB_XM), (uint32_t)(k & 1), p.err, 1026);
                        if (!ok) break;
                        m = fmaxf(s_m[row], s_m[128 + row]);         // key 0 is visible to every row: finite
                        if (NWG == 4) m = fmaxf(m, fmaxf(s_m[256 + row], s_m[384 + row]));
                    } else if (mt > m + PA_RANGE) {
                        p.flags[w] = 1;                              // out of the range this form covers: the exact form redoes the item
                        atomicAdd(p.counter + 2, 1);
                    }
                } else {
                    // tcgen05.ld / st are warp-wide instructions: the warp decides together, and a lane that has no
                    // need of it rescales by 1
                    const bool mine = (i != 0) && (mt > m + PA_LAZY);
                    if (i == 0) m = mt;
                    if (__any_sync(0xffffffffu, mine)) {
                        // some row's scores outran its reference exponent: rescale what it has accumulated. A row is its
                        // thread's TMEM lane; the value MMAs of the previous tile must have finished writing it.
                        ok = mbar_wait(bar(PB_PEMPTY + ((tc - 1) & 1)), (uint32_t)(((tc - 1) >> 1) & 1), p.err, 1022);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        tc_fence_after();
                        const float alpha = mine ? exp2f(m - mt) : 1.f;
                        l *= alpha;
                        if (mine) m = mt;
                        for (int c = 0; c < PA_DV / 16; c++) {
                            uint32_t o[16];
                            TMEM_LD16(o, 0, tlane + PA_COL_O + c * 16);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                            for (int j = 0; j < 16; j++) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
                            TMEM_ST16(o, 0, tlane + PA_COL_O + c * 16);
                        }
                        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    }
                }
                uint32_t pk[NC / 2];
                float lsum = 0.f;
#pragma unroll
                for (int j = 0; j < NC; j += 2) {
                    const float p0 = exp2f(s[j] - m), p1 = exp2f(s[j + 1] - m);
                    lsum += p0 + p1;
                    pk[j >> 1] = pack_bf16x2(p0, p1);
                }
                l += lsum;
                // the P buffer of this parity was read by the value MMAs two tiles ago
                ok = mbar_wait(bar(PB_PEMPTY + sb), (uint32_t)((su & 1) ^ 1), p.err, 1023);
                if (!ok) break;
                uint8_t *prow = sm + PA_OFF_P + sb * PA_P_BYTES + row * 128;
#pragma unroll
                for (int c = 0; c < NC / 8; c++)
                    *reinterpret_cast<uint4 *>(prow + (((wg * (NC / 8) + c) ^ (row & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tc_fence_before();
                mbar_arrive(bar(PB_PFULL + sb));
            }
            if (!ok) break;
            {
                // the next item's query tile: the score MMAs of this item are done with theirs (they precede its last value MMAs)
                int wn;
                ok = next_item(k + 1, wn);
                if (!ok) break;
                if (wn >= 0) {
                    ok = mbar_wait(bar(PB_QEMPTY), (uint32_t)(k & 1), p.err, 1025);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    const AttnItem nx = attn_item(wn, p, nq);
                    load_query(nx.q0, nx.h);
                }
            }
            // ---- epilogue of the item: O / l -> bf16 -> out[t][h][half * 256 ..], full lines through a staging tile
            ok = mbar_wait(bar(PB_ODONE), (uint32_t)(k & 1), p.err, 1024);
            if (!ok) break;
            tc_fence_after();
            if (NWG >= 2) {                                          // the row's sum is the groups' sums
                s_l[wg * 128 + row] = l;
                mbar_arrive(bar(PB_XL));
                ok = mbar_wait(bar(PB_XL), (uint32_t)(k & 1), p.err, 1027);
                if (!ok) break;
                l = s_l[row] + s_l[128 + row];
                if (NWG == 4) l += s_l[256 + row] + s_l[384 + row];
            }
            const float inv = l > 0.f ? 1.f / l : 0.f;
            uint8_t *stg = sm + PA_OFF_P + (warp - 4) * 4096;         // 4 KB per warp: [32 rows][128 B], in the P buffers (idle: the item's value MMAs are done, and the next item's P comes from these threads)
            const int t0w = q0 + q4 * 32;
            constexpr int EG = NWG > 2 ? 2 : NWG;                     // groups that write out (the staging tiles are the two P buffers: eight warps)
            constexpr int NCH = PA_DV / 64 / EG;                      // 64-column chunks per writing thread
#pragma unroll 1
            for (int c = 0; c < (wg < EG ? NCH : 0); c++) {
                const int col = (wg * NCH + c) * 64;
                uint32_t o[64];
                TMEM_LD16(o, 0, tlane + PA_COL_O + col);
                TMEM_LD16(o, 16, tlane + PA_COL_O + col + 16);
                TMEM_LD16(o, 32, tlane + PA_COL_O + col + 32);
                TMEM_LD16(o, 48, tlane + PA_COL_O + col + 48);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    uint4 wv;
                    wv.x = pack_bf16x2(__uint_as_float(o[8 * j]) * inv, __uint_as_float(o[8 * j + 1]) * inv);
                    wv.y = pack_bf16x2(__uint_as_float(o[8 * j + 2]) * inv, __uint_as_float(o[8 * j + 3]) * inv);
                    wv.z = pack_bf16x2(__uint_as_float(o[8 * j + 4]) * inv, __uint_as_float(o[8 * j + 5]) * inv);
                    wv.w = pack_bf16x2(__uint_as_float(o[8 * j + 6]) * inv, __uint_as_float(o[8 * j + 7]) * inv);
                    *reinterpret_cast<uint4 *>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) = wv;
                }
                __syncwarp();
#pragma unroll
                for (int r8 = 0; r8 < 8; r8++) {
                    const int rr = r8 * 4 + (lane >> 3), jj = lane & 7;
                    const uint4 wv = *reinterpret_cast<const uint4 *>(stg + rr * 128 + ((jj ^ (rr & 7)) << 4));
                    if (t0w + rr < p.n)
                        *reinterpret_cast<uint4 *>(p.out + ((int64_t)(t0w + rr) * p.nh + h) * (GQA ? PA_DV : PA_L) + half * PA_DV + col + jj * 8) = wv;
                }
                __syncwarp();
            }
            tc_fence_before();
            mbar_arrive(bar(PB_OFREE));                              // the value MMAs of the next item may overwrite the accumulator
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Key expansion: Kx[h][c][0:128] = W_uk[h] lat[c], Kx[h][c][128:192] = k_rope[c].
constexpr int KX_TOK = 128, KX_NOPE = 128;
constexpr int KX_W_BYTES = KX_NOPE * PA_L * 2;        // 131072: eight [128 d][64 l] blocks
constexpr int KX_A_BYTES = KX_TOK * 128 * 2;          // 32768: two [128 tok][64 l] blocks = one 128-wide chunk of the latent
constexpr int KX_OFF_W = 0, KX_OFF_A = KX_W_BYTES, KX_OFF_STG = KX_OFF_A + 2 * KX_A_BYTES, KX_OFF_BAR = KX_OFF_STG + 4 * 4096;
constexpr int KX_SMEM = KX_OFF_BAR + 256 + 1024;
enum { KB_WFULL = 0, KB_AFULL = 1, KB_AEMPTY = 3, KB_DFULL = 5, KB_DEMPTY = 7, KB_COUNT = 9 };

struct KexpParams {
    const uint16_t *cache;    // bf16 [T][576]
    uint16_t *kx;             // bf16 [nh][T][192]: head-major, so that a head's key tile is one contiguous 24 KB
    int T, nh;
    int *err;
};

__global__ void __launch_bounds__(256, 1)
kexp_tc_kernel(const __grid_constant__ CUtensorMap tm_lat, const __grid_constant__ CUtensorMap tm_w, const KexpParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const uint32_t bar0 = base + KX_OFF_BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(sm + KX_OFF_BAR + 8 * KB_COUNT + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y;
    const int ntiles = (p.T + KX_TOK - 1) / KX_TOK;
    const int nt = (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;     // tiles g, g + G, ...
    if (nt <= 0) return;
    const int nch = nt * 4;                                                              // 128-wide chunks of the 512 latent dims

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_lat) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
        for (int i = 0; i < KB_COUNT; i++) mbar_init(bar(i), i >= KB_DEMPTY ? 128u : 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(bar(KB_WFULL), KX_W_BYTES);
            tma_load_3d(base + KX_OFF_W, &tm_w, 0, h * KX_NOPE, 0, bar(KB_WFULL));
            bool ok = true;
            int issued = 0;
            for (int c = 0; c < nch && ok; c++) {
                const int slot = c & 1, use = c >> 1;
                ok = mbar_wait(bar(KB_AEMPTY + slot), (uint32_t)((use & 1) ^ 1), p.err, 1101);
                if (!ok) break;
                const int tile = (int)blockIdx.x + (c >> 2) * (int)gridDim.x;
                mbar_expect_tx(bar(KB_AFULL + slot), KX_A_BYTES);
                tma_load_3d(base + KX_OFF_A + slot * KX_A_BYTES, &tm_lat, 0, tile * KX_TOK, (c & 3) * 2, bar(KB_AFULL + slot));
                issued = c + 1;
            }
            if (!ok) {
                mbar_wait(bar(KB_WFULL), 0, p.err, 1102);
                for (int c = (issued > 2 ? issued - 2 : 0); c < issued; c++) mbar_wait(bar(KB_AFULL + (c & 1)), (uint32_t)((c >> 1) & 1), p.err, 1103);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t ID = idesc_bf16(128, KX_NOPE, 0, 0);
            const uint64_t dW = smem_desc(base + KX_OFF_W, 16, 1024);
            bool ok = mbar_wait(bar(KB_WFULL), 0, p.err, 1104);
            for (int c = 0; c < nch && ok; c++) {
                const int slot = c & 1, use = c >> 1, ti = c >> 2, kc = c & 3, db = ti & 1;
                if (kc == 0) ok = mbar_wait(bar(KB_DEMPTY + db), (uint32_t)(((ti >> 1) & 1) ^ 1), p.err, 1105);
                if (ok) ok = mbar_wait(bar(KB_AFULL + slot), (uint32_t)(use & 1), p.err, 1106);
                if (!ok) break;
                tc_fence_after();
                const uint64_t dA = smem_desc(base + KX_OFF_A + slot * KX_A_BYTES, 16, 1024);
#pragma unroll
                for (int s = 0; s < 8; s++)       // chunk kc covers W blocks 2 kc and 2 kc + 1
                    umma_bf16(tmem + db * KX_NOPE, dA + (uint64_t)(((s >> 2) * (KX_TOK * 128) + (s & 3) * 32) >> 4),
                              dW + (uint64_t)((((kc * 2 + (s >> 2)) * (KX_NOPE * 128)) + (s & 3) * 32) >> 4), ID, (kc | s) != 0);
                umma_commit(bar(KB_AEMPTY + slot));
                if (kc == 3) umma_commit(bar(KB_DFULL + db));
            }
        }
    } else if (warp >= 4) {
        const int q4 = warp & 3;
        const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
        uint8_t *stg = sm + KX_OFF_STG + q4 * 4096;
        bool ok = true;
        for (int ti = 0; ti < nt && ok; ti++) {
            const int db = ti & 1;
            const int t0w = ((int)blockIdx.x + ti * (int)gridDim.x) * KX_TOK + q4 * 32;
            // rope tail first (independent of the MMAs): 128 bytes per token, eight lanes per row
#pragma unroll
            for (int r8 = 0; r8 < 8; r8++) {
                const int rr = r8 * 4 + (lane >> 3), jj = lane & 7;
                if (t0w + rr < p.T) {
                    const uint4 w = *reinterpret_cast<const uint4 *>(p.cache + (int64_t)(t0w + rr) * PA_ROW + PA_L + jj * 8);
                    *reinterpret_cast<uint4 *>(p.kx + ((int64_t)h * p.T + t0w + rr) * PaMla::DQK + KX_NOPE + jj * 8) = w;
                }
            }
            ok = mbar_wait(bar(KB_DFULL + db), (uint32_t)((ti >> 1) & 1), p.err, 1107);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < 2; c++) {
                uint32_t v[64];
                TMEM_LD16(v, 0, tlane + db * KX_NOPE + c * 64);
                TMEM_LD16(v, 16, tlane + db * KX_NOPE + c * 64 + 16);
                TMEM_LD16(v, 32, tlane + db * KX_NOPE + c * 64 + 32);
                TMEM_LD16(v, 48, tlane + db * KX_NOPE + c * 64 + 48);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    uint4 w;
                    w.x = pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
                    w.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                    w.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                    w.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                    *reinterpret_cast<uint4 *>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) = w;
                }
                __syncwarp();
#pragma unroll
                for (int r8 = 0; r8 < 8; r8++) {
                    const int rr = r8 * 4 + (lane >> 3), jj = lane & 7;
                    const uint4 w = *reinterpret_cast<const uint4 *>(stg + rr * 128 + ((jj ^ (rr & 7)) << 4));
                    if (t0w + rr < p.T)
                        *reinterpret_cast<uint4 *>(p.kx + ((int64_t)h * p.T + t0w + rr) * PaMla::DQK + c * 64 + jj * 8) = w;
                }
                __syncwarp();
            }
            tc_fence_before();
            mbar_arrive(bar(KB_DEMPTY + db));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
    }
}

bool encode3(CUtensorMap *tm, const void *ptr, uint64_t rows, uint64_t blocks, uint64_t row_bytes, uint32_t box_rows, uint32_t box_blocks) {
    CwkEncodeTiledFn enc = cwk_encode_tiled_fn();
    if (!enc) return false;
    cuuint64_t dims[3] = {64, rows, blocks};
    cuuint64_t strides[2] = {row_bytes, 128};
    cuuint32_t box[3] = {64, box_rows, box_blocks};
    cuuint32_t es[3] = {1, 1, 1};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Whether cwk_mla_prefill_attn_tc can take these operands (asked before the caller rotates Q in place).
bool cwk_mla_prefill_attn_tc_ok(const void *Q, const void *cache, const void *Wuk, const void *kx, const void *out) {
    if (!cwk_encode_tiled_fn()) return false;
    return ((reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(Wuk) | reinterpret_cast<uintptr_t>(kx) |
             reinterpret_cast<uintptr_t>(out)) & 15) == 0;
}

// Q bf16 [n][nh][192] with the rope part already rotated; cache bf16 [pos0 + n][576] (latent | rope key);
// Wuk bf16 [nh][128][512]; kx = workspace bf16 [nh][pos0 + n][192]; flags = workspace int32, one per item of the
// attention (ceil(n / 128) x nh x 2) plus three counters; out bf16 [n][nh][512]. exact_only: skip the fast form and run
// the exact form on every item (for tests).
// Returns CWK_ERR_UNSUPPORTED (no error text) when the tensor path cannot run.
int cwk_mla_prefill_attn_tc(cwk_ctx *ctx, const void *Q, const void *cache, const void *Wuk, void *kx, int *flags, int64_t pos0, int n, int nh,
                            float scale, void *out, int exact_only) {
    if (!cwk_encode_tiled_fn()) return CWK_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(cache) | reinterpret_cast<uintptr_t>(Wuk) | reinterpret_cast<uintptr_t>(kx) |
         reinterpret_cast<uintptr_t>(out)) & 15)
        return CWK_ERR_UNSUPPORTED;
    int s = cwk_ensure_err_word(ctx);
    if (s != CWK_OK) return s;
    const int T = (int)(pos0 + n);
    CUtensorMap tm_lat, tm_w, tm_k, tm_c;
    if (!encode3(&tm_lat, cache, (uint64_t)T, PA_L / 64, PA_ROW * 2, KX_TOK, 2) ||                 // latent dims only: block index 8 (rope) stays out
        !encode3(&tm_w, Wuk, (uint64_t)nh * KX_NOPE, PA_L / 64, PA_L * 2, KX_NOPE, PA_L / 64) ||
        !encode3(&tm_k, kx, (uint64_t)nh * T, 3, PaMla::DQK * 2, PA_KT, 3) ||            // rows past a head's last key belong to the next head: every such key is masked

        !encode3(&tm_c, cache, (uint64_t)T, PA_L / 64, PA_ROW * 2, PA_KT, 4))
        return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled failed for the prefill attention operands");
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(kexp_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, KX_SMEM));
        CWK_CUDA(ctx, cudaFuncSetAttribute(prefill_attn_kernel<1, PaMla, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PaMla::SMEM));
        CWK_CUDA(ctx, cudaFuncSetAttribute(prefill_attn_kernel<4, PaMla, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PaMla::SMEM));
        attr_set[ctx->device & 15] = true;
    }
    {
        KexpParams kp;
        kp.cache = (const uint16_t *)cache; kp.kx = (uint16_t *)kx; kp.T = T; kp.nh = nh; kp.err = ctx->dev_err;
        const int ntiles = (T + KX_TOK - 1) / KX_TOK;
        const int G = std::max(1, std::min(ntiles, ctx->sm_count / std::max(1, nh)));
        CwkKernelTimer timer(ctx);
        kexp_tc_kernel<<<dim3(G, nh), 256, KX_SMEM, ctx->stream>>>(tm_lat, tm_w, kp);
        CWK_LAUNCH_CHECK(ctx, "kexp_tc_kernel");
    }
    {
        AttnParams ap;
        ap.q = (const uint16_t *)Q; ap.out = (uint16_t *)out; ap.n = n; ap.nh = nh; ap.T = T; ap.pos0 = pos0; ap.group = 1; ap.scale_log2 = scale * 1.4426950408889634f; ap.flags = flags;
        ap.err = ctx->dev_err;
        const int total = ((n + PA_QT - 1) / PA_QT) * nh * 2;
        ap.counter = flags + total;
        CWK_CUDA(ctx, cudaMemsetAsync(flags, 0, (size_t)(total + 3) * sizeof(int), ctx->stream));
        if (exact_only) {       // every item flagged (any non-zero word), the flag count non-zero, the two item counters back to zero
            CWK_CUDA(ctx, cudaMemsetAsync(flags, 1, (size_t)(total + 3) * sizeof(int), ctx->stream));
            CWK_CUDA(ctx, cudaMemsetAsync(flags + total, 0, 2 * sizeof(int), ctx->stream));
        }
        const int grid = std::min(total, ctx->sm_count);
        if (!exact_only) {
            CwkKernelTimer timer(ctx);
            prefill_attn_kernel<4, PaMla, false><<<grid, 640, PaMla::SMEM, ctx->stream>>>(tm_k, tm_c, ap);
            CWK_LAUNCH_CHECK(ctx, "prefill_attn_kernel<4>");
        }
        // the repair pass: items whose flag is clear are skipped
        prefill_attn_kernel<1, PaMla, false><<<grid, 256, PaMla::SMEM, ctx->stream>>>(tm_k, tm_c, ap);
        CWK_LAUNCH_CHECK(ctx, "prefill_attn_kernel<1>");
    }
    return CWK_OK;
}

// Causal GQA prefill on the same kernel (Qwen3.5 full-attention layers, src/q35_model.c:1713-1746): per query head,
// 128 consecutive queries are the MMA's rows; keys and values are the 256-wide rows of the head's KV head, streamed in
// 64-key tiles by TMA straight from the caches. Q bf16 [n][nh][256]; K, V bf16 [pos + n][nkv][256]; out bf16
// [n][nh][256]; flags = workspace int32 [ceil(n / 128) * nh + 3]. Returns CWK_ERR_UNSUPPORTED (no error text) when the
// tensor path cannot take the operands.
int cwk_gqa_prefill_tc(cwk_ctx *ctx, const void *Q, const void *K, const void *V, int64_t pos, int n, int nh, int nkv, int hd,
                       float scale, void *out, int *flags) {
    if (!cwk_encode_tiled_fn() || hd != 256 || nkv <= 0 || nh % nkv) return CWK_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(K) | reinterpret_cast<uintptr_t>(V) | reinterpret_cast<uintptr_t>(out)) & 15)
        return CWK_ERR_UNSUPPORTED;
    int s = cwk_ensure_err_word(ctx);
    if (s != CWK_OK) return s;
    const int T = (int)(pos + n);
    CUtensorMap tm_k, tm_v;
    // the caches as [64][rows][nkv * 4 column blocks]: a tile is one box of 64 keys x the 4 blocks of one KV head
    if (!encode3(&tm_k, K, (uint64_t)T, (uint64_t)nkv * 4, (uint64_t)nkv * hd * 2, PA_KT, 4) ||
        !encode3(&tm_v, V, (uint64_t)T, (uint64_t)nkv * 4, (uint64_t)nkv * hd * 2, PA_KT, 4))
        return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled failed for the GQA prefill operands");
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(prefill_attn_kernel<1, PaGqa, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PaGqa::SMEM));
        CWK_CUDA(ctx, cudaFuncSetAttribute(prefill_attn_kernel<2, PaGqa, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PaGqa::SMEM));
        attr_set[ctx->device & 15] = true;
    }
    AttnParams ap;
    ap.q = (const uint16_t *)Q; ap.out = (uint16_t *)out; ap.n = n; ap.nh = nh; ap.T = T; ap.pos0 = pos; ap.group = nh / nkv;
    ap.scale_log2 = scale * 1.4426950408889634f; ap.flags = flags; ap.err = ctx->dev_err;
    const int total = ((n + PA_QT - 1) / PA_QT) * nh;
    ap.counter = flags + total;
    CWK_CUDA(ctx, cudaMemsetAsync(flags, 0, (size_t)(total + 3) * sizeof(int), ctx->stream));
    const int grid = std::min(total, ctx->sm_count);
    {
        CwkKernelTimer timer(ctx);
        prefill_attn_kernel<2, PaGqa, true><<<grid, 384, PaGqa::SMEM, ctx->stream>>>(tm_k, tm_v, ap);
        CWK_LAUNCH_CHECK(ctx, "prefill_attn_kernel<2, gqa>");
    }
    prefill_attn_kernel<1, PaGqa, true><<<grid, 256, PaGqa::SMEM, ctx->stream>>>(tm_k, tm_v, ap);      // repairs flagged items only
    CWK_LAUNCH_CHECK(ctx, "prefill_attn_kernel<1, gqa>");
    return CWK_OK;
}
