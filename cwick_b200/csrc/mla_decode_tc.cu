// mla_decode_tc.cu -- MLA absorbed decode on the Blackwell tensor path:
// TMA-staged cache tiles, tcgen05.mma with accumulators in tensor memory.
//
// Shape: 64 heads, 512-d latent + 64-d rope key, bf16. The 64 heads are too few
// rows for a full-rate MMA (M = 128), so both products are issued transposed,
// with the 128 TOKENS of a tile as the MMA's M dimension:
//
//   S^T[128 tok][64 heads] = K[128 tok][576] . Q[64 heads][576]^T        (A, B K-major)
//   O^T[512 dv ][64 heads] += V^T[512 dv][128 tok] . P^T[128 tok][64 heads]   (A, B MN-major)
//
// K and V are the same shared-memory bytes: a tile is nine [128 tok][64 dim]
// blocks (8 latent + 1 rope) written by TMA with the 128-byte swizzle, read
// K-major for the first product and MN-major for the second. P^T (bf16) is
// written by the softmax warps into the rope block's slot, which is dead once
// S^T is complete. Tensor memory holds O^T (4 x 64 columns) and S^T (64).
//
// One tile is resident at a time (Q 72 KB + tile 144 KB of the 227 KB), and its
// blocks are recycled as soon as the second product has consumed them, so the
// next tile streams in behind the MMAs of this one. A TMA operation costs some
// 400 cycles however small its box, and operations of one block queue behind one
// another, so the cache is described as [64][rows][9 blocks] and a tile arrives
// as three boxes of two column blocks (32 KB) and one of three (the last latent pair with the
// rope block, which come free together); Q is one box.
//
// Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps
// 4..19 = softmax / correction / epilogue: four groups of four warps, 16 heads
// each (TMEM lane quarter = warp % 4). The exponentials of a tile are computed
// against the current reference exponents before the block agrees (one barrier
// with an OR reduction) on whether any score outran them; only then are they
// redone.
// Every mbarrier wait is bounded; a wait that gives up records a code in a
// device word and the block tears down (TMEM freed, copies drained).
#include <cuda.h>

#include <algorithm>

#include "tc_common.cuh"

namespace {

constexpr int NH = 64, L = 512, DK = 576;
constexpr int TILE = 128;                       // tokens per tile = MMA M
constexpr int NBLK = 9;                         // 64-element column blocks per row
constexpr int RP = 8;                           // index of the rope block / P^T slot
constexpr int KV_BLK = TILE * 128;              // 16384 B
constexpr int Q_BLK = NH * 128;                 // 8192 B
constexpr int OFF_Q = 0;
constexpr int OFF_KV = NBLK * Q_BLK;            // 73728
constexpr int OFF_BAR = OFF_KV + NBLK * KV_BLK; // 221184
constexpr int OFF_MISC = OFF_BAR + 256;
constexpr int SMEM_USED = OFF_MISC + 2048;
constexpr int SMEM_TOTAL = SMEM_USED + 1024;    // slack to align the base to 1024 B
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_O = 0, COL_S = 256;
constexpr int HG = 16;                          // heads per softmax warp group
constexpr int NG = NH / HG;                     // 4 groups of four warps
constexpr float LAZY_LOG2 = 16.f;               // a score may outrun the reference exponent by 2^16 before a rescale
constexpr int NSOFT = NG * 128;                 // 512 softmax threads
constexpr int NTHREADS = 128 + NSOFT;           // 640

// barrier slots (8 bytes each) inside OFF_BAR
enum { B_FULL = 0, B_EMPTY_L = 9, B_EMPTY_RP = 13, B_QFULL = 14, B_SFULL = 15, B_PFULL = 16, B_COUNT = 17 };

__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

// v[0..15] per lane -> lane L returns the reduction over the 32 lanes of v[L & 15]: the two half-warps
// are folded first, then the live values halve at every stage (31 shuffles in all).
template <bool IS_MAX>
__device__ __forceinline__ float warp_transpose_reduce16(float (&v)[16], int lane) {
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const float r = __shfl_xor_sync(0xffffffffu, v[i], 16);
        v[i] = IS_MAX ? fmaxf(v[i], r) : v[i] + r;
    }
#pragma unroll
    for (int off = 8; off >= 1; off >>= 1) {
        const bool hi = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < off; i++) {
            const float send = hi ? v[i] : v[i + off];
            const float keep = hi ? v[i + off] : v[i];
            const float recv = __shfl_xor_sync(0xffffffffu, send, off);
            v[i] = IS_MAX ? fmaxf(keep, recv) : keep + recv;
        }
    }
    return v[0];
}
struct TcParams {
    const int32_t *kv_len; // [B] device, or NULL: every sequence has kv_len_imm rows
    int kv_len_imm;
    float *partial;        // [B][nsplit][NH*(L+2)]
    int nsplit;
    float scale_log2;
    int *err;              // device word, 0 = fine
    int batch_coord_zero;  // all sequences read cache slice 0 (shared cache)
    uint16_t *out;         // direct mode (nsplit == 1): normalised bf16 [B][NH][L]; NULL = write partial records
    int reverse_b;         // schedule sequences last-to-first (causal prefill: longest first)
    int halves;            // 2: blockIdx.z picks one half of the 512 value columns (two blocks share a tile's scores)
    int stagger;           // cycles between the start times of eight groups of blocks (0 = all at once)
    // gather mode (sel != NULL): the tile's rows are cache rows sel[b][j], fetched with 16-byte asynchronous copies into
    // the same swizzled blocks the tiled loads fill (a TMA box cannot follow a row list): the first tile by the 16
    // softmax warps, which have nothing else to do yet, the following ones by two otherwise idle warps
    const int32_t *sel;    // [B][sel_ld] device
    int64_t sel_ld;
    const uint16_t *cache;
    int64_t seq_stride, ld;
    int rope_cols;         // 64, or 0: the ninth block is zeros
#ifdef CWK_TRACE
    long long *trace;      // developer build only: per-phase clock64 stamps of block (0,0); NULL = off
#endif
};

__global__ void __launch_bounds__(NTHREADS, 1)
mla_decode_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                     const __grid_constant__ CUtensorMap tm_kr, const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;             // 1024-byte aligned (swizzle atom)
    uint8_t *sm = smem_raw + (base - raw);
    const uint32_t bar0 = base + OFF_BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(sm + OFF_MISC);
    float *s_mref = reinterpret_cast<float *>(sm + OFF_MISC + 128);   // [64]
    float *s_alpha = s_mref + 64;                                     // [64]
    float *s_w = s_alpha + 64;                                        // [16 warps][16] per-warp max / sum

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, b = p.reverse_b ? (int)(gridDim.y - 1 - blockIdx.y) : (int)blockIdx.y;
    // With few blocks in the launch (one short sequence), two blocks take each tile: both compute the tile's scores
    // and probabilities, each accumulates and writes one half of the value columns. Half the value MMAs per block,
    // and the records leave through twice as many SMs.
    const int mb0 = p.halves == 2 ? 2 * (int)blockIdx.z : 0, mb1 = p.halves == 2 ? mb0 + 2 : 4;
    const int kv = p.kv_len ? p.kv_len[b] : p.kv_len_imm;
    const int ntiles = (kv + TILE - 1) / TILE;
    const int t0 = (int)((int64_t)ntiles * split / p.nsplit);
    const int t1 = (int)((int64_t)ntiles * (split + 1) / p.nsplit);
    const int n = t1 - t0;
    float *rec = p.partial + ((int64_t)b * p.nsplit + split) * (int64_t)(NH * (L + 2));

    if (n <= 0) {                       // empty split: a record the merge ignores (direct mode: zeros)
        if (p.out) {
            for (int i = tid; i < NH * L / 2; i += NTHREADS) reinterpret_cast<uint32_t *>(p.out + (int64_t)b * NH * L)[i] = 0u;
        } else {
            for (int i = tid; i < NH * (L + 2); i += NTHREADS) rec[i] = (i < NH) ? -INFINITY : 0.f;
        }
        return;
    }

    const int bz = p.batch_coord_zero ? 0 : b;
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_kv) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_kr) : "memory");
        for (int i = 0; i < B_COUNT; i++)
            mbar_init(bar(i), i == B_PFULL ? (uint32_t)NSOFT : (p.sel && i < B_EMPTY_L) ? (uint32_t)NSOFT : 1u);      // gather: 512 arrivals fill a block
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // A full wave of blocks with many tiles each: blocks that start together stay in lockstep for their first tiles
        // (every SM loads, then every SM computes, and HBM idles through the compute phases: 10 k cycles per tile against
        // 7 k once they have drifted apart), so eight groups of blocks start a fraction of a tile period apart.
        // Blocks that have one tile more than the others start first when they are few; when they are most of the
        // launch they are the ones to spread.
        if (p.stagger) {
            const int nlong = ntiles % p.nsplit;                            // blocks with one tile more (0: all alike)
            const bool longest = nlong != 0 && n == (ntiles + p.nsplit - 1) / p.nsplit;
            int group;
            if (nlong == 0) group = (split + 3 * b) & 7;
            else if (nlong * 4 <= p.nsplit) group = longest ? 0 : 1 + (split + 3 * b) % 7;      // a few long blocks: they go first
            else group = longest ? (split + 3 * b) % 7 : 7;                 // mostly long blocks: they spread, the few short ones last
            const long long until = clock64() + (long long)group * p.stagger;
            while (clock64() < until) { }
        }
        // The first tile's loads go out before the block-wide set-up (TMEM allocation, the
        // barrier below): nothing they touch depends on it, and their latency is the longest
        // single item of a short call.
        mbar_expect_tx(bar(B_QFULL), NBLK * Q_BLK);
        tma_load_3d(base + OFF_Q, &tm_q, 0, b * NH, 0, bar(B_QFULL));
        if (!p.sel) {
            for (int k = 0; k < 6; k += 2) {
                mbar_expect_tx(bar(B_FULL + k), 2 * KV_BLK);
                tma_load_4d(base + OFF_KV + k * KV_BLK, &tm_kv, 0, t0 * TILE, k, bz, bar(B_FULL + k));
            }
            mbar_expect_tx(bar(B_FULL + 6), 3 * KV_BLK);
            tma_load_4d(base + OFF_KV + 6 * KV_BLK, &tm_kr, 0, t0 * TILE, 6, bz, bar(B_FULL + 6));
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;
#ifdef CWK_TRACE
    // trace slots: [role][tile][event]; only block (0,0) writes
    long long *tr = (p.trace && split == 0 && blockIdx.y == 0) ? p.trace : nullptr;
#define TRACE(role, it, ev) do { if (tr && (it) < 16) tr[((role) * 16 + (it)) * 8 + (ev)] = clock64(); } while (0)
    if (tr && tid == 0) tr[3 * 16 * 8] = clock64();
#else
#define TRACE(role, it, ev) do { } while (0)
#endif

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0 && !p.sel) {
            bool ok = true;
            int issued_it[NBLK];
            for (int k = 0; k < NBLK; k++) issued_it[k] = 0;      // tile 0 went out during set-up
            for (int it = 1; it < n && ok; it++) {
                const uint32_t par_free = (uint32_t)((it & 1) ^ 1);
                const int row = (t0 + it) * TILE;
                for (int k = 0; k < 8 && ok; k += 2) {
                    ok = mbar_wait(bar(B_EMPTY_L + (k >> 1)), par_free, p.err, 102);
                    // the last latent pair and the rope block (= the P^T slot) come free together, at the end of
                    // the second product, and return as one box of three blocks
                    if (ok && k == 6) ok = mbar_wait(bar(B_EMPTY_RP), par_free, p.err, 101);
                    if (!ok) break;
                    if (k == 0) TRACE(0, it, 0);
                    if (k == 2) TRACE(0, it, 2);
                    if (k == 4) TRACE(0, it, 3);
                    if (k == 6) TRACE(0, it, 1);
                    if (k == 6) {
                        mbar_expect_tx(bar(B_FULL + k), 3 * KV_BLK);
                        tma_load_4d(base + OFF_KV + k * KV_BLK, &tm_kr, 0, row, k, bz, bar(B_FULL + k));
                    } else {
                        mbar_expect_tx(bar(B_FULL + k), 2 * KV_BLK);
                        tma_load_4d(base + OFF_KV + k * KV_BLK, &tm_kv, 0, row, k, bz, bar(B_FULL + k));
                    }
                    issued_it[k] = it;
                }
            }
            if (!ok) {      // drain: do not leave the block with bulk copies in flight
                mbar_wait(bar(B_QFULL), 0, p.err, 103);
                for (int k = 0; k < 8; k += 2)
                    if (issued_it[k] >= 0) mbar_wait(bar(B_FULL + k), (uint32_t)(issued_it[k] & 1), p.err, 104);
            }
        }
    } else if ((warp == 2 || warp == 3) && p.sel) {
        // ------------------------------------------------------------ gather producer (row lists)
        // 64 threads, two rows of the tile each: a row's 1152 bytes go out as 72 copies of 16 bytes, each to its place
        // in the 128-byte-swizzled block of its 64 columns. One commit group per pair of blocks (three for the last),
        // so that the score MMAs start on the first pair while the others are still arriving.
        const int pt = tid - 64;
        const uint16_t *cbase = p.cache + (p.batch_coord_zero ? 0 : (int64_t)b * p.seq_stride);
        const int32_t *selb = p.sel + (int64_t)b * p.sel_ld;
        bool ok = true;
        for (int it = 1; it < n && ok; it++) {          // (the first tile is fetched by the softmax warps, idle until its scores exist)
            const uint32_t par_free = (uint32_t)((it & 1) ^ 1);
            const uint16_t *src[2];
            bool val[2];
#pragma unroll
            for (int rr = 0; rr < 2; rr++) {
                const int j = (t0 + it) * TILE + pt + 64 * rr;
                val[rr] = j < kv;
                src[rr] = cbase + (int64_t)(val[rr] ? selb[j] : 0) * p.ld;
            }
#pragma unroll
            for (int k = 0; k < 8; k += 2) {
                ok = mbar_wait(bar(B_EMPTY_L + (k >> 1)), par_free, p.err, 105);
                if (ok && k == 6) ok = mbar_wait(bar(B_EMPTY_RP), par_free, p.err, 106);
                if (ok) {
#pragma unroll
                    for (int kb = k; kb < (k == 6 ? 9 : k + 2); kb++) {
#pragma unroll
                        for (int rr = 0; rr < 2; rr++) {
                            const int r = pt + 64 * rr;
                            const bool v = val[rr] && (kb < 8 || p.rope_cols != 0);
                            const uint32_t dst = base + OFF_KV + kb * KV_BLK + r * 128;
#pragma unroll
                            for (int c = 0; c < 8; c++)
                                cp_async16(dst + (uint32_t)((c ^ (r & 7)) << 4), src[rr] + kb * 64 + c * 8, v);
                        }
                    }
                }
                cp_async_commit();        // (an empty group after a failed wait keeps the counts below in step)
            }
            // a group's bytes are in shared memory -> visible to the tensor-core (asynchronous) proxy -> the block pair is full
            cp_async_wait<3>();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive_n(bar(B_FULL + 0), NSOFT / 64);
            cp_async_wait<2>();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive_n(bar(B_FULL + 2), NSOFT / 64);
            cp_async_wait<1>();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive_n(bar(B_FULL + 4), NSOFT / 64);
            cp_async_wait<0>();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive_n(bar(B_FULL + 6), NSOFT / 64);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t ID_QK = idesc_bf16(128, 64, 0, 0);
            constexpr uint32_t ID_PV = idesc_bf16(128, 64, 1, 1);
            // Descriptors are built once; every MMA adds a compile-time constant to the address field
            // (the issue loop is one thread, and its instruction count bounds the MMA rate at N = 64).
            const uint64_t dK = smem_desc(base + OFF_KV, 16, 1024), dQ = smem_desc(base + OFF_Q, 16, 1024);
            const uint64_t dV = smem_desc(base + OFF_KV, KV_BLK, 1024), dP = smem_desc(base + OFF_KV + RP * KV_BLK, KV_BLK, 1024);
            bool ok = mbar_wait(bar(B_QFULL), 0, p.err, 201);
            for (int it = 0; it < n && ok; it++) {
                const uint32_t par = (uint32_t)(it & 1);
                // S^T = K Q^T over the nine column blocks (4 k-steps of 16 each)
#pragma unroll
                for (int k = 0; k < NBLK; k++) {
                    if (ok && (k & 1) == 0 && k < 8) ok = mbar_wait(bar(B_FULL + k), par, p.err, 202);     // blocks arrive in pairs, the rope block with the last pair
                    if (ok) {
                        if (k == 0) TRACE(1, it, 0);
                        if (k == RP) TRACE(1, it, 1);
                        tc_fence_after();
#pragma unroll
                        for (int ks = 0; ks < 4; ks++)
                            umma_bf16(tmem + COL_S, dK + (uint64_t)((k * KV_BLK + ks * 32) >> 4), dQ + (uint64_t)((k * Q_BLK + ks * 32) >> 4),
                                      ID_QK, (k | ks) != 0);
                    }
                }
                if (!ok) break;
                umma_commit(bar(B_SFULL));
                TRACE(1, it, 2);
                // O^T += V^T P^T, four 128-row blocks of dv, 8 k-steps of 16 tokens each
                ok = mbar_wait(bar(B_PFULL), par, p.err, 203);
                if (!ok) break;
                TRACE(1, it, 3);
                tc_fence_after();
                const uint32_t acc0 = it != 0;
#pragma unroll
                for (int mb = 0; mb < 4; mb++) {
                    if (mb >= mb0 && mb < mb1) {
#pragma unroll
                        for (int ks = 0; ks < 8; ks++)
                            umma_bf16(tmem + COL_O + mb * 64, dV + (uint64_t)((2 * mb * KV_BLK + ks * 2048) >> 4), dP + (uint64_t)((ks * 2048) >> 4),
                                      ID_PV, ks != 0 ? 1u : acc0);
                    }
                    umma_commit(bar(B_EMPTY_L + mb));      // also for the other half's blocks: their slots are free once the scores are done
                }
                umma_commit(bar(B_EMPTY_RP));
                TRACE(1, it, 4);
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------ softmax / correction / epilogue
        // Four groups of four warps: group g owns heads [16g, 16g+16) (S^T / O^T columns); inside a
        // group, warp w owns TMEM lanes 32*(w%4).. = token rows (S^T) or dv rows (O^T).
        const int q = warp & 3;                       // TMEM lane quarter
        const int g = (warp - 4) >> 2;                // head group
        const int hb = g * HG;                        // first head of the group
        const int row = q * 32 + lane;                // token row inside the tile == TMEM lane
        const int st = tid - 128;                     // 0..511
        const uint32_t tlane = tmem + ((uint32_t)(q * 32) << 16);
        float lpart[HG];
#pragma unroll
        for (int h = 0; h < HG; h++) lpart[h] = 0.f;
        if (p.sel) {
            // gather mode: these 512 threads have nothing to do until the first tile's scores exist, so they fetch the
            // first tile (four threads per row; 16-byte copies into the swizzled blocks, one commit group per block pair)
            const int r = st >> 2, part = st & 3;
            const int j = t0 * TILE + r;
            const bool val = j < kv;
            const uint16_t *src = p.cache + (p.batch_coord_zero ? 0 : (int64_t)b * p.seq_stride) +
                                  (int64_t)(val ? p.sel[(int64_t)b * p.sel_ld + j] : 0) * p.ld;
            const uint32_t drow = base + OFF_KV + r * 128;
#pragma unroll
            for (int k = 0; k < 8; k += 2) {
                const int per = (k == 6) ? 6 : 4;                // 16-byte pieces of the pair (or triple) for this thread
#pragma unroll
                for (int x = 0; x < 6; x++) {
                    if (x < per) {
                        const int cc = part * per + x, kb = k + (cc >> 3), c = cc & 7;
                        cp_async16(drow + (uint32_t)(kb * KV_BLK) + (uint32_t)((c ^ (r & 7)) << 4), src + kb * 64 + c * 8,
                                   val && (kb < 8 || p.rope_cols != 0));
                    }
                }
                cp_async_commit();
            }
            cp_async_wait<3>();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(bar(B_FULL + 0));
            cp_async_wait<2>();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(bar(B_FULL + 2));
            cp_async_wait<1>();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(bar(B_FULL + 4));
            cp_async_wait<0>();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(bar(B_FULL + 6));
        }
        bool ok = true;
        for (int it = 0; it < n; it++) {
            ok = mbar_wait(bar(B_SFULL), (uint32_t)(it & 1), p.err, 301);
            if (!ok) break;
            if (st == 0) TRACE(2, it, 0);
            tc_fence_after();
            uint32_t sr[HG];
            TMEM_LD16(sr, 0, tlane + COL_S + hb);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (st == 0) TRACE(2, it, 5);
            const bool valid = (t0 + it) * TILE + row < kv;
            float s[HG];
#pragma unroll
            for (int h = 0; h < HG; h++) s[h] = valid ? __uint_as_float(sr[h]) * p.scale_log2 : -INFINITY;

            if (it == 0) {
                // Reference exponent per head: the score of the tile's first token. Any value works
                // as long as no score outruns it by more than 2^LAZY_LOG2 (checked next, every tile).
                if (row == 0) {
#pragma unroll
                    for (int h = 0; h < HG; h++) s_mref[hb + h] = s[h];
                }
                softmax_bar();
            }
            // Probabilities against the current reference exponent, computed BEFORE the block agrees on
            // whether a rescale is needed: the exponentials fill the time the barrier spends waiting for
            // the slowest warp, and in the common case (no rescale) they are the final values.
            float pv[HG];
            bool ex = false;
#pragma unroll
            for (int h = 0; h < HG; h += 4) {
                const float4 mr = *reinterpret_cast<const float4 *>(s_mref + hb + h);
                const float d0 = s[h] - mr.x, d1 = s[h + 1] - mr.y, d2 = s[h + 2] - mr.z, d3 = s[h + 3] - mr.w;
                ex |= (d0 > LAZY_LOG2) | (d1 > LAZY_LOG2) | (d2 > LAZY_LOG2) | (d3 > LAZY_LOG2);
                pv[h] = exp2f(d0); pv[h + 1] = exp2f(d1); pv[h + 2] = exp2f(d2); pv[h + 3] = exp2f(d3);
            }
            uint32_t need;
            asm volatile("{\n.reg .pred pi, po;\nsetp.ne.b32 pi, %1, 0;\nbar.red.or.pred po, 1, 512, pi;\nselp.u32 %0, 1, 0, po;\n}\n"
                         : "=r"(need) : "r"((uint32_t)ex) : "memory");
            if (st == 0) TRACE(2, it, 6);
            if (need) {
                // exact column maxima over the 128 tokens, new reference, rescale what exists
                float v[HG];
#pragma unroll
                for (int h = 0; h < HG; h++) v[h] = s[h];
                const float mine = warp_transpose_reduce16<true>(v, lane);   // lane L: max of head hb+(L&15) over this warp's rows
                if (lane < HG) s_w[(warp - 4) * HG + lane] = mine;
                softmax_bar();
                if (st < NH) {
                    const int gg = st / HG, hh = st % HG;
                    const float *w4 = s_w + gg * 4 * HG + hh;
                    const float M = fmaxf(fmaxf(w4[0], w4[HG]), fmaxf(w4[2 * HG], w4[3 * HG]));
                    const float mo = s_mref[st];
                    const float mn = fmaxf(mo, M);
                    s_alpha[st] = exp2f(mo - mn);
                    s_mref[st] = mn;
                }
                softmax_bar();
#pragma unroll
                for (int h = 0; h < HG; h++) lpart[h] *= s_alpha[hb + h];
                if (it > 0) {
                    // O^T columns are heads: scale column h of every dv block by alpha[h]
                    for (int mb = 0; mb < 4; mb++) {
                        uint32_t o[16];
                        const uint32_t ta = tlane + COL_O + mb * 64 + hb;
                        TMEM_LD16(o, 0, ta);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            o[j] = __float_as_uint(__uint_as_float(o[j]) * s_alpha[hb + j]);
                        TMEM_ST16(o, 0, ta);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
            }
            if (need) {         // the reference moved: probabilities against the new one
#pragma unroll
                for (int h = 0; h < HG; h++) pv[h] = exp2f(s[h] - s_mref[hb + h]);
            }
            // P^T row of this token -> the rope block's slot, MN-major, 128-byte swizzle
            uint8_t *prow = sm + OFF_KV + RP * KV_BLK + row * 128;
#pragma unroll
            for (int c = 0; c < HG / 8; c++) {
#pragma unroll
                for (int j = 0; j < 8; j++) lpart[c * 8 + j] += pv[c * 8 + j];
                uint4 w;
                w.x = pack_bf16x2(pv[c * 8 + 0], pv[c * 8 + 1]); w.y = pack_bf16x2(pv[c * 8 + 2], pv[c * 8 + 3]);
                w.z = pack_bf16x2(pv[c * 8 + 4], pv[c * 8 + 5]); w.w = pack_bf16x2(pv[c * 8 + 6], pv[c * 8 + 7]);
                *reinterpret_cast<uint4 *>(prow + (((g * (HG / 8) + c) ^ (row & 7)) << 4)) = w;
            }
            if (!valid) {       // rows past the sequence end hold whatever the cache holds: 0 x NaN would poison O
                const uint4 z = make_uint4(0, 0, 0, 0);
                for (int k = g * 2; k < g * 2 + 2; k++) {
                    uint8_t *vrow = sm + OFF_KV + k * KV_BLK + row * 128;
#pragma unroll
                    for (int c = 0; c < 8; c++) *reinterpret_cast<uint4 *>(vrow + (c << 4)) = z;
                }
            }
            if (st == 0) TRACE(2, it, 7);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            tc_fence_before();
            mbar_arrive(bar(B_PFULL));
            if (st == 0) TRACE(2, it, 1);
        }
        // ---- epilogue: the row sums need only the last softmax; each 128-row block of O^T is written as soon
        // as its own MMAs have completed (their commit is the barrier that frees the block's latent slot), so
        // the write-out of block 0 runs under the MMAs of blocks 1-3
        if (ok) {
            const float mine = warp_transpose_reduce16<false>(lpart, lane);  // lane L: sum of head hb+(L&15) over this warp's rows
            if (lane < HG) s_w[(warp - 4) * HG + lane] = mine;
            if (st == 0) TRACE(2, 15, 3);
            softmax_bar();
            if (st < NH) {
                const int gg = st / HG, hh = st % HG;
                const float *w4 = s_w + gg * 4 * HG + hh;
                const float lsum = (w4[0] + w4[HG]) + (w4[2 * HG] + w4[3 * HG]);
                if (p.out) {
                    s_alpha[st] = lsum > 0.f ? 1.f / lsum : 0.f;
                } else if (mb0 == 0) {         // both halves hold the same (m, l): one writes them
                    rec[st] = s_mref[st] * 0.6931471805599453f;
                    rec[NH + st] = lsum;
                }
            }
            if (p.out) softmax_bar();
            if (st == 0) TRACE(2, 15, 4);
            for (int mb = mb0; mb < mb1 && ok; mb++) {
                ok = mbar_wait(bar(mb == 3 ? B_EMPTY_RP : B_EMPTY_L + mb), (uint32_t)((n - 1) & 1), p.err, 302);
                ok = __all_sync(0xffffffffu, ok);                  // the TMEM load below is warp-wide
                if (!ok) break;
                if (st == 0 && mb == 0) TRACE(2, 15, 2);
                tc_fence_after();
                uint32_t o[16];
                const int h0 = hb;
                TMEM_LD16(o, 0, tlane + COL_O + mb * 64 + h0);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (p.out) {
                    uint16_t *dst = p.out + ((int64_t)b * NH + h0) * L + mb * 128 + row;
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        dst[j * L] = (uint16_t)(pack_bf16x2(__uint_as_float(o[j]) * s_alpha[h0 + j], 0.f) & 0xffffu);
                } else {
                    float *dst = rec + 2 * NH + mb * 128 + row + (int64_t)h0 * L;      // o[h][dv], dv = mb*128 + row
#pragma unroll
                    for (int j = 0; j < 16; j++) dst[j * L] = __uint_as_float(o[j]);
                }
            }
        }
    }
#ifdef CWK_TRACE
    if (tr && tid == 128) tr[3 * 16 * 8 + 1] = clock64();
#endif
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

bool cwk_mla_decode_tc_available() { return true; }

int cwk_mla_decode_tc_launch(cwk_ctx *ctx, const void *q, const void *cache, int64_t seq_stride, int64_t ld,
                             const int32_t *kv_len, int max_kv_len, int B, int nh, int R, float scale, float *partial,
                             int nsplit, void *out_direct, const int32_t *sel, int64_t sel_ld) {
    const int width = L + R;          // 576, or 512 for a rope-free latent (the rope block then reads as zeros)
    if (nh != NH) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "tcgen05 MLA decode is built for 64 heads");
    if (max_kv_len <= 0) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "tcgen05 MLA decode needs a non-empty cache");
    {
        int es = cwk_ensure_err_word(ctx);
        if (es != CWK_OK) return es;
    }
    const CUtensorMap *tm_q = nullptr, *tm_kv = nullptr, *tm_kr = nullptr;
    {
        int ts = cwk_mla_tensor_maps(ctx, q, cache, seq_stride, ld, max_kv_len, B, width, &tm_q, &tm_kv, &tm_kr);
        if (ts != CWK_OK) return ts;
    }
    const bool shared_cache = (seq_stride == 0);
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(mla_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        attr_set[ctx->device & 15] = true;
    }
    TcParams p;
    p.kv_len = kv_len; p.kv_len_imm = max_kv_len; p.partial = partial; p.nsplit = nsplit; p.scale_log2 = scale * 1.4426950408889634f;
    p.err = ctx->dev_err; p.batch_coord_zero = shared_cache ? 1 : 0;
#ifdef CWK_TRACE
    p.trace = (long long *)ctx->tc_trace;
#endif
    p.out = (uint16_t *)out_direct;
    p.sel = sel; p.sel_ld = sel_ld; p.cache = (const uint16_t *)cache; p.seq_stride = seq_stride; p.ld = ld; p.rope_cols = R;
    p.reverse_b = shared_cache ? 1 : 0;
    p.halves = ((int64_t)nsplit * B * 2 <= ctx->sm_count) ? 2 : 1;
    {
        const int tiles_per_block = ((max_kv_len + TILE - 1) / TILE + nsplit - 1) / nsplit;
        p.stagger = ((int64_t)nsplit * B * 2 > ctx->sm_count && tiles_per_block >= 6) ? 700 : 0;
    }
    mla_decode_tc_kernel<<<dim3(nsplit, B, p.halves), NTHREADS, SMEM_TOTAL, ctx->stream>>>(*tm_q, *tm_kv, *tm_kr, p);
    CWK_LAUNCH_CHECK(ctx, "mla_decode_tc_kernel");
    return CWK_OK;
}
