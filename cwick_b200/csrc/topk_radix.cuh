// topk_radix.cuh -- exact k-th largest of a float row by radix select, shared by the selection kernels.
//
// A row is handled by a thread-block cluster of TK_CL blocks of 1024 threads: each block owns a
// contiguous slice of the row, 8 consecutive scores per thread. A slice of up to 8192 scores stays
// in registers for all four radix passes and the compaction (rows up to 65536 scores are read from
// memory once); longer slices are re-read chunk by chunk. Per pass every block histograms its own
// slice in shared memory, one cluster barrier publishes the histograms, and every block adds up
// all of them through distributed shared memory and reaches the same digit.
#pragma once
#include <cstdint>

#include <cooperative_groups.h>
#include <cuda_runtime.h>

namespace cg = cooperative_groups;

constexpr int TK_CL = 8;                 // blocks per row (the portable cluster size)
constexpr int TK_THREADS = 1024;
constexpr int TK_PT = 8;                 // scores per thread and chunk
constexpr int TK_CHUNK = TK_THREADS * TK_PT;

// order-preserving map float -> uint32 (larger float <=> larger integer; -0 < +0)
__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float order_key_inverse(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

struct TkShared {
    uint32_t hist[2][256];               // this block's digit counts, double-buffered across passes
    uint32_t tot[256];                   // the cluster's digit counts
    uint32_t sel[2];                     // chosen prefix, remaining rank
    unsigned long long cnt[32], off[32], total;   // block scan of (above | equal << 32)
    unsigned long long pub;              // this block's totals, read by the blocks of higher rank
    unsigned long long base;             // totals of the blocks of lower rank
    int tbase;
    float fmax;
};

struct TkSlice {
    int begin, end;                      // this block's part of the row
    bool cached;                         // the slice fits the registers
};

__device__ __forceinline__ TkSlice tk_slice(int nb, unsigned rank) {
    const int per = (((nb + TK_CL - 1) / TK_CL) + 7) & ~7;
    TkSlice s;
    s.begin = min(nb, (int)rank * per);
    s.end = min(nb, s.begin + per);
    s.cached = per <= TK_CHUNK;
    return s;
}

// keys of scores c0 + 8*tid .. +7 (those below `end`)
__device__ __forceinline__ void tk_load(const float *s, int c0, int end, uint32_t (&k)[TK_PT]) {
    const int i0 = c0 + (int)threadIdx.x * TK_PT;
    if (i0 + TK_PT <= end && (reinterpret_cast<uintptr_t>(s + i0) & 15u) == 0) {
        const float4 a = __ldcg(reinterpret_cast<const float4 *>(s + i0)), b = __ldcg(reinterpret_cast<const float4 *>(s + i0 + 4));   // L2: the row may have been written by this launch
        k[0] = order_key(a.x); k[1] = order_key(a.y); k[2] = order_key(a.z); k[3] = order_key(a.w);
        k[4] = order_key(b.x); k[5] = order_key(b.y); k[6] = order_key(b.z); k[7] = order_key(b.w);
    } else {
#pragma unroll
        for (int j = 0; j < TK_PT; j++) k[j] = (i0 + j < end) ? order_key(__ldcg(s + i0 + j)) : 0u;
    }
}

// Warp 0 of a block: the bin of a 256-bin digit histogram where the count from the top reaches
// `remaining`. sel[0] = prefix extended by that digit, sel[1] = the rank still wanted inside the bin.
__device__ __forceinline__ void tk_pick_bin(const uint32_t *hist, int lane, uint32_t prefix, int shift, int remaining, uint32_t *sel) {
    uint32_t c[8], tot = 0;                    // 8 bins per lane, suffix sums across the lanes
#pragma unroll
    for (int j = 0; j < 8; j++) { c[j] = hist[lane * 8 + j]; tot += c[j]; }
    uint32_t incl = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_down_sync(0xffffffffu, incl, o);
        if (lane + o < 32) incl += t;
    }
    uint32_t above = incl - tot;               // elements in the bins of higher lanes
    const uint32_t r = (uint32_t)remaining;
    if (above < r && r <= above + tot) {
#pragma unroll
        for (int j = 7; j >= 0; j--) {
            if (r <= above + c[j]) {
                sel[0] = prefix | ((uint32_t)(lane * 8 + j) << shift);
                sel[1] = r - above;
                break;
            }
            above += c[j];
        }
    }
}

// The same selection over a short list of row positions (one block's worth of work, no cluster
// traffic): the rank-th largest of s[list[0..cnt)]. Every thread of the block calls it.
__device__ __forceinline__ void tk_list_select(const float *s, const int32_t *list, int cnt, int rank, TkShared &sh, uint32_t &prefix,
                                               int &remaining) {
    const int tid = threadIdx.x, lane = tid & 31;
    prefix = 0;
    uint32_t mask = 0;
    remaining = rank;
    // a thread's first entry stays in a register over the four passes (two dependent loads from L2 each time otherwise)
    const uint32_t first = tid < cnt ? order_key(__ldcg(s + __ldcg(list + tid))) : 0u;
    for (int pass = 0; pass < 4; pass++) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) sh.tot[tid] = 0;
        __syncthreads();
        if (tid < cnt && (first & mask) == prefix) atomicAdd(&sh.tot[(first >> shift) & 255u], 1u);
        for (int i = tid + TK_THREADS; i < cnt; i += TK_THREADS) {
            const uint32_t k = order_key(__ldcg(s + __ldcg(list + i)));
            if ((k & mask) == prefix) atomicAdd(&sh.tot[(k >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid < 32) tk_pick_bin(sh.tot, lane, prefix, shift, remaining, sh.sel);
        __syncthreads();
        prefix = sh.sel[0];
        remaining = (int)sh.sel[1];
        mask |= 255u << shift;
    }
}

// Exact want-th largest value of the row: 4 passes of 8 bits over the order-preserving integer
// image. On return `prefix` is that image and `remaining` how many rows equal to it are wanted.
// Every thread of every block of the cluster calls it; nb > want >= 1. Scores of one row usually
// share their leading digits, so the lanes of a warp that hit the first active lane's bin are
// counted with one atomic, not 32. kc holds the slice's keys when sl.cached (loaded by the caller).
__device__ __forceinline__ void tk_radix_select(const float *s, const TkSlice sl, uint32_t (&kc)[TK_PT], int want, TkShared &sh,
                                                uint32_t &prefix, int &remaining) {
    cg::cluster_group cl = cg::this_cluster();
    const int tid = threadIdx.x, lane = tid & 31;
    prefix = 0;
    uint32_t mask = 0;
    remaining = want;
    for (int pass = 0; pass < 4; pass++) {
        const int shift = 24 - 8 * pass;
        uint32_t *h = sh.hist[pass & 1];
        if (tid < 256) h[tid] = 0;
        __syncthreads();
        for (int c0 = sl.begin; c0 < sl.end; c0 += TK_CHUNK) {
            if (!sl.cached) tk_load(s, c0, sl.end, kc);
            const int i0 = c0 + tid * TK_PT;
#pragma unroll
            for (int j = 0; j < TK_PT; j++) {
                const bool act = (i0 + j < sl.end) && ((kc[j] & mask) == prefix);
                const uint32_t d = (kc[j] >> shift) & 255u;
                // the first active lane's digit is counted once for every lane that shares it; the others add singly
                const uint32_t am = __ballot_sync(0xffffffffu, act);
                if (am) {
                    const int leader = __ffs(am) - 1;
                    const uint32_t d0 = __shfl_sync(0xffffffffu, d, leader);
                    const uint32_t same = __ballot_sync(0xffffffffu, act && d == d0);
                    if (lane == leader) atomicAdd(&h[d0], (uint32_t)__popc(same));
                    else if (act && d != d0) atomicAdd(&h[d], 1u);
                }
            }
        }
        cl.sync();
        if (tid < 256) {
            uint32_t t = 0;
#pragma unroll
            for (unsigned r = 0; r < TK_CL; r++) t += cl.map_shared_rank(h, r)[tid];
            sh.tot[tid] = t;
        }
        __syncthreads();
        if (tid < 32) tk_pick_bin(sh.tot, lane, prefix, shift, remaining, sh.sel);
        __syncthreads();
        prefix = sh.sel[0];
        remaining = (int)sh.sel[1];
        mask |= 255u << shift;
    }
}

// The second half of a selection, for every thread of every block of the row's cluster: the exact threshold (radix select
// over the row, or, when the row holds +inf / -inf outside a short list of re-scored positions, over that list only), then
// the ordered compaction into out[]: rows above the threshold in index order, then rows equal to it in index order, `want`
// in all (ascending: one list in index order). kc holds the slice's keys when sl.cached.
__device__ __forceinline__ void tk_threshold_and_compact(const float *s, const TkSlice sl, uint32_t (&kc)[TK_PT], int nb, int want,
                                                         int keep_self, int ascending, int32_t *out, int32_t *nsel_b,
                                                         const int32_t *band_list, int band_cnt, int band_above, TkShared &sh) {
    cg::cluster_group cl = cg::this_cluster();
    const unsigned rank = cl.block_rank();
    const int tid = threadIdx.x;
    if (tid == 0) sh.pub = 0;
    uint32_t thr;
    int need_eq;
    if (band_list) {
        // The row holds +inf / -inf outside a short list of re-scored positions (cwk_dsa_select): the exact
        // threshold is the (want - certainly selected)-th largest score of that list. Every block of the
        // cluster finds it for itself; the list is a few hundred entries.
        const int kth = max(1, min(want - band_above, band_cnt));   // holds by construction; clamped against a violated error bound
        tk_list_select(s, band_list, band_cnt, kth, sh, thr, need_eq);
    } else {
        tk_radix_select(s, sl, kc, want, sh, thr, need_eq);
    }
    // thr is the integer image of the threshold; need_eq rows equal to it are wanted (the first
    // ones in index order); want - need_eq rows lie above it.
    const int n_gt = want - need_eq;
    const int lane = tid & 31, warp = tid >> 5;
    // this block's totals, for the offsets of the blocks after it
    {
        unsigned long long mine = 0;
        for (int c0 = sl.begin; c0 < sl.end; c0 += TK_CHUNK) {
            if (!sl.cached) tk_load(s, c0, sl.end, kc);
            const int i0 = c0 + tid * TK_PT;
#pragma unroll
            for (int j = 0; j < TK_PT; j++)
                if (i0 + j < sl.end) mine += (kc[j] > thr ? 1ull : 0ull) + (kc[j] == thr ? (1ull << 32) : 0ull);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
        if (lane == 0 && mine) atomicAdd(&sh.pub, mine);
    }
    cl.sync();
    if (tid < 32) {
        // totals of the blocks of lower rank: the lanes fetch them from the neighbours' shared memory together
        // (one round trip instead of one per block), lane 0 adds them up in rank order
        const unsigned long long mine = (unsigned)tid < rank ? *cl.map_shared_rank(&sh.pub, (unsigned)tid) : 0ull;
        unsigned long long base = 0;
        int tbase = 0;
#pragma unroll
        for (unsigned r = 0; r < TK_CL; r++) {
            const unsigned long long v = __shfl_sync(0xffffffffu, mine, (int)r);
            if (r < rank) {
                const int g = (int)(v & 0xffffffffull), e = (int)(v >> 32), eb = (int)(base >> 32);
                tbase += g + max(0, min(e, need_eq - eb));
                base += v;
            }
        }
        if (tid == 0) {
            sh.base = base;
            sh.tbase = tbase;
        }
    }
    __syncthreads();
    unsigned long long running = sh.base;
    const int eq_before_block = (int)(sh.base >> 32);
    const int tbase = sh.tbase;
    const int eq_quota = max(0, need_eq - eq_before_block);     // ties this block may still take
    unsigned long long local = 0;                                // (above | equal) in this block's earlier chunks
    for (int c0 = sl.begin; c0 < sl.end; c0 += TK_CHUNK) {
        if (!sl.cached) tk_load(s, c0, sl.end, kc);
        const int i0 = c0 + tid * TK_PT;
        unsigned long long mine = 0;
#pragma unroll
        for (int j = 0; j < TK_PT; j++)
            if (i0 + j < sl.end) mine += (kc[j] > thr ? 1ull : 0ull) + (kc[j] == thr ? (1ull << 32) : 0ull);
        unsigned long long incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) sh.cnt[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const unsigned long long v = sh.cnt[lane];
            unsigned long long wi = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long t = __shfl_up_sync(0xffffffffu, wi, o);
                if (lane >= o) wi += t;
            }
            sh.off[lane] = wi - v;
            if (lane == 31) sh.total = wi;
        }
        __syncthreads();
        const unsigned long long before = local + sh.off[warp] + incl - mine;   // within this block
        int lg = (int)(before & 0xffffffffull), le = (int)(before >> 32);
        const int og0 = (int)(running & 0xffffffffull), oe0 = (int)(running >> 32);
#pragma unroll
        for (int j = 0; j < TK_PT; j++) {
            if (i0 + j < sl.end) {
                const bool gt = kc[j] > thr, eq = kc[j] == thr;
                const bool take = gt || (eq && le < eq_quota);
                if (take) {
                    if (ascending) out[tbase + lg + min(le, eq_quota)] = i0 + j;
                    else if (gt) out[og0 + lg] = i0 + j;
                    else out[n_gt + oe0 + le] = i0 + j;
                }
                lg += gt ? 1 : 0;
                le += eq ? 1 : 0;
            }
        }
        local += sh.total;
    }
    cl.sync();                              // every block's part of the list is written; nobody reads a neighbour's shared memory after this
    if (rank == 0 && tid == 0) {
        int cnt = want;
        if (keep_self && out[cnt - 1] != nb - 1) out[cnt++] = nb - 1;
        *nsel_b = cnt;
    }
}
