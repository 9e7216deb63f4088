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
        const float4 a = *reinterpret_cast<const float4 *>(s + i0), b = *reinterpret_cast<const float4 *>(s + i0 + 4);
        k[0] = order_key(a.x); k[1] = order_key(a.y); k[2] = order_key(a.z); k[3] = order_key(a.w);
        k[4] = order_key(b.x); k[5] = order_key(b.y); k[6] = order_key(b.z); k[7] = order_key(b.w);
    } else {
#pragma unroll
        for (int j = 0; j < TK_PT; j++) k[j] = (i0 + j < end) ? order_key(s[i0 + j]) : 0u;
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
    for (int pass = 0; pass < 4; pass++) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) sh.tot[tid] = 0;
        __syncthreads();
        for (int i = tid; i < cnt; i += TK_THREADS) {
            const uint32_t k = order_key(s[list[i]]);
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
