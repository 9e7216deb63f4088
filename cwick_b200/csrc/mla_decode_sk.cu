// mla_decode_sk.cu -- MLA absorbed decode as ONE persistent launch: the tcgen05/TMA tile pipeline of
// mla_decode_tc.cu, with the work dealt out tile by tile instead of split by split, and the
// cross-block reduction done inside the kernel.
//
// Work: the 128-token tiles of all B sequences form one line of `total` tiles; block c of G takes
// tiles [c*total/G, (c+1)*total/G). Its range is a list of SEGMENTS (sequence, first tile, tile
// count): every SM gets the same number of tiles (+-1) whatever the batch looks like, so there is
// no partial last wave, and a sequence is cut only where a block boundary falls inside it.
//
// A segment that covers its whole sequence is normalised and written as bf16 straight from tensor
// memory. A sequence that several blocks share is reduced through one accumulator record in
// global memory: every contributing block uses the SAME reference exponent per head (the score of
// the sequence's first cached row, which each block computes for itself from q and that row), so
// un-normalised partial sums simply add: red.global.add.f32 into {l[64], o[64][512]}. A ticket per
// sequence tells the last contributor that it is the last; that block reads the accumulator back,
// normalises, writes the bf16 rows (or one folded record) and leaves accumulator and ticket zeroed
// for the next launch. No split records, no merge kernel, no second launch.
//
// A block whose scores outran the common reference by more than 2^64 (the lazy rescale moved its own
// reference that far) cannot add into the accumulator without risking overflow: it parks a full
// {m, l, o} record in a small pool instead, and the finishing block folds such records in with a
// proper log-sum-exp merge. The pool has EXC_CAP entries; running out of them is reported through
// the context's error word, never silently.
//
// Sums through atomics are not ordered: two runs on the same inputs can differ in the last bits of
// the f32 accumulator (before the bf16 rounding of the output). cwk_ctx_force_mla_path(ctx, 2)
// selects the split-record kernel, whose results are reproducible bit for bit.
#include <cuda.h>

#include <algorithm>

#include "tc_common.cuh"

namespace {

constexpr int NH = 64, L = 512;
constexpr int TILE = 128;                       // tokens per tile = MMA M
constexpr int NBLK = 9;                         // 64-element column blocks per row
constexpr int RP = 8;                           // index of the rope block / P^T slot
constexpr int KV_BLK = TILE * 128;              // 16384 B
constexpr int Q_BLK = NH * 128;                 // 8192 B
constexpr int OFF_Q = 0;
constexpr int OFF_KV = NBLK * Q_BLK;            // 73728
constexpr int OFF_BAR = OFF_KV + NBLK * KV_BLK; // 221184
constexpr int OFF_MISC = OFF_BAR + 256;
constexpr int MISC_BYTES = 3840;
constexpr int SMEM_USED = OFF_MISC + MISC_BYTES;
constexpr int SMEM_TOTAL = SMEM_USED + 1024;    // slack to align the base to 1024 B
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_O = 0, COL_S = 256;
constexpr int HG = 16;                          // heads per softmax warp group
constexpr int NG = NH / HG;                     // 4 groups of four warps
constexpr float LAZY_LOG2 = 16.f;               // a score may outrun the reference exponent by 2^16 before a rescale
constexpr float EXC_LOG2 = 64.f;                // a block's reference may outrun the common one by 2^64 before it parks a record
constexpr int NSOFT = NG * 128;                 // 512 softmax threads
constexpr int NTHREADS = 128 + NSOFT;           // 640
constexpr int NWARPS = NTHREADS / 32;
constexpr int SEGCAP = 48;                      // segments per table fill
constexpr int EMPTYCAP = 32;
constexpr int REC = NH * (L + 2);               // floats per accumulator / record
constexpr float LN2 = 0.6931471805599453f;

enum { B_FULL = 0, B_EMPTY_L = 9, B_EMPTY_RP = 13, B_QFULL = 14, B_SFULL = 15, B_PFULL = 16, B_QFREE = 17, B_COUNT = 18 };

struct Seg {
    int b;          // sequence
    int t0;         // first tile inside the sequence
    int n;          // tiles
    int kv;         // rows of the sequence
    int slot;       // accumulator slot (= first block that touches the sequence)
    int ncontrib;   // blocks that touch the sequence (1 = this segment is the whole sequence)
};

// misc area layout (byte offsets from OFF_MISC)
constexpr int M_TMEM = 0, M_FLAGS = 16, M_MREF = 128, M_MREF0 = 384, M_ALPHA = 640, M_W = 896, M_SCAN = 1920,
              M_SEG = 2048, M_EMPTY = M_SEG + SEGCAP * 24;
static_assert(sizeof(Seg) == 24, "segment record size");
static_assert(M_EMPTY + EMPTYCAP * 4 + 8 <= MISC_BYTES, "misc area too small");

struct SkParams {
    const int32_t *kv_len;   // [B] device, or NULL: every sequence has kv_len_imm rows
    int kv_len_imm;
    int B;
    const uint16_t *q;       // the same memory tm_q describes (the common reference is computed with plain loads)
    const uint16_t *cache;
    int64_t seq_stride, ld;
    int width;               // 576, or 512 for a rope-free latent
    float scale_log2;
    float *acc;              // [G][REC] {unused[NH], l[NH], o[NH][L]}; zero between launches
    unsigned int *ctl;       // [0] exit ticket, [1] pool counter, [2, 2+slots) sequence tickets; zero between launches
    unsigned int *tags;      // [exc_cap] which sequence slot (+1) a parked record belongs to, 0 = free; zero between launches
                             // tags[exc_cap] counts the records parked since the buffers were created (never reset)
    float *exc;              // [exc_cap][REC] parked records, m in log2 units
    int exc_cap;
    uint16_t *out;           // bf16 [B][NH][L], or NULL
    float *rec_out;          // out == NULL: one folded record {m, l, o} per sequence, [B][REC]
    int *err;                // device word, 0 = fine
};

__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

// v[0..15] per lane -> lane L returns the reduction over the 32 lanes of v[L & 15].
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

__device__ __forceinline__ int ntiles_of(int kv) { return kv > 0 ? (kv + TILE - 1) / TILE : 0; }
// the block whose range [c*total/G, (c+1)*total/G) holds tile x
__device__ __forceinline__ int block_of(int64_t x, int64_t total, int G) { return (int)(((x + 1) * G - 1) / total); }

// Exclusive scan of one int per thread over the whole block (NTHREADS threads); `total` = the sum.
__device__ __forceinline__ int block_excl_scan(int v, int *s_scan, int &total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) s_scan[warp] = x;
    __syncthreads();
    if (warp == 0) {
        int w = lane < NWARPS ? s_scan[lane] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += y;
        }
        s_scan[lane] = w;
    }
    __syncthreads();
    const int woff = warp > 0 ? s_scan[warp - 1] : 0;
    total = s_scan[NWARPS - 1];
    __syncthreads();
    return woff + x - v;
}

__device__ __forceinline__ void fill_seg(Seg &s, int b, int kv, int64_t p, int nt, int64_t r0, int64_t r1, int64_t total, int G) {
    const int64_t lo = p > r0 ? p : r0, hi = (p + nt) < r1 ? (p + nt) : r1;
    s.b = b; s.kv = kv; s.t0 = (int)(lo - p); s.n = (int)(hi - lo);
    const int first = block_of(p, total, G), last = block_of(p + nt - 1, total, G);
    s.slot = first; s.ncontrib = last - first + 1;
}

// Ragged lengths. Two block-wide scans give every thread the tiles before its chunk of sequences and the table
// index of its first segment; segments [round0, round0 + SEGCAP) are then written to s_seg. round0 < 0: only count
// (and write the zeros of the empty sequences this block is responsible for). Returns the block's segment count.
// Ends with a block barrier.
__device__ __noinline__ int fill_table(const SkParams &p, int c, int G, int round0, int *s_scan, Seg *s_seg, int *s_flags, int *s_empty) {
    const int tid = threadIdx.x;
    const int chunk = (p.B + NTHREADS - 1) / NTHREADS;
    const int bb0 = min(p.B, tid * chunk), bb1 = min(p.B, bb0 + chunk);
    int mine = 0;
    for (int b = bb0; b < bb1; b++) mine += ntiles_of(p.kv_len[b]);
    int tot32 = 0;
    const int64_t poff = block_excl_scan(mine, s_scan, tot32);
    const int64_t total = tot32;
    const int Ge = (int)min((int64_t)G, total);              // blocks that get tiles: never more blocks than tiles
    const int64_t r0 = c < Ge ? (int64_t)c * total / Ge : 0, r1 = c < Ge ? (int64_t)(c + 1) * total / Ge : 0;
    int cnt = 0;
    int64_t pp = poff;
    for (int b = bb0; b < bb1; b++) {
        const int nt = ntiles_of(p.kv_len[b]);
        if (nt > 0 && r1 > r0 && pp < r1 && pp + nt > r0) cnt++;
        if (round0 < 0 && nt == 0 && (b % G) == c) {         // an empty sequence: this block writes its zeros
            const int e = atomicAdd(&s_flags[4], 1);
            if (e < EMPTYCAP) s_empty[e] = b;
            else if (p.out) for (int i = 0; i < NH * L / 2; i++) reinterpret_cast<uint32_t *>(p.out + (int64_t)b * NH * L)[i] = 0u;
            else for (int i = 0; i < REC; i++) p.rec_out[(int64_t)b * REC + i] = (i < NH) ? -INFINITY : 0.f;
        }
        pp += nt;
    }
    int nseg = 0;
    const int coff = block_excl_scan(cnt, s_scan, nseg);
    if (round0 < 0) {
        const int ne = min(s_flags[4], EMPTYCAP);
        for (int e = 0; e < ne; e++) {
            const int b = s_empty[e];
            if (p.out) for (int i = tid; i < NH * L / 2; i += NTHREADS) reinterpret_cast<uint32_t *>(p.out + (int64_t)b * NH * L)[i] = 0u;
            else for (int i = tid; i < REC; i += NTHREADS) p.rec_out[(int64_t)b * REC + i] = (i < NH) ? -INFINITY : 0.f;
        }
    } else {
        const int nround = min(SEGCAP, nseg - round0);
        int idx = coff - round0;
        pp = poff;
        for (int b = bb0; b < bb1 && idx < nround; b++) {
            const int kv = p.kv_len[b], nt = ntiles_of(kv);
            if (nt > 0 && r1 > r0 && pp < r1 && pp + nt > r0) {
                if (idx >= 0) fill_seg(s_seg[idx], b, kv, pp, nt, r0, r1, total, Ge);
                idx++;
            }
            pp += nt;
        }
    }
    __syncthreads();
    return nseg;
}

// The end of a segment, after the row sums of the 16 softmax warps are in s_w: the segment's O^T leaves tensor memory
// as bf16 rows (the segment is the whole sequence), or is added into the sequence's accumulator, after which the
// last contributor finishes the sequence. Kept out of line so that its registers do not count against the tile loop.
// Called by the 512 softmax threads; returns false when a bounded wait gave up.
__device__ __noinline__ bool segment_epilogue(const SkParams &p, const Seg &s, uint8_t *sm, uint32_t bar0, uint32_t tmem, int itl) {
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint8_t *misc = sm + OFF_MISC;
    int *s_flags = reinterpret_cast<int *>(misc + M_FLAGS);
    float *s_mref = reinterpret_cast<float *>(misc + M_MREF);
    float *s_mref0 = reinterpret_cast<float *>(misc + M_MREF0);
    float *s_alpha = reinterpret_cast<float *>(misc + M_ALPHA);
    float *s_w = reinterpret_cast<float *>(misc + M_W);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q4 = warp & 3, g = (warp - 4) >> 2, hb = g * HG, row = q4 * 32 + lane, st = tid - 128;
    const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
    const bool sole = s.ncontrib == 1;
    bool ok = true;
    if (st == 0) s_flags[1] = 0;
    softmax_bar();
    float *A = p.acc + (int64_t)s.slot * REC;
    float lsum = 0.f, delta = 0.f;
    if (st < NH) {
        const int gg = st / HG, hh = st % HG;
        const float *w4 = s_w + gg * 4 * HG + hh;
        lsum = (w4[0] + w4[HG]) + (w4[2 * HG] + w4[3 * HG]);
        if (sole) {
            if (p.out) {
                s_alpha[st] = lsum > 0.f ? 1.f / lsum : 0.f;
            } else {
                float *rec = p.rec_out + (int64_t)s.b * REC;
                rec[st] = s_mref[st] * LN2;
                rec[NH + st] = lsum;
                s_alpha[st] = 1.f;
            }
        } else {
            delta = s_mref[st] - s_mref0[st];                 // >= 0: how far this block's reference moved
            if (delta > EXC_LOG2) s_flags[1] = 1;
        }
    }
    softmax_bar();
    const bool park = !sole && s_flags[1] != 0;
    float *X = nullptr;                                       // parked record
    if (!sole) {
        if (park) {
            if (st == 0) {
                const unsigned int e = atomicAdd(&p.ctl[1], 1u);
                atomicAdd(&p.tags[p.exc_cap], 1u);
                s_flags[2] = (e < (unsigned int)p.exc_cap) ? (int)e : -1;
                if (e >= (unsigned int)p.exc_cap) atomicCAS(p.err, 0, 401);   // more parked records than the pool holds
            }
            softmax_bar();
            if (s_flags[2] >= 0) X = p.exc + (int64_t)s_flags[2] * REC;
            if (st < NH) {
                if (X) { X[st] = s_mref[st]; X[NH + st] = lsum; }
                s_alpha[st] = 1.f;
            }
        } else if (st < NH) {
            const float f = exp2f(delta);
            s_alpha[st] = f;
            atomicAdd(A + NH + st, lsum * f);
        }
        softmax_bar();
    }
    // Each 128-row block of O^T leaves as soon as its own MMAs have completed (their commit is the
    // barrier that frees the block's latent slot).
    for (int mb = 0; mb < 4 && ok; mb++) {
        ok = mbar_wait(bar(mb == 3 ? B_EMPTY_RP : B_EMPTY_L + mb), (uint32_t)(itl & 1), p.err, 302);
        ok = __all_sync(0xffffffffu, ok);                  // the TMEM load below is warp-wide
        if (!ok) break;
        tc_fence_after();
        uint32_t o[16];
        TMEM_LD16(o, 0, tlane + COL_O + mb * 64 + hb);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int dv = mb * 128 + row;
        if (sole && p.out) {
            uint16_t *dst = p.out + ((int64_t)s.b * NH + hb) * L + dv;
#pragma unroll
            for (int j = 0; j < 16; j++)
                dst[j * L] = (uint16_t)(pack_bf16x2(__uint_as_float(o[j]) * s_alpha[hb + j], 0.f) & 0xffffu);
        } else if (sole || park) {
            float *dst = sole ? p.rec_out + (int64_t)s.b * REC : X;
            if (dst) {
                dst += 2 * NH + (int64_t)hb * L + dv;
#pragma unroll
                for (int j = 0; j < 16; j++) dst[j * L] = __uint_as_float(o[j]);
            }
        } else {
            float *dst = A + 2 * NH + (int64_t)hb * L + dv;
#pragma unroll
            for (int j = 0; j < 16; j++) atomicAdd(dst + j * L, __uint_as_float(o[j]) * s_alpha[hb + j]);
        }
    }
    // A wait that gave up must not leave some warps at a barrier the others never reach: the decision to stop is
    // taken by all 512 threads together.
    if (!ok) s_flags[5] = 1;
    softmax_bar();
    if (s_flags[5]) return false;
    if (!sole) {
        // ---- ticket: is this block the sequence's last contributor? -----------------------------
        __threadfence();
        softmax_bar();
        if (st == 0) {
            if (park && s_flags[2] >= 0) {
                p.tags[s_flags[2]] = (unsigned int)s.slot + 1u;    // the record is complete: tag it
                __threadfence();
            }
            const unsigned int tk = atomicAdd(&p.ctl[2 + s.slot], 1u);
            s_flags[0] = (tk == (unsigned int)s.ncontrib - 1u) ? 1 : 0;
            s_flags[3] = 0;
            if (s_flags[0]) {
                __threadfence();
                s_flags[3] = (int)min(__ldcg(&p.ctl[1]), (unsigned int)p.exc_cap);
            }
        }
        softmax_bar();
        if (s_flags[0]) {
            __threadfence();
            // ---- the finishing block ----------------------------------------------------------
            // s_mref0 becomes the running reference of the accumulator while parked records are folded in.
            const int nexc = s_flags[3];
            for (int e = 0; e < nexc; e++) {
                if (__ldcg(&p.tags[e]) != (unsigned int)s.slot + 1u) continue;     // block-uniform
                const float *Xe = p.exc + (int64_t)e * REC;
                if (st < NH) {
                    const float me = __ldcg(Xe + st), le = __ldcg(Xe + NH + st), m0 = s_mref0[st], l0 = __ldcg(A + NH + st);
                    const float mn = (le > 0.f) ? fmaxf(m0, me) : m0;
                    const float a = exp2f(m0 - mn), bsc = (le > 0.f) ? exp2f(me - mn) : 0.f;
                    s_alpha[st] = a; s_w[st] = bsc;
                    s_mref0[st] = mn;
                    __stcg(A + NH + st, l0 * a + le * bsc);
                }
                softmax_bar();
                for (int i = st; i < NH * L / 4; i += NSOFT) {
                    const int h = i >> 7;
                    float4 v = __ldcg(reinterpret_cast<const float4 *>(A + 2 * NH) + i);
                    const float4 x = __ldcg(reinterpret_cast<const float4 *>(Xe + 2 * NH) + i);
                    const float a = s_alpha[h], bsc = s_w[h];
                    v.x = v.x * a + x.x * bsc; v.y = v.y * a + x.y * bsc; v.z = v.z * a + x.z * bsc; v.w = v.w * a + x.w * bsc;
                    __stcg(reinterpret_cast<float4 *>(A + 2 * NH) + i, v);
                }
                softmax_bar();
                if (st == 0) p.tags[e] = 0u;
            }
            if (st < NH) {
                const float l = __ldcg(A + NH + st);
                if (p.out) {
                    s_alpha[st] = l > 0.f ? 1.f / l : 0.f;
                } else {
                    float *rec = p.rec_out + (int64_t)s.b * REC;
                    rec[st] = s_mref0[st] * LN2;
                    rec[NH + st] = l;
                    s_alpha[st] = 1.f;
                }
                __stcg(A + NH + st, 0.f);
            }
            if (st == 0) p.ctl[2 + s.slot] = 0u;
            softmax_bar();
            const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
            for (int i = st; i < NH * L / 4; i += NSOFT) {
                const int h = i >> 7;
                float4 v = __ldcg(reinterpret_cast<const float4 *>(A + 2 * NH) + i);
                __stcg(reinterpret_cast<float4 *>(A + 2 * NH) + i, z4);
                const float a = s_alpha[h];
                if (p.out) {
                    uint2 w;
                    w.x = pack_bf16x2(v.x * a, v.y * a); w.y = pack_bf16x2(v.z * a, v.w * a);
                    *reinterpret_cast<uint2 *>(p.out + (int64_t)s.b * NH * L + (int64_t)i * 4) = w;
                } else {
                    *(reinterpret_cast<float4 *>(p.rec_out + (int64_t)s.b * REC + 2 * NH) + i) = v;
                }
            }
        }
        softmax_bar();       // s_mref0 / s_alpha are reused by the next segment
    }
    return true;
}

__global__ void __launch_bounds__(NTHREADS, 1)
mla_decode_sk_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv,
                     const __grid_constant__ CUtensorMap tm_kr, const SkParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;             // 1024-byte aligned (swizzle atom)
    uint8_t *sm = smem_raw + (base - raw);
    const uint32_t bar0 = base + OFF_BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint8_t *misc = sm + OFF_MISC;
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(misc + M_TMEM);
    int *s_flags = reinterpret_cast<int *>(misc + M_FLAGS);           // [0] last contributor, [1] park a record, [2] pool entry, [3] pool count seen, [4] empties, [5] a softmax thread's wait gave up
    float *s_mref = reinterpret_cast<float *>(misc + M_MREF);         // [64] this block's reference exponents (log2 units)
    float *s_mref0 = reinterpret_cast<float *>(misc + M_MREF0);       // [64] the sequence's common reference
    float *s_alpha = reinterpret_cast<float *>(misc + M_ALPHA);       // [64]
    float *s_w = reinterpret_cast<float *>(misc + M_W);               // [16 warps][16]
    int *s_scan = reinterpret_cast<int *>(misc + M_SCAN);             // [32]
    Seg *s_seg = reinterpret_cast<Seg *>(misc + M_SEG);
    int *s_empty = reinterpret_cast<int *>(misc + M_EMPTY);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c = blockIdx.x, G = gridDim.x;
    const bool uniform = (p.kv_len == nullptr) || p.B == 1;
    const bool shared_cache = (p.seq_stride == 0);

    // ---- this block's share of the tile line ----------------------------------------------
    // Uniform lengths: everything follows from (B, length) by arithmetic. Ragged lengths: fill_table() scans
    // kv_len. Either way the table is (re)computed from scratch for every round of SEGCAP segments, so that
    // nothing but the role counters stays in registers across the pipeline code.
    int nseg = 0;
    if (uniform) {
        const int u_nt = ntiles_of(p.kv_len ? p.kv_len[0] : p.kv_len_imm);
        const int64_t total = (int64_t)p.B * u_nt;
        const int Ge = (int)min((int64_t)G, total);          // blocks that get tiles: never more blocks than tiles
        if (c < Ge) {
            const int64_t r0 = (int64_t)c * total / Ge, r1 = (int64_t)(c + 1) * total / Ge;
            nseg = (int)((r1 - 1) / u_nt) - (int)(r0 / u_nt) + 1;
        }
    }
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_kv) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_kr) : "memory");
        for (int i = 0; i < B_COUNT; i++) mbar_init(bar(i), i == B_PFULL ? (uint32_t)NSOFT : 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_flags[4] = 0;
        s_flags[5] = 0;
    }
    if (uniform && nseg > 0 && tid == 0) {
        // One sequence length for all: the first segment is known without a scan, so its loads go out
        // before the block-wide set-up; their latency is the longest single item of a short call.
        const int u_kv = p.kv_len ? p.kv_len[0] : p.kv_len_imm, u_nt = ntiles_of(u_kv);
        const int64_t total = (int64_t)p.B * u_nt;
        const int Ge = (int)min((int64_t)G, total);
        const int64_t r0 = (int64_t)c * total / Ge, r1 = (int64_t)(c + 1) * total / Ge;
        const int u_b0 = (int)(r0 / u_nt);
        Seg s0;
        fill_seg(s0, u_b0, u_kv, (int64_t)u_b0 * u_nt, u_nt, r0, r1, total, Ge);
        const int bz = shared_cache ? 0 : s0.b;
        mbar_expect_tx(bar(B_QFULL), NBLK * Q_BLK);
        tma_load_3d(base + OFF_Q, &tm_q, 0, s0.b * NH, 0, bar(B_QFULL));
        for (int k = 0; k < 6; k += 2) {
            mbar_expect_tx(bar(B_FULL + k), 2 * KV_BLK);
            tma_load_4d(base + OFF_KV + k * KV_BLK, &tm_kv, 0, s0.t0 * TILE, k, bz, bar(B_FULL + k));
        }
        mbar_expect_tx(bar(B_FULL + 6), 3 * KV_BLK);
        tma_load_4d(base + OFF_KV + 6 * KV_BLK, &tm_kr, 0, s0.t0 * TILE, 6, bz, bar(B_FULL + 6));
    }
    const bool early = uniform && nseg > 0;      // the first segment's Q and first tile were requested during set-up
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    __syncthreads();

    if (!uniform) {
        nseg = fill_table(p, c, G, -1, s_scan, s_seg, s_flags, s_empty);      // counts the segments, zeroes the empty sequences' outputs
    } else if (nseg == 0 && ntiles_of(p.kv_len ? p.kv_len[0] : p.kv_len_imm) == 0) {
        // every sequence is empty
        for (int b = c; b < p.B; b += G) {
            if (p.out) for (int i = tid; i < NH * L / 2; i += NTHREADS) reinterpret_cast<uint32_t *>(p.out + (int64_t)b * NH * L)[i] = 0u;
            else for (int i = tid; i < REC; i += NTHREADS) p.rec_out[(int64_t)b * REC + i] = (i < NH) ? -INFINITY : 0.f;
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;

    // Running counters of each role; they continue across table fills so the barrier phases stay in step.
    int it = 0;            // tiles this role has gone through
    int sg = 0;            // segments this role has gone through
    bool ok = true;

    for (int round0 = 0; round0 < nseg; round0 += SEGCAP) {
        const int nround = min(SEGCAP, nseg - round0);
        // ---- fill the segment table for this round -------------------------------------------------
        if (uniform) {
            if (tid < nround) {
                const int u_kv = p.kv_len ? p.kv_len[0] : p.kv_len_imm, u_nt = ntiles_of(u_kv);
                const int64_t total = (int64_t)p.B * u_nt;
                const int Ge = (int)min((int64_t)G, total);
                const int64_t r0 = (int64_t)c * total / Ge, r1 = (int64_t)(c + 1) * total / Ge;
                const int b = (int)(r0 / u_nt) + round0 + tid;
                fill_seg(s_seg[tid], b, u_kv, (int64_t)b * u_nt, u_nt, r0, r1, total, Ge);
            }
            __syncthreads();
        } else {
            fill_table(p, c, G, round0, s_scan, s_seg, s_flags, s_empty);
        }

        if (warp == 0) {
            // ------------------------------------------------------------ TMA producer
            if (lane == 0) {
                for (int si = 0; si < nround && ok; si++, sg++) {
                    const Seg &s = s_seg[si];
                    const int bz = shared_cache ? 0 : s.b;
                    const bool skip_first = early && sg == 0;     // requested during set-up
                    if (!skip_first) {
                        if (sg > 0) ok = mbar_wait(bar(B_QFREE), (uint32_t)((sg - 1) & 1), p.err, 105);
                        if (!ok) break;
                        mbar_expect_tx(bar(B_QFULL), NBLK * Q_BLK);
                        tma_load_3d(base + OFF_Q, &tm_q, 0, s.b * NH, 0, bar(B_QFULL));
                    }
                    for (int t = 0; t < s.n && ok; t++, it++) {
                        if (skip_first && t == 0) continue;
                        const uint32_t par_free = (uint32_t)((it & 1) ^ 1);
                        const int row = (s.t0 + t) * TILE;
                        for (int k = 0; k < 8 && ok; k += 2) {
                            if (it > 0) {
                                ok = mbar_wait(bar(B_EMPTY_L + (k >> 1)), par_free, p.err, 102);
                                // the last latent pair and the rope block (= the P^T slot) come free together
                                if (ok && k == 6) ok = mbar_wait(bar(B_EMPTY_RP), par_free, p.err, 101);
                                if (!ok) break;
                            }
                            if (k == 6) {
                                mbar_expect_tx(bar(B_FULL + k), 3 * KV_BLK);
                                tma_load_4d(base + OFF_KV + k * KV_BLK, &tm_kr, 0, row, k, bz, bar(B_FULL + k));
                            } else {
                                mbar_expect_tx(bar(B_FULL + k), 2 * KV_BLK);
                                tma_load_4d(base + OFF_KV + k * KV_BLK, &tm_kv, 0, row, k, bz, bar(B_FULL + k));
                            }
                        }
                    }
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------ MMA issuer
            if (lane == 0) {
                constexpr uint32_t ID_QK = idesc_bf16(128, 64, 0, 0);
                constexpr uint32_t ID_PV = idesc_bf16(128, 64, 1, 1);
                const uint64_t dK = smem_desc(base + OFF_KV, 16, 1024), dQ = smem_desc(base + OFF_Q, 16, 1024);
                const uint64_t dV = smem_desc(base + OFF_KV, KV_BLK, 1024), dP = smem_desc(base + OFF_KV + RP * KV_BLK, KV_BLK, 1024);
                for (int si = 0; si < nround && ok; si++, sg++) {
                    const int n = s_seg[si].n;
                    ok = mbar_wait(bar(B_QFULL), (uint32_t)(sg & 1), p.err, 201);
                    for (int t = 0; t < n && ok; t++, it++) {
                        const uint32_t par = (uint32_t)(it & 1);
                        // S^T = K Q^T over the nine column blocks (4 k-steps of 16 each)
#pragma unroll
                        for (int k = 0; k < NBLK; k++) {
                            if (ok && (k & 1) == 0 && k < 8) ok = mbar_wait(bar(B_FULL + k), par, p.err, 202);
                            if (ok) {
                                tc_fence_after();
#pragma unroll
                                for (int ks = 0; ks < 4; ks++)
                                    umma_bf16(tmem + COL_S, dK + (uint64_t)((k * KV_BLK + ks * 32) >> 4), dQ + (uint64_t)((k * Q_BLK + ks * 32) >> 4),
                                              ID_QK, (k | ks) != 0);
                            }
                        }
                        if (!ok) break;
                        umma_commit(bar(B_SFULL));
                        if (t == n - 1) umma_commit(bar(B_QFREE));        // the segment's last scores: Q may be replaced
                        // O^T += V^T P^T. The softmax threads arrive on B_PFULL for a segment's first tile only after
                        // they have read the previous segment's O^T out of tensor memory, so no further wait is needed
                        // before the accumulator is overwritten.
                        ok = mbar_wait(bar(B_PFULL), par, p.err, 203);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t acc0 = t != 0;
#pragma unroll
                        for (int mb = 0; mb < 4; mb++) {
#pragma unroll
                            for (int ks = 0; ks < 8; ks++)
                                umma_bf16(tmem + COL_O + mb * 64, dV + (uint64_t)((2 * mb * KV_BLK + ks * 2048) >> 4), dP + (uint64_t)((ks * 2048) >> 4),
                                          ID_PV, ks != 0 ? 1u : acc0);
                            umma_commit(bar(B_EMPTY_L + mb));
                        }
                        umma_commit(bar(B_EMPTY_RP));
                    }
                }
            }
        } else if (warp >= 4) {
            // ------------------------------------------------------------ softmax / correction / epilogue
            const int q4 = warp & 3;                      // TMEM lane quarter
            const int g = (warp - 4) >> 2;                // head group
            const int hb = g * HG;                        // first head of the group
            const int row = q4 * 32 + lane;               // token row inside the tile == TMEM lane
            const int st = tid - 128;                     // 0..511
            const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
            for (int si = 0; si < nround && ok; si++, sg++) {
                const Seg &s = s_seg[si];
                const bool sole = s.ncontrib == 1;
                if (!sole) {
                    // The common reference: scale * (q_h . row 0 of the sequence), by eight threads per head with
                    // plain loads, the same instructions on the same data in every contributing block.
                    const int h = st >> 3, part = st & 7, nch = p.width >> 6;        // 16-byte pieces per thread
                    const uint4 *qp = reinterpret_cast<const uint4 *>(p.q + ((int64_t)s.b * NH + h) * p.width) + part * nch;
                    const uint4 *kp = reinterpret_cast<const uint4 *>(p.cache + (shared_cache ? 0 : (int64_t)s.b * p.seq_stride)) + part * nch;
                    float d = 0.f;
                    for (int i = 0; i < nch; i++) {
                        const uint4 a = __ldg(qp + i), k4 = __ldg(kp + i);
                        const uint32_t au[4] = {a.x, a.y, a.z, a.w}, ku[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            d = fmaf(__uint_as_float(au[e] << 16), __uint_as_float(ku[e] << 16), d);
                            d = fmaf(__uint_as_float(au[e] & 0xffff0000u), __uint_as_float(ku[e] & 0xffff0000u), d);
                        }
                    }
                    d += __shfl_xor_sync(0xffffffffu, d, 1);
                    d += __shfl_xor_sync(0xffffffffu, d, 2);
                    d += __shfl_xor_sync(0xffffffffu, d, 4);
                    if (part == 0) { s_mref[h] = d * p.scale_log2; s_mref0[h] = d * p.scale_log2; }
                    softmax_bar();
                }
                float lpart[HG];
#pragma unroll
                for (int h = 0; h < HG; h++) lpart[h] = 0.f;
                const int vlim = s.kv - s.t0 * TILE - row;            // this thread's row of tile t is a cached row while t*TILE < vlim
                const int ntile = s.n;
                for (int t = 0; t < ntile; t++, it++) {
                    if (!mbar_wait(bar(B_SFULL), (uint32_t)(it & 1), p.err, 301)) s_flags[5] = 1;   // acted on by all threads together, below
                    tc_fence_after();
                    uint32_t sr[HG];
                    TMEM_LD16(sr, 0, tlane + COL_S + hb);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const bool valid = t * TILE < vlim;
                    float sv[HG];
#pragma unroll
                    for (int h = 0; h < HG; h++) sv[h] = valid ? __uint_as_float(sr[h]) * p.scale_log2 : -INFINITY;

                    if (sole && t == 0) {
                        // nobody to agree with: the reference is the score of the segment's first token
                        if (row == 0) {
#pragma unroll
                            for (int h = 0; h < HG; h++) s_mref[hb + h] = sv[h];
                        }
                        softmax_bar();
                    }
                    // Probabilities against the current reference, computed BEFORE the block agrees on whether a
                    // rescale is needed; in the common case (no rescale) they are the final values.
                    float pv[HG];
                    bool ex = false;
#pragma unroll
                    for (int h = 0; h < HG; h += 4) {
                        const float4 mr = *reinterpret_cast<const float4 *>(s_mref + hb + h);
                        const float d0 = sv[h] - mr.x, d1 = sv[h + 1] - mr.y, d2 = sv[h + 2] - mr.z, d3 = sv[h + 3] - mr.w;
                        ex |= (d0 > LAZY_LOG2) | (d1 > LAZY_LOG2) | (d2 > LAZY_LOG2) | (d3 > LAZY_LOG2);
                        pv[h] = exp2f(d0); pv[h + 1] = exp2f(d1); pv[h + 2] = exp2f(d2); pv[h + 3] = exp2f(d3);
                    }
                    uint32_t need;
                    asm volatile("{\n.reg .pred pi, po;\nsetp.ne.b32 pi, %1, 0;\nbar.red.or.pred po, 1, 512, pi;\nselp.u32 %0, 1, 0, po;\n}\n"
                                 : "=r"(need) : "r"((uint32_t)ex) : "memory");
                    if (s_flags[5]) { ok = false; break; }            // some thread's wait gave up: every thread stops here
                    if (need) {
                        // exact column maxima over the 128 tokens, new reference, rescale what exists
                        float v[HG];
#pragma unroll
                        for (int h = 0; h < HG; h++) v[h] = sv[h];
                        const float mine = warp_transpose_reduce16<true>(v, lane);
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
                        if (t > 0) {
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
#pragma unroll
                        for (int h = 0; h < HG; h++) pv[h] = exp2f(sv[h] - s_mref[hb + h]);
                    }
                    // P^T row of this token -> the rope block's slot, MN-major, 128-byte swizzle
                    uint8_t *prow = sm + OFF_KV + RP * KV_BLK + row * 128;
#pragma unroll
                    for (int cc = 0; cc < HG / 8; cc++) {
#pragma unroll
                        for (int j = 0; j < 8; j++) lpart[cc * 8 + j] += pv[cc * 8 + j];
                        uint4 w;
                        w.x = pack_bf16x2(pv[cc * 8 + 0], pv[cc * 8 + 1]); w.y = pack_bf16x2(pv[cc * 8 + 2], pv[cc * 8 + 3]);
                        w.z = pack_bf16x2(pv[cc * 8 + 4], pv[cc * 8 + 5]); w.w = pack_bf16x2(pv[cc * 8 + 6], pv[cc * 8 + 7]);
                        *reinterpret_cast<uint4 *>(prow + (((g * (HG / 8) + cc) ^ (row & 7)) << 4)) = w;
                    }
                    if (!valid) {       // rows past the sequence end hold whatever the cache holds: 0 x NaN would poison O
                        const uint4 z = make_uint4(0, 0, 0, 0);
                        for (int k = g * 2; k < g * 2 + 2; k++) {
                            uint8_t *vrow = sm + OFF_KV + k * KV_BLK + row * 128;
#pragma unroll
                            for (int cc = 0; cc < 8; cc++) *reinterpret_cast<uint4 *>(vrow + (cc << 4)) = z;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    tc_fence_before();
                    mbar_arrive(bar(B_PFULL));
                }
                if (!ok) break;
                // ---- end of the segment --------------------------------------------------------------
                const int itl = it - 1;                                   // the segment's last tile
                {
                    const float mine = warp_transpose_reduce16<false>(lpart, lane);
                    if (lane < HG) s_w[(warp - 4) * HG + lane] = mine;
                }
                ok = segment_epilogue(p, s, sm, bar0, tmem, itl);
                if (!ok) break;
            }
        }
        __syncthreads();                 // everyone is done with this table
    }

    // ---- the last block out resets the pool counter for the next launch ----------------------------
    if (tid == 0) {
        __threadfence();
        const unsigned int d = atomicAdd(&p.ctl[0], 1u);
        if (d == (unsigned int)G - 1u) {
            p.ctl[0] = 0u;
            p.ctl[1] = 0u;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

constexpr int CWK_SK_EXC_CAP = 16;

void cwk_sk_free(cwk_ctx *ctx) {
    if (ctx->sk_acc) cudaFree(ctx->sk_acc);
    ctx->sk_acc = nullptr;
    delete (CwkMlaTmapCache *)ctx->sk_tmaps;
    ctx->sk_tmaps = nullptr;
}

// How many records blocks have parked so far on this context (see the file comment); synchronises the stream.
extern "C" CWK_API int cwk_mla_decode_parked_records(cwk_ctx *ctx, uint64_t *count) {
    if (!ctx || !count) return CWK_ERR_ARGUMENT;
    *count = 0;
    if (!ctx->sk_acc) return CWK_OK;
    const int slots = ctx->sm_count;
    const unsigned int *tags = (const unsigned int *)((const float *)ctx->sk_acc + (size_t)(slots + CWK_SK_EXC_CAP) * REC) + 2 + slots;
    unsigned int v = 0;
    CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    CWK_CUDA(ctx, cudaMemcpy(&v, tags + CWK_SK_EXC_CAP, sizeof(v), cudaMemcpyDeviceToHost));
    *count = v;
    return CWK_OK;
}

// After a kernel gave up a wait: accumulators and tickets may hold a half-finished step.
void cwk_sk_reset(cwk_ctx *ctx) {
    if (ctx->sk_acc) cudaMemsetAsync(ctx->sk_acc, 0, ctx->sk_bytes, ctx->stream);
}

int cwk_mla_decode_sk_launch(cwk_ctx *ctx, const void *q, const void *cache, int64_t seq_stride, int64_t ld,
                             const int32_t *kv_len, int max_kv_len, int B, int nh, int R, float scale, void *out,
                             float *rec_out, int blocks) {
    const int width = L + R;          // 576, or 512 for a rope-free latent (the rope block then reads as zeros)
    if (nh != NH) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "tcgen05 MLA decode is built for 64 heads");
    if (max_kv_len <= 0) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "tcgen05 MLA decode needs a non-empty cache");
    if (!out && !rec_out) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mla_decode: no output");
    {
        int es = cwk_ensure_err_word(ctx);
        if (es != CWK_OK) return es;
    }
    const int slots = ctx->sm_count;
    if (!ctx->sk_acc) {
        // accumulators [slots][REC] | parked records [EXC_CAP][REC] | control words: one allocation, zeroed once;
        // the kernel leaves everything it touched zeroed again
        const size_t acc_b = (size_t)slots * REC * 4, exc_b = (size_t)CWK_SK_EXC_CAP * REC * 4;
        const size_t ctl_b = ((size_t)(2 + slots + CWK_SK_EXC_CAP + 1) * 4 + 255) & ~(size_t)255;
        CWK_CUDA(ctx, cudaMalloc(&ctx->sk_acc, acc_b + exc_b + ctl_b));
        ctx->sk_bytes = acc_b + exc_b + ctl_b;
        CWK_CUDA(ctx, cudaMemsetAsync(ctx->sk_acc, 0, ctx->sk_bytes, ctx->stream));
    }
    const CUtensorMap *tm_q = nullptr, *tm_kv = nullptr, *tm_kr = nullptr;
    {
        int ts = cwk_mla_tensor_maps(ctx, q, cache, seq_stride, ld, max_kv_len, B, width, &tm_q, &tm_kv, &tm_kr);
        if (ts != CWK_OK) return ts;
    }
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(mla_decode_sk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
        attr_set[ctx->device & 15] = true;
    }
    const int64_t max_tiles = (int64_t)B * ((max_kv_len + TILE - 1) / TILE);
    int G = (int)std::min<int64_t>(slots, max_tiles);
    if (blocks > 0) G = std::min(G, blocks);
    if (G < 1) G = 1;
    SkParams p;
    p.kv_len = kv_len; p.kv_len_imm = max_kv_len; p.B = B;
    p.q = (const uint16_t *)q; p.cache = (const uint16_t *)cache; p.seq_stride = seq_stride; p.ld = ld; p.width = width;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.acc = (float *)ctx->sk_acc;
    p.exc = p.acc + (size_t)slots * REC;
    p.ctl = (unsigned int *)(p.exc + (size_t)CWK_SK_EXC_CAP * REC);
    p.tags = p.ctl + 2 + slots;
    p.exc_cap = CWK_SK_EXC_CAP;
    p.out = (uint16_t *)out; p.rec_out = out ? nullptr : rec_out;
    p.err = ctx->dev_err;
    mla_decode_sk_kernel<<<G, NTHREADS, SMEM_TOTAL, ctx->stream>>>(*tm_q, *tm_kv, *tm_kr, p);
    CWK_LAUNCH_CHECK(ctx, "mla_decode_sk_kernel");
    return CWK_OK;
}
