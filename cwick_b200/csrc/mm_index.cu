// mm_index.cu -- the MiniMax block indexer: per-position index scores over bf16 keys and the selection of
// blocks a query may attend to (src/mm_model.c:1733-1781). The attention over the selected positions is the
// gathered GQA decode of csrc/gqa.cu (cwk_gqa_decode_sel).
//   mm_index_scores_kernel   sc[s] = sum_h ReLU(q_h . k_s): one thread per key (rows staged through shared memory),
//                            heads in order, sequential f32 dots (the reference's order, so block maxima and ties
//                            are the reference's)
//   mm_select_fused_kernel   block maxima, exact top blocks and the position list in one launch (up to 1024 blocks)
//   mm_block_max_kernel      (longer rows: three launches) maximum of every block of `bs` scores (fmaxf from -1e30,
//                            partial last block included)
//   mm_expand_blocks_kernel  the top blocks (exact top-k of csrc/dsa.cu, ascending) plus the block holding the next
//                            position when it is missing, expanded to the list of positions (at most `cap`)
#include "cwk_common.cuh"

namespace {

// 128 keys per block: their rows (ID bf16 each) come into shared memory by 16-byte asynchronous copies, coalesced, into
// rows padded by 4 words, so that a thread's 16-byte reads of its own row are conflict-free.
template <int ID>
__global__ void __launch_bounds__(128, 5) mm_index_scores_kernel(const uint16_t *keys, int64_t n, const float *q, int ih, float *sc) {
    constexpr int WPR = ID / 2, LD = WPR + 4;      // words per key row, padded row stride
    extern __shared__ float s_dyn[];
    float *s_q = s_dyn;                            // [ih][ID]
    uint32_t *s_k = reinterpret_cast<uint32_t *>(s_dyn + ih * ID);       // [128][LD]
    const int64_t s0 = (int64_t)blockIdx.x * 128;
    const int nk = (int)min((int64_t)128, n - s0);
    {
        const uint32_t kb = (uint32_t)__cvta_generic_to_shared(s_k);
        const uint16_t *src = keys + s0 * ID;
        for (int ch = threadIdx.x; ch < nk * (WPR / 4); ch += 128) {
            const int row = ch / (WPR / 4), c4 = ch % (WPR / 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kb + (uint32_t)(row * LD + c4 * 4) * 4u), "l"(src + (int64_t)ch * 8) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int i = threadIdx.x; i < ih * ID; i += blockDim.x) s_q[i] = q[i];
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if ((int)threadIdx.x >= nk) return;
    uint32_t kw[WPR];                               // the key row as it is stored: two bf16 per word (half the registers of f32)
#pragma unroll
    for (int c = 0; c < WPR / 4; c++) {
        const uint4 v = *reinterpret_cast<const uint4 *>(s_k + threadIdx.x * LD + c * 4);
        kw[c * 4] = v.x; kw[c * 4 + 1] = v.y; kw[c * 4 + 2] = v.z; kw[c * 4 + 3] = v.w;
    }
    auto kf = [&](int i) { return (i & 1) ? __uint_as_float(kw[i >> 1] & 0xFFFF0000u) : __uint_as_float(kw[i >> 1] << 16); };
    // Four heads at a time: each head's dot stays one sequential chain (the reference's order), the four chains are
    // independent of each other and fill the adder's latency; the heads' ReLU'd dots are then added in head order.
    float tot = 0.f;
    int h = 0;
    for (; h + 4 <= ih; h += 4) {
        const float *q0 = s_q + h * ID, *q1 = q0 + ID, *q2 = q1 + ID, *q3 = q2 + ID;
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
        for (int i = 0; i < ID; i++) {
            d0 = __fadd_rn(d0, __fmul_rn(q0[i], kf(i)));
            d1 = __fadd_rn(d1, __fmul_rn(q1[i], kf(i)));
            d2 = __fadd_rn(d2, __fmul_rn(q2[i], kf(i)));
            d3 = __fadd_rn(d3, __fmul_rn(q3[i], kf(i)));
        }
        if (d0 > 0.f) tot = __fadd_rn(tot, d0);
        if (d1 > 0.f) tot = __fadd_rn(tot, d1);
        if (d2 > 0.f) tot = __fadd_rn(tot, d2);
        if (d3 > 0.f) tot = __fadd_rn(tot, d3);
    }
    for (; h < ih; h++) {
        const float *qh = s_q + h * ID;
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < ID; i++) d = __fadd_rn(d, __fmul_rn(qh[i], kf(i)));
        if (d > 0.f) tot = __fadd_rn(tot, d);
    }
    sc[s0 + threadIdx.x] = tot;
}

__global__ void mm_block_max_kernel(const float *sc, int64_t limit, int bs, float *bsc, int32_t *nblk_out) {
    const int nblk = (int)((limit + bs - 1) / bs);
    const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (blockIdx.x == 0 && threadIdx.x == 0) *nblk_out = nblk;
    if (b >= nblk) return;
    const int64_t s0 = (int64_t)b * bs, s1 = min((int64_t)limit, s0 + bs);
    float mx = -1e30f;
    for (int64_t t = s0 + lane; t < s1; t += 32) mx = fmaxf(mx, sc[t]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) bsc[b] = mx;
}

// One block. blk: the ascending top blocks (count in *cnt). Appends block limit / bs when it is not among them and
// the list is shorter than topk + 4, then writes the positions of the blocks in list order, clipped to `limit` and
// to `cap` entries; *nsel = number of positions, *nblk_sel = number of blocks.
__global__ void __launch_bounds__(256) mm_expand_blocks_kernel(int32_t *blk, const int32_t *cnt, int64_t limit, int bs, int topk, int cap,
                                                               int32_t *sel, int32_t *nsel, int32_t *nblk_sel) {
    __shared__ int s_off[1024 + 8];
    __shared__ int s_nb;
    if (threadIdx.x == 0) {
        int nb = *cnt;
        const int last = (int)(limit / bs);
        bool have = false;
        for (int i = 0; i < nb; i++) have |= (blk[i] == last);
        if (!have && nb < topk + 4) blk[nb++] = last;
        int off = 0;
        for (int i = 0; i < nb; i++) {
            s_off[i] = off;
            const int64_t s0 = (int64_t)blk[i] * bs;
            const int64_t s1 = min(limit, s0 + bs);
            off += (int)max((int64_t)0, s1 - s0);
        }
        s_off[nb] = off;
        s_nb = nb;
        *nsel = min(off, cap);
        *nblk_sel = nb;
    }
    __syncthreads();
    const int nb = s_nb;
    for (int i = 0; i < nb; i++) {
        const int64_t s0 = (int64_t)blk[i] * bs;
        const int len = s_off[i + 1] - s_off[i];
        for (int t = threadIdx.x; t < len; t += blockDim.x)
            if (s_off[i] + t < cap) sel[s_off[i] + t] = (int32_t)(s0 + t);
    }
}

// The whole selection in one launch, for up to 1024 blocks of a multiple of four scores: one block of 1024 threads.
//   1. block maxima: a thread takes 16-byte groups t, t + 1024, ... of the scores (all its loads in flight at once) and
//      folds each group's maximum into its block's slot with a shared-memory atomic on order-preserving keys;
//   2. exact top blocks: the topk-th largest maximum by radix select; a block is kept when its maximum is larger, or
//      equal and among the first of the equal ones in index order (the rule of the exact top-k kernel);
//   3. the kept blocks in ascending order by a block-wide scan, the most recent block appended as the reference does,
//      and the positions of the list written by all threads (a binary search per position over the blocks' offsets).
__device__ __forceinline__ int mm_block_scan_1024(int v, int *s_warp, int &total) {      // exclusive scan over 1024 threads
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += u;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = s_warp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += u;
        }
        s_warp[lane] = w;
    }
    __syncthreads();
    total = s_warp[31];
    const int base = warp ? s_warp[warp - 1] : 0;
    __syncthreads();
    return base + inc - v;
}

__global__ void __launch_bounds__(1024) mm_select_fused_kernel(const float *sc, int64_t limit, int bs, int topk, int cap, int32_t *sel,
                                                               int32_t *nsel, int32_t *blk_out, int32_t *nblk_out) {
    __shared__ uint32_t s_key[1024];
    __shared__ int s_blk[1024 + 8], s_off[1024 + 8 + 1], s_warp[32], s_have, s_hist[256], s_pick[2];
    const int tid = threadIdx.x;
    const int nblk = (int)((limit + bs - 1) / bs);
    auto key_of = [](float f) { const uint32_t u = __float_as_uint(f); return (u & 0x80000000u) ? ~u : (u | 0x80000000u); };
    if (tid < nblk) s_key[tid] = key_of(-1e30f);
    __syncthreads();
    {
        const int64_t ngroups = (limit + 3) / 4;
        constexpr int AHEAD = 8;
        for (int64_t g0 = tid; g0 < ngroups; g0 += 1024 * AHEAD) {
            float4 v[AHEAD];
#pragma unroll
            for (int u = 0; u < AHEAD; u++) {
                const int64_t g = g0 + (int64_t)u * 1024;
                v[u] = make_float4(-1e30f, -1e30f, -1e30f, -1e30f);
                if (g < ngroups) {
                    if (g * 4 + 4 <= limit) v[u] = __ldg(reinterpret_cast<const float4 *>(sc) + g);
                    else {
                        v[u].x = sc[g * 4];
                        if (g * 4 + 1 < limit) v[u].y = sc[g * 4 + 1];
                        if (g * 4 + 2 < limit) v[u].z = sc[g * 4 + 2];
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < AHEAD; u++) {
                const int64_t g = g0 + (int64_t)u * 1024;
                if (g < ngroups) atomicMax(&s_key[(int)(g * 4 / bs)], key_of(fmaxf(fmaxf(fmaxf(fmaxf(-1e30f, v[u].x), v[u].y), v[u].z), v[u].w)));
            }
        }
    }
    __syncthreads();
    // The topk-th largest key by radix select (four passes of eight bits over a 256-bin histogram in shared memory),
    // then: kept = larger than it, or equal to it and among the first `need` equal ones in index order.
    const uint32_t mine = tid < nblk ? s_key[tid] : 0u;
    int keep = 0;
    if (nblk <= topk) {
        keep = tid < nblk;
    } else {
        uint32_t prefix = 0, mask = 0;
        int need = topk;
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) s_hist[tid] = 0;
            __syncthreads();
            if (tid < nblk && (mine & mask) == prefix) atomicAdd(&s_hist[(mine >> shift) & 255u], 1);
            __syncthreads();
            if (tid < 32) {                              // warp 0: the bin in which the `need`-th largest candidate lies
                int c[8], mysum = 0;
#pragma unroll
                for (int u = 0; u < 8; u++) { c[u] = s_hist[tid * 8 + u]; mysum += c[u]; }
                int above = mysum;                       // candidates in this lane's bins and in the bins of higher lanes
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int u = __shfl_down_sync(0xffffffffu, above, o);
                    if (tid + o < 32) above += u;
                }
                const int higher = above - mysum;        // candidates in the bins of higher lanes only
                if (higher < need && above >= need) {    // exactly one lane
                    int left = need - higher, d = 7;
                    for (; d > 0; d--) {
                        if (c[d] >= left) break;
                        left -= c[d];
                    }
                    s_pick[0] = tid * 8 + d;
                    s_pick[1] = left;                    // still to take inside bin d
                }
            }
            __syncthreads();
            prefix |= (uint32_t)s_pick[0] << shift;
            mask |= 255u << shift;
            need = s_pick[1];
            __syncthreads();
        }
        int ntie;
        const int eq = tid < nblk && mine == prefix;
        const int eqrank = mm_block_scan_1024(eq, s_warp, ntie);
        keep = tid < nblk && (mine > prefix || (eq && eqrank < need));
    }
    const int last = (int)(limit / bs);                  // the block of the next position: always listed (it may hold no score yet)
    if (tid == 0) s_have = 0;
    int nb;
    const int pos = mm_block_scan_1024(keep, s_warp, nb);      // (its barriers order the flag's reset before the write below)
    if (keep) {
        s_blk[pos] = tid;
        if (tid == last) s_have = 1;
    }
    __syncthreads();
    if (!s_have && nb < topk + 4) {                      // every thread takes the same branch
        if (tid == 0) s_blk[nb] = last;
        nb++;
    }
    __syncthreads();
    // positions per listed block, their offsets
    int len = 0;
    if (tid < nb) {
        const int64_t s0 = (int64_t)s_blk[tid] * bs, s1 = min(limit, s0 + bs);
        len = (int)max((int64_t)0, s1 - s0);
    }
    int total;
    const int off = mm_block_scan_1024(len, s_warp, total);
    if (tid < nb) s_off[tid] = off;
    if (tid == 0) s_off[nb] = total;
    __syncthreads();                                     // (topk <= 1020: the list, the appended block included, fits the 1024 threads)
    const int nout = min(total, cap);
    for (int q = tid; q < nout; q += 1024) {
        int lo = 0, hi = nb - 1;                         // the listed block that holds position q: s_off[lo] <= q < s_off[lo + 1]
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_off[mid] <= q) lo = mid; else hi = mid - 1;
        }
        sel[q] = (int32_t)((int64_t)s_blk[lo] * bs + (q - s_off[lo]));
    }
    if (blk_out)
        for (int i = tid; i < nb; i += 1024) blk_out[i] = s_blk[i];
    if (tid == 0) {
        *nsel = nout;
        if (nblk_out) *nblk_out = nb;
    }
}

}  // namespace

extern "C" {

int cwk_ds_topk(cwk_ctx *ctx, const float *sc, int64_t sc_stride, const int32_t *n, int B, int k, int32_t *out, int64_t out_ld,
                int32_t *count);

int cwk_mm_index_scores(cwk_ctx *ctx, const void *keys, int64_t n, int id, const float *q, int ih, float *sc) {
    if (!ctx || !keys || !q || !sc || n < 0 || ih <= 0) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mm_index_scores: bad argument");
    if (id != 64 && id != 128) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "mm_index_scores is built for index dims 64 and 128 (got %d)", id);
    if (reinterpret_cast<uintptr_t>(keys) & 15) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mm_index_scores: keys must be 16-byte aligned");
    const size_t smem = (size_t)ih * id * 4 + (size_t)128 * (id / 2 + 4) * 4;
    if (smem > 48 * 1024) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "mm_index_scores: too many index heads");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (n == 0) return CWK_OK;
    CwkKernelTimer timer(ctx);
    const unsigned grid = (unsigned)((n + 127) / 128);
    if (id == 128) mm_index_scores_kernel<128><<<grid, 128, smem, ctx->stream>>>((const uint16_t *)keys, n, q, ih, sc);
    else mm_index_scores_kernel<64><<<grid, 128, smem, ctx->stream>>>((const uint16_t *)keys, n, q, ih, sc);
    CWK_LAUNCH_CHECK(ctx, "mm_index_scores_kernel");
    return CWK_OK;
}

int cwk_mm_select_blocks(cwk_ctx *ctx, const float *sc, int64_t limit, int bs, int topk, int cap, int32_t *sel, int32_t *nsel,
                         int32_t *blk_out, int32_t *nblk_out) {
    if (!ctx || !sc || !sel || !nsel || limit <= 0 || bs <= 0 || topk <= 0 || topk + 4 > 1024 || cap <= 0)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mm_select_blocks: bad argument (topk <= 1020)");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const int nblk = (int)((limit + bs - 1) / bs);
    if (nblk <= 1024 && bs % 4 == 0 && (reinterpret_cast<uintptr_t>(sc) & 15) == 0) {      // one launch
        CwkKernelTimer timer(ctx);
        mm_select_fused_kernel<<<1, 1024, 0, ctx->stream>>>(sc, limit, bs, topk, cap, sel, nsel, blk_out, nblk_out);
        CWK_LAUNCH_CHECK(ctx, "mm_select_fused_kernel");
        return CWK_OK;
    }
    // work: block maxima [nblk + 1] | kept blocks [topk + 4] | block count | kept count | blocks selected
    int s = cwk_reserve_work(ctx, ((size_t)nblk + 1 + topk + 4 + 3) * sizeof(float));
    if (s != CWK_OK) return s;
    float *bsc = (float *)ctx->work;
    int32_t *blk = blk_out ? blk_out : (int32_t *)(bsc + nblk + 1);
    int32_t *nb = (int32_t *)(bsc + nblk + 1) + topk + 4, *cnt = nb + 1, *nbs = nblk_out ? nblk_out : nb + 2;
    mm_block_max_kernel<<<(nblk + 7) / 8, 256, 0, ctx->stream>>>(sc, limit, bs, bsc, nb);
    CWK_LAUNCH_CHECK(ctx, "mm_block_max_kernel");
    s = cwk_ds_topk(ctx, bsc, nblk, nb, 1, topk, blk, topk, cnt);
    if (s != CWK_OK) return s;
    mm_expand_blocks_kernel<<<1, 256, 0, ctx->stream>>>(blk, cnt, limit, bs, topk, cap, sel, nsel, nbs);
    CWK_LAUNCH_CHECK(ctx, "mm_expand_blocks_kernel");
    return CWK_OK;
}

}  // extern "C"
