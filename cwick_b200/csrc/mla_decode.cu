// mla_decode.cu -- MLA absorbed decode over the bf16 latent cache: launch
// planning, the general-dimension kernel, the split merge, and the C entry
// points. The 512+64 / 64-row-block case runs on tensor cores (flash_rows.cuh,
// and the tcgen05 kernel in mla_decode_tc.cu when present); any other
// dimensions take the general kernel below.
#include <algorithm>
#include <cmath>

#include "flash_rows.cuh"

// tcgen05/TMA path (mla_decode_tc.cu). Returns CWK_ERR_UNSUPPORTED when it does
// not apply so the caller can take the mma.sync path.
int cwk_mla_decode_tc_launch(cwk_ctx *ctx, const void *q, const void *cache, int64_t seq_stride,
                             int64_t ld, const int32_t *kv_len, int max_kv_len, int B, int nh,
                             int R, float scale, float *partial, int nsplit, void *out_direct, const int32_t *sel, int64_t sel_ld);
bool cwk_mla_decode_tc_available();
// persistent tcgen05/TMA kernel with the cross-block reduction inside (mla_decode_sk.cu): bf16 rows to `out`, or one
// folded record per sequence to `rec_out`
int cwk_mla_decode_sk_launch(cwk_ctx *ctx, const void *q, const void *cache, int64_t seq_stride, int64_t ld,
                             const int32_t *kv_len, int max_kv_len, int B, int nh, int R, float scale, void *out,
                             float *rec_out, int blocks);

// ---------------------------------------------------------------------------
// General kernel: any nh, L <= 512 (multiple of 2), any R. One block per
// (split, head, sequence); each of 4 warps walks a quarter of the split's keys
// with a running (m, l, o) and the four are merged in shared memory.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) mla_decode_general_kernel(
    const uint16_t *q, const uint16_t *cache, int64_t seq_stride, int64_t ld, const int32_t *kv_len,
    const int32_t *sel, int64_t sel_ld, int nh, int L, int R, float scale, float *partial,
    int nsplit, int kv_len_imm) {
    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = kv_len ? kv_len[b] : kv_len_imm;
    const int t0 = (int)((int64_t)n * split / nsplit), t1 = (int)((int64_t)n * (split + 1) / nsplit);
    const int DKq = L + R;
    const uint16_t *qh = q + ((int64_t)b * nh + h) * DKq;
    const uint16_t *base = cache + (int64_t)b * seq_stride;
    constexpr int MAXJ = 16;
    float acc[MAXJ];
#pragma unroll
    for (int j = 0; j < MAXJ; j++) acc[j] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int t = t0 + warp; t < t1; t += 4) {
        const int64_t row = sel ? sel[(int64_t)b * sel_ld + t] : t;
        const uint16_t *c = base + row * ld;
        float d = 0.f;
        for (int i = lane; i < DKq; i += 32) d += bf16_bits_to_f32(qh[i]) * bf16_bits_to_f32(c[i]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        d *= scale;
        const float mn = fmaxf(m, d);
        const float alpha = (m == -INFINITY) ? 0.f : __expf(m - mn);
        const float pw = __expf(d - mn);
        l = l * alpha + pw;
#pragma unroll
        for (int j = 0; j < MAXJ; j++) {
            const int i = lane + 32 * j;
            if (i < L) acc[j] = acc[j] * alpha + pw * bf16_bits_to_f32(c[i]);
        }
        m = mn;
    }
    __shared__ float sm[4], sl[4], so[4][512];
    if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
    for (int j = 0; j < MAXJ; j++) {
        const int i = lane + 32 * j;
        if (i < L) so[warp][i] = acc[j];
    }
    __syncthreads();
    float M = fmaxf(fmaxf(sm[0], sm[1]), fmaxf(sm[2], sm[3]));
    float *rec = partial + ((int64_t)b * nsplit + split) * ((int64_t)nh * (L + 2));
    float w[4], lt = 0.f;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        w[k] = (sm[k] == -INFINITY) ? 0.f : __expf(sm[k] - M);
        lt += w[k] * sl[k];
    }
    if (threadIdx.x == 0) { rec[h] = M; rec[nh + h] = lt; }
    for (int i = threadIdx.x; i < L; i += 128)
        rec[2 * nh + (int64_t)h * L + i] = w[0] * so[0][i] + w[1] * so[1][i] + w[2] * so[2][i] + w[3] * so[3][i];
}

// ---------------------------------------------------------------------------
// launch planning
// ---------------------------------------------------------------------------
// Pick the split count that minimises (waves of blocks) x (tiles per block),
// with a small charge per split for the partial it writes and the merge reads.
static int plan_splits(int sm_count, int blocks_per_split, int max_tiles, int requested) {
    if (max_tiles < 1) max_tiles = 1;
    if (requested > 0) return std::min(std::min(requested, max_tiles), CWK_MAX_SPLITS);
    int best = 1;
    double best_cost = 1e30;
    const int cap = std::min(max_tiles, 256);
    for (int ns = 1; ns <= cap; ns++) {
        const int64_t blocks = (int64_t)blocks_per_split * ns;
        const double waves = std::ceil((double)blocks / sm_count);
        const double tiles = std::ceil((double)max_tiles / ns);
        const double cost = waves * (tiles + 1.5) + 0.02 * ns;
        if (cost < best_cost - 1e-9) { best_cost = cost; best = ns; }
    }
    return best;
}

using MlaSmem = FlashRowsSmem<64, 576, 512, 64, 8, false>;

static int mla_launch(cwk_ctx *ctx, const void *q, const void *cache, int64_t seq_stride, int64_t ld,
                      const int32_t *kv_len, int max_kv_len, const int32_t *sel, int64_t sel_ld, int B,
                      int nh, int L, int R, float scale, void *out, float *partial_out, int n_splits) {
    if (!ctx || !q || !cache || (!kv_len && B != 1) || (!out && !partial_out && !ctx->keep_splits)) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mla_decode: null argument");
    if (B <= 0 || nh <= 0 || L <= 0 || R < 0 || max_kv_len < 0 || ld < L + R)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mla_decode: bad dimensions B=%d nh=%d L=%d R=%d ld=%lld", B, nh, L, R, (long long)ld);
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));

    const bool aligned = (ld % 8) == 0 && (seq_stride % 8) == 0 && ((uintptr_t)cache % 16) == 0 && ((uintptr_t)q % 16) == 0;
    int path = (L == 512 && R == 64 && aligned) ? 1 : 0;
    // the tcgen05 kernel also takes the rope-free 512-wide latent: its ninth column block is then
    // out of the tensor's bounds and arrives as zeros
    // (a row list goes to the same kernel: two of its warps fetch the listed rows with 16-byte copies instead of TMA boxes)
    const bool tc_ok = L == 512 && (R == 64 || R == 0) && aligned && nh == 64 && max_kv_len > 0 && cwk_mla_decode_tc_available();
    if (tc_ok) path = 2;
    if (ctx->force_mla_path >= 0 && ctx->force_mla_path != 3) {
        // 4 = the persistent kernel: same conditions as 2, taken only on request (its cross-block sums go through f32
        // atomics, which the split records + merge launch of 2 beat at every shape measured so far)
        const int best = tc_ok ? (sel ? 2 : 4) : path;
        if (ctx->force_mla_path > best || (ctx->force_mla_path == 3))
            return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "mla_decode: forced path %d not applicable (best %d)", ctx->force_mla_path, path);
        path = ctx->force_mla_path;
    }
    if (path == 4) {
        // one persistent launch: no split records, no merge
        const size_t recb = (size_t)nh * (L + 2) * sizeof(float);
        float *rec_dst = partial_out;
        if (!out && !partial_out) {           // keep_splits: one folded record in the context's scratch
            int s = cwk_reserve_scratch(ctx, recb);
            if (s != CWK_OK) return s;
            rec_dst = ctx->scratch;
        }
        {
            CwkKernelTimer timer(ctx);
            int s = cwk_mla_decode_sk_launch(ctx, q, cache, seq_stride, ld, kv_len, max_kv_len, B, nh, R, scale, out, rec_dst,
                                             n_splits > 0 ? n_splits * B : -n_splits);
            if (s != CWK_OK) return s;
        }
        ctx->last_nsplit = 1;
        return CWK_OK;
    }
    if (path == 0 && (L > 512 || (L & 1)))
        return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "mla_decode: general kernel needs even L <= 512 (got %d)", L);

    const int tile = (path >= 2) ? 128 : (path == 1 ? 64 : 32);
    const int max_tiles = (max_kv_len + tile - 1) / tile;
    const int hblocks = (path == 0) ? nh : (nh + 63) / 64;
    int ns = plan_splits(ctx->sm_count, B * hblocks, max_tiles, n_splits > 0 ? n_splits : 0);
    // One split per sequence needs no records at all: the kernel normalises and writes bf16.
    const bool direct = (ns == 1 && out && !partial_out && path != 0);
    const size_t rec = (size_t)nh * (L + 2) * sizeof(float);
    if (!direct) {
        int s = cwk_reserve_scratch(ctx, rec * ((size_t)ns * B + (ctx->keep_splits ? 1 : 0)));      // keep_splits: room for one folded record behind them
        if (s != CWK_OK) return s;
    }
    float *partial = ctx->scratch;

    {
    CwkKernelTimer timer(ctx);
    if (path == 2) {
        int s = cwk_mla_decode_tc_launch(ctx, q, cache, seq_stride, ld, kv_len, max_kv_len, B, nh, R, scale, partial, ns,
                                         direct ? out : nullptr, sel, sel_ld);
        if (s != CWK_OK) return s;
    } else if (path == 1) {
        static bool attr_set[16] = {false};
        auto kern = flash_rows_kernel<MODE_MLA, 64, 576, 512, 64, 8, false>;
        if (!attr_set[ctx->device & 15]) {
            CWK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MlaSmem::TOTAL));
            attr_set[ctx->device & 15] = true;
        }
        FlashRowsParams p{};
        p.q = (const uint16_t *)q; p.k = (const uint16_t *)cache; p.v = p.k;
        p.seq_stride = seq_stride; p.ld = ld; p.kv_len = kv_len; p.kv_len_imm = max_kv_len; p.sel = sel; p.sel_ld = sel_ld;
        p.nh = nh; p.nkv = 1; p.group = nh; p.scale_log2 = scale * 1.4426950408889634f;
        p.partial = partial; p.out = direct ? (uint16_t *)out : nullptr; p.nsplit = ns; p.direct = direct ? 1 : 0;
        kern<<<dim3(ns, hblocks, B), 256, MlaSmem::TOTAL, ctx->stream>>>(p);
        CWK_LAUNCH_CHECK(ctx, "flash_rows_kernel<MLA>");
    } else {
        mla_decode_general_kernel<<<dim3(ns, nh, B), 128, 0, ctx->stream>>>(
            (const uint16_t *)q, (const uint16_t *)cache, seq_stride, ld, kv_len, sel, sel_ld, nh, L, R,
            scale, partial, ns, max_kv_len);
        CWK_LAUNCH_CHECK(ctx, "mla_decode_general_kernel");
    }
    }
    if (out && !direct) {
        lse_combine_launch(ctx->stream, partial, ns, nh, L, B, (uint16_t *)out);
        CWK_LAUNCH_CHECK(ctx, "lse_merge_kernel");
    }
    ctx->last_nsplit = ns;
    if (partial_out && !ctx->keep_splits) {          // B == 1 here
        lse_fold_launch(ctx->stream, partial, ns, nh, L, partial_out);
        CWK_LAUNCH_CHECK(ctx, "lse_merge_kernel<fold>");
    }
    return CWK_OK;
}

// One sequence whose row count is known on the host (no device length array): used by the
// reference-named decode entry point.
int cwk_mla_decode_rows(cwk_ctx *ctx, const void *q, const void *cache, int64_t ld, int rows, int nh, int L, int R,
                        float scale, void *out) {
    return mla_launch(ctx, q, cache, 0, ld, nullptr, rows, nullptr, 0, 1, nh, L, R, scale, out, nullptr, 0);
}

// Split-KV decode of one sequence whose result stays as split records in the context's scratch
// (the KV-range exchange folds and ships them itself).
int cwk_mla_launch_splits(cwk_ctx *ctx, const void *q, const void *cache, int64_t ld, int rows, int nh, int L, int R,
                          float scale, float **partial_out, int *nsplit_out) {
    ctx->keep_splits = true;
    int s = mla_launch(ctx, q, cache, 0, ld, nullptr, rows, nullptr, 0, 1, nh, L, R, scale, nullptr, nullptr, 0);
    ctx->keep_splits = false;
    *partial_out = ctx->scratch;
    *nsplit_out = ctx->last_nsplit;
    return s;
}

extern "C" {

int cwk_mla_decode_path(const cwk_ctx *ctx, int nh, int L, int R) {
    if (!ctx) return -1;
    int path = (L == 512 && R == 64) ? 1 : 0;
    const bool tc_ok = L == 512 && (R == 64 || R == 0) && nh == 64 && cwk_mla_decode_tc_available();
    if (tc_ok) path = 2;
    if (ctx->force_mla_path >= 0 && ctx->force_mla_path != 3 && ctx->force_mla_path <= (tc_ok ? 4 : path)) path = ctx->force_mla_path;
    return path;
}

int cwk_mla_decode(cwk_ctx *ctx, const void *q, const void *cache, int64_t seq_stride, int64_t ld,
                   const int32_t *kv_len, int max_kv_len, const int32_t *sel, int64_t sel_ld, int B,
                   int nh, int L, int R, float scale, void *out, int n_splits) {
    if (!out) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mla_decode: out is null");
    return mla_launch(ctx, q, cache, seq_stride, ld, kv_len, max_kv_len, sel, sel_ld, B, nh, L, R, scale,
                      out, nullptr, n_splits);
}

static bool is_pinned_host(const void *p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeHost;
}

int cwk_mla_decode_host(cwk_ctx *ctx, const void *q_host, const void *cache_dev, int64_t seq_stride,
                        int64_t ld, const int32_t *kv_len_host, const int32_t *sel_host, int64_t sel_ld,
                        int B, int nh, int L, int R, float scale, void *out_host, int n_splits) {
    if (!ctx || !q_host || !cache_dev || !kv_len_host || !out_host || B <= 0 || nh <= 0 || L <= 0 || R < 0)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mla_decode_host: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t qb = (size_t)B * nh * (L + R) * 2, ob = (size_t)B * nh * L * 2, lb = (size_t)B * 4;
    const size_t sb = sel_host ? (size_t)B * sel_ld * 4 : 0;
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const size_t total = up(qb) + up(ob) + up(lb) + up(sb);
    int s = cwk_reserve_stage(ctx, total, total);
    if (s != CWK_OK) return s;
    uint8_t *pin = (uint8_t *)ctx->stage_pin, *dev = (uint8_t *)ctx->stage_dev;
    const size_t o_q = 0, o_l = up(qb), o_s = o_l + up(lb), o_o = o_s + up(sb);
    // Caller buffers that are already page-locked are copied from and to directly; pageable ones
    // go through the context's pinned staging.
    const bool q_pinned = is_pinned_host(q_host), o_pinned = is_pinned_host(out_host);
    int max_len = 0;
    for (int i = 0; i < B; i++) max_len = std::max(max_len, (int)kv_len_host[i]);
    const bool lens_imm = (B == 1);                 // one sequence: its length travels as a kernel argument
    if (q_pinned) {
        CWK_CUDA(ctx, cudaMemcpyAsync(dev + o_q, q_host, qb, cudaMemcpyHostToDevice, ctx->stream));
    } else {
        memcpy(pin + o_q, q_host, qb);
        CWK_CUDA(ctx, cudaMemcpyAsync(dev + o_q, pin + o_q, qb, cudaMemcpyHostToDevice, ctx->stream));
    }
    if (!lens_imm || sb) {
        memcpy(pin + o_l, kv_len_host, lb);
        if (sb) memcpy(pin + o_s, sel_host, sb);
        CWK_CUDA(ctx, cudaMemcpyAsync(dev + o_l, pin + o_l, o_o - o_l, cudaMemcpyHostToDevice, ctx->stream));
    }
    // A page-locked output buffer that the device can address (mapped pinned memory) is written by the last kernel
    // itself: one copy operation less between the kernels and the caller.
    void *out_alias = nullptr;
    if (o_pinned && cudaHostGetDevicePointer(&out_alias, out_host, 0) != cudaSuccess) {
        (void)cudaGetLastError();
        out_alias = nullptr;
    }
    s = mla_launch(ctx, dev + o_q, cache_dev, seq_stride, ld, lens_imm ? nullptr : (const int32_t *)(dev + o_l), max_len,
                   sb ? (const int32_t *)(dev + o_s) : nullptr, sel_ld, B, nh, L, R, scale, out_alias ? out_alias : (void *)(dev + o_o),
                   nullptr, n_splits);
    if (s != CWK_OK) return s;
    if (!out_alias)
        CWK_CUDA(ctx, cudaMemcpyAsync(o_pinned ? out_host : (void *)(pin + o_o), dev + o_o, ob, cudaMemcpyDeviceToHost, ctx->stream));
    CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    s = cwk_check_device_error(ctx);
    if (s != CWK_OK) return s;
    if (!o_pinned) memcpy(out_host, pin + o_o, ob);
    return CWK_OK;
}

int cwk_mla_decode_partial(cwk_ctx *ctx, const void *q, const void *cache, int64_t ld, int64_t row0,
                           int64_t rows, int nh, int L, int R, float scale, float *partial) {
    if (!ctx || !partial || rows < 0 || row0 < 0) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mla_decode_partial: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    // Split inside the GPU as usual, then fold the splits into ONE un-normalised record.
    const uint16_t *base = (const uint16_t *)cache + row0 * ld;
    return mla_launch(ctx, q, base, 0, ld, nullptr, (int)rows, nullptr, 0, 1, nh, L, R,
                      scale, nullptr, partial, 0);
}

int cwk_lse_combine(cwk_ctx *ctx, const float *partials, int G, int nh, int L, void *out) {
    if (!ctx || !partials || !out || G <= 0 || G > CWK_MAX_SPLITS || nh <= 0 || L <= 0 || (L & 1))
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "lse_combine: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    lse_combine_launch(ctx->stream, partials, G, nh, L, 1, (uint16_t *)out);
    CWK_LAUNCH_CHECK(ctx, "lse_merge_kernel");
    return CWK_OK;
}

}  // extern "C"
