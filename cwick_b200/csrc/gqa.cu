// gqa.cu -- Qwen3.5-style grouped-query attention: single-query decode
// (split over the key range, merged by lse_merge_kernel) and causal prefill.
// Both run flash_rows_kernel with K and V as separate streams.
#include <algorithm>
#include <cmath>

#include "flash_rows.cuh"

template <int HD>
static int gqa_decode_launch(cwk_ctx *ctx, const FlashRowsParams &p, int B, int nkv, int ns) {
    // A decode step is 4 FLOP per cached byte: nothing but latency to hide. A ring of three tiles (two in flight, 128 KB per
    // SM at head dimension 256) and eight warps (two per scheduler; each owns eight keys of a tile's scores and 1/8 of the
    // value columns), since the shared memory of a tile ring leaves room for one block per SM only.
    using SM = FlashRowsSmem<16, HD, HD, 64, 8, true, 3>;
    auto kern = flash_rows_kernel<MODE_GQA_DEC, 16, HD, HD, 64, 8, true, 3>;
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL));
        attr_set[ctx->device & 15] = true;
    }
    kern<<<dim3(ns, nkv, B), 256, SM::TOTAL, ctx->stream>>>(p);
    CWK_LAUNCH_CHECK(ctx, "flash_rows_kernel<GQA_DEC>");
    return CWK_OK;
}

template <int HD>
static int gqa_prefill_launch(cwk_ctx *ctx, const FlashRowsParams &p, int nblocks, int nkv) {
    using SM = FlashRowsSmem<64, HD, HD, 64, 8, true>;
    auto kern = flash_rows_kernel<MODE_GQA_PRE, 64, HD, HD, 64, 8, true>;
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL));
        attr_set[ctx->device & 15] = true;
    }
    kern<<<dim3(nblocks, nkv, 1), 256, SM::TOTAL, ctx->stream>>>(p);
    CWK_LAUNCH_CHECK(ctx, "flash_rows_kernel<GQA_PRE>");
    return CWK_OK;
}

int cwk_gqa_prefill_tc(cwk_ctx *ctx, const void *Q, const void *K, const void *V, int64_t pos, int n, int nh, int nkv, int hd,
                       float scale, void *out, int *flags);

extern "C" {

// sel != NULL: the keys of sequence b are rows sel[b*sel_ld + 0 .. kv_len[b]) of its cache, in that order.
static int gqa_decode_impl(cwk_ctx *ctx, const void *q, const void *K, const void *V, int64_t seq_stride,
                           const int32_t *kv_len, int max_kv_len, const int32_t *sel, int64_t sel_ld, int B, int nh, int nkv, int hd,
                           float scale, void *out, int n_splits) {
    if (!ctx || !q || !K || !V || !kv_len || !out) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "gqa_decode: null argument");
    if (B <= 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || max_kv_len < 0)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "gqa_decode: bad dimensions");
    const int group = nh / nkv;
    if (group > 16 || (hd != 256 && hd != 128))
        return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "gqa_decode: head_dim %d / group %d not built (128 or 256, group <= 16)", hd, group);
    if (((uintptr_t)K | (uintptr_t)V | (uintptr_t)q) % 16 != 0 || (seq_stride % 8) != 0)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "gqa_decode: pointers must be 16-byte aligned");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const int max_tiles = std::max(1, (max_kv_len + 63) / 64);
    int ns = n_splits > 0 ? std::min(std::min(n_splits, max_tiles), CWK_MAX_SPLITS) : 1;
    if (n_splits <= 0) {
        double best = 1e30;
        for (int c = 1; c <= std::min(max_tiles, 256); c++) {
            double waves = std::ceil((double)B * nkv * c / ctx->sm_count);
            double cost = waves * (std::ceil((double)max_tiles / c) + 1.0) + 0.02 * c;
            if (cost < best - 1e-9) { best = cost; ns = c; }
        }
    }
    int s = cwk_reserve_scratch(ctx, (size_t)B * ns * nh * (hd + 2) * sizeof(float));
    if (s != CWK_OK) return s;
    FlashRowsParams p{};
    p.q = (const uint16_t *)q; p.k = (const uint16_t *)K; p.v = (const uint16_t *)V;
    p.seq_stride = seq_stride; p.ld = (int64_t)nkv * hd; p.kv_len = kv_len; p.sel = sel; p.sel_ld = sel_ld;
    p.nh = nh; p.nkv = nkv; p.group = group; p.scale_log2 = scale * 1.4426950408889634f;
    p.partial = ctx->scratch; p.nsplit = ns; p.direct = 0;
    {
        CwkKernelTimer timer(ctx);
        s = (hd == 256) ? gqa_decode_launch<256>(ctx, p, B, nkv, ns) : gqa_decode_launch<128>(ctx, p, B, nkv, ns);
    }
    if (s != CWK_OK) return s;
    lse_combine_launch(ctx->stream, ctx->scratch, ns, nh, hd, B, (uint16_t *)out);
    CWK_LAUNCH_CHECK(ctx, "lse_merge_kernel");
    return CWK_OK;
}

int cwk_gqa_decode(cwk_ctx *ctx, const void *q, const void *K, const void *V, int64_t seq_stride,
                   const int32_t *kv_len, int max_kv_len, int B, int nh, int nkv, int hd, float scale,
                   void *out, int n_splits) {
    return gqa_decode_impl(ctx, q, K, V, seq_stride, kv_len, max_kv_len, nullptr, 0, B, nh, nkv, hd, scale, out, n_splits);
}

int cwk_gqa_decode_sel(cwk_ctx *ctx, const void *q, const void *K, const void *V, int64_t seq_stride,
                       const int32_t *nsel, int max_nsel, const int32_t *sel, int64_t sel_ld, int B, int nh, int nkv, int hd,
                       float scale, void *out, int n_splits) {
    if (!sel || sel_ld < max_nsel) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "gqa_decode_sel: bad selection list");
    return gqa_decode_impl(ctx, q, K, V, seq_stride, nsel, max_nsel, sel, sel_ld, B, nh, nkv, hd, scale, out, n_splits);
}

int cwk_gqa_prefill(cwk_ctx *ctx, const void *Q, const void *K, const void *V, int64_t pos, int n, int nh,
                    int nkv, int hd, float scale, void *out) {
    if (!ctx || !Q || !K || !V || !out) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "gqa_prefill: null argument");
    if (n <= 0 || pos < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "gqa_prefill: bad dimensions");
    const int group = nh / nkv;
    if (64 % group != 0 || (hd != 256 && hd != 128))
        return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "gqa_prefill: head_dim %d / group %d not built", hd, group);
    if (((uintptr_t)K | (uintptr_t)V | (uintptr_t)Q) % 16 != 0)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "gqa_prefill: pointers must be 16-byte aligned");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    // head dim 256 on the tcgen05/TMA prefill kernel (queries as MMA rows, K/V tiles by TMA from the caches); forcing a
    // general path on the context (cwk_ctx_force_mla_path 0 or 1) keeps the mma.sync kernel for A/B runs
    if (hd == 256 && ctx->force_mla_path != 0 && ctx->force_mla_path != 1) {
        const size_t flags_bytes = ((size_t)((n + 127) / 128) * nh + 3) * sizeof(int);
        int s = cwk_reserve_work(ctx, flags_bytes);
        if (s != CWK_OK) return s;
        s = cwk_gqa_prefill_tc(ctx, Q, K, V, pos, n, nh, nkv, hd, scale, out, (int *)ctx->work);
        if (s != CWK_ERR_UNSUPPORTED) return s;
    }
    const int QT = 64 / group;
    FlashRowsParams p{};
    p.q = (const uint16_t *)Q; p.k = (const uint16_t *)K; p.v = (const uint16_t *)V;
    p.seq_stride = 0; p.ld = (int64_t)nkv * hd; p.kv_len = nullptr; p.sel = nullptr;
    p.nh = nh; p.nkv = nkv; p.group = group; p.scale_log2 = scale * 1.4426950408889634f;
    p.partial = nullptr; p.out = (uint16_t *)out; p.nsplit = 1; p.direct = 1; p.pos = pos; p.nq = n;
    const int nblocks = (n + QT - 1) / QT;
    CwkKernelTimer timer(ctx);
    return (hd == 256) ? gqa_prefill_launch<256>(ctx, p, nblocks, nkv) : gqa_prefill_launch<128>(ctx, p, nblocks, nkv);
}

}  // extern "C"
