// dsa.cu -- DSA lightning indexer: exact-order scores over FP8 keys and exact
// top-k selection with the reference's ordering rule.
#include "cwk_common.cuh"
#include "topk_radix.cuh"

__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    float mag;
    if (e == 0) mag = (float)m * 0.001953125f;                        // m * 2^-9
    else if (e == 15 && m == 7) mag = __int_as_float(0x7fc00000);
    else mag = __uint_as_float(((e + 120u) << 23) | (m << 20));      // (1+m/8) * 2^(e-7)
    return (b & 0x80u) ? -mag : mag;
}

// One thread per key, the dequantised key row held in registers for all heads; q and the head
// weights sit in shared memory and are read as float4 broadcasts. The arithmetic is the
// reference's: per head four strided f32 accumulators with separate multiply and add (no fused
// multiply-add), combined (s0+s1)+(s2+s3); ReLU; times the head weight; heads summed in order.
template <int HD>
__global__ void __launch_bounds__(128) indexer_scores_fp8_kernel(
    const uint8_t *keys, const float *kscale, int64_t key_stride, const float *q, const float *wt,
    const int32_t *n, int ih, float *sc) {
    extern __shared__ __align__(16) float sm[];
    float *sq = sm;                      // [ih][HD]
    float *sw = sq + ih * HD;            // [ih]
    const int b = blockIdx.y, tid = threadIdx.x;
    const int nb = n[b];
    const int c0 = blockIdx.x * 128;
    if (c0 >= nb) return;
    for (int i = tid; i < ih * HD; i += 128) sq[i] = q[(int64_t)b * ih * HD + i];
    for (int i = tid; i < ih; i += 128) sw[i] = wt[(int64_t)b * ih + i];
    __syncthreads();
    const int c = c0 + tid;
    if (c >= nb) return;
    float kf[HD];
    {
        const uint4 *kr = reinterpret_cast<const uint4 *>(keys + ((int64_t)b * key_stride + c) * HD);
        const float s = kscale[(int64_t)b * key_stride + c];
#pragma unroll
        for (int ch = 0; ch < HD / 16; ch++) {
            const uint4 v = kr[ch];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; k++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    kf[ch * 16 + k * 4 + j] = __fmul_rn(e4m3_to_f32((w[k] >> (8 * j)) & 0xffu), s);
        }
    }
    float total = 0.f;
    for (int h = 0; h < ih; h++) {
        const float4 *qh = reinterpret_cast<const float4 *>(sq + h * HD);
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
        for (int i = 0; i < HD / 4; i++) {
            const float4 qv = qh[i];
            s0 = __fadd_rn(s0, __fmul_rn(kf[4 * i + 0], qv.x));
            s1 = __fadd_rn(s1, __fmul_rn(kf[4 * i + 1], qv.y));
            s2 = __fadd_rn(s2, __fmul_rn(kf[4 * i + 2], qv.z));
            s3 = __fadd_rn(s3, __fmul_rn(kf[4 * i + 3], qv.w));
        }
        float d = __fadd_rn(__fadd_rn(s0, s1), __fadd_rn(s2, s3));
        if (d < 0.f) d = 0.f;
        total = __fadd_rn(total, __fmul_rn(d, sw[h]));
    }
    sc[(int64_t)b * key_stride + c] = total;
}

// ---- exact top-k ---------------------------------------------------------------
// One cluster of TK_CL blocks of 1024 threads per sequence. Radix select (4 passes of 8 bits over
// an order-preserving integer image of the score) finds the want-th largest value exactly; an
// ordered compaction then writes the rows above it in index order followed by the rows equal to
// it in index order, `want` in all (ascending: one list in index order).
__global__ void __cluster_dims__(TK_CL, 1, 1) __launch_bounds__(TK_THREADS, 1)
topk_select_kernel(const float *sc, int64_t sc_stride, const int32_t *n, int want, int keep_self, int32_t *sel, int64_t sel_ld,
                   int32_t *nsel, int ascending, const int32_t *band_list, const int32_t *band_count) {
    cg::cluster_group cl = cg::this_cluster();
    const unsigned rank = cl.block_rank();
    const int b = blockIdx.y, tid = threadIdx.x;
    const int nb = n[b];
    const float *s = sc + (int64_t)b * sc_stride;
    int32_t *out = sel + (int64_t)b * sel_ld;
    const TkSlice sl = tk_slice(nb, rank);
    if (nb <= want) {                       // the whole prefix is the top-k
        for (int i = sl.begin + tid; i < sl.end; i += TK_THREADS) out[i] = i;
        if (rank == 0 && tid == 0) nsel[b] = nb;
        return;
    }
    __shared__ TkShared sh;
    uint32_t kc[TK_PT];
    if (sl.cached) tk_load(s, sl.begin, sl.end, kc);
    tk_threshold_and_compact(s, sl, kc, nb, want, keep_self, ascending, out, nsel + b,
                             band_list ? band_list + (int64_t)b * sc_stride : nullptr, band_list ? band_count[2 * b] : 0,
                             band_list ? band_count[2 * b + 1] : 0, sh);
}

extern "C" {

int cwk_indexer_scores_fp8(cwk_ctx *ctx, const void *keys, const float *kscale, int64_t key_stride,
                           const float *q, const float *wt, const int32_t *n, int max_n, int B, int ih,
                           int hd, float *sc) {
    if (!ctx || !keys || !kscale || !q || !wt || !n || !sc || B <= 0 || ih <= 0 || max_n < 0)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "indexer_scores: bad argument");
    if (hd != 128) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "indexer_scores: head dim %d not built (128)", hd);
    if (((uintptr_t)keys % 16) != 0) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "indexer_scores: keys must be 16-byte aligned");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (max_n == 0) return CWK_OK;
    const size_t smem = (size_t)(ih * 128 + ih) * sizeof(float);
    auto kern = indexer_scores_fp8_kernel<128>;
    if (smem > 48 * 1024) CWK_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CwkKernelTimer timer(ctx);
    kern<<<dim3((max_n + 127) / 128, B), 128, smem, ctx->stream>>>((const uint8_t *)keys, kscale, key_stride, q, wt, n, ih, sc);
    CWK_LAUNCH_CHECK(ctx, "indexer_scores_fp8_kernel");
    return CWK_OK;
}

int cwk_topk_select(cwk_ctx *ctx, const float *sc, int64_t sc_stride, const int32_t *n, int max_n, int B,
                    int want, int keep_self, int32_t *sel, int64_t sel_ld, int32_t *nsel) {
    if (!ctx || !sc || !n || !sel || !nsel || B <= 0 || want <= 0 || sel_ld < want + 1)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "topk_select: bad argument");
    (void)max_n;
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    CwkKernelTimer timer(ctx);
    topk_select_kernel<<<dim3(TK_CL, B), TK_THREADS, 0, ctx->stream>>>(sc, sc_stride, n, want, keep_self, sel, sel_ld, nsel, 0, nullptr, nullptr);
    CWK_LAUNCH_CHECK(ctx, "topk_select_kernel");
    return CWK_OK;
}

}  // extern "C"

extern "C" {

int cwk_ds_topk(cwk_ctx *ctx, const float *sc, int64_t sc_stride, const int32_t *n, int B, int k, int32_t *out, int64_t out_ld,
                int32_t *count) {
    if (!ctx || !sc || !n || !out || !count || B <= 0 || k <= 0 || out_ld < k)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_topk: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    CwkKernelTimer timer(ctx);
    topk_select_kernel<<<dim3(TK_CL, B), TK_THREADS, 0, ctx->stream>>>(sc, sc_stride, n, k, 0, out, out_ld, count, 1, nullptr, nullptr);
    CWK_LAUNCH_CHECK(ctx, "topk_select_kernel<ascending>");
    return CWK_OK;
}

}  // extern "C"
