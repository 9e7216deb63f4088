// fp8_linear_tc.cu -- the FP8-E4M3 block-scaled projection on tcgen05.
//
//   Y[n][cols] = sum over 128-wide K blocks kb of  scale[col/128][kb] * ( X[:, kb] . W[:, kb]^T )
//
// The E4M3 codes are first widened to bf16 by a small kernel (exact: every E4M3
// value is a bf16 value), so the contraction is a bf16 x bf16 MMA with exact
// products and f32 accumulation. The F32 block scale changes every 128 along K
// and is not representable in the operands without rounding, so each K block is
// accumulated on its own in tensor memory and then multiplied by its scale and
// added into f32 registers by the epilogue warps ("block sum times scale", the
// order of src/tensor.c:511-520). Two TMEM accumulators alternate so the MMA of
// block kb+1 runs while block kb is being promoted.
//
// Block tile 128 (rows of X) x 128 (cols = one scale column block), K step 64
// (one 128-byte swizzle atom of bf16). Warp 0 = TMA producer, warp 1 = MMA
// issuer + TMEM owner, warps 4..7 = promotion / epilogue.
#include "tc_common.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;      // 16 KB each
constexpr int G_OFF_BAR = STAGES * (A_BYTES + B_BYTES);          // 196608
constexpr int G_SMEM = G_OFF_BAR + 256 + 1024;
constexpr uint32_t G_TMEM_COLS = 256;                             // two 128-column partial accumulators
enum { GB_FULL = 0, GB_EMPTY = STAGES, GB_PFULL = 2 * STAGES, GB_PEMPTY = 2 * STAGES + 2, GB_COUNT = 2 * STAGES + 4 };

// E4M3 -> bf16, exact. 16 codes per thread.
__global__ void __launch_bounds__(256) e4m3_to_bf16_kernel(const uint8_t *src, uint16_t *dst, int64_t n16) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n16) return;
    const uint4 v = reinterpret_cast<const uint4 *>(src)[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int k = 0; k < 4; k++)
#pragma unroll
        for (int hlf = 0; hlf < 2; hlf++) {
            uint32_t r = 0;
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const uint32_t b = (w[k] >> (16 * hlf + 8 * j)) & 0xffu;
                const uint32_t e = (b >> 3) & 15u, m = b & 7u;
                uint32_t h;
                if (e == 0) {
                    if (m == 0) h = 0;
                    else {
                        const int lz = (m >= 4) ? 0 : (m >= 2 ? 1 : 2);
                        h = ((uint32_t)(120 - lz) << 7) | (((m << (lz + 1)) & 7u) << 4);
                    }
                } else if (e == 15 && m == 7) h = 0x7fc0u;
                else h = ((e + 120u) << 7) | (m << 4);
                h |= (b & 0x80u) << 8;
                r |= h << (16 * j);
            }
            o[k * 2 + hlf] = r;
        }
    reinterpret_cast<uint4 *>(dst)[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    reinterpret_cast<uint4 *>(dst)[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
}

struct GemmParams {
    const float *scale_inv;
    int64_t n, k, cols;
    void *Y;
    int out_bf16;
    int *err;
};

__global__ void __launch_bounds__(256, 1)
fp8_linear_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                     const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const uint32_t bar0 = base + G_OFF_BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(sm + G_OFF_BAR + 8 * GB_COUNT + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col0 = blockIdx.x * BN, row0 = blockIdx.y * BM;
    const int nkb = (int)(p.k / 128);              // scale blocks along K
    const int nst = nkb * 2;                       // K steps of 64

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_x) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
        for (int i = 0; i < GB_COUNT; i++) mbar_init(bar(i), (i >= GB_PEMPTY) ? 128u : 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(G_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            int last_issued = -1;
            for (int s = 0; s < nst && ok; s++) {
                const int slot = s % STAGES, use = s / STAGES;
                ok = mbar_wait(bar(GB_EMPTY + slot), (uint32_t)((use & 1) ^ 1), p.err, 401);
                if (!ok) break;
                mbar_expect_tx(bar(GB_FULL + slot), A_BYTES + B_BYTES);
                tma_load_2d(base + slot * (A_BYTES + B_BYTES), &tm_x, s * BK, row0, bar(GB_FULL + slot));
                tma_load_2d(base + slot * (A_BYTES + B_BYTES) + A_BYTES, &tm_w, s * BK, col0, bar(GB_FULL + slot));
                last_issued = s;
            }
            if (!ok)      // drain the copies still in flight before leaving
                for (int s = last_issued; s >= 0 && s > last_issued - STAGES; s--)
                    mbar_wait(bar(GB_FULL + s % STAGES), (uint32_t)((s / STAGES) & 1), p.err, 402);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t ID = idesc_bf16(BM, BN, 0, 0);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; kb++) {
                const int pb = kb & 1, puse = kb >> 1;
                ok = mbar_wait(bar(GB_PEMPTY + pb), (uint32_t)((puse & 1) ^ 1), p.err, 403);
                if (!ok) break;
                tc_fence_after();
                for (int h2 = 0; h2 < 2 && ok; h2++) {
                    const int s = kb * 2 + h2, slot = s % STAGES, use = s / STAGES;
                    ok = mbar_wait(bar(GB_FULL + slot), (uint32_t)(use & 1), p.err, 404);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a0 = base + slot * (A_BYTES + B_BYTES), b0 = a0 + A_BYTES;
                    const uint64_t da = smem_desc(a0, 16, 1024), db = smem_desc(b0, 16, 1024);   // one build per stage, constant adds per MMA
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        umma_bf16(tmem + pb * 128, da + (uint64_t)((ks * 32) >> 4), db + (uint64_t)((ks * 32) >> 4), ID, (h2 | ks) != 0);
                    umma_commit(bar(GB_EMPTY + slot));        // stage may be refilled once these MMAs are done
                }
                if (ok) umma_commit(bar(GB_PFULL + pb));
            }
        }
    } else if (warp >= 4) {
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const uint32_t tlane = tmem + ((uint32_t)(q * 32) << 16);
        const int64_t ncb = (p.k + 127) / 128;
        const float *srow = p.scale_inv + (int64_t)(col0 / 128) * ncb;
        float acc[BN];
#pragma unroll
        for (int j = 0; j < BN; j++) acc[j] = 0.f;
        bool ok = true;
        for (int kb = 0; kb < nkb; kb++) {
            const int pb = kb & 1, puse = kb >> 1;
            ok = mbar_wait(bar(GB_PFULL + pb), (uint32_t)(puse & 1), p.err, 405);
            if (!ok) break;
            tc_fence_after();
            const float sc = __ldg(srow + kb);
#pragma unroll
            for (int c = 0; c < BN / 64; c++) {
                uint32_t v[64];                              // four loads in flight per wait
                TMEM_LD16(v, 0, tlane + pb * 128 + c * 64);
                TMEM_LD16(v, 16, tlane + pb * 128 + c * 64 + 16);
                TMEM_LD16(v, 32, tlane + pb * 128 + c * 64 + 32);
                TMEM_LD16(v, 48, tlane + pb * 128 + c * 64 + 48);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 64; j++) acc[c * 64 + j] = fmaf(__uint_as_float(v[j]), sc, acc[c * 64 + j]);
            }
            tc_fence_before();
            mbar_arrive(bar(GB_PEMPTY + pb));
        }
        if (ok && row0 + row < p.n) {
            const int64_t r = row0 + row;
            if (p.out_bf16) {
                uint16_t *y = (uint16_t *)p.Y + r * p.cols + col0;
#pragma unroll
                for (int j = 0; j < BN; j += 8) {
                    if (col0 + j + 8 <= p.cols) {
                        uint4 w;
                        w.x = pack_bf16x2(acc[j], acc[j + 1]); w.y = pack_bf16x2(acc[j + 2], acc[j + 3]);
                        w.z = pack_bf16x2(acc[j + 4], acc[j + 5]); w.w = pack_bf16x2(acc[j + 6], acc[j + 7]);
                        *reinterpret_cast<uint4 *>(y + j) = w;
                    } else {
                        for (int e = 0; e < 8; e++)
                            if (col0 + j + e < p.cols) y[j + e] = (uint16_t)(pack_bf16x2(acc[j + e], 0.f) & 0xffffu);
                    }
                }
            } else {
                float *y = (float *)p.Y + r * p.cols + col0;
#pragma unroll
                for (int j = 0; j < BN; j += 4) {
                    if (col0 + j + 4 <= p.cols) {
                        *reinterpret_cast<float4 *>(y + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                    } else {
                        for (int e = 0; e < 4; e++)
                            if (col0 + j + e < p.cols) y[j + e] = acc[j + e];
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(G_TMEM_COLS) : "memory");
    }
}

}  // namespace

bool cwk_fp8_linear_tc_available() { return true; }

int cwk_fp8_linear_tc_launch(cwk_ctx *ctx, const void *X, const void *W, const float *scale_inv, int64_t n, int64_t k,
                             int64_t cols, void *Y, int out_bf16) {
    // vector stores in the epilogue want 16-byte aligned rows
    if ((cols % 8) != 0 || (k % 128) != 0 || ((uintptr_t)Y % 16) != 0)
        return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "tcgen05 FP8 GEMM needs cols %% 8 == 0 and k %% 128 == 0");
    if (!cwk_encode_tiled_fn()) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled not available");
    {
        int es = cwk_ensure_err_word(ctx);
        if (es != CWK_OK) return es;
    }
    // widened weights live in their own buffer (the split scratch and the prefill workspace are in use around this call)
    const size_t wbytes = (size_t)cols * k * 2;
    if (wbytes > ctx->wbf16_bytes) {
        if (ctx->wbf16) {
            CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            CWK_CUDA(ctx, cudaFree(ctx->wbf16));
            ctx->wbf16 = nullptr;
            ctx->wbf16_bytes = 0;
        }
        CWK_CUDA(ctx, cudaMalloc(&ctx->wbf16, wbytes));
        ctx->wbf16_bytes = wbytes;
    }
    const int64_t n16 = cols * k / 16;
    e4m3_to_bf16_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, ctx->stream>>>((const uint8_t *)W, (uint16_t *)ctx->wbf16, n16);
    CWK_LAUNCH_CHECK(ctx, "e4m3_to_bf16_kernel");
    CUtensorMap tm_x, tm_w;
    if (!cwk_make_tmap_bf16_2d(&tm_x, X, (uint64_t)n, (uint64_t)k, (uint64_t)k, BM) ||
        !cwk_make_tmap_bf16_2d(&tm_w, ctx->wbf16, (uint64_t)cols, (uint64_t)k, (uint64_t)k, BN))
        return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled failed for the projection operands");
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(fp8_linear_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM));
        attr_set[ctx->device & 15] = true;
    }
    GemmParams p;
    p.scale_inv = scale_inv; p.n = n; p.k = k; p.cols = cols; p.Y = Y; p.out_bf16 = out_bf16; p.err = ctx->dev_err;
    dim3 grid((unsigned)((cols + BN - 1) / BN), (unsigned)((n + BM - 1) / BM));
    CwkKernelTimer timer(ctx);
    fp8_linear_tc_kernel<<<grid, 256, G_SMEM, ctx->stream>>>(tm_x, tm_w, p);
    CWK_LAUNCH_CHECK(ctx, "fp8_linear_tc_kernel");
    return CWK_OK;
}
