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
// Block tile 128 (rows of X) x 256 (two scale column blocks), K step 128 = one scale block per
// pipeline stage, two stages. An operand tile arrives as ONE TMA box of two 64-wide column blocks
// (a TMA operation costs some 400 cycles whatever its size, and a 128 x 128 tile with 64-wide steps
// is bound by that, not by the MMAs). The MMA is M 128 x N 256: at N = 256 the operand reads leave
// shared-memory bandwidth for the incoming tiles. Warp 0 = TMA producer, warp 1 = MMA issuer + TMEM
// owner, warps 4..11 = promotion / epilogue (TMEM lane quarter = warp % 4; warps 4-7 own output
// columns 0-127 of the tile, warps 8-11 columns 128-255).
#include <map>
#include <tuple>

#include "tc_common.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 128;
constexpr int STAGES = 2;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;      // 32 KB + 64 KB
constexpr int G_OFF_BAR = STAGES * (A_BYTES + B_BYTES);          // 196608
constexpr int G_SMEM = G_OFF_BAR + 256 + 1024;
constexpr uint32_t G_TMEM_COLS = 512;                             // two 256-column partial accumulators
constexpr int G_THREADS = 384;
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

// One launch serves one projection, or two that share the activations X (q_a and kv_a of the MLA
// prefill: alone they fill 1.3 and 0.65 waves of the SMs): column tiles [0, tiles_a) belong to the
// first weight matrix, the rest to the second.
struct GemmProblem {
    const float *scale_inv;
    int64_t cols;
    void *Y;
    int out_bf16;
};
struct GemmParams {
    GemmProblem pr[2];
    int tiles_a;               // column tiles of the first problem
    int64_t n, k;
    int *err;
};

__global__ void __launch_bounds__(G_THREADS, 1)
fp8_linear_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                     const __grid_constant__ CUtensorMap tm_w2, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const uint32_t bar0 = base + G_OFF_BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(sm + G_OFF_BAR + 8 * GB_COUNT + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int second = (int)blockIdx.x >= p.tiles_a;
    GemmProblem pp;            // field-wise select: indexing the parameter struct with a run-time index would copy it to local memory
    pp.scale_inv = second ? p.pr[1].scale_inv : p.pr[0].scale_inv;
    pp.cols = second ? p.pr[1].cols : p.pr[0].cols;
    pp.Y = second ? p.pr[1].Y : p.pr[0].Y;
    pp.out_bf16 = second ? p.pr[1].out_bf16 : p.pr[0].out_bf16;
    const int col0 = ((int)blockIdx.x - (second ? p.tiles_a : 0)) * BN, row0 = blockIdx.y * BM;
    const int nkb = (int)(p.k / 128);              // scale blocks along K = pipeline steps

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_x) : "memory");
        if (second) asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w2) : "memory");
        else asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
        for (int i = 0; i < GB_COUNT; i++) mbar_init(bar(i), (i >= GB_PEMPTY) ? 256u : 1u);
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
            int issued = 0;
            for (int s = 0; s < nkb && ok; s++) {
                const int slot = s % STAGES, use = s / STAGES;
                ok = mbar_wait(bar(GB_EMPTY + slot), (uint32_t)((use & 1) ^ 1), p.err, 401);
                if (!ok) break;
                mbar_expect_tx(bar(GB_FULL + slot), A_BYTES + B_BYTES);
                tma_load_3d(base + slot * (A_BYTES + B_BYTES), &tm_x, 0, row0, s * 2, bar(GB_FULL + slot));
                // (the maps are kernel parameters: their addresses must stay in parameter space, so no pointer select)
                if (second) tma_load_3d(base + slot * (A_BYTES + B_BYTES) + A_BYTES, &tm_w2, 0, col0, s * 2, bar(GB_FULL + slot));
                else tma_load_3d(base + slot * (A_BYTES + B_BYTES) + A_BYTES, &tm_w, 0, col0, s * 2, bar(GB_FULL + slot));
                issued = s + 1;
            }
            if (!ok)      // drain the copies still in flight before leaving
                for (int s = (issued > STAGES ? issued - STAGES : 0); s < issued; s++)
                    mbar_wait(bar(GB_FULL + s % STAGES), (uint32_t)((s / STAGES) & 1), p.err, 402);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t ID = idesc_bf16(BM, BN, 0, 0);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; kb++) {
                const int pb = kb & 1, puse = kb >> 1, slot = kb % STAGES, use = kb / STAGES;
                ok = mbar_wait(bar(GB_PEMPTY + pb), (uint32_t)((puse & 1) ^ 1), p.err, 403);
                if (ok) ok = mbar_wait(bar(GB_FULL + slot), (uint32_t)(use & 1), p.err, 404);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a0 = base + slot * (A_BYTES + B_BYTES), b0 = a0 + A_BYTES;
                const uint64_t da = smem_desc(a0, 16, 1024), db = smem_desc(b0, 16, 1024);   // one build per stage, constant adds per MMA
#pragma unroll
                for (int ks = 0; ks < 8; ks++)          // 64-wide column block ks >> 2 of each operand, 32 bytes per 16-wide step
                    umma_bf16(tmem + pb * 256, da + (uint64_t)(((ks >> 2) * (BM * 128) + (ks & 3) * 32) >> 4),
                              db + (uint64_t)(((ks >> 2) * (BN * 128) + (ks & 3) * 32) >> 4), ID, ks != 0);
                umma_commit(bar(GB_EMPTY + slot));        // stage may be refilled once these MMAs are done
                umma_commit(bar(GB_PFULL + pb));
            }
        }
    } else if (warp >= 4) {
        const int q = warp & 3, ch = (warp - 4) >> 2;
        const int row = q * 32 + lane;
        const int cbase = col0 + ch * 128;             // first output column of this warp's 128
        const bool live = cbase < pp.cols;              // a tile past the last column block: only keep the barriers moving
        const uint32_t tlane = tmem + ((uint32_t)(q * 32) << 16);
        const int64_t ncb = (p.k + 127) / 128;
        const float *srow = pp.scale_inv + (int64_t)(live ? cbase / 128 : 0) * ncb;
        float acc[128];
#pragma unroll
        for (int j = 0; j < 128; j++) acc[j] = 0.f;
        bool ok = true;
        for (int kb = 0; kb < nkb; kb++) {
            const int pb = kb & 1, puse = kb >> 1;
            ok = mbar_wait(bar(GB_PFULL + pb), (uint32_t)(puse & 1), p.err, 405);
            if (!ok) break;
            tc_fence_after();
            if (live) {
                const float sc = __ldg(srow + kb);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    uint32_t v[32];                              // two loads in flight per wait
                    TMEM_LD16(v, 0, tlane + pb * 256 + ch * 128 + c * 32);
                    TMEM_LD16(v, 16, tlane + pb * 256 + ch * 128 + c * 32 + 16);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; j++) acc[c * 32 + j] = fmaf(__uint_as_float(v[j]), sc, acc[c * 32 + j]);
                }
            }
            tc_fence_before();
            mbar_arrive(bar(GB_PEMPTY + pb));
        }
        if (ok && live && row0 + row < p.n) {
            const int64_t r = row0 + row;
            if (pp.out_bf16) {
                uint16_t *y = (uint16_t *)pp.Y + r * pp.cols + cbase;
#pragma unroll
                for (int j = 0; j < 128; j += 8) {
                    if (cbase + j + 8 <= pp.cols) {
                        uint4 w;
                        w.x = pack_bf16x2(acc[j], acc[j + 1]); w.y = pack_bf16x2(acc[j + 2], acc[j + 3]);
                        w.z = pack_bf16x2(acc[j + 4], acc[j + 5]); w.w = pack_bf16x2(acc[j + 6], acc[j + 7]);
                        *reinterpret_cast<uint4 *>(y + j) = w;
                    } else {
                        for (int e = 0; e < 8; e++)
                            if (cbase + j + e < pp.cols) y[j + e] = (uint16_t)(pack_bf16x2(acc[j + e], 0.f) & 0xffffu);
                    }
                }
            } else {
                float *y = (float *)pp.Y + r * pp.cols + cbase;
#pragma unroll
                for (int j = 0; j < 128; j += 4) {
                    if (cbase + j + 4 <= pp.cols) {
                        *reinterpret_cast<float4 *>(y + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                    } else {
                        for (int e = 0; e < 4; e++)
                            if (cbase + j + e < pp.cols) y[j + e] = acc[j + e];
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

// Widened copies of weight tensors, kept per context. A serving loop applies the same few projections to every
// chunk, and checkpoints are immutable (the reference maps them read-only), so the exact E4M3 -> bf16 widening of a
// weight is done once per (pointer, shape) and reused, up to a byte budget; beyond it, or after
// cwk_ctx_drop_weight_cache, a call widens into the context's transient buffer as before.
struct WideEntry {
    void *dev;
    CUtensorMap tm;
};
struct WideCache {
    std::map<std::tuple<const void *, int64_t, int64_t>, WideEntry> m;
    size_t bytes = 0;
};

void cwk_fp8_weight_cache_free(cwk_ctx *ctx) {
    WideCache *wc = (WideCache *)ctx->wide_cache;
    if (!wc) return;
    for (auto &kv : wc->m) cudaFree(kv.second.dev);
    delete wc;
    ctx->wide_cache = nullptr;
}

static int encode_weight_map(cwk_ctx *ctx, const void *dst, int64_t cols, int64_t k, CUtensorMap *tm);

// Widens W (E4M3 [cols][k]) to bf16 and encodes its tensor map: from the context's cache when the weight has been
// seen, into the cache when it has room, else into the context's transient buffer at element offset `at`.
static int prepare_weights(cwk_ctx *ctx, const void *W, int64_t cols, int64_t k, size_t at, CUtensorMap *tm) {
    const int64_t n16 = cols * k / 16;
    const size_t bytes = (size_t)cols * k * 2;
    if (!ctx->wide_cache) ctx->wide_cache = new WideCache();
    WideCache *wc = (WideCache *)ctx->wide_cache;
    const auto key = std::make_tuple(W, cols, k);
    auto it = wc->m.find(key);
    if (it != wc->m.end()) { *tm = it->second.tm; return CWK_OK; }
    uint16_t *dst = (uint16_t *)ctx->wbf16 + at;
    bool cached = false;
    if (wc->bytes + bytes <= ctx->wide_cache_budget) {
        void *d = nullptr;
        if (cudaMalloc(&d, bytes) == cudaSuccess) { dst = (uint16_t *)d; cached = true; }
        else (void)cudaGetLastError();
    }
    e4m3_to_bf16_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, ctx->stream>>>((const uint8_t *)W, dst, n16);
    CWK_LAUNCH_CHECK(ctx, "e4m3_to_bf16_kernel");
    int s = encode_weight_map(ctx, dst, cols, k, tm);
    if (s != CWK_OK) { if (cached) cudaFree(dst); return s; }
    if (cached) {
        wc->m[key] = WideEntry{dst, *tm};
        wc->bytes += bytes;
    }
    return CWK_OK;
}

static int encode_weight_map(cwk_ctx *ctx, const void *dst_c, int64_t cols, int64_t k, CUtensorMap *tm) {
    void *dst = const_cast<void *>(dst_c);
    CwkEncodeTiledFn enc = cwk_encode_tiled_fn();
    cuuint32_t es[3] = {1, 1, 1};
    cuuint64_t wd[3] = {64, (cuuint64_t)cols, (cuuint64_t)(k / 64)};
    cuuint64_t st[2] = {(cuuint64_t)k * 2, 128};
    cuuint32_t wb[3] = {64, BN, 2};
    if (enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dst, wd, st, wb, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled failed for the projection weights");
    return CWK_OK;
}

// Y1 = X . W1^T (block-scaled), and, when W2 is given, Y2 = X . W2^T in the same launch.
int cwk_fp8_linear_tc_launch2(cwk_ctx *ctx, const void *X, int64_t n, int64_t k, const void *W1, const float *scale1, int64_t cols1,
                              void *Y1, int out_bf16_1, const void *W2, const float *scale2, int64_t cols2, void *Y2, int out_bf16_2) {
    // vector stores in the epilogue want 16-byte aligned rows
    if ((cols1 % 8) != 0 || (k % 128) != 0 || ((uintptr_t)Y1 % 16) != 0 || ((uintptr_t)X % 16) != 0 ||
        (W2 && ((cols2 % 8) != 0 || ((uintptr_t)Y2 % 16) != 0)))
        return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "tcgen05 FP8 GEMM needs cols %% 8 == 0 and k %% 128 == 0");
    if (!cwk_encode_tiled_fn()) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled not available");
    {
        int es = cwk_ensure_err_word(ctx);
        if (es != CWK_OK) return es;
    }
    // widened weights live in their own buffer (the split scratch and the prefill workspace are in use around this call)
    const size_t e1 = (size_t)cols1 * k, e2 = W2 ? (size_t)cols2 * k : 0;
    const size_t wbytes = (e1 + e2) * 2;
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
    CUtensorMap tm_x, tm_w, tm_w2;
    int s = prepare_weights(ctx, W1, cols1, k, 0, &tm_w);
    if (s != CWK_OK) return s;
    tm_w2 = tm_w;
    if (W2) {
        s = prepare_weights(ctx, W2, cols2, k, e1, &tm_w2);
        if (s != CWK_OK) return s;
    }
    {
        // activations as [64][rows][k / 64 column blocks]: one box = all rows of a tile x two column blocks (one 128-wide scale block)
        CwkEncodeTiledFn enc = cwk_encode_tiled_fn();
        cuuint32_t es[3] = {1, 1, 1};
        cuuint64_t xd[3] = {64, (cuuint64_t)n, (cuuint64_t)(k / 64)};
        cuuint64_t st[2] = {(cuuint64_t)k * 2, 128};
        cuuint32_t xb[3] = {64, BM, 2};
        if (enc(&tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(X), xd, st, xb, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled failed for the projection activations");
    }
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(fp8_linear_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM));
        attr_set[ctx->device & 15] = true;
    }
    GemmParams p;
    p.pr[0].scale_inv = scale1; p.pr[0].cols = cols1; p.pr[0].Y = Y1; p.pr[0].out_bf16 = out_bf16_1;
    p.pr[1] = p.pr[0];
    if (W2) { p.pr[1].scale_inv = scale2; p.pr[1].cols = cols2; p.pr[1].Y = Y2; p.pr[1].out_bf16 = out_bf16_2; }
    p.tiles_a = (int)((cols1 + BN - 1) / BN);
    p.n = n; p.k = k; p.err = ctx->dev_err;
    const int tiles_b = W2 ? (int)((cols2 + BN - 1) / BN) : 0;
    dim3 grid((unsigned)(p.tiles_a + tiles_b), (unsigned)((n + BM - 1) / BM));
    CwkKernelTimer timer(ctx);
    fp8_linear_tc_kernel<<<grid, G_THREADS, G_SMEM, ctx->stream>>>(tm_x, tm_w, tm_w2, p);
    CWK_LAUNCH_CHECK(ctx, "fp8_linear_tc_kernel");
    return CWK_OK;
}

int cwk_fp8_linear_tc_launch(cwk_ctx *ctx, const void *X, const void *W, const float *scale_inv, int64_t n, int64_t k,
                             int64_t cols, void *Y, int out_bf16) {
    return cwk_fp8_linear_tc_launch2(ctx, X, n, k, W, scale_inv, cols, Y, out_bf16, nullptr, nullptr, 0, nullptr, 0);
}
