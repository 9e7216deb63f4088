// unabsorb_tc.cu -- the un-absorb of the attention output through W_v on the Blackwell tensor path.
//
//   out[t][h][0:128] = attn[t][h][0:512] . W_v[h]^T      (W_v[h] is [128][512] row-major bf16)
//
// The identity is attn_out[h] = W_v c_acc[h] of src/attention.c:812-815 (gemv_bf16_n), batched over the
// tokens of a prefill chunk: per head a [tokens][512] x [512][128] product, the step between the absorbed
// attention and o_proj (src/attention.c:1020-1023). One block owns one head: W_v[h] (128 KB) is brought into
// shared memory once by one TMA box and stays there as the MMA's B operand (K-contiguous); 128-token tiles of
// the attention output stream through a two-stage ring, 128 of the 512 latent columns (32 KB, one box) at a
// time. Two 128-column accumulators in tensor memory: the epilogue of one tile (TMEM -> bf16 -> global through
// a per-warp staging tile, whole 128-byte lines) runs under the MMAs of the next. The kernel reads
// 1024 B and writes 256 B per (token, head) for 131 kFLOP (102 FLOP/B): a 32 KB ring fill feeds 8 MMAs of 64
// cycles, 64 B/clk per SM, more than twice an SM's share of HBM, so the kernel is HBM-bound.
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer and TMEM owner, 4-7 = epilogue (TMEM lane quarter = warp % 4).
// Every mbarrier wait is bounded and records a code in the context's error word when it gives up.
#include <algorithm>

#include "tc_common.cuh"

namespace {

constexpr int UT_TOK = 128, UT_V = 128, UT_L = 512;
constexpr int UT_W_BYTES = UT_V * UT_L * 2;         // 131072: eight [128 n][64 k] blocks
constexpr int UT_A_BYTES = UT_TOK * 128 * 2;        // 32768: two [128 tok][64 k] blocks = 128 latent columns
constexpr int UT_CHUNKS = UT_L / 128;               // 4 ring fills per tile
constexpr int UT_OFF_W = 0;
constexpr int UT_OFF_A = UT_W_BYTES;                // two stages
constexpr int UT_OFF_STG = UT_OFF_A + 2 * UT_A_BYTES;   // 4 epilogue warps x [32 rows][128 B]
constexpr int UT_OFF_BAR = UT_OFF_STG + 4 * 4096;
constexpr int UT_SMEM = UT_OFF_BAR + 256 + 1024;
constexpr int UT_THREADS = 256;
enum { UB_WFULL = 0, UB_AFULL = 1, UB_AEMPTY = 3, UB_DFULL = 5, UB_DEMPTY = 7, UB_COUNT = 9 };

struct UnabsorbParams {
    uint16_t *out;            // bf16 [n][nh][128]
    int n, nh, w_head_rows;
    int *err;
};

__global__ void __launch_bounds__(UT_THREADS, 1)
unabsorb_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w, const UnabsorbParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const uint32_t bar0 = base + UT_OFF_BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(sm + UT_OFF_BAR + 8 * UB_COUNT + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y;
    const int ntiles = (p.n + UT_TOK - 1) / UT_TOK;
    const int nt = (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;      // tiles g, g + G, ... of this head
    if (nt <= 0) return;

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
        for (int i = 0; i < UB_COUNT; i++) mbar_init(bar(i), i >= UB_DEMPTY ? 128u : 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // W_v[h] and the first two ring fills go out before the block-wide set-up
        mbar_expect_tx(bar(UB_WFULL), UT_W_BYTES);
        tma_load_3d(base + UT_OFF_W, &tm_w, 0, h * p.w_head_rows, 0, bar(UB_WFULL));
        for (int f = 0; f < 2; f++) {
            mbar_expect_tx(bar(UB_AFULL + f), UT_A_BYTES);
            tma_load_3d(base + UT_OFF_A + f * UT_A_BYTES, &tm_a, 0, (int)blockIdx.x * UT_TOK, h * 8 + f * 2, bar(UB_AFULL + f));
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;
    const int nfill = nt * UT_CHUNKS;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            int issued = nfill < 2 ? nfill : 2;            // fills 0 and 1 went out during set-up
            for (int f = 2; f < nfill && ok; f++) {
                const int slot = f & 1, use = f >> 1, i = f / UT_CHUNKS, c = f % UT_CHUNKS;
                ok = mbar_wait(bar(UB_AEMPTY + slot), (uint32_t)((use & 1) ^ 1), p.err, 911);
                if (!ok) break;
                mbar_expect_tx(bar(UB_AFULL + slot), UT_A_BYTES);
                tma_load_3d(base + UT_OFF_A + slot * UT_A_BYTES, &tm_a, 0, ((int)blockIdx.x + i * (int)gridDim.x) * UT_TOK, h * 8 + c * 2,
                            bar(UB_AFULL + slot));
                issued = f + 1;
            }
            if (!ok) {     // drain the copies still in flight before leaving
                mbar_wait(bar(UB_WFULL), 0, p.err, 912);
                for (int f = (issued > 2 ? issued - 2 : 0); f < issued; f++) mbar_wait(bar(UB_AFULL + (f & 1)), (uint32_t)((f >> 1) & 1), p.err, 913);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t ID = idesc_bf16(128, UT_V, 0, 0);
            const uint64_t dW = smem_desc(base + UT_OFF_W, 16, 1024);
            bool ok = mbar_wait(bar(UB_WFULL), 0, p.err, 914);
            for (int i = 0; i < nt && ok; i++) {
                const int db = i & 1;
                ok = mbar_wait(bar(UB_DEMPTY + db), (uint32_t)(((i >> 1) & 1) ^ 1), p.err, 916);
                for (int c = 0; c < UT_CHUNKS && ok; c++) {
                    const int f = i * UT_CHUNKS + c, slot = f & 1, use = f >> 1;
                    ok = mbar_wait(bar(UB_AFULL + slot), (uint32_t)(use & 1), p.err, 915);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t dA = smem_desc(base + UT_OFF_A + slot * UT_A_BYTES, 16, 1024);
#pragma unroll
                    for (int ks = 0; ks < 8; ks++)
                        umma_bf16(tmem + db * 128, dA + (uint64_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4),
                                  dW + (uint64_t)(((c * 2 + (ks >> 2)) * 16384 + (ks & 3) * 32) >> 4), ID, (c | ks) != 0);
                    umma_commit(bar(UB_AEMPTY + slot));
                }
                if (ok) umma_commit(bar(UB_DFULL + db));
            }
        }
    } else if (warp >= 4) {
        // ---------------- epilogue: TMEM -> bf16 -> out
        const int q4 = warp & 3;
        const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
        uint8_t *stg = sm + UT_OFF_STG + (warp - 4) * 4096;
        bool ok = true;
        for (int i = 0; i < nt && ok; i++) {
            const int db = i & 1;
            const int t0w = ((int)blockIdx.x + i * (int)gridDim.x) * UT_TOK + q4 * 32;       // first token row of this warp
            ok = mbar_wait(bar(UB_DFULL + db), (uint32_t)((i >> 1) & 1), p.err, 917);
            ok = __all_sync(0xffffffffu, ok);            // the TMEM loads below are warp-wide
            if (!ok) break;
            tc_fence_after();
            // A thread holds one token row of the accumulator, and rows of `out` lie nh * 256 bytes apart: the 64
            // columns of a pass go through the warp's staging tile and leave as whole 128-byte lines.
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t v[64];
                const uint32_t col = (uint32_t)(db * 128 + c * 64);
                TMEM_LD16(v, 0, tlane + col);
                TMEM_LD16(v, 16, tlane + col + 16);
                TMEM_LD16(v, 32, tlane + col + 32);
                TMEM_LD16(v, 48, tlane + col + 48);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    uint4 w;
                    w.x = pack_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
                    w.y = pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
                    w.z = pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
                    w.w = pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
                    *reinterpret_cast<uint4 *>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) = w;
                }
                __syncwarp();
#pragma unroll
                for (int r = 0; r < 8; r++) {
                    const int rr = r * 4 + (lane >> 3), jj = lane & 7;
                    const uint4 w = *reinterpret_cast<const uint4 *>(stg + rr * 128 + ((jj ^ (rr & 7)) << 4));
                    if (t0w + rr < p.n)
                        *reinterpret_cast<uint4 *>(p.out + ((int64_t)(t0w + rr) * p.nh + h) * UT_V + c * 64 + jj * 8) = w;
                }
                __syncwarp();
            }
            tc_fence_before();
            mbar_arrive(bar(UB_DEMPTY + db));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
    }
}

}  // namespace

extern "C" int cwk_mla_unabsorb(cwk_ctx *ctx, const void *attn, const void *Wv, int64_t w_head_rows, int n, int nh, void *out) {
    if (!ctx || !attn || !Wv || !out || n <= 0 || nh <= 0 || w_head_rows < UT_V)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mla_unabsorb: bad argument");
    CwkEncodeTiledFn enc = cwk_encode_tiled_fn();
    if (!enc) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "mla_unabsorb: cuTensorMapEncodeTiled is not available");
    if ((reinterpret_cast<uintptr_t>(attn) | reinterpret_cast<uintptr_t>(Wv) | reinterpret_cast<uintptr_t>(out)) & 15)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mla_unabsorb: buffers must be 16-byte aligned");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    int s = cwk_ensure_err_word(ctx);
    if (s != CWK_OK) return s;
    CUtensorMap tm_a, tm_w;
    {
        // the attention output as [64][n tokens][nh * 8 column blocks]: head h's latent columns are blocks 8h .. 8h + 7
        cuuint64_t dims[3] = {64, (cuuint64_t)n, (cuuint64_t)nh * 8};
        cuuint64_t strides[2] = {(cuuint64_t)nh * UT_L * 2, 128};
        cuuint32_t box[3] = {64, UT_TOK, 2};
        cuuint32_t es[3] = {1, 1, 1};
        if (enc(&tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(attn), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled(attention output) failed");
    }
    {
        // W_v as [64][rows][8 column blocks]: one box brings a head's whole [128][512]
        cuuint64_t dims[3] = {64, (cuuint64_t)(nh - 1) * (cuuint64_t)w_head_rows + UT_V, UT_L / 64};
        cuuint64_t strides[2] = {(cuuint64_t)UT_L * 2, 128};
        cuuint32_t box[3] = {64, UT_V, UT_L / 64};
        cuuint32_t es[3] = {1, 1, 1};
        if (enc(&tm_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(Wv), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled(W_v) failed");
    }
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(unabsorb_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, UT_SMEM));
        attr_set[ctx->device & 15] = true;
    }
    UnabsorbParams p;
    p.out = (uint16_t *)out; p.n = n; p.nh = nh; p.w_head_rows = (int)w_head_rows; p.err = ctx->dev_err;
    const int ntiles = (n + UT_TOK - 1) / UT_TOK;
    const int G = std::max(1, std::min(ntiles, ctx->sm_count / std::max(1, nh)));
    CwkKernelTimer timer(ctx);
    unabsorb_tc_kernel<<<dim3(G, nh), UT_THREADS, UT_SMEM, ctx->stream>>>(tm_a, tm_w, p);
    CWK_LAUNCH_CHECK(ctx, "unabsorb_tc_kernel");
    return CWK_OK;
}
