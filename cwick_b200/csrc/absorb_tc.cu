// absorb_tc.cu -- the absorb of q_nope through W_uk on the Blackwell tensor path.
//
//   Qfull[t][h][0:512]   = q[t][h][0:128] . W_uk[h]      (W_uk[h] is [128][512] row-major bf16)
// (the rope tail Qfull[t][h][512:576] is written by a kernel of its own)
//
// The identity is q_abs = W_k^T q of src/attention.c:741-744 (gemv_bf16_t), batched over the tokens
// of a prefill chunk: per head a [tokens][128] x [128][512] product. One block owns one head: W_uk[h]
// (128 KB) is brought into shared memory once by one TMA box and stays there as the MMA's B
// operand (N-contiguous, so "MN-major"), while 128-token tiles of q stream through a two-stage
// ring (one 32 KB box each). The 512 output columns are two accumulators of 256 columns in
// tensor memory: the epilogue of one half (TMEM -> bf16 -> global) runs under the MMAs of the
// other half and of the next tile.
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer and TMEM owner, 4-11 = epilogue
// (TMEM lane quarter = warp % 4; warps 4-7 take the low 128 columns of a half, 8-11 the high).
// Every mbarrier wait is bounded and records a code in the context's error word when it gives up.
#include <algorithm>

#include "tc_common.cuh"

namespace {

constexpr int AT_TOK = 128, AT_NOPE = 128, AT_L = 512, AT_ROPE = 64;
constexpr int AT_QD = AT_NOPE + AT_ROPE, AT_ROW = AT_L + AT_ROPE;
constexpr int AT_W_BYTES = AT_NOPE * AT_L * 2;      // 131072: eight [128 k][64 n] blocks
constexpr int AT_A_BYTES = AT_TOK * AT_NOPE * 2;    // 32768: two [128 tok][64 k] blocks
constexpr int AT_OFF_W = 0;
constexpr int AT_OFF_A = AT_W_BYTES;                // two stages
constexpr int AT_OFF_STG = AT_OFF_A + 2 * AT_A_BYTES;   // 8 epilogue warps x [32 rows][128 B] staging for full-line stores
constexpr int AT_OFF_BAR = AT_OFF_STG + 8 * 4096;
constexpr int AT_SMEM = AT_OFF_BAR + 256 + 1024;
constexpr int AT_THREADS = 384;
enum { AB_WFULL = 0, AB_AFULL = 1, AB_AEMPTY = 3, AB_DFULL = 5, AB_DEMPTY = 7, AB_COUNT = 9 };

struct AbsorbParams {
    const uint16_t *q;        // bf16 [n][nh][192]
    uint16_t *qfull;          // bf16 [n][nh][576]
    int n, nh;
    int *err;
};

__global__ void __launch_bounds__(AT_THREADS, 1)
absorb_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_w, const AbsorbParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const uint32_t bar0 = base + AT_OFF_BAR;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t *s_tmem = reinterpret_cast<uint32_t *>(sm + AT_OFF_BAR + 8 * AB_COUNT + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y;
    const int ntiles = (p.n + AT_TOK - 1) / AT_TOK;
    // tiles g, g + G, ... of this head
    const int nt = (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    if (nt <= 0) return;

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
        for (int i = 0; i < AB_COUNT; i++) mbar_init(bar(i), i >= AB_DEMPTY ? 256u : 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(bar(AB_WFULL), AT_W_BYTES);
            tma_load_3d(base + AT_OFF_W, &tm_w, 0, h * AT_NOPE, 0, bar(AB_WFULL));
            bool ok = true;
            int issued = 0;
            for (int i = 0; i < nt && ok; i++) {
                const int slot = i & 1, use = i >> 1;
                ok = mbar_wait(bar(AB_AEMPTY + slot), (uint32_t)((use & 1) ^ 1), p.err, 901);
                if (!ok) break;
                mbar_expect_tx(bar(AB_AFULL + slot), AT_A_BYTES);
                tma_load_3d(base + AT_OFF_A + slot * AT_A_BYTES, &tm_q, 0, ((int)blockIdx.x + i * (int)gridDim.x) * AT_TOK, h * 3,
                            bar(AB_AFULL + slot));
                issued = i + 1;
            }
            if (!ok) {     // drain the copies still in flight before leaving
                mbar_wait(bar(AB_WFULL), 0, p.err, 902);
                for (int i = (issued > 2 ? issued - 2 : 0); i < issued; i++) mbar_wait(bar(AB_AFULL + (i & 1)), (uint32_t)((i >> 1) & 1), p.err, 903);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t ID = idesc_bf16(128, 256, 0, 1);
            const uint64_t dW = smem_desc(base + AT_OFF_W, 16384, 1024);
            bool ok = mbar_wait(bar(AB_WFULL), 0, p.err, 904);
            for (int i = 0; i < nt && ok; i++) {
                const int slot = i & 1, use = i >> 1;
                ok = mbar_wait(bar(AB_AFULL + slot), (uint32_t)(use & 1), p.err, 905);
                if (!ok) break;
                const uint64_t dA = smem_desc(base + AT_OFF_A + slot * AT_A_BYTES, 16, 1024);
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    if (ok) ok = mbar_wait(bar(AB_DEMPTY + half), (uint32_t)((i & 1) ^ 1), p.err, 906);
                    if (ok) {
                        tc_fence_after();
#pragma unroll
                        for (int ks = 0; ks < 8; ks++)
                            umma_bf16(tmem + half * 256, dA + (uint64_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4),
                                      dW + (uint64_t)((half * 4 * 16384 + ks * 2048) >> 4), ID, ks != 0);
                        umma_commit(bar(AB_DFULL + half));
                    }
                }
                if (ok) umma_commit(bar(AB_AEMPTY + slot));
            }
        }
    } else if (warp < 4) {
        // idle
    } else {
        // ---------------- epilogue: TMEM -> bf16 -> Qfull
        const int q4 = warp & 3, g2 = (warp - 4) >> 2;
        const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
        bool ok = true;
        for (int i = 0; i < nt && ok; i++) {
            const int t = ((int)blockIdx.x + i * (int)gridDim.x) * AT_TOK + q4 * 32 + lane;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                if (ok) ok = mbar_wait(bar(AB_DFULL + half), (uint32_t)(i & 1), p.err, 907);
                if (!ok) break;
                tc_fence_after();
                // A thread holds one token row of the accumulator, and rows of Qfull lie 73 KB apart: storing from
                // the registers would touch 32 lines per instruction, 16 bytes each. The 64 columns of a pass go
                // through a per-warp staging tile instead, and leave as whole 128-byte lines, four rows per instruction.
                uint8_t *stg = sm + AT_OFF_STG + (warp - 4) * 4096;
                const int t0w = t - lane;                   // first token row of this warp
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t v[64];
                    const uint32_t col = (uint32_t)(half * 256 + g2 * 128 + c * 64);
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
                    for (int i = 0; i < 8; i++) {
                        const int rr = i * 4 + (lane >> 3), jj = lane & 7;
                        const uint4 w = *reinterpret_cast<const uint4 *>(stg + rr * 128 + ((jj ^ (rr & 7)) << 4));
                        if (t0w + rr < p.n)
                            *reinterpret_cast<uint4 *>(p.qfull + ((int64_t)(t0w + rr) * p.nh + h) * AT_ROW + col + jj * 8) = w;
                    }
                    __syncwarp();
                }
                tc_fence_before();
                mbar_arrive(bar(AB_DEMPTY + half));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

}  // namespace

// Returns CWK_ERR_UNSUPPORTED (without touching the context's error text) when the tensor path
// cannot run, so that the caller may take the mma.sync kernel instead.
int cwk_absorb_tc_launch(cwk_ctx *ctx, const void *Q, int n, int nh, const void *Wuk, void *Qfull) {
    CwkEncodeTiledFn enc = cwk_encode_tiled_fn();
    if (!enc) return CWK_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(Wuk) | reinterpret_cast<uintptr_t>(Qfull)) & 15) return CWK_ERR_UNSUPPORTED;
    int s = cwk_ensure_err_word(ctx);
    if (s != CWK_OK) return s;
    CUtensorMap tm_q, tm_w;
    {
        // q as [64][n tokens][nh * 3 column blocks]: head h's nope dims are blocks 3h and 3h + 1
        cuuint64_t dims[3] = {64, (cuuint64_t)n, (cuuint64_t)nh * 3};
        cuuint64_t strides[2] = {(cuuint64_t)nh * AT_QD * 2, 128};
        cuuint32_t box[3] = {64, AT_TOK, 2};
        cuuint32_t es[3] = {1, 1, 1};
        if (enc(&tm_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(Q), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled(q_nope) failed");
    }
    {
        // W_uk as [64][nh * 128 rows][8 column blocks]: one box brings a head's whole [128][512]
        cuuint64_t dims[3] = {64, (cuuint64_t)nh * AT_NOPE, AT_L / 64};
        cuuint64_t strides[2] = {(cuuint64_t)AT_L * 2, 128};
        cuuint32_t box[3] = {64, AT_NOPE, AT_L / 64};
        cuuint32_t es[3] = {1, 1, 1};
        if (enc(&tm_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(Wuk), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled(W_uk) failed");
    }
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(absorb_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM));
        attr_set[ctx->device & 15] = true;
    }
    AbsorbParams p;
    p.q = (const uint16_t *)Q; p.qfull = (uint16_t *)Qfull; p.n = n; p.nh = nh; p.err = ctx->dev_err;
    const int ntiles = (n + AT_TOK - 1) / AT_TOK;
    const int G = std::max(1, std::min(ntiles, ctx->sm_count / std::max(1, nh)));
    CwkKernelTimer timer(ctx);
    absorb_tc_kernel<<<dim3(G, nh), AT_THREADS, AT_SMEM, ctx->stream>>>(tm_q, tm_w, p);
    CWK_LAUNCH_CHECK(ctx, "absorb_tc_kernel");
    return CWK_OK;
}
