// fp8_linear.cu -- Y = X . W^T with W in E4M3 and one F32 multiplier per
// 128x128 block. General kernel on mma.sync: the E4M3 codes are widened to bf16
// (exact) on their way into shared memory, each 128-wide K block is
// accumulated on its own in f32 and then scaled into the running sum, which is
// the reference's "block sum times scale" order (src/tensor.c:511-520).
#include "cwk_common.cuh"

int cwk_fp8_linear_tc_launch(cwk_ctx *ctx, const void *X, const void *W, const float *scale_inv, int64_t n,
                             int64_t k, int64_t cols, void *Y, int out_bf16);
bool cwk_fp8_linear_tc_available();

__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2(uint32_t two) {
    // two E4M3 codes in the low 16 bits -> two bf16 (exact: 3-bit mantissa, bias 7 -> bias 127)
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const uint32_t b = (two >> (8 * i)) & 0xffu;
        const uint32_t e = (b >> 3) & 15u, m = b & 7u;
        uint32_t h;
        if (e == 0) {
            // subnormal m * 2^-9: normalise by hand
            if (m == 0) h = 0;
            else {
                const int lz = (m >= 4) ? 0 : (m >= 2 ? 1 : 2);          // shifts to reach bit 2
                const uint32_t mm = (m << (lz + 1)) & 7u;               // drop the leading one
                h = ((uint32_t)(127 - 7 - lz) << 7) | (mm << 4);
            }
        } else if (e == 15 && m == 7) {
            h = 0x7fc0u;
        } else {
            h = ((e + 120u) << 7) | (m << 4);
        }
        h |= (b & 0x80u) << 8;
        r |= h << (16 * i);
    }
    return r;
}

template <bool OUT_BF16>
__global__ void __launch_bounds__(256) fp8_linear_kernel(const uint16_t *X, const uint8_t *W,
                                                         const float *scale_inv, int64_t n, int64_t k,
                                                         int64_t cols, void *Y) {
    constexpr int BM = 128, BN = 128, BK = 64;
    __shared__ __align__(128) uint8_t sX[BM * BK * 2];
    __shared__ __align__(128) uint8_t sW[BN * BK * 2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp & 1, wn = warp >> 1;        // 2 x 4 warps, warp tile 64 x 32
    const int64_t row0 = (int64_t)blockIdx.y * BM, col0 = (int64_t)blockIdx.x * BN;
    const int64_t ncb = (k + 127) / 128;
    const float *srow = scale_inv + (col0 / 128) * ncb;

    float acc[4][4][4], part[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[i][j][e] = part[i][j][e] = 0.f;

    for (int64_t k0 = 0; k0 < k; k0 += BK) {
        __syncthreads();
        // X tile: 128 rows x 8 chunks of 16 bytes
        for (int i = tid; i < BM * 8; i += 256) {
            const int r = i >> 3, c = i & 7;
            const bool ok = row0 + r < n;
            cp_async16(smem_u32(sX + r * 128 + ((c ^ (r & 7)) << 4)),
                       ok ? (const void *)(X + (row0 + r) * k + k0 + c * 8) : (const void *)X, ok);
        }
        cp_async_commit();
        // W tile: 128 rows x 64 codes = 4 loads of 16 bytes per row, widened to 2 chunks each
        for (int i = tid; i < BN * 4; i += 256) {
            const int r = i >> 2, q4 = i & 3;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (col0 + r < cols) v = *reinterpret_cast<const uint4 *>(W + (col0 + r) * k + k0 + q4 * 16);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int hfl = 0; hfl < 2; hfl++) {
                uint4 o;
                o.x = e4m3x2_to_bf16x2(w[hfl * 2] & 0xffffu);
                o.y = e4m3x2_to_bf16x2(w[hfl * 2] >> 16);
                o.z = e4m3x2_to_bf16x2(w[hfl * 2 + 1] & 0xffffu);
                o.w = e4m3x2_to_bf16x2(w[hfl * 2 + 1] >> 16);
                const int c = q4 * 2 + hfl;
                *reinterpret_cast<uint4 *>(sW + r * 128 + ((c ^ (r & 7)) << 4)) = o;
            }
        }
        cp_async_wait<0>();
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < BK / 16; ks++) {
            uint32_t a[4][4];
#pragma unroll
            for (int mi = 0; mi < 4; mi++) {
                const int r = wm * 64 + mi * 16 + (lane & 15);
                ldmatrix_x4(a[mi][0], a[mi][1], a[mi][2], a[mi][3],
                            smem_u32(sX + r * 128) + (((ks * 2 + (lane >> 4)) ^ (r & 7)) << 4));
            }
#pragma unroll
            for (int np = 0; np < 2; np++) {
                const int r = wn * 32 + np * 16 + (lane & 7) + ((lane >> 4) << 3);
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3, smem_u32(sW + r * 128) + (((ks * 2 + ((lane >> 3) & 1)) ^ (r & 7)) << 4));
#pragma unroll
                for (int mi = 0; mi < 4; mi++) {
                    mma_bf16_16816(part[mi][np * 2], a[mi], b0, b1);
                    mma_bf16_16816(part[mi][np * 2 + 1], a[mi], b2, b3);
                }
            }
        }
        if (((k0 + BK) & 127) == 0 || k0 + BK >= k) {      // a 128-wide scale block just closed
            const float sc = srow[k0 / 128];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++)
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        acc[i][j][e] += part[i][j][e] * sc;
                        part[i][j][e] = 0.f;
                    }
        }
    }
#pragma unroll
    for (int mi = 0; mi < 4; mi++)
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int64_t r = row0 + wm * 64 + mi * 16 + (lane >> 2) + half * 8;
            if (r >= n) continue;
#pragma unroll
            for (int nj = 0; nj < 4; nj++) {
                const int64_t c = col0 + wn * 32 + nj * 8 + (lane & 3) * 2;
                const float v0 = acc[mi][nj][half * 2], v1 = acc[mi][nj][half * 2 + 1];
                if (OUT_BF16) {
                    uint16_t *y = (uint16_t *)Y + r * cols + c;
                    if (c + 1 < cols) *reinterpret_cast<uint32_t *>(y) = pack_bf16x2(v0, v1);
                    else if (c < cols) y[0] = (uint16_t)(pack_bf16x2(v0, 0.f) & 0xffffu);
                } else {
                    float *y = (float *)Y + r * cols + c;
                    if (c < cols) y[0] = v0;
                    if (c + 1 < cols) y[1] = v1;
                }
            }
        }
}

extern "C" int cwk_fp8_linear(cwk_ctx *ctx, const void *X, const void *W, const float *scale_inv, int64_t n,
                              int64_t k, int64_t cols, void *Y, int out_bf16) {
    if (!ctx || !X || !W || !scale_inv || !Y || n <= 0 || k <= 0 || cols <= 0)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "fp8_linear: bad argument");
    if (k % 128 != 0 || (cols & 1))
        return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "fp8_linear: k must be a multiple of 128 and cols even (k=%lld cols=%lld)", (long long)k, (long long)cols);
    if (((uintptr_t)X | (uintptr_t)W) % 16 != 0) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "fp8_linear: X and W must be 16-byte aligned");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (cwk_fp8_linear_tc_available() && ctx->force_mla_path != 1 && ctx->force_mla_path != 0) {
        int s = cwk_fp8_linear_tc_launch(ctx, X, W, scale_inv, n, k, cols, Y, out_bf16);
        if (s != CWK_ERR_UNSUPPORTED) return s;
    }
    dim3 grid((unsigned)((cols + 127) / 128), (unsigned)((n + 127) / 128));
    CwkKernelTimer timer(ctx);
    if (out_bf16)
        fp8_linear_kernel<true><<<grid, 256, 0, ctx->stream>>>((const uint16_t *)X, (const uint8_t *)W, scale_inv, n, k, cols, Y);
    else
        fp8_linear_kernel<false><<<grid, 256, 0, ctx->stream>>>((const uint16_t *)X, (const uint8_t *)W, scale_inv, n, k, cols, Y);
    CWK_LAUNCH_CHECK(ctx, "fp8_linear_kernel");
    return CWK_OK;
}
