// dropin.cu -- the reference-named attention entry points (include/cwick_compat.h): a link-level
// replacement of the reference's cwick_attention_mla_decode, latent (absorbed) path, that keeps
// the reference's calling convention -- host pointers, caller-owned cache, void return -- and
// runs every stage on the GPU. Device mirrors of the weights and of the latent cache are kept
// in a process-wide registry, created on first sight.
#include <cmath>
#include <cstdarg>
#include <cstdlib>
#include <map>
#include <mutex>
#include <vector>
#include <unordered_map>

#include "../../include/cwick_compat.h"
#include <cuda_fp16.h>

#include "cwk_common.cuh"

int cwk_mla_decode_rows(cwk_ctx *ctx, const void *q, const void *cache, int64_t ld, int rows, int nh, int L, int R,
                        float scale, void *out);

int cwk_mla_decode(cwk_ctx *ctx, const void *q, const void *cache, int64_t seq_stride, int64_t ld, const int32_t *kv_len,
                   int max_kv_len, const int32_t *sel, int64_t sel_ld, int B, int nh, int L, int R, float scale, void *out,
                   int n_splits);

namespace {

// ---- projections ------------------------------------------------------------------------------------------------
// y[t][r] = W[r] . x[t] for one token per blockIdx.y: W [rows][k] row-major in BF16, F32 or FP8-E4M3 (one F32 multiplier
// per 128 x 128 block), x and y f32 (cwick_linear with rows == 1: src/tensor.c:745-765 -> gemv_bf16_range :143-176,
// cwick_gemv_fp8 :674-691 -> gemv_fp8_range :495-532). A projection of one token is its weights read once: the kernel
// is there to keep enough of them in flight. A block of eight warps takes RPB rows, 8 / RPB warps per row (the host
// picks RPB so that the grid is several blocks per SM even for a 512-row matrix); a lane reads 16 bytes of its row per
// step, eight steps ahead of their use, f32 accumulate; the row's warps add up through shared memory.
__device__ __forceinline__ float e4m3_val(uint32_t b) {
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    float mag;
    if (e == 0) mag = (float)m * 0.001953125f;
    else if (e == 15 && m == 7) mag = __int_as_float(0x7fc00000);
    else mag = __uint_as_float(((e + 120u) << 23) | (m << 20));
    return (b & 0x80u) ? -mag : mag;
}

enum { GEMV_BF16 = 0, GEMV_F32 = 1, GEMV_FP8 = 2 };

// 16 bytes of a weight row: read once, so they are kept out of L1, where the activations they meet are read again and again
__device__ __forceinline__ uint4 ld_weight16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Four E4M3 codes against four activations, 256 times too small. A code's seven magnitude bits, moved to bits 7..13 of a
// half, are a half of 2^-8 times the code's value -- subnormal codes land on subnormal halves -- so two codes widen with one
// half2 -> float2 conversion and no table or branch; the power of two goes into the block's multiplier. Only the NaN code
// (magnitude 0x7f) has no such half: a word that holds one takes the code-by-code path.
__device__ __forceinline__ float e4m3x4_dot_by_256th(uint32_t v, const float4 &xq) {
    const uint32_t mag = v & 0x7f7f7f7fu;
    if (__vcmpeq4(mag, 0x7f7f7f7fu))
        return (e4m3_val(v & 0xffu) * xq.x + e4m3_val((v >> 8) & 0xffu) * xq.y + e4m3_val((v >> 16) & 0xffu) * xq.z + e4m3_val(v >> 24) * xq.w) *
               0.00390625f;
    const uint32_t sg = v & 0x80808080u;
    const uint32_t h01 = ((mag & 0x7fu) << 7) | ((mag & 0x7f00u) << 15) | ((sg & 0x80u) << 8) | ((sg & 0x8000u) << 16);
    const uint32_t h23 = ((mag >> 9) & 0x3f80u) | ((mag >> 1) & 0x3f800000u) | ((sg >> 8) & 0x8000u) | (sg & 0x80000000u);
    const float2 f01 = __half22float2(*reinterpret_cast<const __half2 *>(&h01));
    const float2 f23 = __half22float2(*reinterpret_cast<const __half2 *>(&h23));
    return f01.x * xq.x + f01.y * xq.y + f23.x * xq.z + f23.y * xq.w;
}

template <int KIND>
__device__ __forceinline__ float gemv_piece(const uint4 &v, const float *x, int j, const float *sc) {
    // the 16 bytes at element j of the row against x[j ..]: 8 bf16, 4 f32 or 16 e4m3 (times their block's multiplier)
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    float a = 0.f;
    if (KIND == GEMV_BF16) {
        const float4 x0 = *reinterpret_cast<const float4 *>(x + j), x1 = *reinterpret_cast<const float4 *>(x + j + 4);
        a += __uint_as_float(u[0] << 16) * x0.x + __uint_as_float(u[0] & 0xffff0000u) * x0.y;
        a += __uint_as_float(u[1] << 16) * x0.z + __uint_as_float(u[1] & 0xffff0000u) * x0.w;
        a += __uint_as_float(u[2] << 16) * x1.x + __uint_as_float(u[2] & 0xffff0000u) * x1.y;
        a += __uint_as_float(u[3] << 16) * x1.z + __uint_as_float(u[3] & 0xffff0000u) * x1.w;
    } else if (KIND == GEMV_F32) {
        const float4 x0 = *reinterpret_cast<const float4 *>(x + j);
        a = __uint_as_float(u[0]) * x0.x + __uint_as_float(u[1]) * x0.y + __uint_as_float(u[2]) * x0.z + __uint_as_float(u[3]) * x0.w;
    } else {
#pragma unroll
        for (int q = 0; q < 4; q++) a += e4m3x4_dot_by_256th(u[q], *reinterpret_cast<const float4 *>(x + j + 4 * q));
        a *= sc[j >> 7] * 256.0f;                         // 16 elements from a multiple of 16: inside one 128-wide block
    }
    return a;
}

// (A second matrix over the same x may ride in the same launch: blocks [nb1, gridDim.x) belong to it. A chunk's tokens are
// taken TOK at a time, blockIdx.y = group of tokens: a weight piece is read once for the group's tokens -- each token's sum
// runs in the same order as when it is alone.)
template <int KIND, int TOK>
__global__ void __launch_bounds__(256) gemv_rows_kernel(const void *Wv, const float *scales, const float *x, float *y, int rows, int k,
                                                        int64_t ldx, int64_t ldy, int rpb, int nb1, const void *W2, const float *scales2,
                                                        float *y2, int rows2, int64_t ldy2, int ntok) {
    constexpr int E = KIND == GEMV_BF16 ? 8 : KIND == GEMV_F32 ? 4 : 16;      // elements per 16 bytes
    constexpr int EB = 16 / E;                                                // bytes per element
    __shared__ float s_part[TOK][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wpr = 8 / rpb;                               // warps per row
    int bx = blockIdx.x;
    if (bx >= nb1) { bx -= nb1; Wv = W2; scales = scales2; y = y2; rows = rows2; ldy = ldy2; }
    const int r = bx * rpb + warp / wpr, part = warp % wpr;
    const int t0 = blockIdx.y * TOK;
    const float *xt[TOK];
#pragma unroll
    for (int t = 0; t < TOK; t++) xt[t] = x + (int64_t)min(t0 + t, ntok - 1) * ldx;      // a group's missing tokens repeat the last one
    float acc[TOK];
#pragma unroll
    for (int t = 0; t < TOK; t++) acc[t] = 0.f;
    if (r < rows) {
        const uint8_t *w = reinterpret_cast<const uint8_t *>(Wv) + (int64_t)r * k * EB;
        const float *sc = KIND == GEMV_FP8 ? scales + (int64_t)(r / 128) * ((k + 127) / 128) : nullptr;
        const bool vec = (k % E) == 0 && ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) & 15) == 0 && (ldx & 3) == 0;
        if (vec) {
            const int step = wpr * 32 * E;                 // elements per step of the row's warps
            int j = (part * 32 + lane) * E;
            for (; j + 7 * step + E <= k; j += 8 * step) {       // eight loads in flight
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; u++) v[u] = ld_weight16(w + (int64_t)(j + u * step) * EB);
#pragma unroll
                for (int t = 0; t < TOK; t++)
#pragma unroll
                    for (int u = 0; u < 8; u++) acc[t] += gemv_piece<KIND>(v[u], xt[t], j + u * step, sc);
            }
            for (; j + 3 * step + E <= k; j += 4 * step) {       // four
                const uint4 v0 = ld_weight16(w + (int64_t)j * EB);
                const uint4 v1 = ld_weight16(w + (int64_t)(j + step) * EB);
                const uint4 v2 = ld_weight16(w + (int64_t)(j + 2 * step) * EB);
                const uint4 v3 = ld_weight16(w + (int64_t)(j + 3 * step) * EB);
#pragma unroll
                for (int t = 0; t < TOK; t++) {
                    acc[t] += gemv_piece<KIND>(v0, xt[t], j, sc) + gemv_piece<KIND>(v1, xt[t], j + step, sc);
                    acc[t] += gemv_piece<KIND>(v2, xt[t], j + 2 * step, sc) + gemv_piece<KIND>(v3, xt[t], j + 3 * step, sc);
                }
            }
            for (; j + E <= k; j += step) {
                const uint4 v0 = ld_weight16(w + (int64_t)j * EB);
#pragma unroll
                for (int t = 0; t < TOK; t++) acc[t] += gemv_piece<KIND>(v0, xt[t], j, sc);
            }
        } else {
            for (int j = part * 32 + lane; j < k; j += wpr * 32) {
                float wv;
                if (KIND == GEMV_BF16) wv = bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(w)[j]);
                else if (KIND == GEMV_F32) wv = reinterpret_cast<const float *>(w)[j];
                else wv = e4m3_val(w[j]) * sc[j >> 7];
#pragma unroll
                for (int t = 0; t < TOK; t++) acc[t] += wv * xt[t][j];
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TOK; t++)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], o);
    if (wpr == 1) {
        if (lane == 0 && r < rows)
#pragma unroll
            for (int t = 0; t < TOK; t++)
                if (t0 + t < ntok) y[(int64_t)(t0 + t) * ldy + r] = acc[t];
        return;
    }
    if (lane == 0)
#pragma unroll
        for (int t = 0; t < TOK; t++) s_part[t][warp] = acc[t];
    __syncthreads();
    if (part == 0 && lane == 0 && r < rows) {
#pragma unroll
        for (int t = 0; t < TOK; t++) {
            float sum = 0.f;
            for (int i = 0; i < wpr; i++) sum += s_part[t][warp + i];
            if (t0 + t < ntok) y[(int64_t)(t0 + t) * ldy + r] = sum;
        }
    }
}

// A chunk of tokens: four rows x four tokens per warp, so that a lane's 16 bytes of a weight row meet four tokens' activations
// and a token's activations meet four rows -- the one-token form, run per token, reads every activation from L1 once per row
// and is bound by that. A warp covers the whole width of its rows (lane l takes pieces l, l + 32, ...), eight warps = 32 rows
// per block, blockIdx.y = group of four tokens; f32 accumulate, the lanes' sums by shuffles.
template <int KIND>
__device__ __forceinline__ void unpack16(const uint4 &v, float *o) {      // 8 bf16, 4 f32 or 16 e4m3 (those 256 times too small)
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
    if (KIND == GEMV_BF16) {
#pragma unroll
        for (int q = 0; q < 4; q++) { o[2 * q] = __uint_as_float(u[q] << 16); o[2 * q + 1] = __uint_as_float(u[q] & 0xffff0000u); }
    } else if (KIND == GEMV_F32) {
#pragma unroll
        for (int q = 0; q < 4; q++) o[q] = __uint_as_float(u[q]);
    } else {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint32_t mag = u[q] & 0x7f7f7f7fu, sg = u[q] & 0x80808080u;
            if (__vcmpeq4(mag, 0x7f7f7f7fu)) {             // a NaN code in the word: code by code
#pragma unroll
                for (int e = 0; e < 4; e++) o[4 * q + e] = e4m3_val((u[q] >> (8 * e)) & 0xffu) * 0.00390625f;
            } else {
                const uint32_t h01 = ((mag & 0x7fu) << 7) | ((mag & 0x7f00u) << 15) | ((sg & 0x80u) << 8) | ((sg & 0x8000u) << 16);
                const uint32_t h23 = ((mag >> 9) & 0x3f80u) | ((mag >> 1) & 0x3f800000u) | ((sg >> 8) & 0x8000u) | (sg & 0x80000000u);
                const float2 f01 = __half22float2(*reinterpret_cast<const __half2 *>(&h01));
                const float2 f23 = __half22float2(*reinterpret_cast<const __half2 *>(&h23));
                o[4 * q] = f01.x; o[4 * q + 1] = f01.y; o[4 * q + 2] = f23.x; o[4 * q + 3] = f23.y;
            }
        }
    }
}

template <int KIND>
__global__ void __launch_bounds__(256) gemm_rows_kernel(const void *Wv, const float *scales, const float *x, float *y, int rows, int k,
                                                        int64_t ldx, int64_t ldy, int ntok) {
    constexpr int E = KIND == GEMV_BF16 ? 8 : KIND == GEMV_F32 ? 4 : 16, EB = 16 / E, R = 4, TOK = 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r0 = (blockIdx.x * 8 + warp) * R, t0 = blockIdx.y * TOK;
    if (r0 >= rows) return;
    const float *xt[TOK];
#pragma unroll
    for (int t = 0; t < TOK; t++) xt[t] = x + (int64_t)min(t0 + t, ntok - 1) * ldx;
    const uint8_t *w[R];
#pragma unroll
    for (int r = 0; r < R; r++) w[r] = reinterpret_cast<const uint8_t *>(Wv) + (int64_t)min(r0 + r, rows - 1) * k * EB;
    const int nkb = (k + 127) / 128;
    float acc[R][TOK];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int t = 0; t < TOK; t++) acc[r][t] = 0.f;
    // (loads of the next step issued ahead of this step's arithmetic were measured: the registers they hold cost more
    // in resident warps than the overlap gives -- 2.37 against 1.67 ms for the widest projection of a 512-token chunk)
    for (int j = lane * E; j + E <= k; j += 32 * E) {
        uint4 wv[R];
#pragma unroll
        for (int r = 0; r < R; r++) wv[r] = ld_weight16(w[r] + (int64_t)j * EB);
        float xv[TOK][E];
#pragma unroll
        for (int t = 0; t < TOK; t++)
#pragma unroll
            for (int q = 0; q < E / 4; q++) {
                const float4 f = *reinterpret_cast<const float4 *>(xt[t] + j + 4 * q);
                xv[t][4 * q] = f.x; xv[t][4 * q + 1] = f.y; xv[t][4 * q + 2] = f.z; xv[t][4 * q + 3] = f.w;
            }
#pragma unroll
        for (int r = 0; r < R; r++) {
            float o[E];
            unpack16<KIND>(wv[r], o);
            float m = 1.f;
            if (KIND == GEMV_FP8) m = scales[(int64_t)(min(r0 + r, rows - 1) / 128) * nkb + (j >> 7)] * 256.0f;
#pragma unroll
            for (int t = 0; t < TOK; t++) {
                float d = 0.f;
#pragma unroll
                for (int e = 0; e < E; e++) d += o[e] * xv[t][e];
                acc[r][t] += KIND == GEMV_FP8 ? d * m : d;
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int t = 0; t < TOK; t++) {
            float a = acc[r][t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
            if (lane == 0 && r0 + r < rows && t0 + t < ntok) y[(int64_t)(t0 + t) * ldy + r0 + r] = a;
        }
}

// Whether gemm_rows_kernel takes the operands: whole 16-byte pieces, aligned rows.
bool gemm_rows_ok(const void *W, const float *x, int64_t k, int64_t ldx, int kind) {
    const int E = kind == GEMV_BF16 ? 8 : kind == GEMV_F32 ? 4 : 16;
    return k % (32 * E) == 0 && (ldx & 3) == 0 && ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(x)) & 15) == 0;
}

// y[t][0..rows) = W . x[t] for n tokens. kind: GEMV_BF16 / GEMV_F32 / GEMV_FP8. W2 != NULL: also y2 = W2 . x[t] (same kind,
// same k) in the same launch.
template <int TOK>
void launch_gemv_tok(cwk_ctx *ctx, int kind, const void *W, const float *scales, const float *x, float *y, int64_t rows, int64_t k, int n,
                     int64_t ldx, int64_t ldy, const void *W2, const float *scales2, float *y2, int64_t rows2, int64_t ldy2) {
    const int groups = (n + TOK - 1) / TOK;
    int rpb = 8;                                           // fewer rows per block until the grid is a few blocks per SM
    while (rpb > 1 && ((rows + rpb - 1) / rpb + (rows2 + rpb - 1) / rpb) * groups < 4 * (int64_t)ctx->sm_count) rpb >>= 1;
    const int nb1 = (int)((rows + rpb - 1) / rpb), nb2 = W2 ? (int)((rows2 + rpb - 1) / rpb) : 0;
    const dim3 grid((unsigned)(nb1 + nb2), (unsigned)groups);
    if (kind == GEMV_BF16)
        gemv_rows_kernel<GEMV_BF16, TOK><<<grid, 256, 0, ctx->stream>>>(W, scales, x, y, (int)rows, (int)k, ldx, ldy, rpb, nb1, W2, scales2, y2, (int)rows2, ldy2, n);
    else if (kind == GEMV_F32)
        gemv_rows_kernel<GEMV_F32, TOK><<<grid, 256, 0, ctx->stream>>>(W, scales, x, y, (int)rows, (int)k, ldx, ldy, rpb, nb1, W2, scales2, y2, (int)rows2, ldy2, n);
    else
        gemv_rows_kernel<GEMV_FP8, TOK><<<grid, 256, 0, ctx->stream>>>(W, scales, x, y, (int)rows, (int)k, ldx, ldy, rpb, nb1, W2, scales2, y2, (int)rows2, ldy2, n);
    ctx->launches++;
}
void launch_gemv(cwk_ctx *ctx, int kind, const void *W, const float *scales, const float *x, float *y, int64_t rows, int64_t k, int n,
                 int64_t ldx, int64_t ldy, const void *W2 = nullptr, const float *scales2 = nullptr, float *y2 = nullptr, int64_t rows2 = 0,
                 int64_t ldy2 = 0) {
    if (n >= 4 && !W2 && gemm_rows_ok(W, x, k, ldx, kind)) {
        const dim3 grid((unsigned)((rows + 31) / 32), (unsigned)((n + 3) / 4));
        if (kind == GEMV_BF16) gemm_rows_kernel<GEMV_BF16><<<grid, 256, 0, ctx->stream>>>(W, scales, x, y, (int)rows, (int)k, ldx, ldy, n);
        else if (kind == GEMV_F32) gemm_rows_kernel<GEMV_F32><<<grid, 256, 0, ctx->stream>>>(W, scales, x, y, (int)rows, (int)k, ldx, ldy, n);
        else gemm_rows_kernel<GEMV_FP8><<<grid, 256, 0, ctx->stream>>>(W, scales, x, y, (int)rows, (int)k, ldx, ldy, n);
        ctx->launches++;
        return;
    }
    if (n >= 4) launch_gemv_tok<4>(ctx, kind, W, scales, x, y, rows, k, n, ldx, ldy, W2, scales2, y2, rows2, ldy2);
    else launch_gemv_tok<1>(ctx, kind, W, scales, x, y, rows, k, n, ldx, ldy, W2, scales2, y2, rows2, ldy2);
}

// The KDA layer's projections keep the one-warp-per-row form: a lane's strided partial sums and the shuffle tree are the
// order in which the values of the convolution window (copies of these outputs) were pinned bit for bit.
__global__ void __launch_bounds__(256) gemv_bf16_kernel(const uint16_t *W, const float *x, float *y, int rows, int k, int64_t ldx,
                                                        int64_t ldy) {
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= rows) return;
    x += (int64_t)blockIdx.y * ldx;
    y += (int64_t)blockIdx.y * ldy;
    const uint16_t *w = W + (int64_t)r * k;
    float acc = 0.f;
    if ((k & 7) == 0) {
        for (int j = lane * 8; j + 8 <= k; j += 256) {
            const uint4 v = *reinterpret_cast<const uint4 *>(w + j);
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                acc += bf16_bits_to_f32((uint16_t)(u[e] & 0xffffu)) * x[j + 2 * e];
                acc += bf16_bits_to_f32((uint16_t)(u[e] >> 16)) * x[j + 2 * e + 1];
            }
        }
    } else {
        for (int j = lane; j < k; j += 32) acc += bf16_bits_to_f32(w[j]) * x[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[r] = acc;
}

// In place: x <- x / sqrt(mean(x^2) + eps) * w (cwick_rms_norm + apply_bf16_vec, src/tensor.c:780-791,
// src/attention.c:70-73), one block per row (blockIdx.x). Optionally also narrows the result to bf16 the way the
// reference narrows a latent-cache row (src/util.c:202-210) into row_out + row * row_ld.
__device__ __forceinline__ void rms_scale_row(float *x, int n, const uint16_t *w, float eps, uint16_t *row_out, void *host_row, int host_bf16) {
    __shared__ double red[8];
    double ss = 0.0;
    for (int i = threadIdx.x; i < n; i += 256) ss += (double)x[i] * (double)x[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const double tot = ((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]));
    const float inv = __fdiv_rn(1.0f, (float)sqrt(tot / (double)n + (double)eps));
    for (int i = threadIdx.x; i < n; i += 256) {
        const float v = x[i] * inv * bf16_bits_to_f32(w[i]);
        x[i] = v;
        const uint32_t u = __float_as_uint(v);
        const uint16_t nb = (uint16_t)((u + ((u >> 15) & 1u) + ((u >> 16) & 1u)) >> 16);
        if (row_out) row_out[i] = nb;
        if (host_row) {                                    // the caller's copy of the row, in the caller's element width
            if (host_bf16) reinterpret_cast<uint16_t *>(host_row)[i] = nb;
            else reinterpret_cast<float *>(host_row)[i] = v;
        }
    }
}
__global__ void __launch_bounds__(256) rms_scale_kernel(float *x, int n, int64_t ldx, const uint16_t *w, float eps, uint16_t *row_out,
                                                        int64_t row_ld) {
    rms_scale_row(x + (int64_t)blockIdx.x * ldx, n, w, eps, row_out ? row_out + (int64_t)blockIdx.x * row_ld : nullptr, nullptr, 0);
}
// The two norms of a decode step in one launch: block 0 the q_a row, block 1 the kv_a row (which is also the new cache row,
// on the device and -- through page-locked memory the device can address -- in the staging buffer the caller's array is
// filled from).
__global__ void __launch_bounds__(256) rms_scale_pair_kernel(float *xa, int na, const uint16_t *wa, float *xb, int nb, const uint16_t *wb,
                                                             float eps, uint16_t *row_out, void *host_row, int host_bf16) {
    if (blockIdx.x == 0) rms_scale_row(xa, na, wa, eps, nullptr, nullptr, 0);
    else rms_scale_row(xb, nb, wb, eps, row_out, host_row, host_bf16);
}

// q_abs[t][h][c] = sum_r q[t][h][r] * W_k[h][r][c] (src/attention.c:741-744), W_k = rows [h*kv_dim, +nope) of
// kv_b_proj [nh*kv_dim][kv_lora]. grid (nh, tokens), thread per column, bf16 out.
__global__ void absorb_q_kernel(const float *q, const uint16_t *kvb, int nh, int nope, int kv_dim, int kv_lora, uint16_t *qabs) {
    const int h = blockIdx.x;
    q += (int64_t)blockIdx.y * nh * nope;
    qabs += (int64_t)blockIdx.y * nh * kv_lora;
    const uint16_t *wk = kvb + (int64_t)h * kv_dim * kv_lora;
    for (int c = threadIdx.x; c < kv_lora; c += blockDim.x) {
        float acc = 0.f;
        for (int r = 0; r < nope; r++) acc += q[h * nope + r] * bf16_bits_to_f32(wk[(int64_t)r * kv_lora + c]);
        qabs[(int64_t)h * kv_lora + c] = (uint16_t)(pack_bf16x2(acc, 0.f) & 0xffffu);
    }
}

// The same for a latent width that is a multiple of 8 with 512 % (kv_lora / 8) == 0 (512: 64 threads across a row of
// W_k, 8 columns = 16 bytes each, eight groups of rows): a head is 128 KB of weights read once by one block, so what
// counts is loads in flight -- eight rows ahead per thread -- not the arithmetic. The row groups add up through shared
// memory. grid (nh, tokens), 512 threads, dynamic shared memory (512 / (kv_lora / 8)) * kv_lora floats.
__global__ void __launch_bounds__(512) absorb_q_rows_kernel(const float *q, const uint16_t *kvb, int nh, int nope, int kv_dim, int kv_lora,
                                                            uint16_t *qabs) {
    extern __shared__ float s_abs[];
    const int h = blockIdx.x;
    q += (int64_t)blockIdx.y * nh * nope + (int64_t)h * nope;
    qabs += (int64_t)blockIdx.y * nh * kv_lora + (int64_t)h * kv_lora;
    const int tpr = kv_lora / 8, ng = 512 / tpr;           // threads per row, row groups
    const int rg = threadIdx.x / tpr, c8 = (threadIdx.x % tpr) * 8;
    const uint16_t *wk = kvb + (int64_t)h * kv_dim * kv_lora + c8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto fma8 = [&](const uint4 &v, float qv) {
        acc[0] += qv * __uint_as_float(v.x << 16); acc[1] += qv * __uint_as_float(v.x & 0xffff0000u);
        acc[2] += qv * __uint_as_float(v.y << 16); acc[3] += qv * __uint_as_float(v.y & 0xffff0000u);
        acc[4] += qv * __uint_as_float(v.z << 16); acc[5] += qv * __uint_as_float(v.z & 0xffff0000u);
        acc[6] += qv * __uint_as_float(v.w << 16); acc[7] += qv * __uint_as_float(v.w & 0xffff0000u);
    };
    int r = rg;
    for (; r + 7 * ng < nope; r += 8 * ng) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = __ldg(reinterpret_cast<const uint4 *>(wk + (int64_t)(r + u * ng) * kv_lora));
#pragma unroll
        for (int u = 0; u < 8; u++) fma8(v[u], q[r + u * ng]);
    }
    for (; r < nope; r += ng) fma8(__ldg(reinterpret_cast<const uint4 *>(wk + (int64_t)r * kv_lora)), q[r]);
#pragma unroll
    for (int e = 0; e < 8; e++) s_abs[rg * kv_lora + c8 + e] = acc[e];
    __syncthreads();
    for (int c = threadIdx.x; c < kv_lora; c += 512) {
        float t = 0.f;
        for (int gi = 0; gi < ng; gi++) t += s_abs[gi * kv_lora + c];
        qabs[c] = (uint16_t)(pack_bf16x2(t, 0.f) & 0xffffu);
    }
}

// For a chunk: four tokens per block (blockIdx.y = group of four), so that a thread's 16 bytes of a W_k row meet four
// tokens' q values: 32 multiply-adds per load instead of 8. Otherwise as absorb_q_rows_kernel; dynamic shared memory
// 4 x (512 / (kv_lora / 8)) * kv_lora floats would be too much, so the row groups add up token by token through one
// token's worth of it.
__global__ void __launch_bounds__(512) absorb_q_rows4_kernel(const float *q, const uint16_t *kvb, int nh, int nope, int kv_dim, int kv_lora,
                                                             uint16_t *qabs, int ntok) {
    extern __shared__ float s_abs[];
    constexpr int TOK = 4;
    const int h = blockIdx.x, t0 = blockIdx.y * TOK;
    const float *qt[TOK];
#pragma unroll
    for (int t = 0; t < TOK; t++) qt[t] = q + (int64_t)min(t0 + t, ntok - 1) * nh * nope + (int64_t)h * nope;
    const int tpr = kv_lora / 8, ng = 512 / tpr;           // threads per row, row groups
    const int rg = threadIdx.x / tpr, c8 = (threadIdx.x % tpr) * 8;
    const uint16_t *wk = kvb + (int64_t)h * kv_dim * kv_lora + c8;
    float acc[TOK][8];
#pragma unroll
    for (int t = 0; t < TOK; t++)
#pragma unroll
        for (int e = 0; e < 8; e++) acc[t][e] = 0.f;
    auto fma8 = [&](const uint4 &v, int r) {
        const float wv[8] = {__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u),
                             __uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u), __uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u)};
#pragma unroll
        for (int t = 0; t < TOK; t++) {
            const float qv = qt[t][r];
#pragma unroll
            for (int e = 0; e < 8; e++) acc[t][e] += qv * wv[e];
        }
    };
    int r = rg;
    for (; r + 3 * ng < nope; r += 4 * ng) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] = ld_weight16(wk + (int64_t)(r + u * ng) * kv_lora);
#pragma unroll
        for (int u = 0; u < 4; u++) fma8(v[u], r + u * ng);
    }
    for (; r < nope; r += ng) fma8(ld_weight16(wk + (int64_t)r * kv_lora), r);
#pragma unroll
    for (int t = 0; t < TOK; t++) {
#pragma unroll
        for (int e = 0; e < 8; e++) s_abs[rg * kv_lora + c8 + e] = acc[t][e];
        __syncthreads();
        if (t0 + t < ntok)
            for (int c = threadIdx.x; c < kv_lora; c += 512) {
                float sum = 0.f;
                for (int gi = 0; gi < ng; gi++) sum += s_abs[gi * kv_lora + c];
                qabs[((int64_t)(t0 + t) * nh + h) * kv_lora + c] = (uint16_t)(pack_bf16x2(sum, 0.f) & 0xffffu);
            }
        __syncthreads();
    }
}

void launch_absorb_q(cudaStream_t st, const float *q, const uint16_t *kvb, int nh, int nope, int kv_dim, int kv_lora, uint16_t *qabs,
                     int tokens) {
    const int tpr = kv_lora / 8;
    if (kv_lora % 8 == 0 && tpr <= 512 && 512 % tpr == 0 && (reinterpret_cast<uintptr_t>(kvb) & 15) == 0 &&
        (size_t)(512 / tpr) * kv_lora * 4 <= 48 * 1024) {
        if (tokens >= 4)
            absorb_q_rows4_kernel<<<dim3(nh, (tokens + 3) / 4), 512, (size_t)(512 / tpr) * kv_lora * 4, st>>>(q, kvb, nh, nope, kv_dim, kv_lora, qabs, tokens);
        else
            absorb_q_rows_kernel<<<dim3(nh, tokens), 512, (size_t)(512 / tpr) * kv_lora * 4, st>>>(q, kvb, nh, nope, kv_dim, kv_lora, qabs);
    }
    else
        absorb_q_kernel<<<dim3(nh, tokens), 256, 0, st>>>(q, kvb, nh, nope, kv_dim, kv_lora, qabs);
}

// attn_out[t][h][r] = W_v[h][r] . c_acc[t][h] (src/attention.c:812-815). One warp per (h, r); blockIdx.y = token.
__global__ void __launch_bounds__(256) unabsorb_kernel(const uint16_t *cacc, const uint16_t *kvb, int nh, int nope, int vdim,
                                                       int kv_lora, float *attn) {
    const int idx = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (idx >= nh * vdim) return;
    cacc += (int64_t)blockIdx.y * nh * kv_lora;
    attn += (int64_t)blockIdx.y * nh * vdim;
    const int h = idx / vdim, r = idx % vdim;
    const uint16_t *w = kvb + ((int64_t)h * (nope + vdim) + nope + r) * kv_lora;
    const uint16_t *c = cacc + (int64_t)h * kv_lora;
    float acc = 0.f;
    for (int j = lane; j < kv_lora; j += 32) acc += bf16_bits_to_f32(w[j]) * bf16_bits_to_f32(c[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) attn[idx] = acc;
}

// The same for a chunk of tokens: four value rows x four tokens per warp (a lane's 16 bytes of a W_v row meet four tokens'
// accumulators and the other way round), eight warps = 32 rows per block; grid (vdim / 32, groups of four tokens, heads).
// kv_lora a multiple of 256, vdim a multiple of 4, 16-byte aligned operands.
__global__ void __launch_bounds__(256) unabsorb_rows_kernel(const uint16_t *cacc, const uint16_t *kvb, int nh, int nope, int vdim,
                                                            int kv_lora, float *attn, int ntok) {
    constexpr int R = 4, TOK = 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.z, r0 = (blockIdx.x * 8 + warp) * R, t0 = blockIdx.y * TOK;
    if (r0 >= vdim) return;
    const uint16_t *w[R], *c[TOK];
#pragma unroll
    for (int r = 0; r < R; r++) w[r] = kvb + ((int64_t)h * (nope + vdim) + nope + min(r0 + r, vdim - 1)) * kv_lora;
#pragma unroll
    for (int t = 0; t < TOK; t++) c[t] = cacc + ((int64_t)min(t0 + t, ntok - 1) * nh + h) * kv_lora;
    float acc[R][TOK];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int t = 0; t < TOK; t++) acc[r][t] = 0.f;
    for (int j = lane * 8; j + 8 <= kv_lora; j += 256) {
        uint4 wv[R], cv[TOK];
#pragma unroll
        for (int r = 0; r < R; r++) wv[r] = ld_weight16(w[r] + j);
#pragma unroll
        for (int t = 0; t < TOK; t++) cv[t] = *reinterpret_cast<const uint4 *>(c[t] + j);
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint32_t wu[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
#pragma unroll
            for (int t = 0; t < TOK; t++) {
                const uint32_t cu[4] = {cv[t].x, cv[t].y, cv[t].z, cv[t].w};
                float d = 0.f;
#pragma unroll
                for (int q = 0; q < 4; q++)
                    d += __uint_as_float(wu[q] << 16) * __uint_as_float(cu[q] << 16) +
                         __uint_as_float(wu[q] & 0xffff0000u) * __uint_as_float(cu[q] & 0xffff0000u);
                acc[r][t] += d;
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int t = 0; t < TOK; t++) {
            float a = acc[r][t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
            if (lane == 0 && r0 + r < vdim && t0 + t < ntok) attn[((int64_t)(t0 + t) * nh + h) * vdim + r0 + r] = a;
        }
}

void launch_unabsorb(cudaStream_t st, const uint16_t *cacc, const uint16_t *kvb, int nh, int nope, int vdim, int kv_lora, float *attn, int tokens) {
    if (tokens >= 4 && kv_lora % 256 == 0 && ((reinterpret_cast<uintptr_t>(kvb) | reinterpret_cast<uintptr_t>(cacc)) & 15) == 0)
        unabsorb_rows_kernel<<<dim3((vdim + 31) / 32, (tokens + 3) / 4, nh), 256, 0, st>>>(cacc, kvb, nh, nope, vdim, kv_lora, attn, tokens);
    else
        unabsorb_kernel<<<dim3((nh * vdim + 7) / 8, tokens), 256, 0, st>>>(cacc, kvb, nh, nope, vdim, kv_lora, attn);
}

// Indexer scores over the f32 pool rows, the reference's order (src/attention.c:573-582 with dot_f32's scalar
// grouping :249-258): per head four strided accumulators with separate multiply and add, (s0+s1)+(s2+s3), then any
// remainder in order; ReLU; times the head weight; heads summed in order. One thread per pool row.
__global__ void __launch_bounds__(128) pool_scores_kernel(const float *pool, int n, int hd, const float *q, const float *wt, int ih,
                                                          float *sc) {
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c >= n) return;
    const float *kv = pool + (int64_t)c * hd;
    float total = 0.f;
    for (int h = 0; h < ih; h++) {
        const float *qh = q + (int64_t)h * hd;
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        int i = 0;
        for (; i + 4 <= hd; i += 4) {
            s0 = __fadd_rn(s0, __fmul_rn(kv[i], qh[i]));
            s1 = __fadd_rn(s1, __fmul_rn(kv[i + 1], qh[i + 1]));
            s2 = __fadd_rn(s2, __fmul_rn(kv[i + 2], qh[i + 2]));
            s3 = __fadd_rn(s3, __fmul_rn(kv[i + 3], qh[i + 3]));
        }
        float d = __fadd_rn(__fadd_rn(s0, s1), __fadd_rn(s2, s3));
        for (; i < hd; i++) d = __fadd_rn(d, __fmul_rn(kv[i], qh[i]));
        if (d < 0.f) d = 0.f;
        total = __fadd_rn(total, __fmul_rn(d, wt[h]));
    }
    sc[c] = total;
}

__global__ void scale_vec_kernel(float *x, int n, float s) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = __fmul_rn(x[i], s);
}

// ---- device mirrors ---------------------------------------------------------------------------------------------
struct WeightMirror {
    void *data = nullptr;
    float *scales = nullptr;
    int kind = 0;
    int64_t rows = 0, cols = 0;
};
struct WeightKey {
    const void *ptr;
    int64_t rows, cols;
    int kind;
    bool operator<(const WeightKey &o) const {
        if (ptr != o.ptr) return ptr < o.ptr;
        if (rows != o.rows) return rows < o.rows;
        if (cols != o.cols) return cols < o.cols;
        return kind < o.kind;
    }
};
struct CacheMirror {
    uint16_t *dev = nullptr;
    int64_t capacity = 0, width = 0, next_pos = 0;
    std::vector<uint8_t> last_row;          // the caller's row next_pos-1 as it was when the mirror last agreed with it
};
struct IndexMirror {
    float *pool = nullptr, *tails = nullptr;      // [pool_cap][hd]; tail_k [kp][hd] then tail_g [kp][hd]
    int64_t pool_cap = 0, hd = 0, kp = 0, n_pools = 0;
    std::vector<float> last_row;
};

struct Registry {
    std::mutex mu;
    cwk_ctx *ctx = nullptr;
    std::map<WeightKey, WeightMirror> weights;
    std::map<std::pair<const void *, int64_t>, CacheMirror> caches;
    std::map<const void *, IndexMirror> indexers;
    float *d_buf = nullptr;       // activations
    size_t d_buf_bytes = 0;
    void *pin = nullptr;          // page-locked staging; pin_dev: the same memory as the device addresses it (NULL: not addressable)
    void *pin_dev = nullptr;
    size_t pin_bytes = 0;
} g;

void set_err(cwkc_error *err, int status, const char *fmt, ...) {
    if (!err) return;
    err->status = status;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err->message, sizeof(err->message), fmt, ap);
    va_end(ap);
}

bool latent_ok(const cwkc_model_spec *s, const cwkc_tensor *kvb) {
    // src/attention.c:102-113 (mla_latent_ok)
    if (getenv("CWICK_MLA_EXPANDED") != nullptr) return false;
    const int64_t kv_dim = s->qk_nope_head_dim + s->value_head_dim;
    if (kv_dim <= 0 || s->num_attention_heads <= 0 || s->qk_rope_head_dim != 0 || s->kv_lora_rank <= 0) return false;
    return kvb->rows == s->num_attention_heads * kv_dim && kvb->cols >= s->kv_lora_rank;
}

bool kind_ok(int kind) { return kind == CWKC_WEIGHT_BF16 || kind == CWKC_WEIGHT_F32 || kind == CWKC_WEIGHT_FP8_E4M3; }

// The device copy of a weight tensor, made on first sight. Keyed by data pointer, shape and kind.
const WeightMirror *mirror_weight(const cwkc_tensor *t) {
    if (!t || !t->data || !kind_ok(t->kind)) return nullptr;
    const WeightKey key{t->data, t->rows, t->cols, t->kind};
    auto it = g.weights.find(key);
    if (it != g.weights.end()) return &it->second;
    WeightMirror m;
    m.kind = t->kind; m.rows = t->rows; m.cols = t->cols;
    const size_t el = t->kind == CWKC_WEIGHT_BF16 ? 2 : (t->kind == CWKC_WEIGHT_F32 ? 4 : 1);
    const size_t bytes = (size_t)t->rows * (size_t)t->cols * el;
    if (cudaMalloc(&m.data, bytes) != cudaSuccess) return nullptr;
    if (cudaMemcpy(m.data, t->data, bytes, cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(m.data); return nullptr; }
    if (t->kind == CWKC_WEIGHT_FP8_E4M3) {
        const size_t ns = (size_t)((t->rows + 127) / 128) * (size_t)((t->cols + 127) / 128);
        if (!t->scales || cudaMalloc((void **)&m.scales, ns * 4) != cudaSuccess) { cudaFree(m.data); return nullptr; }
        if (cudaMemcpy(m.scales, t->scales, ns * 4, cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(m.data); cudaFree(m.scales); return nullptr; }
    }
    return &(g.weights[key] = m);
}

// y[t][0..rows) = W . x[t] for n tokens (cwick_linear, src/tensor.c:745-765), whatever the weight's kind.
void dev_linear(cwk_ctx *ctx, const WeightMirror *w, const float *x, float *y, int n, int64_t ldx, int64_t ldy) {
    const int kind = w->kind == CWKC_WEIGHT_BF16 ? GEMV_BF16 : w->kind == CWKC_WEIGHT_F32 ? GEMV_F32 : GEMV_FP8;
    launch_gemv(ctx, kind, w->data, w->scales, x, y, w->rows, w->cols, n, ldx, ldy);
}

// Values of a small vector tensor as f32 on the device (cwick_tensor_value, src/tensor.c:767-774).
float *mirror_vector_f32(const cwkc_tensor *t, int64_t n) {
    if (!t || !t->data) return nullptr;
    const WeightKey key{t->data, -n, 1, t->kind};       // negative rows: the widened-vector form of the tensor
    auto it = g.weights.find(key);
    if (it != g.weights.end()) return (float *)it->second.data;
    std::vector<float> v((size_t)n);
    for (int64_t i = 0; i < n; i++) {
        if (t->kind == CWKC_WEIGHT_BF16) {
            const uint32_t u = (uint32_t)((const uint16_t *)t->data)[i] << 16;
            memcpy(&v[(size_t)i], &u, 4);
        } else if (t->kind == CWKC_WEIGHT_F32) v[(size_t)i] = ((const float *)t->data)[i];
        else v[(size_t)i] = 0.0f;
    }
    WeightMirror m;
    m.kind = t->kind; m.rows = -n; m.cols = 1;
    if (cudaMalloc(&m.data, (size_t)n * 4) != cudaSuccess) return nullptr;
    if (cudaMemcpy(m.data, v.data(), (size_t)n * 4, cudaMemcpyHostToDevice) != cudaSuccess) { cudaFree(m.data); return nullptr; }
    g.weights[key] = m;
    return (float *)m.data;
}

bool ensure_ctx(cwkc_error *err) {
    if (g.ctx) return true;
    const char *d = getenv("CWK_DEVICE");
    if (cwk_ctx_create(d ? atoi(d) : 0, &g.ctx) != CWK_OK) { set_err(err, CWK_ERR_STATE, "no usable sm_100 GPU"); return false; }
    return true;
}
bool ensure_bufs(size_t dev_bytes, size_t pin_bytes, cwkc_error *err) {
    if (dev_bytes > g.d_buf_bytes) {
        if (g.d_buf) { cudaStreamSynchronize(g.ctx->stream); cudaFree(g.d_buf); }
        if (cudaMalloc(&g.d_buf, dev_bytes) != cudaSuccess) { g.d_buf = nullptr; g.d_buf_bytes = 0; set_err(err, CWK_ERR_MEMORY, "device scratch"); return false; }
        g.d_buf_bytes = dev_bytes;
    }
    if (pin_bytes > g.pin_bytes) {
        if (g.pin) { cudaStreamSynchronize(g.ctx->stream); cudaFreeHost(g.pin); }
        if (cudaMallocHost(&g.pin, pin_bytes) != cudaSuccess) { g.pin = nullptr; g.pin_bytes = 0; set_err(err, CWK_ERR_MEMORY, "pinned staging"); return false; }
        g.pin_bytes = pin_bytes;
        if (cudaHostGetDevicePointer(&g.pin_dev, g.pin, 0) != cudaSuccess) { (void)cudaGetLastError(); g.pin_dev = nullptr; }
    }
    return true;
}

// Moves the k largest values to the front by Hoare partitions around the middle element, exactly as the reference's
// score_select does (src/attention.c:528-543): the value left at v[k-1] is what the reference takes as its
// threshold, which is one of the k largest but not always the smallest of them. Reproducing the procedure, not just
// "the k-th largest", is what makes the selection below the reference's own, entry for entry.
void select_front(float *v, int64_t n, int64_t k) {
    int64_t lo = 0, hi = n - 1;
    while (lo < hi) {
        const float pivot = v[(size_t)((lo + hi) >> 1)];
        int64_t i = lo, j = hi;
        while (i <= j) {
            while (v[i] > pivot) i++;
            while (v[j] < pivot) j--;
            if (i <= j) { std::swap(v[i], v[j]); i++; j--; }
        }
        if (k <= j) hi = j;
        else if (k >= i) lo = i;
        else break;
    }
}

// Everything one layer call needs, resolved once.
struct Layer {
    const cwkc_model_spec *spec;
    const WeightMirror *qa, *qb, *kva, *kvb, *o;
    const uint16_t *qa_n, *kva_n;
    int64_t H;
    int nh, nope, vdim, q_lora, kv_lora, kv_dim;
    bool lbf;                       // the caller's cache array holds bf16 (CWICK_LATENT_BF16) or f32
    CacheMirror *cm;
    uint8_t *host_layer;            // the caller's rows of this layer
    size_t host_row_bytes;
    // indexer (all null when the layer has none)
    const cwkc_indexer_weights *idx_w = nullptr;
    cwkc_indexer_state *idx = nullptr;
    IndexMirror *im = nullptr;
    const WeightMirror *wq_b = nullptr, *wk = nullptr, *gate = nullptr, *weights_proj = nullptr;
    const uint16_t *ape = nullptr;
    float *k_norm = nullptr, *k_norm_b = nullptr;
    int ih = 0, ihd = 0, kp = 1;
};

// Bring the device mirror of the latent cache in step with the caller's rows 0..pos-1.
int sync_cache(cwk_ctx *ctx, Layer &ly, int64_t capacity, int64_t pos) {
    CacheMirror &cm = *ly.cm;
    const int kv_lora = ly.kv_lora;
    if (!cm.dev || cm.capacity != capacity || cm.width != kv_lora) {
        if (cm.dev) { cudaStreamSynchronize(ctx->stream); cudaFree(cm.dev); }
        if (cudaMalloc(&cm.dev, (size_t)capacity * kv_lora * 2) != cudaSuccess) { cm.dev = nullptr; return CWK_ERR_MEMORY; }
        cm.capacity = capacity; cm.width = kv_lora; cm.next_pos = -1;
    }
    bool stale = pos != cm.next_pos;
    if (!stale && pos > 0)      // same length: trust the mirror only while the caller's last row is the one written through it
        stale = cm.last_row.size() != ly.host_row_bytes || memcmp(cm.last_row.data(), ly.host_layer + (size_t)(pos - 1) * ly.host_row_bytes, ly.host_row_bytes) != 0;
    if (stale && pos > 0) {
        if (ly.lbf) {
            if (cudaMemcpyAsync(cm.dev, ly.host_layer, (size_t)pos * kv_lora * 2, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) return CWK_ERR_CUDA;
            if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return CWK_ERR_CUDA;      // the source is pageable caller memory
        } else {
            int s = cwk_cache_import_f32(ctx, (const float *)ly.host_layer, pos, kv_lora, cm.dev, kv_lora, 1);
            if (s != CWK_OK) return s;
        }
    }
    return CWK_OK;
}

void note_row_written(Layer &ly, int64_t pos) {
    CacheMirror &cm = *ly.cm;
    cm.last_row.assign(ly.host_layer + (size_t)pos * ly.host_row_bytes, ly.host_layer + (size_t)(pos + 1) * ly.host_row_bytes);
    cm.next_pos = pos + 1;
}

// The indexer's device state in step with the caller's (pool rows 0..n_pools-1, both tails).
int sync_indexer(cwk_ctx *ctx, Layer &ly) {
    IndexMirror &im = *ly.im;
    cwkc_indexer_state *st = ly.idx;
    const int64_t hd = ly.ihd, kp = ly.kp;
    if (!im.pool || im.pool_cap != st->pool_cap || im.hd != hd || im.kp != kp) {
        if (im.pool) { cudaStreamSynchronize(ctx->stream); cudaFree(im.pool); cudaFree(im.tails); }
        im.pool = im.tails = nullptr;
        if (cudaMalloc((void **)&im.pool, (size_t)std::max<int64_t>(1, st->pool_cap) * hd * 4) != cudaSuccess) return CWK_ERR_MEMORY;
        if (cudaMalloc((void **)&im.tails, (size_t)2 * kp * hd * 4) != cudaSuccess) return CWK_ERR_MEMORY;
        im.pool_cap = st->pool_cap; im.hd = hd; im.kp = kp; im.n_pools = -1;
    }
    bool stale = im.n_pools != st->n_pools;
    if (!stale && st->n_pools > 0)
        stale = im.last_row.size() != (size_t)hd || memcmp(im.last_row.data(), st->pool + (size_t)(st->n_pools - 1) * hd, (size_t)hd * 4) != 0;
    if (stale && st->n_pools > 0)
        if (cudaMemcpyAsync(im.pool, st->pool, (size_t)st->n_pools * hd * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) return CWK_ERR_CUDA;
    // the tails are small and the caller may have rewritten them (reset, prefix restore): they travel every call
    if (cudaMemcpyAsync(im.tails, st->tail_k, (size_t)kp * hd * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) return CWK_ERR_CUDA;
    if (cudaMemcpyAsync(im.tails + kp * hd, st->tail_g, (size_t)kp * hd * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) return CWK_ERR_CUDA;
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return CWK_ERR_CUDA;
    im.n_pools = st->n_pools;
    if (st->n_pools > 0) im.last_row.assign(st->pool + (size_t)(st->n_pools - 1) * hd, st->pool + (size_t)st->n_pools * hd);
    return CWK_OK;
}

// One token of one layer, the reference's mla_latent_decode (src/attention.c:642-902) stage by stage on the device.
// x_host/out_host: H floats each. Returns a cwk status; the message goes to err.
int token_step(cwk_ctx *ctx, Layer &ly, int64_t capacity, int64_t pos, const float *x_host, float *out_host, cwkc_error *err) {
    cudaStream_t st = ctx->stream;
    const int64_t H = ly.H;
    const int nh = ly.nh, nope = ly.nope, vdim = ly.vdim, q_lora = ly.q_lora, kv_lora = ly.kv_lora, kv_dim = ly.kv_dim;
    const int ih = ly.ih, ihd = ly.ihd, kp = ly.kp;
    // floats: x[H] qa[q_lora] q[nh*nope] kva[kv_lora] attn[nh*vdim] out[H] iq[ih*ihd] iwt[ih] isc[pool_cap] | bf16: qabs, cacc | int32: sel
    const int64_t pool_cap = ly.idx ? ly.idx->pool_cap : 0;
    const int64_t topk = ly.idx ? ly.spec->index_topk : 0;
    const size_t nf = (size_t)H * 2 + q_lora + (size_t)nh * nope + kv_lora + (size_t)nh * vdim + (size_t)ih * ihd + ih + pool_cap + 64;
    const size_t nsel = (size_t)topk + kp + 4;
    const size_t need = nf * 4 + (size_t)nh * kv_lora * 2 * 2 + nsel * 4 + 512;
    const size_t pin_need = (size_t)H * 4 * 2 + (size_t)kv_lora * 4 + (size_t)(2 * ihd + ih * ihd + ih + pool_cap) * 4 + nsel * 4 + 256;
    if (!ensure_bufs(need, pin_need, err)) return CWK_ERR_MEMORY;
    float *d_x = g.d_buf, *d_qa = d_x + H, *d_q = d_qa + q_lora, *d_kva = d_q + (size_t)nh * nope;
    float *d_attn = d_kva + kv_lora, *d_out = d_attn + (size_t)nh * vdim, *d_iq = d_out + H, *d_iwt = d_iq + (size_t)ih * ihd;
    float *d_isc = d_iwt + ih;
    uint16_t *d_qabs = (uint16_t *)(((uintptr_t)(d_isc + pool_cap) + 63) & ~(uintptr_t)63), *d_cacc = d_qabs + (size_t)nh * kv_lora;
    int32_t *d_sel = (int32_t *)(d_cacc + (size_t)nh * kv_lora);
    float *p_x = (float *)g.pin, *p_out = p_x + H, *p_row = p_out + H;          // p_row: kv_lora f32, or kv_lora bf16
    float *p_tail = p_row + kv_lora, *p_iq = p_tail + 2 * ihd, *p_iwt = p_iq + (size_t)ih * ihd, *p_sc = p_iwt + ih;
    int32_t *p_sel = (int32_t *)(p_sc + pool_cap);

    int s = sync_cache(ctx, ly, capacity, pos);
    if (s != CWK_OK) { set_err(err, s, "latent cache mirror failed"); return s; }
    CacheMirror &cm = *ly.cm;

    // Outputs the host reads after the call's one synchronise -- the new cache row, the layer's output -- are written by
    // the kernels straight into the page-locked staging buffer when the device can address it: two copy operations less.
    uint8_t *pin_dev = (uint8_t *)g.pin_dev;
    void *a_row = pin_dev ? (void *)(pin_dev + ((uint8_t *)p_row - (uint8_t *)g.pin)) : nullptr;
    float *a_out = pin_dev ? (float *)(pin_dev + ((uint8_t *)p_out - (uint8_t *)g.pin)) : nullptr;
    memcpy(p_x, x_host, (size_t)H * 4);
    cudaMemcpyAsync(d_x, p_x, (size_t)H * 4, cudaMemcpyHostToDevice, st);
    if (ly.qa->kind == ly.kva->kind && ly.qa->cols == ly.kva->cols) {      // q_a and kv_a read the same x: one launch
        const int kind = ly.qa->kind == CWKC_WEIGHT_BF16 ? GEMV_BF16 : ly.qa->kind == CWKC_WEIGHT_F32 ? GEMV_F32 : GEMV_FP8;
        launch_gemv(ctx, kind, ly.qa->data, ly.qa->scales, d_x, d_qa, ly.qa->rows, ly.qa->cols, 1, 0, 0, ly.kva->data, ly.kva->scales, d_kva,
                    ly.kva->rows, 0);
    } else {
        dev_linear(ctx, ly.qa, d_x, d_qa, 1, 0, 0);
        dev_linear(ctx, ly.kva, d_x, d_kva, 1, 0, 0);
    }
    // the caller's array stays the source of truth: the row goes back in the caller's element width
    rms_scale_pair_kernel<<<2, 256, 0, st>>>(d_qa, q_lora, ly.qa_n, d_kva, kv_lora, ly.kva_n, ly.spec->rms_norm_eps_f,
                                             cm.dev + (size_t)pos * kv_lora, a_row, ly.lbf ? 1 : 0);
    dev_linear(ctx, ly.qb, d_qa, d_q, 1, 0, 0);
    if (!a_row) {
        if (ly.lbf) cudaMemcpyAsync(p_row, cm.dev + (size_t)pos * kv_lora, (size_t)kv_lora * 2, cudaMemcpyDeviceToHost, st);
        else cudaMemcpyAsync(p_row, d_kva, (size_t)kv_lora * 4, cudaMemcpyDeviceToHost, st);
    }
    launch_absorb_q(st, d_q, (const uint16_t *)ly.kvb->data, nh, nope, kv_dim, kv_lora, d_qabs, 1);
    ctx->launches += 2;

    // ---- DSA indexer (src/attention.c:716-735): absorb this position, then pick the rows to attend to ----
    int64_t nlist = pos + 1;
    bool use_sel = false;
    if (ly.idx) {
        cwkc_indexer_state *ist = ly.idx;
        IndexMirror &im = *ly.im;
        s = sync_indexer(ctx, ly);
        if (s != CWK_OK) { set_err(err, s, "indexer state mirror failed"); return s; }
        const int64_t r = pos % kp;
        // indexer_absorb (:472-526): this position's raw key and gate rows
        dev_linear(ctx, ly.wk, d_x, im.tails + r * ihd, 1, 0, 0);
        dev_linear(ctx, ly.gate, d_x, im.tails + (kp + r) * ihd, 1, 0, 0);
        cudaMemcpyAsync(p_tail, im.tails + r * ihd, (size_t)ihd * 4, cudaMemcpyDeviceToHost, st);
        cudaMemcpyAsync(p_tail + ihd, im.tails + (kp + r) * ihd, (size_t)ihd * 4, cudaMemcpyDeviceToHost, st);
        bool closed = false;
        if (r == kp - 1 && ist->n_pools < ist->pool_cap && kp <= 8) {
            s = cwk_indexer_pool_compress(ctx, im.tails, im.tails + kp * ihd, ly.ape, ly.k_norm, ly.k_norm_b, 1, kp, ihd,
                                          ly.spec->rms_norm_eps_f, im.pool + ist->n_pools * ihd);
            if (s != CWK_OK) { set_err(err, s, "%s", cwk_last_error(ctx)); return s; }
            closed = true;
        }
        if (cudaStreamSynchronize(st) != cudaSuccess) { set_err(err, CWK_ERR_CUDA, "indexer absorb failed"); return CWK_ERR_CUDA; }
        memcpy(ist->tail_k + r * ihd, p_tail, (size_t)ihd * 4);
        memcpy(ist->tail_g + r * ihd, p_tail + ihd, (size_t)ihd * 4);
        if (closed) {
            if (cudaMemcpy(ist->pool + (size_t)ist->n_pools * ihd, im.pool + ist->n_pools * ihd, (size_t)ihd * 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
                set_err(err, CWK_ERR_CUDA, "pool row read-back failed");
                return CWK_ERR_CUDA;
            }
            im.last_row.assign(ist->pool + (size_t)ist->n_pools * ihd, ist->pool + (size_t)(ist->n_pools + 1) * ihd);
            ist->n_pools++;
            im.n_pools = ist->n_pools;
        }
        // indexer_select (:548-622)
        const int64_t n_comp = ist->n_pools, want = (topk + kp - 1) / kp, npos = pos + 1;
        if (want > 0 && n_comp > want) {
            dev_linear(ctx, ly.wq_b, d_qa, d_iq, 1, 0, 0);
            dev_linear(ctx, ly.weights_proj, d_x, d_iwt, 1, 0, 0);
            const float wscale = 1.0f / sqrtf((float)((double)ihd * (double)ih));
            scale_vec_kernel<<<(ih + 127) / 128, 128, 0, st>>>(d_iwt, ih, wscale);
            pool_scores_kernel<<<(unsigned)((n_comp + 127) / 128), 128, 0, st>>>(im.pool, (int)n_comp, ihd, d_iq, d_iwt, ih, d_isc);
            ctx->launches += 2;
            cudaMemcpyAsync(p_iq, d_iq, (size_t)ih * ihd * 4, cudaMemcpyDeviceToHost, st);
            cudaMemcpyAsync(p_iwt, d_iwt, (size_t)ih * 4, cudaMemcpyDeviceToHost, st);
            cudaMemcpyAsync(p_sc, d_isc, (size_t)n_comp * 4, cudaMemcpyDeviceToHost, st);
            if (cudaStreamSynchronize(st) != cudaSuccess) { set_err(err, CWK_ERR_CUDA, "indexer scores failed"); return CWK_ERR_CUDA; }
            // the reference leaves q, wt and the scores in the state's scratch: so does this
            memcpy(ist->q, p_iq, (size_t)ih * ihd * 4);
            memcpy(ist->wt, p_iwt, (size_t)ih * 4);
            memcpy(ist->sc, p_sc, (size_t)n_comp * 4);
            memcpy(ist->sc2, p_sc, (size_t)n_comp * 4);
            select_front(ist->sc2, n_comp, want);
            const float thr = ist->sc2[want - 1];
            const int64_t cap = want * kp;
            int64_t n = 0;
            int64_t *sel = ist->sel;
            for (int pass = 0; pass < 2 && n < cap; pass++)
                for (int64_t c = 0; c < n_comp && n < cap; c++) {
                    const bool take = pass == 0 ? (ist->sc[c] > thr) : (ist->sc[c] == thr);
                    if (take) for (int64_t rr = 0; rr < kp; rr++) sel[n++] = c * kp + rr;      // the pool's positions
                }
            const int64_t tail = npos % kp;              // positions in no closed pool yet: always kept (:600-604)
            for (int64_t rr = 0; rr < tail; rr++) sel[n++] = npos - tail + rr;
            if (getenv("CWICK_INDEXER_STRICT") == nullptr && (n == 0 || sel[n - 1] != npos - 1)) sel[n++] = npos - 1;   // :618-621
            if (n > 0) {
                for (int64_t i = 0; i < n; i++) p_sel[i] = (int32_t)sel[i];
                cudaMemcpyAsync(d_sel, p_sel, (size_t)n * 4, cudaMemcpyHostToDevice, st);
                nlist = n;
                use_sel = true;
            }
        }
    }

    s = cwk_mla_decode(ctx, d_qabs, cm.dev, 0, kv_lora, nullptr, (int)nlist, use_sel ? d_sel : nullptr, use_sel ? (int64_t)nlist : 0, 1, nh,
                       kv_lora, 0, 1.0f / sqrtf((float)nope), d_cacc, 0);
    if (s != CWK_OK) { set_err(err, s, "%s", cwk_last_error(ctx)); return s; }
    unabsorb_kernel<<<dim3((nh * vdim + 7) / 8, 1), 256, 0, st>>>(d_cacc, (const uint16_t *)ly.kvb->data, nh, nope, vdim, kv_lora, d_attn);
    ctx->launches += 1;
    if (a_out) dev_linear(ctx, ly.o, d_attn, a_out, 1, 0, 0);
    else {
        dev_linear(ctx, ly.o, d_attn, d_out, 1, 0, 0);
        cudaMemcpyAsync(p_out, d_out, (size_t)H * 4, cudaMemcpyDeviceToHost, st);
    }
    if (cudaStreamSynchronize(st) != cudaSuccess || cudaGetLastError() != cudaSuccess) {
        set_err(err, CWK_ERR_CUDA, "GPU decode failed: %s", cudaGetErrorString(cudaGetLastError()));
        return CWK_ERR_CUDA;
    }
    if (cwk_check_device_error(ctx) != CWK_OK) { set_err(err, CWK_ERR_STATE, "%s", cwk_last_error(ctx)); return CWK_ERR_STATE; }
    memcpy(out_host, p_out, (size_t)H * 4);
    memcpy(ly.host_layer + (size_t)pos * ly.host_row_bytes, p_row, ly.host_row_bytes);
    note_row_written(ly, pos);
    return CWK_OK;
}

// A chunk of n tokens of a layer without an indexer: every stage batched over the tokens, the attention as n
// decode-shaped problems over one shared cache (row t sees rows 0..pos0+t), src/attention.c:943-1024.
int chunk_steps(cwk_ctx *ctx, Layer &ly, int64_t capacity, int64_t pos0, int64_t n, const float *X_host, float *Out_host, cwkc_error *err) {
    cudaStream_t st = ctx->stream;
    const int64_t H = ly.H;
    const int nh = ly.nh, nope = ly.nope, vdim = ly.vdim, q_lora = ly.q_lora, kv_lora = ly.kv_lora, kv_dim = ly.kv_dim;
    const size_t per_f = (size_t)H * 2 + q_lora + (size_t)nh * nope + kv_lora + (size_t)nh * vdim;
    const size_t need = (size_t)n * (per_f * 4 + (size_t)nh * kv_lora * 2 * 2 + 4) + 1024;
    if (!ensure_bufs(need, 64, err)) return CWK_ERR_MEMORY;
    float *d_x = g.d_buf, *d_qa = d_x + n * H, *d_q = d_qa + n * q_lora, *d_kva = d_q + n * (size_t)nh * nope;
    float *d_attn = d_kva + n * kv_lora, *d_out = d_attn + n * (size_t)nh * vdim;
    uint16_t *d_qabs = (uint16_t *)(((uintptr_t)(d_out + n * H) + 63) & ~(uintptr_t)63), *d_cacc = d_qabs + n * (size_t)nh * kv_lora;
    int32_t *d_len = (int32_t *)(d_cacc + n * (size_t)nh * kv_lora);
    int s = sync_cache(ctx, ly, capacity, pos0);
    if (s != CWK_OK) { set_err(err, s, "latent cache mirror failed"); return s; }
    CacheMirror &cm = *ly.cm;
    std::vector<int32_t> lens((size_t)n);
    for (int64_t t = 0; t < n; t++) lens[(size_t)t] = (int32_t)(pos0 + t + 1);
    if (cudaMemcpyAsync(d_x, X_host, (size_t)n * H * 4, cudaMemcpyHostToDevice, st) != cudaSuccess ||
        cudaMemcpyAsync(d_len, lens.data(), (size_t)n * 4, cudaMemcpyHostToDevice, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess) {
        set_err(err, CWK_ERR_CUDA, "chunk upload failed");
        return CWK_ERR_CUDA;
    }
    dev_linear(ctx, ly.qa, d_x, d_qa, (int)n, H, q_lora);
    dev_linear(ctx, ly.kva, d_x, d_kva, (int)n, H, kv_lora);
    rms_scale_kernel<<<(unsigned)n, 256, 0, st>>>(d_qa, q_lora, q_lora, ly.qa_n, ly.spec->rms_norm_eps_f, nullptr, 0);
    rms_scale_kernel<<<(unsigned)n, 256, 0, st>>>(d_kva, kv_lora, kv_lora, ly.kva_n, ly.spec->rms_norm_eps_f, cm.dev + (size_t)pos0 * kv_lora, kv_lora);
    dev_linear(ctx, ly.qb, d_qa, d_q, (int)n, q_lora, (int64_t)nh * nope);
    launch_absorb_q(st, d_q, (const uint16_t *)ly.kvb->data, nh, nope, kv_dim, kv_lora, d_qabs, (int)n);
    ctx->launches += 3;
    s = cwk_mla_decode(ctx, d_qabs, cm.dev, 0, kv_lora, d_len, (int)(pos0 + n), nullptr, 0, (int)n, nh, kv_lora, 0, 1.0f / sqrtf((float)nope),
                       d_cacc, 0);
    if (s != CWK_OK) { set_err(err, s, "%s", cwk_last_error(ctx)); return s; }
    launch_unabsorb(st, d_cacc, (const uint16_t *)ly.kvb->data, nh, nope, vdim, kv_lora, d_attn, (int)n);
    ctx->launches += 1;
    dev_linear(ctx, ly.o, d_attn, d_out, (int)n, (int64_t)nh * vdim, H);
    // results and the chunk's cache rows back to the caller (pageable memory: synchronous copies)
    bool ok = cudaMemcpyAsync(Out_host, d_out, (size_t)n * H * 4, cudaMemcpyDeviceToHost, st) == cudaSuccess;
    if (ly.lbf) ok = ok && cudaMemcpyAsync(ly.host_layer + (size_t)pos0 * ly.host_row_bytes, cm.dev + (size_t)pos0 * kv_lora, (size_t)n * kv_lora * 2, cudaMemcpyDeviceToHost, st) == cudaSuccess;
    else ok = ok && cudaMemcpyAsync(ly.host_layer + (size_t)pos0 * ly.host_row_bytes, d_kva, (size_t)n * kv_lora * 4, cudaMemcpyDeviceToHost, st) == cudaSuccess;
    if (!ok || cudaStreamSynchronize(st) != cudaSuccess || cudaGetLastError() != cudaSuccess) {
        set_err(err, CWK_ERR_CUDA, "GPU chunk failed: %s", cudaGetErrorString(cudaGetLastError()));
        return CWK_ERR_CUDA;
    }
    if (cwk_check_device_error(ctx) != CWK_OK) { set_err(err, CWK_ERR_STATE, "%s", cwk_last_error(ctx)); return CWK_ERR_STATE; }
    note_row_written(ly, pos0 + n - 1);
    return CWK_OK;
}

// Resolve a layer call: checks, device context, mirrors. Returns a cwk status.
int resolve_layer(Layer &ly, const cwkc_model_spec *spec, const cwkc_tensor *qa, const cwkc_tensor *qb, const cwkc_tensor *kva,
                  const cwkc_tensor *kvb, const cwkc_tensor *o, const cwkc_tensor *qa_n, const cwkc_tensor *kva_n, float *keys,
                  int64_t capacity, int64_t layer, const cwkc_indexer_weights *idx_w, cwkc_indexer_state *idx, cwkc_error *err) {
    ly.spec = spec;
    ly.H = spec->hidden_size;
    ly.nh = (int)spec->num_attention_heads; ly.nope = (int)spec->qk_nope_head_dim; ly.vdim = (int)spec->value_head_dim;
    ly.q_lora = (int)spec->q_lora_rank; ly.kv_lora = (int)spec->kv_lora_rank; ly.kv_dim = ly.nope + ly.vdim;
    if (ly.kv_lora > 512 || (ly.kv_lora & 7)) { set_err(err, CWK_ERR_UNSUPPORTED, "kv_lora_rank %d not built (multiple of 8, <= 512)", ly.kv_lora); return CWK_ERR_UNSUPPORTED; }
    if (kvb->kind != CWKC_WEIGHT_BF16 || qa_n->kind != CWKC_WEIGHT_BF16 || kva_n->kind != CWKC_WEIGHT_BF16) {
        set_err(err, CWK_ERR_UNSUPPORTED, "kv_b_proj and the two layer norms are handled as BF16 tensors only");
        return CWK_ERR_UNSUPPORTED;
    }
    for (const cwkc_tensor *t : {qa, qb, kva, o})
        if (!kind_ok(t->kind)) { set_err(err, CWK_ERR_UNSUPPORTED, "projection weight kind %d is not handled (BF16, F32, FP8-E4M3)", t->kind); return CWK_ERR_UNSUPPORTED; }
    if (!ensure_ctx(err)) return CWK_ERR_STATE;
    ly.qa = mirror_weight(qa); ly.qb = mirror_weight(qb); ly.kva = mirror_weight(kva); ly.kvb = mirror_weight(kvb); ly.o = mirror_weight(o);
    const WeightMirror *n1 = mirror_weight(qa_n), *n2 = mirror_weight(kva_n);
    if (!ly.qa || !ly.qb || !ly.kva || !ly.kvb || !ly.o || !n1 || !n2) { set_err(err, CWK_ERR_MEMORY, "device mirror of a weight failed"); return CWK_ERR_MEMORY; }
    ly.qa_n = (const uint16_t *)n1->data; ly.kva_n = (const uint16_t *)n2->data;
    ly.lbf = cwick_latent_bf16_enabled();
    ly.host_row_bytes = (size_t)ly.kv_lora * (ly.lbf ? 2 : 4);
    ly.host_layer = (uint8_t *)keys + (size_t)layer * (size_t)capacity * ly.host_row_bytes;
    ly.cm = &g.caches[{(const void *)keys, layer}];
    if (idx_w && idx && spec->index_head_dim > 0 && spec->index_n_heads > 0) {
        ly.idx_w = idx_w; ly.idx = idx;
        ly.ih = (int)spec->index_n_heads; ly.ihd = (int)spec->index_head_dim; ly.kp = spec->index_kpool > 0 ? (int)spec->index_kpool : 1;
        if (!idx_w->wq_b || !idx_w->wk || !idx_w->gate || !idx_w->ape || !idx_w->k_norm || !idx_w->k_norm_b || !idx_w->weights_proj ||
            !idx->pool || !idx->tail_k || !idx->tail_g || !idx->sel || !idx->q || !idx->wt || !idx->sc || !idx->sc2) {
            set_err(err, CWK_ERR_ARGUMENT, "indexer weights or state incomplete");
            return CWK_ERR_ARGUMENT;
        }
        if (idx_w->ape->kind != CWKC_WEIGHT_BF16 || ly.ihd > 1024 || ly.kp > 8) {
            set_err(err, CWK_ERR_UNSUPPORTED, "indexer shape not built (ape BF16, head dim <= 1024, kpool <= 8)");
            return CWK_ERR_UNSUPPORTED;
        }
        ly.wq_b = mirror_weight(idx_w->wq_b); ly.wk = mirror_weight(idx_w->wk); ly.gate = mirror_weight(idx_w->gate);
        ly.weights_proj = mirror_weight(idx_w->weights_proj);
        const WeightMirror *ap = mirror_weight(idx_w->ape);
        ly.k_norm = mirror_vector_f32(idx_w->k_norm, ly.ihd);
        ly.k_norm_b = mirror_vector_f32(idx_w->k_norm_b, ly.ihd);
        if (!ly.wq_b || !ly.wk || !ly.gate || !ly.weights_proj || !ap || !ly.k_norm || !ly.k_norm_b) {
            set_err(err, CWK_ERR_MEMORY, "device mirror of an indexer weight failed");
            return CWK_ERR_MEMORY;
        }
        ly.ape = (const uint16_t *)ap->data;
        ly.im = &g.indexers[(const void *)idx];
    }
    return CWK_OK;
}

}  // namespace

extern "C" {

bool cwick_latent_bf16_enabled(void) {
    // src/attention.c:288-296: CWICK_LATENT_BF16=1|on
    const char *e = getenv("CWICK_LATENT_BF16");
    return e && (e[0] == '1' || strcmp(e, "on") == 0);
}
size_t cwick_latent_elem_bytes(void) { return cwick_latent_bf16_enabled() ? sizeof(uint16_t) : sizeof(float); }
bool cwick_mla_latent_enabled(const cwkc_model_spec *spec, const cwkc_tensor *kvb) { return latent_ok(spec, kvb); }
bool cwick_indexer_active(const cwkc_model_spec *spec, int64_t npos) {
    // src/attention.c:120-125
    if (spec->index_topk <= 0 || spec->index_head_dim <= 0 || spec->index_n_heads <= 0) return false;
    return npos > spec->index_topk;
}

void cwk_dropin_reset(void) {
    std::lock_guard<std::mutex> lock(g.mu);
    if (g.ctx) cwk_ctx_sync(g.ctx);
    for (auto &kv : g.weights) { cudaFree(kv.second.data); if (kv.second.scales) cudaFree(kv.second.scales); }
    g.weights.clear();
    for (auto &kv : g.caches) cudaFree(kv.second.dev);
    g.caches.clear();
    for (auto &kv : g.indexers) { cudaFree(kv.second.pool); cudaFree(kv.second.tails); }
    g.indexers.clear();
}

void cwick_attention_mla_decode(const cwkc_model_spec *spec, const cwkc_tensor *qa, const cwkc_tensor *qb,
                                const cwkc_tensor *kva, const cwkc_tensor *kvb, const cwkc_tensor *gate,
                                const cwkc_tensor *o, const cwkc_tensor *qa_n, const cwkc_tensor *kva_n, float *keys,
                                float *values, int64_t capacity, int64_t pos, int64_t layer,
                                const cwkc_indexer_weights *idx_w, cwkc_indexer_state *idx, const float *x, float *out,
                                cwkc_error *err) {
    (void)gate;
    if (!spec || !qa || !qb || !kva || !kvb || !o || !qa_n || !kva_n || !keys || !x || !out || pos < 0 || pos >= capacity)
        return set_err(err, CWK_ERR_ARGUMENT, "cwick_attention_mla_decode: bad argument");
    if (values != nullptr || !latent_ok(spec, kvb))
        return set_err(err, CWK_ERR_UNSUPPORTED, "expanded-cache MLA decode is not built into the GPU attention library");
    std::lock_guard<std::mutex> lock(g.mu);
    Layer ly;
    if (resolve_layer(ly, spec, qa, qb, kva, kvb, o, qa_n, kva_n, keys, capacity, layer, idx_w, idx, err) != CWK_OK) return;
    token_step(g.ctx, ly, capacity, pos, x, out, err);
}

// cwick_attention_kda_decode (src/attention.c:1176-1437) on the GPU: the six projections of x, the two second-stage
// gates, cwk_kda_step, o_proj. The signature leaves the layer's recurrent state and convolution window with the caller
// and says nothing about when the caller rewrites them (a new sequence zeroes them, a prefix restore replaces them),
// so both travel to the device and back on every call: correct for any caller, and dominated by that traffic
// (4 MB each way at 64 heads of 128). A caller that keeps the state on the device calls cwk_kda_step itself.
extern "C" int cwk_kda_step(cwk_ctx *ctx, int B, int nh, int hd, float lower, float rms_eps, const float *q, const float *k,
                            const float *v, const void *q_conv, const void *k_conv, const void *v_conv, float *conv,
                            const float *gate_raw, const float *dt_bias, const float *a_log, const float *beta_raw,
                            const float *gate, const void *o_norm, float *rec, float *core);

static float tensor_value(const cwkc_tensor *t, int64_t i) {       // cwick_tensor_value, src/tensor.c:767-774
    if (t->kind == CWKC_WEIGHT_BF16) {
        const uint32_t u = (uint32_t)((const uint16_t *)t->data)[i] << 16;
        float f;
        memcpy(&f, &u, 4);
        return f;
    }
    return t->kind == CWKC_WEIGHT_F32 ? ((const float *)t->data)[i] : 0.0f;
}

void cwick_attention_kda_decode(const cwkc_model_spec *spec, const cwkc_tensor *q_proj, const cwkc_tensor *k_proj,
                                const cwkc_tensor *v_proj, const cwkc_tensor *q_conv, const cwkc_tensor *k_conv,
                                const cwkc_tensor *v_conv, const cwkc_tensor *a_log, const cwkc_tensor *dt_bias,
                                const cwkc_tensor *o_norm, const cwkc_tensor *fa_proj, const cwkc_tensor *fb_proj,
                                const cwkc_tensor *b_proj, const cwkc_tensor *ga_proj, const cwkc_tensor *gb_proj,
                                const cwkc_tensor *o_proj, float *rec, float *conv, int64_t layer, const float *x, float *out,
                                cwkc_error *err) {
    const cwkc_tensor *ws[] = {q_proj, k_proj, v_proj, fa_proj, b_proj, ga_proj, fb_proj, gb_proj, o_proj, q_conv, k_conv, v_conv, o_norm};
    if (!spec || !a_log || !dt_bias || !rec || !conv || !x || !out || layer < 0)
        return set_err(err, CWK_ERR_ARGUMENT, "cwick_attention_kda_decode: bad argument");
    for (const cwkc_tensor *t : ws) {
        if (!t || !t->data) return set_err(err, CWK_ERR_ARGUMENT, "cwick_attention_kda_decode: missing tensor");
        if (t->kind != CWKC_WEIGHT_BF16) return set_err(err, CWK_ERR_UNSUPPORTED, "only BF16 weights are handled here");
    }
    const int64_t H = spec->hidden_size;
    const int nh = (int)spec->linear_num_heads, hd = (int)spec->linear_head_dim;
    const int64_t proj = (int64_t)nh * hd;
    if (spec->short_conv_kernel_size != 4) return set_err(err, CWK_ERR_UNSUPPORTED, "short convolution width %lld not built (4)", (long long)spec->short_conv_kernel_size);
    if ((hd != 32 && hd != 64 && hd != 128) || (H & 7)) return set_err(err, CWK_ERR_UNSUPPORTED, "KDA head dim %d / hidden %lld not built", hd, (long long)H);

    std::lock_guard<std::mutex> lock(g.mu);
    if (!ensure_ctx(err)) return;
    cwk_ctx *ctx = g.ctx;
    cudaStream_t st = ctx->stream;
    const uint16_t *d_w[13];
    for (int i = 0; i < 13; i++)
        {
            const WeightMirror *wm = mirror_weight(ws[i]);
            if (!wm) return set_err(err, CWK_ERR_MEMORY, "device mirror of a weight failed");
            d_w[i] = (const uint16_t *)wm->data;
        }
    // floats: x[H] q k v gate_raw gate core [proj each] f_a g_a [hd each] beta a_log [nh each] dt[proj] out[H] rec conv
    const size_t n_rec = (size_t)nh * hd * hd, n_conv = (size_t)3 * proj * 3;
    const size_t nf = (size_t)H * 2 + (size_t)proj * 7 + (size_t)hd * 2 + (size_t)nh * 2 + n_rec + n_conv + 64;
    if (nf * 4 > g.d_buf_bytes) {
        if (g.d_buf) cudaFree(g.d_buf);
        if (cudaMalloc(&g.d_buf, nf * 4) != cudaSuccess) { g.d_buf = nullptr; g.d_buf_bytes = 0; return set_err(err, CWK_ERR_MEMORY, "device scratch"); }
        g.d_buf_bytes = nf * 4;
    }
    float *d_x = g.d_buf, *d_q = d_x + H, *d_k = d_q + proj, *d_v = d_k + proj, *d_graw = d_v + proj, *d_gate = d_graw + proj;
    float *d_core = d_gate + proj, *d_dt = d_core + proj, *d_fa = d_dt + proj, *d_ga = d_fa + hd, *d_beta = d_ga + hd, *d_alog = d_beta + nh;
    float *d_out = d_alog + nh;
    float *d_rec = g.d_buf + ((((size_t)(d_out - g.d_buf) + (size_t)H) + 3) & ~(size_t)3), *d_conv = d_rec + n_rec;     // 16-byte aligned state
    std::vector<float> small((size_t)nh + proj);
    for (int h = 0; h < nh; h++) small[h] = tensor_value(a_log, h);
    for (int64_t i = 0; i < proj; i++) small[nh + i] = tensor_value(dt_bias, i);
    float *h_rec = rec + (size_t)layer * n_rec, *h_conv = conv + (size_t)layer * n_conv;
    cudaMemcpyAsync(d_x, x, (size_t)H * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(d_alog, small.data(), (size_t)nh * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(d_dt, small.data() + nh, (size_t)proj * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(d_rec, h_rec, n_rec * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(d_conv, h_conv, n_conv * 4, cudaMemcpyHostToDevice, st);
    const int P = (int)proj;
    gemv_bf16_kernel<<<dim3((P + 7) / 8, 1), 256, 0, st>>>(d_w[0], d_x, d_q, P, (int)H, 0, 0);
    gemv_bf16_kernel<<<dim3((P + 7) / 8, 1), 256, 0, st>>>(d_w[1], d_x, d_k, P, (int)H, 0, 0);
    gemv_bf16_kernel<<<dim3((P + 7) / 8, 1), 256, 0, st>>>(d_w[2], d_x, d_v, P, (int)H, 0, 0);
    gemv_bf16_kernel<<<dim3((hd + 7) / 8, 1), 256, 0, st>>>(d_w[3], d_x, d_fa, hd, (int)H, 0, 0);
    gemv_bf16_kernel<<<dim3((nh + 7) / 8, 1), 256, 0, st>>>(d_w[4], d_x, d_beta, nh, (int)H, 0, 0);
    gemv_bf16_kernel<<<dim3((hd + 7) / 8, 1), 256, 0, st>>>(d_w[5], d_x, d_ga, hd, (int)H, 0, 0);
    gemv_bf16_kernel<<<dim3((P + 7) / 8, 1), 256, 0, st>>>(d_w[6], d_fa, d_graw, P, hd, 0, 0);
    gemv_bf16_kernel<<<dim3((P + 7) / 8, 1), 256, 0, st>>>(d_w[7], d_ga, d_gate, P, hd, 0, 0);
    ctx->launches += 8;
    int s = cwk_kda_step(ctx, 1, nh, hd, spec->gate_lower_bound, spec->rms_norm_eps_f, d_q, d_k, d_v, d_w[9], d_w[10], d_w[11], d_conv,
                         d_graw, d_dt, d_alog, d_beta, d_gate, d_w[12], d_rec, d_core);
    if (s != CWK_OK) return set_err(err, s, "%s", cwk_last_error(ctx));
    gemv_bf16_kernel<<<dim3((unsigned)((H + 7) / 8), 1), 256, 0, st>>>(d_w[8], d_core, d_out, (int)H, P, 0, 0);
    ctx->launches += 1;
    cudaMemcpyAsync(out, d_out, (size_t)H * 4, cudaMemcpyDeviceToHost, st);
    cudaMemcpyAsync(h_rec, d_rec, n_rec * 4, cudaMemcpyDeviceToHost, st);
    cudaMemcpyAsync(h_conv, d_conv, n_conv * 4, cudaMemcpyDeviceToHost, st);
    if (cudaStreamSynchronize(st) != cudaSuccess || cudaGetLastError() != cudaSuccess)
        return set_err(err, CWK_ERR_CUDA, "GPU KDA decode failed: %s", cudaGetErrorString(cudaGetLastError()));
}

// ---- the rest of attention.c's link surface (src/cwick.h:864-938, src/prof.c:78-85) -------------------------
// The phase timers prof.c reads; the GPU entry points do not split their time into these phases.
uint64_t g_attn_proj_ns = 0, g_attn_conv_ns = 0, g_attn_gate_ns = 0, g_attn_rec_ns = 0, g_attn_mla_ns = 0, g_attn_tail_ns = 0;

// src/attention.c:446-458: floats the engine reserves per KV slot for the indexer's pool, tails, selection and scratch.
uint64_t cwick_indexer_bytes(const cwkc_model_spec *spec, int64_t capacity) {
    const int64_t hd = spec->index_head_dim;
    const int64_t kp = spec->index_kpool > 0 ? spec->index_kpool : 1;
    const int64_t topk = spec->index_topk > 0 ? spec->index_topk : 0;
    if (hd <= 0 || spec->index_n_heads <= 0) return 0;
    const int64_t pools = capacity / kp + 2, sel = topk + kp + 2;
    return (uint64_t)((pools * hd) + (2 * kp * hd) + sel + (spec->index_n_heads * hd) + spec->index_n_heads + 2 * pools) * sizeof(float);
}

// src/attention.c:460-468
void cwick_indexer_reset(const cwkc_model_spec *spec, cwkc_indexer_state *st) {
    if (!st) return;
    const int64_t hd = spec->index_head_dim;
    const int64_t kp = spec->index_kpool > 0 ? spec->index_kpool : 1;
    if (hd > 0 && st->pool) {
        memset(st->pool, 0, (size_t)st->pool_cap * (size_t)hd * sizeof(float));
        memset(st->tail_k, 0, (size_t)kp * (size_t)hd * sizeof(float));
        memset(st->tail_g, 0, (size_t)kp * (size_t)hd * sizeof(float));
    }
    st->n_pools = 0;
}

// src/attention.c:932-941: the chunk path runs for the latent layout with BF16 projections (the reference's own
// condition, kept as it is: the engine asks before it commits to the chunk's pre-mix).
bool cwick_mla_chunk_supported(const cwkc_model_spec *spec, const cwkc_tensor *qa, const cwkc_tensor *qb, const cwkc_tensor *kva,
                               const cwkc_tensor *kvb, const cwkc_tensor *o, const float *values) {
    if (!spec || !qa || !qb || !kva || !kvb || !o) return false;
    const char *e = getenv("CWICK_NO_CHUNK_ATTN");
    if (e && *e && *e != '0') return false;
    if (values != nullptr || !latent_ok(spec, kvb)) return false;
    return qa->kind == CWKC_WEIGHT_BF16 && kva->kind == CWKC_WEIGHT_BF16 && qb->kind == CWKC_WEIGHT_BF16 && o->kind == CWKC_WEIGHT_BF16;
}

// src/attention.c:943-1024. Without an indexer every stage is batched over the chunk's tokens; with one, the
// selection depends on token order (each token absorbs into the pools before it selects), so the tokens run one
// after another through the same stages as the decode entry point.
int cwick_attention_mla_prefill_chunk(const cwkc_model_spec *spec, const cwkc_tensor *qa, const cwkc_tensor *qb, const cwkc_tensor *kva,
                                      const cwkc_tensor *kvb, const cwkc_tensor *o, const cwkc_tensor *qa_n, const cwkc_tensor *kva_n,
                                      float *keys, float *values, int64_t capacity, int64_t pos0, int64_t n, int64_t layer,
                                      const cwkc_indexer_weights *idx_w, cwkc_indexer_state *idx, const float *X, float *Out,
                                      cwkc_error *err) {
    if (!spec || n <= 0 || !keys || !qa || !qb || !kva || !kvb || !o || !qa_n || !kva_n || !X || !Out || pos0 < 0 || pos0 + n > capacity)
        return CWK_ERR_ARGUMENT;
    if (!cwick_mla_chunk_supported(spec, qa, qb, kva, kvb, o, values)) return CWK_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g.mu);
    Layer ly;
    int s = resolve_layer(ly, spec, qa, qb, kva, kvb, o, qa_n, kva_n, keys, capacity, layer, idx_w, idx, err);
    if (s != CWK_OK) return s;
    if (!ly.idx) return chunk_steps(g.ctx, ly, capacity, pos0, n, X, Out, err);
    for (int64_t t = 0; t < n; t++) {
        s = token_step(g.ctx, ly, capacity, pos0 + t, X + t * ly.H, Out + t * ly.H, err);
        if (s != CWK_OK) return s;
    }
    return CWK_OK;
}

}  // extern "C"
