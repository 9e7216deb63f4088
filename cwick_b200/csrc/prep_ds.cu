// prep_ds.cu -- the small pieces either side of the attention reductions, and the DeepSeek-V4
// variants of the sparse path: Qwen3.5 q/k norm + partial RoPE + cache store and the sigmoid output
// gate; the GLM indexer's pool compression; DeepSeek's sparse attention with a sink term, its
// indexer scores (bf16-rounded head dots) and its block-scaled FP8 projection with quantised
// activations.
#include "cwk_common.cuh"
#include "ds_codec.cuh"

namespace {

__device__ __forceinline__ uint16_t to_bf16(float v) { return (uint16_t)(pack_bf16x2(v, 0.f) & 0xffffu); }

// One block of `hd` threads per (token, head). Heads 0..nh-1 are query heads (input stride 2*hd, the
// gate half skipped), heads nh..nh+nkv-1 key heads, nh+nkv.. value heads (copied).
// rms_norm_w with (1+w) weights and f32 accumulation in index order (src/q35_model.c:112-122) is
// reproduced by a serial sum in thread 0 -- hd is 256, and this keeps the reference's order;
// rotate-half RoPE on the first `rot` dims with cos/sin of pos * theta^(-2i/rot) formed in double
// (src/q35_model.c:144-153, :459-477).
__global__ void gqa_qk_prep_kernel(const float *qg, const float *k, const float *v, const float *q_norm,
                                   const float *k_norm, float eps, int rot, double theta, int64_t pos0, int nh, int nkv,
                                   int hd, uint16_t *q_out, uint16_t *kc, uint16_t *vc) {
    const int t = blockIdx.y, head = blockIdx.x, i = threadIdx.x;
    extern __shared__ float sh[];          // [hd] values, [1] rstd
    const float *src;
    const float *w = nullptr;
    uint16_t *dst;
    if (head < nh) {
        src = qg + ((int64_t)t * nh + head) * 2 * hd;
        w = q_norm;
        dst = q_out + ((int64_t)t * nh + head) * hd;
    } else if (head < nh + nkv) {
        src = k + ((int64_t)t * nkv + (head - nh)) * hd;
        w = k_norm;
        dst = kc + ((pos0 + t) * nkv + (head - nh)) * hd;
    } else {
        src = v + ((int64_t)t * nkv + (head - nh - nkv)) * hd;
        dst = vc + ((pos0 + t) * nkv + (head - nh - nkv)) * hd;
        dst[i] = to_bf16(src[i]);
        return;
    }
    sh[i] = src[i];
    __syncthreads();
    if (i == 0) {
        float acc = 0.f;
        for (int j = 0; j < hd; j++) acc = __fadd_rn(acc, __fmul_rn(sh[j], sh[j]));
        sh[hd] = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(acc, (float)hd), eps)));
    }
    __syncthreads();
    const float rstd = sh[hd];
    float val = __fmul_rn(__fmul_rn(sh[i], rstd), __fadd_rn(1.0f, w[i]));
    __syncthreads();
    sh[i] = val;
    __syncthreads();
    const int pairs = rot / 2;
    if (i < rot) {
        const int j = i < pairs ? i : i - pairs;
        const double inv = 1.0 / pow(theta, (double)(2 * j) / (double)rot);
        const double a = (double)(pos0 + t) * inv;
        const float c = (float)cos(a), s = (float)sin(a);
        const float lo = sh[j], hi = sh[j + pairs];
        val = (i < pairs) ? __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, s)) : __fadd_rn(__fmul_rn(hi, c), __fmul_rn(lo, s));
    }
    dst[i] = to_bf16(val);
}

// o[t][h][i] = attn[t][h][i] * sigmoid(gate), gate = qg[t][h][hd + i] (src/q35_model.c:1749-1760).
__global__ void gqa_gate_kernel(const uint16_t *attn, const float *qg, int64_t total, int hd, float *out) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int64_t th = idx / hd;
    const int i = (int)(idx % hd);
    const float g = qg[th * 2 * hd + hd + i];
    out[idx] = bf16_bits_to_f32(attn[idx]) * (1.0f / (1.0f + expf(-g)));
}

// One block per pool: layer-norm each of the kp raw key rows (mean/variance in double), softmax over
// the kp rows of gate + ape per dimension, affine k_norm on the way (src/attention.c:490-525).
__global__ void indexer_pool_kernel(const float *tail_k, const float *tail_g, const uint16_t *ape, const float *k_norm,
                                    const float *k_norm_b, int kp, int hd, float eps, float *pool) {
    const int pidx = blockIdx.x, d = threadIdx.x;
    const float *tk = tail_k + (int64_t)pidx * kp * hd, *tg = tail_g + (int64_t)pidx * kp * hd;
    __shared__ float s_mean[8], s_inv[8];
    if (d < kp) {
        const float *row = tk + d * hd;
        double s = 0.0;
        for (int j = 0; j < hd; j++) s += (double)row[j];
        const float mean = (float)(s / (double)hd);
        double var = 0.0;
        for (int j = 0; j < hd; j++) { const double t = (double)row[j] - (double)mean; var += t * t; }
        s_mean[d] = mean;
        s_inv[d] = __fdiv_rn(1.0f, sqrtf(__fadd_rn((float)(var / (double)hd), eps)));
    }
    __syncthreads();
    if (d >= hd) return;
    float mx = -INFINITY;
    for (int i = 0; i < kp; i++) mx = fmaxf(mx, __fadd_rn(tg[i * hd + d], bf16_bits_to_f32(ape[i * hd + d])));
    float den = 0.f, acc = 0.f;
    for (int i = 0; i < kp; i++) {
        const float lg = __fadd_rn(tg[i * hd + d], bf16_bits_to_f32(ape[i * hd + d]));
        const float pw = expf(__fsub_rn(lg, mx));
        den = __fadd_rn(den, pw);
        const float nrm = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(tk[i * hd + d], s_mean[i]), s_inv[i]), k_norm[d]), k_norm_b[d]);
        acc = __fadd_rn(acc, __fmul_rn(pw, nrm));
    }
    pool[(int64_t)pidx * hd + d] = den > 0.f ? __fdiv_rn(acc, den) : 0.f;
}

// DeepSeek sparse attention, one block (256 threads) per head. Keys == values == f32 rows of HD,
// gathered through idx (negative = skip); scores f32, the denominator also takes exp(sink[h]-max)
// (src/ds_model.c:917-966). `total` <= 1024.
__global__ void __launch_bounds__(256) ds_sparse_attn_kernel(const float *q, const float *kv, const int *idx, int total,
                                                             int HD, const float *sink, float scale, float *o) {
    const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __shared__ float sc[1024];
    __shared__ float red[8];
    const float *qh = q + (int64_t)h * HD;
    for (int j = warp; j < total; j += 8) {
        const int t = idx[j];
        float d = 0.f;
        if (t >= 0) {
            const float *kt = kv + (int64_t)t * HD;
            for (int i = lane; i < HD; i += 32) d += qh[i] * kt[i];
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        if (lane == 0) sc[j] = (t >= 0) ? d * scale : -INFINITY;
    }
    __syncthreads();
    float mx = -1e30f;
    for (int j = tid; j < total; j += 256) mx = fmaxf(mx, sc[j]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < 8; w++) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float sum = 0.f;
    for (int j = tid; j < total; j += 256) {
        const float e = (idx[j] >= 0) ? expf(sc[j] - mx) : 0.f;
        sc[j] = e;
        sum += e;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = expf(sink[h] - mx);
    for (int w = 0; w < 8; w++) sum += red[w];
    const float inv = 1.0f / sum;
    for (int i = tid; i < HD; i += 256) {
        float acc = 0.f;
        for (int j = 0; j < total; j++) {
            const int t = idx[j];
            if (t >= 0) acc += sc[j] * kv[(int64_t)t * HD + i];
        }
        o[(int64_t)h * HD + i] = acc * inv;
    }
}

// DeepSeek indexer score of one key per thread: per head a sequential f32 dot (separate multiply and
// add, index order), rounded to bf16, ReLU, times the head weight, heads in order
// (src/ds_model.c:1108-1121). q in shared memory.
__global__ void __launch_bounds__(128) ds_indexer_scores_kernel(const float *keys, const float *q, const float *w, int n,
                                                                int ih, int hd, float *sc) {
    extern __shared__ float sq[];          // [ih][hd] + [ih]
    for (int i = threadIdx.x; i < ih * hd; i += 128) sq[i] = q[i];
    for (int i = threadIdx.x; i < ih; i += 128) sq[ih * hd + i] = w[i];
    __syncthreads();
    const int t = blockIdx.x * 128 + threadIdx.x;
    if (t >= n) return;
    const float *kt = keys + (int64_t)t * hd;
    float acc = 0.f;
    for (int h = 0; h < ih; h++) {
        const float *qh = sq + h * hd;
        float d = 0.f;
        for (int i = 0; i < hd; i++) d = __fadd_rn(d, __fmul_rn(qh[i], kt[i]));
        d = bf16_round_rne(d);
        if (d > 0.f) acc = __fadd_rn(acc, __fmul_rn(d, sq[ih * hd + h]));
    }
    sc[t] = acc;
}

// DeepSeek quantised projection of one activation row. Step 1 (one block): per 32 activations the
// E4M3 codes (round to nearest even with the reference encoder's subnormal quirk) and the
// power-of-two scale (src/ds_quant.c:143-159). Step 2: one warp per output row, lanes over the
// 32-wide blocks: (sum_32 e4m3(w) * a) * a_scale * 2^(w_scale-127), summed, rounded to bf16
// (src/ds_quant.c:653-666, src/ds_model.c:880-885).
__global__ void __launch_bounds__(256) ds_act_quant_kernel(const float *x, int64_t K, float *af, float *asf) {
    for (int64_t b = threadIdx.x; b < K / 32; b += 256) {
        float amax = 0.f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[b * 32 + i]));
        if (amax < 1e-4f) amax = 1e-4f;
        const uint32_t u = __float_as_uint(__fmul_rn(amax, 1.0f / 448.0f));
        const int e = (int)((u >> 23) & 0xFF) - 127 + ((u & 0x7FFFFF) ? 1 : 0);
        const float sc = ldexpf(1.0f, e);
        asf[b] = sc;
        for (int i = 0; i < 32; i++) {
            float qv = __fdiv_rn(x[b * 32 + i], sc);
            qv = fminf(fmaxf(qv, -448.f), 448.f);
            af[b * 32 + i] = e4m3_quantise_dequantise_ref(qv);
        }
    }
}
__global__ void __launch_bounds__(256) ds_fp8_gemv_kernel(const uint8_t *w, const uint8_t *w_scale, const float *af,
                                                          const float *asf, int64_t N, int64_t K, float *out) {
    const int64_t n = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (n >= N) return;
    const int64_t nb = K / 32;
    const uint8_t *row = w + n * K, *rs = w_scale + (n / 32) * nb;
    float acc = 0.f;
    for (int64_t b = lane; b < nb; b += 32) {
        const uint4 *p = reinterpret_cast<const uint4 *>(row + b * 32);
        float part = 0.f;
#pragma unroll
        for (int v = 0; v < 2; v++) {
            const uint4 c = p[v];
            const uint32_t u[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
            for (int k = 0; k < 4; k++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    part = __fadd_rn(part, __fmul_rn(e4m3f((u[k] >> (8 * j)) & 0xffu), af[b * 32 + v * 16 + k * 4 + j]));
        }
        acc += (part * asf[b]) * __uint_as_float((uint32_t)rs[b] << 23);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) out[n] = bf16_round_rne(acc);
}

}  // namespace

extern "C" {

int cwk_gqa_qk_prep(cwk_ctx *ctx, const float *qg, const float *k, const float *v, const float *q_norm, const float *k_norm,
                    float eps, int rot, double theta, int64_t pos0, int n, int nh, int nkv, int hd, void *q_out, void *kcache,
                    void *vcache) {
    if (!ctx || !qg || !k || !v || !q_norm || !k_norm || !q_out || !kcache || !vcache || n <= 0 || hd <= 0 || hd > 1024 ||
        rot < 0 || rot > hd || (rot & 1))
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "gqa_qk_prep: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    gqa_qk_prep_kernel<<<dim3(nh + 2 * nkv, n), hd, (hd + 1) * sizeof(float), ctx->stream>>>(
        qg, k, v, q_norm, k_norm, eps, rot, theta, pos0, nh, nkv, hd, (uint16_t *)q_out, (uint16_t *)kcache, (uint16_t *)vcache);
    CWK_LAUNCH_CHECK(ctx, "gqa_qk_prep_kernel");
    return CWK_OK;
}

int cwk_gqa_gate(cwk_ctx *ctx, const void *attn, const float *qg, int n, int nh, int hd, float *out) {
    if (!ctx || !attn || !qg || !out || n <= 0) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "gqa_gate: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const int64_t total = (int64_t)n * nh * hd;
    gqa_gate_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>((const uint16_t *)attn, qg, total, hd, out);
    CWK_LAUNCH_CHECK(ctx, "gqa_gate_kernel");
    return CWK_OK;
}

int cwk_indexer_pool_compress(cwk_ctx *ctx, const float *tail_k, const float *tail_g, const void *ape, const float *k_norm,
                              const float *k_norm_b, int n_pools, int kp, int hd, float eps, float *pool) {
    if (!ctx || !tail_k || !tail_g || !ape || !k_norm || !k_norm_b || !pool || n_pools <= 0 || kp <= 0 || kp > 8 || hd <= 0 || hd > 1024)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "indexer_pool_compress: bad argument (kpool <= 8)");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    indexer_pool_kernel<<<n_pools, ((hd > kp ? hd : kp) + 31) / 32 * 32, 0, ctx->stream>>>(tail_k, tail_g, (const uint16_t *)ape, k_norm,
                                                                                      k_norm_b, kp, hd, eps, pool);
    CWK_LAUNCH_CHECK(ctx, "indexer_pool_kernel");
    return CWK_OK;
}

int cwk_ds_sparse_attn(cwk_ctx *ctx, const float *q, const float *kv, const int32_t *idx, int total, int nh, int HD,
                       const float *sink, float scale, float *o) {
    if (!ctx || !q || !kv || !idx || !sink || !o || total < 0 || total > 1024 || nh <= 0 || HD <= 0)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_sparse_attn: bad argument (at most 1024 selected rows)");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    CwkKernelTimer timer(ctx);
    ds_sparse_attn_kernel<<<nh, 256, 0, ctx->stream>>>(q, kv, idx, total, HD, sink, scale, o);
    CWK_LAUNCH_CHECK(ctx, "ds_sparse_attn_kernel");
    return CWK_OK;
}

int cwk_ds_indexer_scores(cwk_ctx *ctx, const float *keys, const float *q, const float *w, int n, int ih, int hd, float *sc) {
    if (!ctx || !keys || !q || !w || !sc || n < 0 || ih <= 0 || hd <= 0) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_indexer_scores: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (n == 0) return CWK_OK;
    const size_t smem = (size_t)(ih * hd + ih) * sizeof(float);
    if (smem > 48 * 1024) CWK_CUDA(ctx, cudaFuncSetAttribute(ds_indexer_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CwkKernelTimer timer(ctx);
    ds_indexer_scores_kernel<<<(n + 127) / 128, 128, smem, ctx->stream>>>(keys, q, w, n, ih, hd, sc);
    CWK_LAUNCH_CHECK(ctx, "ds_indexer_scores_kernel");
    return CWK_OK;
}

int cwk_ds_lin_q(cwk_ctx *ctx, const float *x, const void *w, const void *w_scale, int64_t N, int64_t K, float *out) {
    if (!ctx || !x || !w || !w_scale || !out || N <= 0 || K <= 0 || (K % 32) != 0 || ((uintptr_t)w % 16) != 0)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_lin_q: bad argument (K multiple of 32, w 16-byte aligned)");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    int s = cwk_reserve_work(ctx, (size_t)(K + K / 32) * sizeof(float));
    if (s != CWK_OK) return s;
    float *af = (float *)ctx->work, *asf = af + K;
    ds_act_quant_kernel<<<1, 256, 0, ctx->stream>>>(x, K, af, asf);
    CWK_LAUNCH_CHECK(ctx, "ds_act_quant_kernel");
    CwkKernelTimer timer(ctx);
    ds_fp8_gemv_kernel<<<(unsigned)((N + 7) / 8), 256, 0, ctx->stream>>>((const uint8_t *)w, (const uint8_t *)w_scale, af, asf, N, K, out);
    CWK_LAUNCH_CHECK(ctx, "ds_fp8_gemv_kernel");
    return CWK_OK;
}

}  // extern "C"
