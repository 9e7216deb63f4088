// ds_compress.cu -- the DeepSeek-V4 compressor and the candidate-block level of its indexer
// (src/ds_model.c:1002-1077, :1126-1145), in the reference's operation order so that the stored rows are
// the reference's rows bit for bit:
//   ds_pool_norm_kernel        softmax over the ratio axis per element, weighted sum, RMS norm with a
//                              bf16 weight and bf16-rounded result (mean square summed in double, in index order)
//   ds_rmsnorm_bf16w_kernel    the norm alone (index keys)
//   ds_rope_round_qdq_kernel   rotary on a row's tail (cos/sin formed on the host in double with the C library,
//                              as the reference forms them), bf16 rounding of the tail, e2m1
//                              quantise/dequantise of the row (power-of-two scale per 32, or E4M3 scale per block)
//   ds_block_max_kernel, ds_block_mask_kernel   candidate blocks around the exact top-k of csrc/dsa.cu
// These are latency-sized kernels (one row of 128-512 values per position); they exist so that the rows the
// sparse attention and the indexer read are produced on the device, next to the cache they go into.
// Single-precision divisions and products that decide a rounding use the _rn intrinsics: the file is compiled
// with fast-math, and the reference is compiled without contraction.
#include <cmath>

#include "cwk_common.cuh"
#include "ds_codec.cuh"

namespace {

constexpr int DC_THREADS = 256;
constexpr int DC_MAX_RATIO = 64;

// y[i] = bf16(w[i] * (x[i] * r)), r = (float)(1 / sqrt(mean(x^2) + eps)) with the mean in double.
// x in shared memory; thread 0 sums in index order (n is 128-512).
__device__ void rmsnorm_bf16w_row(const float *xs, const uint16_t *w, int n, float eps, float *y, float *s_r) {
    if (threadIdx.x == 0) {
        double acc = 0.0;
        for (int i = 0; i < n; i++) acc += (double)xs[i] * (double)xs[i];
        *s_r = (float)(1.0 / sqrt(acc / n + (double)eps));
    }
    __syncthreads();
    const float r = *s_r;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float t = __fmul_rn(xs[i], r);
        y[i] = bf16_round_rne(w ? __fmul_rn(bf16_bits_to_f32(w[i]), t) : t);
    }
}

// One block per row b: state, score [B][ratio][hd] -> latent [B][hd].
__global__ void __launch_bounds__(DC_THREADS) ds_pool_norm_kernel(const float *state, const float *score, int ratio, int hd,
                                                                  const uint16_t *norm_w, float eps, float *latent) {
    extern __shared__ float xs[];                     // [hd] pooled row, then one word for the norm factor
    const float *st = state + (int64_t)blockIdx.x * ratio * hd, *sc = score + (int64_t)blockIdx.x * ratio * hd;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) {
        float w[DC_MAX_RATIO];
        float mx = -INFINITY, s = 0.f, acc = 0.f;
        for (int r = 0; r < ratio; r++) mx = fmaxf(mx, sc[(int64_t)r * hd + i]);
        for (int r = 0; r < ratio; r++) {
            w[r] = (float)exp((double)__fsub_rn(sc[(int64_t)r * hd + i], mx));      // expf of the C library is correctly rounded in all but rare cases
            s = __fadd_rn(s, w[r]);
        }
        for (int r = 0; r < ratio; r++) acc = __fadd_rn(acc, __fmul_rn(st[(int64_t)r * hd + i], __fdiv_rn(w[r], s)));
        xs[i] = acc;
    }
    __syncthreads();
    rmsnorm_bf16w_row(xs, norm_w, hd, eps, latent + (int64_t)blockIdx.x * hd, xs + hd);
}

__global__ void __launch_bounds__(DC_THREADS) ds_rmsnorm_bf16w_kernel(const float *x, const uint16_t *w, int n, float eps, float *y) {
    extern __shared__ float xs[];
    for (int i = threadIdx.x; i < n; i += blockDim.x) xs[i] = x[(int64_t)blockIdx.x * n + i];
    __syncthreads();
    rmsnorm_bf16w_row(xs, w, n, eps, y + (int64_t)blockIdx.x * n, xs + n);
}

__device__ __forceinline__ float fp4_round_ref(float v) {       // src/ds_ops.c:212-226, as written there
    const float a = fabsf(v);
    float r;
    if (a <= 0.25f) r = 0.f;
    else if (a <= 1.25f) r = 1.f;
    else if (a <= 2.5f) r = 2.f;
    else if (a <= 5.0f) r = 4.f;
    else r = 6.f;
    return v < 0.f ? -r : r;
}

struct RopeTable {
    float c[64], s[64];
};

// One block per row: rotary + bf16 rounding of the last 2*npairs values, then the row's quantise/dequantise.
// mode 0: scale 2^ceil(log2(amax/6)) per 32 values (src/ds_ops.c:254-272); mode 1: scale = E4M3(amax/6) per
// `block` values (:274-293); mode 2: the attention output before its projections (src/ds_model.c:1258-1272):
// the whole row is rounded to bf16 first, the table holds the inverse rotation, nothing is quantised;
// mode 3: rotation and rounding only (the query heads, src/ds_model.c:1188-1193); mode 4: E4M3 with a
// power-of-two scale per 32 values (ds_qdq_fp8_e8m0, src/ds_ops.c:235-252: amax floor 1e-4, scale
// 2^ceil(log2(amax / 448)), clamp to +-448, the reference's own encoder), the window KV row (:1201-1205).
// copy_to (optional): row r is also written to copy_to + r*n (the window ring slot, :1211-1212).
__global__ void __launch_bounds__(DC_THREADS) ds_rope_round_qdq_kernel(float *x, int n, int npairs, const RopeTable tab, int mode, int block,
                                                                       float *copy_to) {
    extern __shared__ float xs[];
    float *row = x + (int64_t)blockIdx.x * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) xs[i] = mode == 2 ? bf16_round_rne(row[i]) : row[i];
    __syncthreads();
    float *t = xs + n - 2 * npairs;
    for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
        const float a = t[2 * i], b = t[2 * i + 1], c = tab.c[i], s = tab.s[i];
        t[2 * i] = bf16_round_rne(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)));
        t[2 * i + 1] = bf16_round_rne(__fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c)));
    }
    __syncthreads();
    const int bl = (mode == 0 || mode == 4) ? 32 : block;
    for (int g = threadIdx.x; mode != 2 && mode != 3 && g < n / bl; g += blockDim.x) {
        float *v = xs + g * bl;
        float amax = 0.f;
        for (int i = 0; i < bl; i++) amax = fmaxf(amax, fabsf(v[i]));
        float sc;
        if (mode == 4) {
            if (amax < 1e-4f) amax = 1e-4f;
            const uint32_t u = __float_as_uint(__fmul_rn(amax, 1.0f / 448.0f));
            const int e = (int)((u >> 23) & 0xFFu) - 127 + ((u & 0x7FFFFFu) ? 1 : 0);
            sc = __uint_as_float((uint32_t)(e + 127) << 23);
            for (int i = 0; i < bl; i++) {
                float q = __fdiv_rn(v[i], sc);
                q = fminf(fmaxf(q, -448.f), 448.f);
                v[i] = __fmul_rn(e4m3_quantise_dequantise_ref(q), sc);
            }
            continue;
        }
        if (mode == 0) {
            const float fl = 6.0f * 1.1754943508222875e-38f;              // 6 * 2^-126
            if (amax <= fl) {
                sc = 1.1754943508222875e-38f;                             // the floor's scale, 2^-126 (its amax / 6 rounds to exactly that)
            } else {
                const uint32_t u = __float_as_uint(__fmul_rn(amax, 1.0f / 6.0f));
                const int e = (int)((u >> 23) & 0xFFu) - 127 + ((u & 0x7FFFFFu) ? 1 : 0);
                sc = __uint_as_float((uint32_t)(e + 127) << 23);
            }
        } else {
            const float fl = 6.0f * 0.001953125f;                         // 6 * 2^-9
            if (amax < fl) amax = fl;
            sc = e4m3_quantise_dequantise_ref(__fmul_rn(amax, 1.0f / 6.0f));
        }
        for (int i = 0; i < bl; i++) {
            float q = __fdiv_rn(v[i], sc);
            q = fminf(fmaxf(q, -6.f), 6.f);
            v[i] = __fmul_rn(fp4_round_ref(q), sc);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        row[i] = xs[i];
        if (copy_to) copy_to[(int64_t)blockIdx.x * n + i] = xs[i];
    }
}

// Maximum of every block of bs scores; the last block is forced in with +inf; word [nblk_out] gets the count.
__global__ void ds_block_max_kernel(const float *sc, int n, int bs, float *bsc, int32_t *nblk_out) {
    const int nblk = (n + bs - 1) / bs;
    const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (blockIdx.x == 0 && threadIdx.x == 0) *nblk_out = nblk;
    if (b >= nblk) return;
    const int hi = min(n, (b + 1) * bs);
    float mx = -INFINITY;
    for (int t = b * bs + lane; t < hi; t += 32) mx = fmaxf(mx, sc[t]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) bsc[b] = (b == (n - 1) / bs) ? INFINITY : mx;
}

// cand[t] = 1 where t's block is in the ascending list of kept blocks.
__global__ void ds_block_mask_kernel(const int32_t *blk, const int32_t *count, int n, int bs, uint8_t *cand) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n) return;
    const int b = t / bs, k = *count;
    int lo = 0, hi = k;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (blk[mid] < b) lo = mid + 1; else hi = mid;
    }
    cand[t] = (lo < k && blk[lo] == b) ? 1 : 0;
}

// What the layers that use the candidates do first: scores outside kept blocks become -inf (src/ds_model.c:1146-1149).
__global__ void ds_mask_scores_kernel(float *sc, const uint8_t *cand, int n) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n && !cand[t]) sc[t] = -INFINITY;
}

}  // namespace

extern "C" {

int cwk_ds_pool_norm(cwk_ctx *ctx, const float *state, const float *score, int B, int ratio, int hd, const void *norm_w,
                     float eps, float *latent) {
    if (!ctx || !state || !score || !latent || B <= 0 || ratio <= 0 || ratio > DC_MAX_RATIO || hd <= 0 || hd > 8192)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_pool_norm: bad argument (ratio 1..%d, hd 1..8192)", DC_MAX_RATIO);
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    ds_pool_norm_kernel<<<B, DC_THREADS, (hd + 1) * sizeof(float), ctx->stream>>>(state, score, ratio, hd, (const uint16_t *)norm_w, eps, latent);
    CWK_LAUNCH_CHECK(ctx, "ds_pool_norm_kernel");
    return CWK_OK;
}

int cwk_ds_rmsnorm_bf16w(cwk_ctx *ctx, const float *x, const void *w, int rows, int n, float eps, float *y) {
    if (!ctx || !x || !y || rows <= 0 || n <= 0 || n > 8192) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_rmsnorm_bf16w: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    ds_rmsnorm_bf16w_kernel<<<rows, DC_THREADS, (n + 1) * sizeof(float), ctx->stream>>>(x, (const uint16_t *)w, n, eps, y);
    CWK_LAUNCH_CHECK(ctx, "ds_rmsnorm_bf16w_kernel");
    return CWK_OK;
}

static int rope_rows_launch(cwk_ctx *ctx, const char *what, float *x, int rows, int n, const float *freq, int npairs, int64_t pos,
                            int mode, int block, float *copy_to = nullptr) {
    if (!ctx || !x || rows <= 0 || n <= 0 || n > 8192 || npairs < 0 || npairs > 64 || 2 * npairs > n || (npairs && !freq))
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "%s: bad argument", what);
    const int bl = (mode == 0 || mode == 4) ? 32 : block;
    if (mode != 2 && mode != 3 && ((mode != 0 && mode != 1 && mode != 4) || bl <= 0 || bl > 128 || n % bl))
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "%s: the row length must be a multiple of the scale block (<= 128)", what);
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    RopeTable tab;
    for (int i = 0; i < npairs; i++) {          // the reference's own expressions (src/ds_ops.c:51-53), on the host's C library
        const double ang = (double)freq[i] * (double)pos;
        tab.c[i] = (float)cos(ang);
        tab.s[i] = (float)sin(ang);
        if (mode == 2) tab.s[i] = -tab.s[i];
    }
    for (int i = npairs; i < 64; i++) tab.c[i] = tab.s[i] = 0.f;
    ds_rope_round_qdq_kernel<<<rows, DC_THREADS, n * sizeof(float), ctx->stream>>>(x, n, npairs, tab, mode, block, copy_to);
    CWK_LAUNCH_CHECK(ctx, "ds_rope_round_qdq_kernel");
    return CWK_OK;
}

int cwk_ds_rope_round_qdq(cwk_ctx *ctx, float *x, int rows, int n, const float *freq, int npairs, int64_t pos, int mode,
                          int block) {
    if (mode < 0 || mode > 3) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_rope_round_qdq: mode is 0..3");
    // public 2 = rotation and rounding only, 3 = E4M3 with power-of-two scales (kernel modes 3 and 4; 2 is the un-rotation)
    return rope_rows_launch(ctx, "ds_rope_round_qdq", x, rows, n, freq, npairs, pos, mode >= 2 ? mode + 1 : mode, block);
}

int cwk_ds_kv_row_store(cwk_ctx *ctx, float *kv, int n, const float *freq, int npairs, int64_t pos, float *win_kv, int window) {
    if (!win_kv || window <= 0 || pos < 0) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_kv_row_store: bad argument");
    return rope_rows_launch(ctx, "ds_kv_row_store", kv, 1, n, freq, npairs, pos, 4, 32, win_kv + (pos % window) * (int64_t)n);
}

int cwk_ds_out_unrope(cwk_ctx *ctx, float *o, int rows, int n, const float *freq, int npairs, int64_t pos) {
    return rope_rows_launch(ctx, "ds_out_unrope", o, rows, n, freq, npairs, pos, 2, 0);
}

int cwk_ds_topk(cwk_ctx *ctx, const float *sc, int64_t sc_stride, const int32_t *n, int B, int k, int32_t *out, int64_t out_ld,
                int32_t *count);

int cwk_ds_candidates(cwk_ctx *ctx, const float *sc, int n, int bs, int kblocks, uint8_t *cand) {
    if (!ctx || !sc || !cand || n <= 0 || bs <= 0 || kblocks <= 0) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_candidates: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const int nblk = (n + bs - 1) / bs;
    // work: block maxima [nblk] | kept blocks [kblocks] | block count | kept count
    int s = cwk_reserve_work(ctx, ((size_t)nblk + kblocks + 2) * sizeof(float));
    if (s != CWK_OK) return s;
    float *bsc = (float *)ctx->work;
    int32_t *blk = (int32_t *)(bsc + nblk), *nb = blk + kblocks, *cnt = nb + 1;
    ds_block_max_kernel<<<(nblk + 7) / 8, 256, 0, ctx->stream>>>(sc, n, bs, bsc, nb);
    CWK_LAUNCH_CHECK(ctx, "ds_block_max_kernel");
    s = cwk_ds_topk(ctx, bsc, nblk, nb, 1, kblocks, blk, kblocks, cnt);
    if (s != CWK_OK) return s;
    ds_block_mask_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>(blk, cnt, n, bs, cand);
    CWK_LAUNCH_CHECK(ctx, "ds_block_mask_kernel");
    return CWK_OK;
}

int cwk_ds_mask_candidates(cwk_ctx *ctx, float *sc, const uint8_t *cand, int n) {
    if (!ctx || !sc || !cand || n <= 0) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "ds_mask_candidates: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    ds_mask_scores_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>(sc, cand, n);
    CWK_LAUNCH_CHECK(ctx, "ds_mask_scores_kernel");
    return CWK_OK;
}

}  // extern "C"
