// mla_prefill.cu -- MLA causal prefill of a chunk of n tokens: FP8 block-scaled
// q/kv projections, RMS norms, RoPE on the 64 rope dims, the absorb of q_nope
// through W_uk, the latent-cache rows, and causal absorbed attention.
//
// The reference does this per token (cwick_attention_mla_prefill_chunk,
// src/attention.c:943-1024: three projection GEMMs, per-token norms and latent
// writes, then mla_latent_decode per token). Here every stage is one batched
// kernel over the chunk, and the attention is one launch in which query i sees
// cache rows 0..pos0+i.
#include <algorithm>

#include "cwk_common.cuh"

// cos/sin of the reference's rope angle, pos / powf(base, 2i/n) (src/attention.c:62), formed the
// way a correctly rounding float libm forms it: the power in double rounded once to float, an
// IEEE float division, then cos/sin of that float angle in double. (The library is compiled
// with fast-math; at positions in the thousands its approximate powf/sincosf would move the
// angle by more than a bf16 step of the result.)
__device__ __forceinline__ void rope_cos_sin(int64_t pos, int i, int n_rope, float base, float &cs, float &sn) {
    const float den = (float)pow((double)base, (double)(2.0f * (float)i / (float)n_rope));
    const float ang = __fdiv_rn((float)pos, den);
    double s, c;
    sincos((double)ang, &s, &c);
    cs = (float)c;
    sn = (float)s;
}

// f32 -> bf16 exactly as the reference narrows a latent-cache row (cwick_f32_to_bf16,
// src/util.c:202-210: add bit15 + lsb, keep the top half -- in effect a truncation). Used for
// the cache rows so that a cache written here is bit-compatible with one the reference wrote.
__device__ __forceinline__ uint16_t narrow_bf16_like_reference(float f) {
    const uint32_t u = __float_as_uint(f);
    return (uint16_t)((u + ((u >> 15) & 1u) + ((u >> 16) & 1u)) >> 16);
}

extern "C" int cwk_fp8_linear(cwk_ctx *ctx, const void *X, const void *W, const float *scale_inv, int64_t n,
                              int64_t k, int64_t cols, void *Y, int out_bf16);
bool cwk_fp8_linear_tc_available();
int cwk_fp8_linear_tc_launch2(cwk_ctx *ctx, const void *X, int64_t n, int64_t k, const void *W1, const float *scale1, int64_t cols1,
                              void *Y1, int out_bf16_1, const void *W2, const float *scale2, int64_t cols2, void *Y2, int out_bf16_2);
extern "C" int cwk_mla_decode(cwk_ctx *ctx, const void *q, const void *cache, int64_t seq_stride, int64_t ld,
                              const int32_t *kv_len, int max_kv_len, const int32_t *sel, int64_t sel_ld, int B,
                              int nh, int L, int R, float scale, void *out, int n_splits);

// Row-wise RMS norm of an f32 matrix (sum of squares in double, as
// cwick_rms_norm does, src/tensor.c:780-791), times a bf16 weight
// (apply_bf16_vec, src/attention.c:70-73), written as bf16. Columns
// [norm_cols, cols) are not normalised: they get the adjacent-pair RoPE of
// src/attention.c:60-68 at position pos0 + row when rope_cols > 0, else are
// copied. One block of 256 threads per row.
__global__ void __launch_bounds__(256) norm_rope_rows_kernel(const float *in, int64_t in_ld, int norm_cols,
                                                             int rope_cols, const uint16_t *weight, float eps,
                                                             float rope_base, int64_t pos0, uint16_t *out,
                                                             int64_t out_ld, int *kv_len_out, int ref_narrow) {
    const int64_t r = blockIdx.x;
    const float *x = in + r * in_ld;
    __shared__ double red[256];
    double ss = 0.0;
    for (int i = threadIdx.x; i < norm_cols; i += 256) ss += (double)x[i] * (double)x[i];
    red[threadIdx.x] = ss;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    const float inv = __fdiv_rn(1.0f, (float)sqrt(red[0] / (double)norm_cols + (double)eps));
    uint16_t *y = out + r * out_ld;
    for (int i = threadIdx.x; i < norm_cols; i += 256) {
        const float v = x[i] * inv * bf16_bits_to_f32(weight[i]);
        y[i] = ref_narrow ? narrow_bf16_like_reference(v) : (uint16_t)(pack_bf16x2(v, 0.f) & 0xffffu);
    }
    for (int i = threadIdx.x; i < rope_cols / 2; i += 256) {
        float sn, cs;
        rope_cos_sin(pos0 + r, i, rope_cols, rope_base, cs, sn);
        const float a = x[norm_cols + 2 * i], b = x[norm_cols + 2 * i + 1];
        const float r0 = a * cs - b * sn, r1 = b * cs + a * sn;
        if (ref_narrow) {
            y[norm_cols + 2 * i] = narrow_bf16_like_reference(r0);
            y[norm_cols + 2 * i + 1] = narrow_bf16_like_reference(r1);
        } else {
            *reinterpret_cast<uint32_t *>(y + norm_cols + 2 * i) = pack_bf16x2(r0, r1);
        }
    }
    if (kv_len_out && threadIdx.x == 0) kv_len_out[r] = (int)(pos0 + r + 1);
}

// The same, one WARP per row, for rows whose normalised part is a multiple of 128 columns (at most 128 * MAXV4) and whose
// rope part is at most 64 columns: a lane keeps its 16-byte pieces of the row in registers, so the row is read once;
// the sum of squares goes through lane-wise doubles and five shuffles, with no shared memory and no block barrier.
// 4096 rows are 4096 warps, all resident at once: the call takes about one row's latency.
template <int MAXV4>
__global__ void __launch_bounds__(256) norm_rope_rows_warp_kernel(const float *in, int64_t in_ld, int norm_cols, int rope_cols,
                                                                  const uint16_t *weight, float eps, float rope_base, int64_t pos0,
                                                                  uint16_t *out, int64_t out_ld, int *kv_len_out, int ref_narrow,
                                                                  int64_t nrows) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= nrows) return;
    const float *x = in + r * in_ld;
    const int np = norm_cols / 128;
    float4 v[MAXV4];
    float ra = 0.f, rb = 0.f;
    if (lane < rope_cols / 2) {
        const float2 ab = *reinterpret_cast<const float2 *>(x + norm_cols + 2 * lane);
        ra = ab.x; rb = ab.y;
    }
    double ss = 0.0;
#pragma unroll
    for (int c = 0; c < MAXV4; c++)
        if (c < np) {
            v[c] = *reinterpret_cast<const float4 *>(x + c * 128 + lane * 4);
            ss += (double)v[c].x * (double)v[c].x;
            ss += (double)v[c].y * (double)v[c].y;
            ss += (double)v[c].z * (double)v[c].z;
            ss += (double)v[c].w * (double)v[c].w;
        }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = __fdiv_rn(1.0f, (float)sqrt(ss / (double)norm_cols + (double)eps));
    uint16_t *y = out + r * out_ld;
#pragma unroll
    for (int c = 0; c < MAXV4; c++)
        if (c < np) {
            const uint2 wb = *reinterpret_cast<const uint2 *>(weight + c * 128 + lane * 4);
            const float o0 = v[c].x * inv * __uint_as_float(wb.x << 16), o1 = v[c].y * inv * __uint_as_float(wb.x & 0xffff0000u);
            const float o2 = v[c].z * inv * __uint_as_float(wb.y << 16), o3 = v[c].w * inv * __uint_as_float(wb.y & 0xffff0000u);
            uint2 pk;
            if (ref_narrow) {
                pk.x = (uint32_t)narrow_bf16_like_reference(o0) | ((uint32_t)narrow_bf16_like_reference(o1) << 16);
                pk.y = (uint32_t)narrow_bf16_like_reference(o2) | ((uint32_t)narrow_bf16_like_reference(o3) << 16);
            } else {
                pk.x = pack_bf16x2(o0, o1);
                pk.y = pack_bf16x2(o2, o3);
            }
            *reinterpret_cast<uint2 *>(y + c * 128 + lane * 4) = pk;
        }
    if (lane < rope_cols / 2) {
        float sn, cs;
        rope_cos_sin(pos0 + r, lane, rope_cols, rope_base, cs, sn);
        const float r0 = ra * cs - rb * sn, r1 = rb * cs + ra * sn;
        *reinterpret_cast<uint32_t *>(y + norm_cols + 2 * lane) =
            ref_narrow ? ((uint32_t)narrow_bf16_like_reference(r0) | ((uint32_t)narrow_bf16_like_reference(r1) << 16)) : pack_bf16x2(r0, r1);
    }
    if (kv_len_out && lane == 0) kv_len_out[r] = (int)(pos0 + r + 1);
}

static bool norm_rope_warp_ok(const float *in, int64_t in_ld, int norm_cols, int rope_cols, const void *weight, const void *out, int64_t out_ld) {
    return norm_cols > 0 && norm_cols % 128 == 0 && norm_cols <= 128 * 12 && rope_cols <= 64 && (rope_cols & 1) == 0 && in_ld % 4 == 0 &&
           out_ld % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(weight) & 7) == 0 &&
           (reinterpret_cast<uintptr_t>(out) & 7) == 0;
}

// Rope tail of the absorbed query: Qfull[t][h][L : L+rope] = RoPE(q[t][h][nope : nope+rope], pos0 + t).
// The angle depends on (t, pair) only: one thread forms it once and rotates that pair of all heads.
__global__ void __launch_bounds__(256) rope_tail_kernel(const uint16_t *q, uint16_t *qfull, int n, int nh, int nope, int n_rope, int L,
                                                        int64_t pos0, float base) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * (n_rope / 2)) return;
    const int t = i / (n_rope / 2), j = i % (n_rope / 2);
    float cs, sn;
    rope_cos_sin(pos0 + t, j, n_rope, base, cs, sn);
    const uint16_t *src = q + (int64_t)t * nh * (nope + n_rope) + nope + 2 * j;
    uint16_t *dst = qfull + (int64_t)t * nh * (L + n_rope) + L + 2 * j;
#pragma unroll 8
    for (int h = 0; h < nh; h++) {
        const uint32_t v = *reinterpret_cast<const uint32_t *>(src + (int64_t)h * (nope + n_rope));
        const float a = __uint_as_float(v << 16), b = __uint_as_float(v & 0xffff0000u);
        *reinterpret_cast<uint32_t *>(dst + (int64_t)h * (L + n_rope)) = pack_bf16x2(a * cs - b * sn, b * cs + a * sn);
    }
}

// RoPE of the rope part of q, in place: q[t][h][nope : nope+rope] at position pos0 + t. One thread per (t, pair) and
// group of heads (blockIdx.y): the angle is formed once per thread and applied to the group's heads. The pairs'
// divisors base^(2j / n_rope) -- the same values rope_cos_sin forms -- are computed once per block (n_rope <= 256).
__global__ void __launch_bounds__(256) rope_q_inplace_kernel(uint16_t *q, int n, int nh, int nope, int n_rope, int64_t pos0, float base) {
    __shared__ float s_den[128];
    for (int jj = threadIdx.x; jj < n_rope / 2; jj += 256) s_den[jj] = (float)pow((double)base, (double)(2.0f * (float)jj / (float)n_rope));
    __syncthreads();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * (n_rope / 2)) return;
    const int t = i / (n_rope / 2), j = i % (n_rope / 2);
    const int hpg = (nh + (int)gridDim.y - 1) / (int)gridDim.y, h0 = (int)blockIdx.y * hpg, h1 = min(nh, h0 + hpg);
    float cs, sn;
    {
        const float ang = __fdiv_rn((float)(pos0 + t), s_den[j]);
        double sd, cd;
        sincos((double)ang, &sd, &cd);
        cs = (float)cd;
        sn = (float)sd;
    }
    uint16_t *src = q + (int64_t)t * nh * (nope + n_rope) + nope + 2 * j;
#pragma unroll 8
    for (int h = h0; h < h1; h++) {
        uint32_t *w = reinterpret_cast<uint32_t *>(src + (int64_t)h * (nope + n_rope));
        const uint32_t v = *w;
        const float a = __uint_as_float(v << 16), b = __uint_as_float(v & 0xffff0000u);
        *w = pack_bf16x2(a * cs - b * sn, b * cs + a * sn);
    }
}

int cwk_absorb_tc_launch(cwk_ctx *ctx, const void *Q, int n, int nh, const void *Wuk, void *Qfull);
bool cwk_mla_prefill_attn_tc_ok(const void *Q, const void *cache, const void *Wuk, const void *kx, const void *out);
int cwk_mla_prefill_attn_tc(cwk_ctx *ctx, const void *Q, const void *cache, const void *Wuk, void *kx, int *flags, int64_t pos0, int n, int nh,
                            float scale, void *out, int exact_only);

// Absorb: Qfull[t][h][0:L] = q[t][h][0:nope] . W_uk[h] ([nope][L] row-major bf16), and
// Qfull[t][h][L:L+rope] = RoPE(q[t][h][nope:nope+rope], pos0+t). The identity is
// q_abs = W_k^T q of src/attention.c:741-744 (gemv_bf16_t), batched over tokens.
// Block = 64 tokens x one head; 8 warps as 4 (16-row blocks) x 2 (halves of L = 512).
constexpr int AB_NOPE = 128, AB_L = 512, AB_ROPE = 64;
constexpr int AB_SMEM = 64 * AB_NOPE * 2 + AB_NOPE * AB_L * 2;   // 16 KB + 128 KB

__global__ void __launch_bounds__(256, 1) absorb_kernel(const uint16_t *q, int n, int nh, const uint16_t *wuk,
                                                        float rope_base, int64_t pos0, uint16_t *qfull) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *sA = smem;                       // [64][128] bf16, 16 chunks per row, swizzled
    uint8_t *sB = smem + 64 * AB_NOPE * 2;    // [128][512] bf16, 64 chunks per row, swizzled
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp & 3, wn = warp >> 2;
    const int t0 = blockIdx.x * 64, h = blockIdx.y;
    const int qd = AB_NOPE + AB_ROPE;
    for (int i = tid; i < 64 * 16; i += 256) {
        const int r = i >> 4, c = i & 15;
        const bool ok = t0 + r < n;
        cp_async16(smem_u32(sA + r * 256 + ((c ^ (r & 7)) << 4)),
                   ok ? (const void *)(q + ((int64_t)(t0 + r) * nh + h) * qd + c * 8) : (const void *)q, ok);
    }
    const uint16_t *wb = wuk + (int64_t)h * AB_NOPE * AB_L;
    for (int i = tid; i < AB_NOPE * 64; i += 256) {
        const int r = i >> 6, c = i & 63;
        cp_async16(smem_u32(sB + r * 1024 + ((c ^ (r & 7)) << 4)), wb + (int64_t)r * AB_L + c * 8, true);
    }
    cp_async_commit();
    // rope tail while the tiles arrive
    for (int i = tid; i < 64 * (AB_ROPE / 2); i += 256) {
        const int r = i / (AB_ROPE / 2), j = i % (AB_ROPE / 2);
        if (t0 + r < n) {
            const uint16_t *src = q + ((int64_t)(t0 + r) * nh + h) * qd + AB_NOPE + 2 * j;
            const float a = bf16_bits_to_f32(src[0]), b = bf16_bits_to_f32(src[1]);
            float sn, cs;
            rope_cos_sin(pos0 + t0 + r, j, AB_ROPE, rope_base, cs, sn);
            *reinterpret_cast<uint32_t *>(qfull + ((int64_t)(t0 + r) * nh + h) * (AB_L + AB_ROPE) + AB_L + 2 * j) =
                pack_bf16x2(a * cs - b * sn, b * cs + a * sn);
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    float acc[32][4];
#pragma unroll
    for (int i = 0; i < 32; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const int arow = wm * 16 + (lane & 15);
#pragma unroll
    for (int kt = 0; kt < AB_NOPE / 16; kt++) {
        uint32_t a[4];
        ldmatrix_x4(a[0], a[1], a[2], a[3], smem_u32(sA + arow * 256) + (((kt * 2 + (lane >> 4)) ^ (arow & 7)) << 4));
        const int brow = kt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const uint32_t bbase = smem_u32(sB + brow * 1024);
#pragma unroll
        for (int np = 0; np < 16; np++) {
            const int chunk = wn * 32 + np * 2 + (lane >> 4);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, bbase + ((chunk ^ (brow & 7)) << 4));
            mma_bf16_16816(acc[np * 2], a, b0, b1);
            mma_bf16_16816(acc[np * 2 + 1], a, b2, b3);
        }
    }
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int r = wm * 16 + (lane >> 2) + half * 8;
        if (t0 + r >= n) continue;
        uint16_t *o = qfull + ((int64_t)(t0 + r) * nh + h) * (AB_L + AB_ROPE) + wn * 256 + (lane & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < 32; nt++)
            *reinterpret_cast<uint32_t *>(o + nt * 8) = pack_bf16x2(acc[nt][half * 2], acc[nt][half * 2 + 1]);
    }
}

extern "C" int cwk_mla_prefill(cwk_ctx *ctx, const void *X, const void *Wqa, const float *Sqa, const void *Wqb,
                               const float *Sqb, const void *Wkva, const float *Skva, const void *qa_norm,
                               const void *kva_norm, const void *Wuk, void *cache, int64_t pos0, int n, int H,
                               int q_lora, int nh, int nope, int rope, int kv_lora, float eps, float rope_base,
                               float scale, void *out) {
    if (!ctx || !X || !Wqa || !Sqa || !Wqb || !Sqb || !Wkva || !Skva || !qa_norm || !kva_norm || !Wuk || !cache || !out)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mla_prefill: null argument");
    if (n <= 0 || pos0 < 0 || H <= 0 || q_lora <= 0 || nh <= 0) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mla_prefill: bad dimensions");
    if (nope != AB_NOPE || rope != AB_ROPE || kv_lora != AB_L)
        return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "mla_prefill is built for nope 128, rope 64, kv_lora 512 (got %d/%d/%d)", nope, rope, kv_lora);
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const int qd = nope + rope, row = kv_lora + rope;
    // workspace: QA f32 [n][q_lora], QAn bf16 [n][q_lora], KVA f32 [n][row], Q bf16 [n][nh*qd],
    // Qfull bf16 [n][nh][row], kv_len int32 [n]
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const size_t b_qa = up((size_t)n * q_lora * 4), b_qan = up((size_t)n * q_lora * 2), b_kva = up((size_t)n * row * 4);
    // The attention takes one of two routes. Queries as MMA rows against per-head expanded keys (mla_prefill_attn.cu)
    // needs Kx bf16 [pos0+n][nh][qd] and no Qfull; the absorbed route (the decode kernel once per query row) needs
    // Qfull bf16 [n][nh][row]. The same workspace region serves whichever runs.
    // The expansion covers every cached row, so it pays when the chunk is a fair share of the context (always for a
    // prompt from position 0); a short chunk after a long history takes the absorbed route.
    const bool expanded_keys = ctx->force_mla_path != 0 && ctx->force_mla_path != 1 && ctx->force_mla_path != 2 && ctx->force_mla_path != 4 && pos0 + n <= 32768 &&
                               (int64_t)n * 4 >= pos0 + n;
    const size_t b_kx = up((size_t)(pos0 + n) * nh * qd * 2);
    const size_t b_q = up((size_t)n * nh * qd * 2), b_qf = expanded_keys ? std::max(b_kx, up((size_t)n * nh * row * 2)) : up((size_t)n * nh * row * 2),
                 b_len = up((size_t)n * 4) + up(((size_t)((n + 127) / 128) * nh * 2 + 3) * 4);
    int s = cwk_reserve_work(ctx, b_qa + b_qan + b_kva + b_q + b_qf + b_len);
    if (s != CWK_OK) return s;
    uint8_t *w = (uint8_t *)ctx->work;
    float *QA = (float *)w;
    uint16_t *QAn = (uint16_t *)(w + b_qa);
    float *KVA = (float *)(w + b_qa + b_qan);
    uint16_t *Q = (uint16_t *)(w + b_qa + b_qan + b_kva);
    uint16_t *Qf = (uint16_t *)(w + b_qa + b_qan + b_kva + b_q);
    int32_t *len = (int32_t *)(w + b_qa + b_qan + b_kva + b_q + b_qf);

    // q_a and kv_a share the activations: one launch of the tensor-core GEMM when it takes the shapes
    bool kva_done = false;
    s = CWK_ERR_UNSUPPORTED;
    if (cwk_fp8_linear_tc_available() && ctx->force_mla_path != 0 && ctx->force_mla_path != 1 && H % 128 == 0 && q_lora % 8 == 0 &&
        row % 8 == 0 && ((uintptr_t)X % 16) == 0) {
        s = cwk_fp8_linear_tc_launch2(ctx, X, n, H, Wqa, Sqa, q_lora, QA, 0, Wkva, Skva, row, KVA, 0);
        if (s == CWK_OK) kva_done = true;
        else if (s != CWK_ERR_UNSUPPORTED) return s;
    }
    if (!kva_done) s = cwk_fp8_linear(ctx, X, Wqa, Sqa, n, H, q_lora, QA, 0);
    if (s != CWK_OK) return s;
    if (norm_rope_warp_ok(QA, q_lora, q_lora, 0, qa_norm, QAn, q_lora))
        norm_rope_rows_warp_kernel<12><<<(n + 7) / 8, 256, 0, ctx->stream>>>(QA, q_lora, q_lora, 0, (const uint16_t *)qa_norm, eps, rope_base,
                                                                             pos0, QAn, q_lora, nullptr, 0, n);
    else
        norm_rope_rows_kernel<<<n, 256, 0, ctx->stream>>>(QA, q_lora, q_lora, 0, (const uint16_t *)qa_norm, eps, rope_base,
                                                          pos0, QAn, q_lora, nullptr, 0);
    CWK_LAUNCH_CHECK(ctx, "norm_rope_rows_kernel(q_a)");
    s = cwk_fp8_linear(ctx, QAn, Wqb, Sqb, n, q_lora, (int64_t)nh * qd, Q, 1);
    if (s != CWK_OK) return s;
    if (!kva_done) {
        s = cwk_fp8_linear(ctx, X, Wkva, Skva, n, H, row, KVA, 0);
        if (s != CWK_OK) return s;
    }
    if (norm_rope_warp_ok(KVA, row, kv_lora, rope, kva_norm, (uint16_t *)cache + pos0 * row, row))
        norm_rope_rows_warp_kernel<12><<<(n + 7) / 8, 256, 0, ctx->stream>>>(KVA, row, kv_lora, rope, (const uint16_t *)kva_norm, eps, rope_base,
                                                                             pos0, (uint16_t *)cache + pos0 * row, row, len, 1, n);
    else
        norm_rope_rows_kernel<<<n, 256, 0, ctx->stream>>>(KVA, row, kv_lora, rope, (const uint16_t *)kva_norm, eps, rope_base,
                                                          pos0, (uint16_t *)cache + pos0 * row, row, len, 1);
    CWK_LAUNCH_CHECK(ctx, "norm_rope_rows_kernel(kv_a)");
    if (expanded_keys && cwk_mla_prefill_attn_tc_ok(Q, cache, Wuk, Qf, out)) {
        rope_q_inplace_kernel<<<dim3((n * (rope / 2) + 255) / 256, nh >= 8 ? 4 : 1), 256, 0, ctx->stream>>>(Q, n, nh, nope, rope, pos0, rope_base);
        CWK_LAUNCH_CHECK(ctx, "rope_q_inplace_kernel");
        return cwk_mla_prefill_attn_tc(ctx, Q, cache, Wuk, Qf, (int *)((uint8_t *)len + up((size_t)n * 4)), pos0, n, nh, scale, out, ctx->force_mla_path == 3);
    }
    // absorb on the tensor path (tcgen05); the mma.sync kernel covers a context without the
    // tensor-map encoder or a caller that forced the general kernels
    s = CWK_ERR_UNSUPPORTED;
    if (ctx->force_mla_path != 0 && ctx->force_mla_path != 1) {
        s = cwk_absorb_tc_launch(ctx, Q, n, nh, Wuk, Qf);
        if (s != CWK_OK && s != CWK_ERR_UNSUPPORTED) return s;
        if (s == CWK_OK) {
            rope_tail_kernel<<<(n * (rope / 2) + 255) / 256, 256, 0, ctx->stream>>>(Q, Qf, n, nh, nope, rope, kv_lora, pos0, rope_base);
            CWK_LAUNCH_CHECK(ctx, "rope_tail_kernel");
        }
    }
    if (s == CWK_ERR_UNSUPPORTED) {
        static bool attr_set[16] = {false};
        if (!attr_set[ctx->device & 15]) {
            CWK_CUDA(ctx, cudaFuncSetAttribute(absorb_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AB_SMEM));
            attr_set[ctx->device & 15] = true;
        }
        absorb_kernel<<<dim3((n + 63) / 64, nh), 256, AB_SMEM, ctx->stream>>>(Q, n, nh, (const uint16_t *)Wuk, rope_base, pos0, Qf);
        CWK_LAUNCH_CHECK(ctx, "absorb_kernel");
    }
    return cwk_mla_decode(ctx, Qf, cache, 0, row, len, (int)(pos0 + n), nullptr, 0, n, nh, kv_lora, rope, scale, out, 0);
}
