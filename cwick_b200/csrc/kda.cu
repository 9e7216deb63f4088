// kda.cu -- one decode step of the KDA (gated delta-rule) linear-attention layers: everything of
// cwick_attention_kda_decode between its projections and o_proj (src/attention.c:1243-1417), for B engine
// slots at once. The projections either side are plain GEMVs and stay with the caller.
//
// One work item per (head, slot), one thread per channel of the head; blocks are persistent and the next item's
// state tile and scalars stream into shared memory (asynchronous copies) while the current item is worked on:
//   1. short convolution over the 3-deep window of projected values + SiLU for q, k, v; the window moves on
//      (:1253-1281)
//   2. L2 norm of q and k over the head, q also / sqrt(hd) (:1285-1301); the squared sums are formed in double
//   3. decay exp(lower * sigmoid(exp(a_log[h]) * (gate_raw + dt_bias))) per key channel, beta = sigmoid (:1314-1342)
//   4. the recurrence on the head's [hd][hd] state (:1352-1396): a thread owns one VALUE column of the state in
//      registers (hd floats, taken from the staged tile), so the state is read once and written once, and the three
//      passes over the key dimension -- delta = v - k.S, S += (beta k) delta, core = q.S -- run in the
//      reference's order on it
//   5. RMS norm of the head's core times o_norm times sigmoid(gate) (:1406-1417)
// The state is the traffic: 2 x hd x hd x 4 bytes per head and token (8.4 MB per layer at 64 heads of 128).
// Products and sums that the reference rounds separately use the _rn intrinsics (this file is compiled with
// fast-math); exp goes through double, so results equal the C library's expf except in rare last-place cases.
#include <algorithm>

#include "cwk_common.cuh"

namespace {

__device__ __forceinline__ float exp_f(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float sigmoid_ref(float x) {             // 1.0f / (1.0f + expf(-x))
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_f(-x)));
}

// Sum of one double per thread over the block (warp shuffles, then the warp sums in warp order). The reference
// adds in index order; a different order moves the double sum by parts in 10^16, which its rounding to float
// hides in all but rare cases (the tests allow for it together with the exp).
template <int HD>
__device__ __forceinline__ double block_sum(double x, double *s_part) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = x;
    __syncthreads();
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < HD / 32; w++) t += s_part[w];
    __syncthreads();
    return t;
}

struct KdaParams {
    const float *q, *k, *v;            // [B][proj] projected inputs
    const uint16_t *q_conv, *k_conv, *v_conv;      // bf16 [proj][4]
    float *conv;                       // [B][3][proj][3]
    const float *gate_raw, *dt_bias, *a_log, *beta_raw, *gate;
    const uint16_t *o_norm;            // bf16 [hd]
    float *rec;                        // [B][nh][hd][hd]
    float *core;                       // [B][proj]
    int nh;
    float lower, rms_eps;
};

// Scalars of one item that come from memory written per slot or per channel, staged in shared memory by 4- and
// 8-byte asynchronous copies together with the item's state tile: [SC_COUNT][HD] words.
enum { SC_X = 0, SC_S = 3, SC_GRAW = 12, SC_GATE = 13, SC_DT = 14, SC_W = 15, SC_COUNT = 21 };      // SC_W: 3 x two words (4 bf16)

template <int HD>
__device__ __forceinline__ void kda_prefetch(const KdaParams &p, int item, float *s_tile, float *s_sc, int j) {
    const int h = item % p.nh, b = item / p.nh;
    const int64_t proj = (int64_t)p.nh * HD, i = (int64_t)h * HD + j;
    const float *r = p.rec + (((int64_t)b * p.nh + h) * HD) * HD;
    const uint32_t tb = (uint32_t)__cvta_generic_to_shared(s_tile), sb = (uint32_t)__cvta_generic_to_shared(s_sc);
#pragma unroll
    for (int c = 0; c < HD / 4; c++) {
        const int ch = c * HD + j;                                    // 16-byte chunk of the [HD][HD] tile
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(tb + (uint32_t)ch * 16u), "l"(r + (int64_t)ch * 4) : "memory");
    }
    auto cp4 = [&](int slot, const float *g) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(sb + (uint32_t)(slot * HD + j) * 4u), "l"(g) : "memory");
    };
    const float *in[3] = {p.q, p.k, p.v};
    const uint16_t *cw[3] = {p.q_conv, p.k_conv, p.v_conv};
#pragma unroll
    for (int w = 0; w < 3; w++) {
        cp4(SC_X + w, in[w] + (int64_t)b * proj + i);
        const float *s = p.conv + (((int64_t)b * 3 + w) * proj + i) * 3;
        cp4(SC_S + 3 * w, s); cp4(SC_S + 3 * w + 1, s + 1); cp4(SC_S + 3 * w + 2, s + 2);
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(sb + (uint32_t)((SC_W + 2 * w) * HD + 2 * j) * 4u), "l"(cw[w] + i * 4) : "memory");
    }
    cp4(SC_GRAW, p.gate_raw + (int64_t)b * proj + i);
    cp4(SC_GATE, p.gate + (int64_t)b * proj + i);
    cp4(SC_DT, p.dt_bias + i);
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// Persistent blocks: block g works on items g, g + G, ... (item = slot * nh + head). While an item is worked on in
// registers, the next item's state tile and scalars stream into shared memory.
template <int HD>
__global__ void __launch_bounds__(HD) kda_step_kernel(const KdaParams p, int nitems) {
    extern __shared__ float4 s_dyn4[];
    float *s_tile = reinterpret_cast<float *>(s_dyn4);                // [HD][HD], the NEXT item's state
    float *s_sc = s_tile + HD * HD;                                   // [SC_COUNT][HD]
    __shared__ float s_q[HD], s_k[HD], s_v[HD], s_eg[HD], s_core[HD];
    __shared__ double s_part[HD / 32];
    const int j = threadIdx.x;
    const int64_t proj = (int64_t)p.nh * HD;

    // One item per block (few slots): nothing to overlap with, the column and the scalars come straight from
    // global memory, the column first.
    const bool single = nitems <= (int)gridDim.x;
    if (!single && (int)blockIdx.x < nitems) kda_prefetch<HD>(p, blockIdx.x, s_tile, s_sc, j);
    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int h = item % p.nh, b = item / p.nh;
        const int64_t i = (int64_t)h * HD + j;
        float st[HD];
        float x[3], sw[3][3], graw, gate_v, dt;
        uint2 wbits[3];
        if (single) {
            const float *r = p.rec + (((int64_t)b * p.nh + h) * HD) * HD + j;
#pragma unroll
            for (int kk = 0; kk < HD; kk++) st[kk] = r[(int64_t)kk * HD];
            const float *in[3] = {p.q, p.k, p.v};
            const uint16_t *cw[3] = {p.q_conv, p.k_conv, p.v_conv};
#pragma unroll
            for (int w = 0; w < 3; w++) {
                x[w] = in[w][(int64_t)b * proj + i];
                const float *sp = p.conv + (((int64_t)b * 3 + w) * proj + i) * 3;
                sw[w][0] = sp[0]; sw[w][1] = sp[1]; sw[w][2] = sp[2];
                wbits[w] = *reinterpret_cast<const uint2 *>(cw[w] + i * 4);
            }
            graw = p.gate_raw[(int64_t)b * proj + i]; gate_v = p.gate[(int64_t)b * proj + i]; dt = p.dt_bias[i];
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
            // this thread's state column and scalars leave shared memory, which then takes the next item
#pragma unroll
            for (int kk = 0; kk < HD; kk++) st[kk] = s_tile[kk * HD + j];
#pragma unroll
            for (int w = 0; w < 3; w++) {
                x[w] = s_sc[(SC_X + w) * HD + j];
#pragma unroll
                for (int t = 0; t < 3; t++) sw[w][t] = s_sc[(SC_S + 3 * w + t) * HD + j];
                wbits[w] = *reinterpret_cast<const uint2 *>(s_sc + (SC_W + 2 * w) * HD + 2 * j);
            }
            graw = s_sc[SC_GRAW * HD + j]; gate_v = s_sc[SC_GATE * HD + j]; dt = s_sc[SC_DT * HD + j];
            __syncthreads();
            if (item + (int)gridDim.x < nitems) kda_prefetch<HD>(p, item + gridDim.x, s_tile, s_sc, j);
        }

        // 1. convolution + SiLU
        {
            float *out[3] = {s_q, s_k, s_v};
#pragma unroll
            for (int w = 0; w < 3; w++) {
                float *s = p.conv + (((int64_t)b * 3 + w) * proj + i) * 3;
                const float c0 = __uint_as_float(wbits[w].x << 16), c1 = __uint_as_float(wbits[w].x & 0xFFFF0000u);
                const float c2 = __uint_as_float(wbits[w].y << 16), c3 = __uint_as_float(wbits[w].y & 0xFFFF0000u);
                float acc = __fmul_rn(sw[w][0], c0);
                acc = __fadd_rn(acc, __fmul_rn(sw[w][1], c1));
                acc = __fadd_rn(acc, __fmul_rn(sw[w][2], c2));
                acc = __fadd_rn(acc, __fmul_rn(x[w], c3));
                out[w][j] = __fmul_rn(acc, sigmoid_ref(acc));
                s[0] = sw[w][1]; s[1] = sw[w][2]; s[2] = x[w];
            }
        }
        // 3. decay factor of this key channel
        {
            const float raw = __fadd_rn(graw, dt);
            const float sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_f(__fmul_rn(-exp_f(p.a_log[h]), raw))));
            s_eg[j] = exp_f(__fmul_rn(p.lower, sg));
        }
        __syncthreads();
        // 2. norms (squared sums in double)
        {
            const double qn = block_sum<HD>((double)s_q[j] * (double)s_q[j], s_part);
            const double kn = block_sum<HD>((double)s_k[j] * (double)s_k[j], s_part);
            const double eps = (double)1.0e-5f;
            const double sq = sqrt(qn), sk = sqrt(kn);
            const float qinv = __fdiv_rn(1.0f, (float)(sq < eps ? eps : sq));
            const float kinv = __fdiv_rn(1.0f, (float)(sk < eps ? eps : sk));
            const float qv = __fdiv_rn(__fmul_rn(s_q[j], qinv), __fsqrt_rn((float)HD));
            const float kv = __fmul_rn(s_k[j], kinv);
            s_q[j] = qv;
            s_k[j] = kv;
        }
        __syncthreads();
        // 4. recurrence: this thread owns value column j of the head's state
        {
            float *r = p.rec + (((int64_t)b * p.nh + h) * HD) * HD + j;
            const float beta = sigmoid_ref(p.beta_raw[(int64_t)b * p.nh + h]);
#pragma unroll
            for (int kk = 0; kk < HD; kk++) st[kk] = __fmul_rn(st[kk], s_eg[kk]);
            float delta = s_v[j];
#pragma unroll
            for (int kk = 0; kk < HD; kk++) delta = __fsub_rn(delta, __fmul_rn(s_k[kk], st[kk]));
#pragma unroll
            for (int kk = 0; kk < HD; kk++) st[kk] = __fadd_rn(st[kk], __fmul_rn(__fmul_rn(beta, s_k[kk]), delta));
            float o = 0.f;
#pragma unroll
            for (int kk = 0; kk < HD; kk++) o = __fadd_rn(o, __fmul_rn(s_q[kk], st[kk]));
#pragma unroll
            for (int kk = 0; kk < HD; kk++) r[(int64_t)kk * HD] = st[kk];
            s_core[j] = o;
        }
        __syncthreads();
        // 5. gated norm
        {
            const double ss = block_sum<HD>((double)s_core[j] * (double)s_core[j], s_part);
            const float inv = __fdiv_rn(1.0f, (float)sqrt(ss / (double)HD + (double)p.rms_eps));
            const float sg = sigmoid_ref(gate_v);
            float o = __fmul_rn(s_core[j], inv);
            o = __fmul_rn(o, bf16_bits_to_f32(p.o_norm[j]));
            p.core[(int64_t)b * proj + i] = __fmul_rn(o, sg);
        }
    }
}

}  // namespace

extern "C" int cwk_kda_step(cwk_ctx *ctx, int B, int nh, int hd, float lower, float rms_eps, const float *q, const float *k,
                            const float *v, const void *q_conv, const void *k_conv, const void *v_conv, float *conv,
                            const float *gate_raw, const float *dt_bias, const float *a_log, const float *beta_raw,
                            const float *gate, const void *o_norm, float *rec, float *core) {
    if (!ctx || !q || !k || !v || !q_conv || !k_conv || !v_conv || !conv || !gate_raw || !dt_bias || !a_log || !beta_raw || !gate ||
        !o_norm || !rec || !core || B <= 0 || nh <= 0)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "kda_step: bad argument");
    if (hd != 32 && hd != 64 && hd != 128) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "kda_step is built for head dims 32, 64, 128 (got %d)", hd);
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    KdaParams p;
    p.q = q; p.k = k; p.v = v;
    p.q_conv = (const uint16_t *)q_conv; p.k_conv = (const uint16_t *)k_conv; p.v_conv = (const uint16_t *)v_conv;
    p.conv = conv; p.gate_raw = gate_raw; p.dt_bias = dt_bias; p.a_log = a_log; p.beta_raw = beta_raw; p.gate = gate;
    p.o_norm = (const uint16_t *)o_norm; p.rec = rec; p.core = core; p.nh = nh; p.lower = lower; p.rms_eps = rms_eps;
    if ((reinterpret_cast<uintptr_t>(rec) & 15) || (reinterpret_cast<uintptr_t>(q_conv) | reinterpret_cast<uintptr_t>(k_conv) | reinterpret_cast<uintptr_t>(v_conv)) & 7)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "kda_step: the state must be 16-byte and the convolution weights 8-byte aligned");
    const int nitems = B * nh;
    const int grid = std::min(nitems, 2 * ctx->sm_count);
    const size_t smem = ((size_t)hd * hd + (size_t)SC_COUNT * hd) * sizeof(float);
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(kda_step_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (128 * 128 + SC_COUNT * 128) * 4));
        CWK_CUDA(ctx, cudaFuncSetAttribute(kda_step_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (64 * 64 + SC_COUNT * 64) * 4));
        attr_set[ctx->device & 15] = true;
    }
    CwkKernelTimer timer(ctx);
    if (hd == 128) kda_step_kernel<128><<<grid, 128, smem, ctx->stream>>>(p, nitems);
    else if (hd == 64) kda_step_kernel<64><<<grid, 64, smem, ctx->stream>>>(p, nitems);
    else kda_step_kernel<32><<<grid, 32, smem, ctx->stream>>>(p, nitems);
    CWK_LAUNCH_CHECK(ctx, "kda_step_kernel");
    return CWK_OK;
}
