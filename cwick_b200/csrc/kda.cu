// kda.cu -- one decode step of the KDA (gated delta-rule) linear-attention layers: everything of
// cwick_attention_kda_decode between its projections and o_proj (src/attention.c:1243-1417), for B engine
// slots at once. The projections either side are plain GEMVs and stay with the caller.
//
// One work item per (head, slot), one thread per channel of the head; blocks are persistent. An item's [hd][hd] state
// comes into shared memory by one bulk copy, is updated there, and goes back by one bulk copy; the item's other inputs
// are fetched into registers an item ahead. Few registers and one tile per block leave room for three blocks per SM,
// which is what overlaps one item's copies with another's arithmetic:
//   1. short convolution over the 3-deep window of projected values + SiLU for q, k, v; the window moves on
//      (:1253-1281)
//   2. L2 norm of q and k over the head, q also / sqrt(hd) (:1285-1301); the squared sums are formed in double
//   3. decay exp(lower * sigmoid(exp(a_log[h]) * (gate_raw + dt_bias))) per key channel, beta = sigmoid (:1314-1342)
//   4. the recurrence on the head's [hd][hd] state (:1352-1396): a thread owns one VALUE column of the tile (lanes read
//      neighbouring words: no bank conflicts), so the state is read once and written once, and the sums over the key
//      dimension -- delta = v - k.S, then S += (beta k) delta with core = q.S -- run in the reference's order on it
//   5. RMS norm of the head's core times o_norm times sigmoid(gate) (:1406-1417)
// The state is the traffic: 2 x hd x hd x 4 bytes per head and token (8.4 MB per layer at 64 heads of 128).
// Products and sums that the reference rounds separately use the _rn intrinsics (this file is compiled with
// fast-math); exp goes through double, so results equal the C library's expf except in rare last-place cases.
#include <algorithm>

#include "tc_common.cuh"

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

constexpr int KDA_ERR_TILE = 0x6b01;

// One item's inputs other than the state, as thread j (channel j of the head) holds them.
struct KdaIn {
    float x[3], sw[3][3], graw, gate_v, dt, a_log, beta_raw;
    uint2 wbits[3];
};
template <int HD> __device__ __forceinline__ void kda_fetch(const KdaParams &p, int item, int j, KdaIn &r) {
    const int h = item % p.nh, b = item / p.nh;
    const int64_t proj = (int64_t)p.nh * HD, i = (int64_t)h * HD + j;
    const float *in[3] = {p.q, p.k, p.v};
    const uint16_t *cw[3] = {p.q_conv, p.k_conv, p.v_conv};
#pragma unroll
    for (int w = 0; w < 3; w++) {
        r.x[w] = __ldg(in[w] + (int64_t)b * proj + i);
        const float *sp = p.conv + (((int64_t)b * 3 + w) * proj + i) * 3;      // written by this kernel, for this item only
        r.sw[w][0] = sp[0]; r.sw[w][1] = sp[1]; r.sw[w][2] = sp[2];
        r.wbits[w] = __ldg(reinterpret_cast<const uint2 *>(cw[w] + i * 4));
    }
    r.graw = __ldg(p.gate_raw + (int64_t)b * proj + i);
    r.gate_v = __ldg(p.gate + (int64_t)b * proj + i);
    r.dt = __ldg(p.dt_bias + i);
    r.a_log = __ldg(p.a_log + h);
    r.beta_raw = __ldg(p.beta_raw + (int64_t)b * p.nh + h);
}

// Persistent blocks: block g works on items g, g + G, ... (item = slot * nh + head).
template <int HD>
__global__ void __launch_bounds__(HD) kda_step_kernel(const KdaParams p, int nitems, int *err) {
    extern __shared__ float4 s_dyn4[];
    float *s_tile = reinterpret_cast<float *>(s_dyn4);                // [HD][HD], this item's state
    __shared__ __align__(16) float s_q[HD], s_k[HD], s_v[HD], s_eg[HD], s_core[HD];
    __shared__ double s_part[HD / 32];
    __shared__ __align__(8) uint64_t s_bar;
    const int j = threadIdx.x;
    const int64_t proj = (int64_t)p.nh * HD;
    const uint32_t bar = smem_u32(&s_bar), tile = smem_u32(s_tile);
    constexpr int COPIER = HD > 32 ? 32 : 0;                          // the thread that issues the tile copies
    constexpr uint32_t TILE_BYTES = HD * HD * 4;
    if (j == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    uint32_t phase = 0;
    KdaIn nxt;
    if ((int)blockIdx.x < nitems) kda_fetch<HD>(p, blockIdx.x, j, nxt);
    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int h = item % p.nh, b = item / p.nh;
        const int64_t i = (int64_t)h * HD + j;
        float *rec = p.rec + (((int64_t)b * p.nh + h) * HD) * HD;
        if (j == COPIER) {
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the last write-back has left the tile
            mbar_expect_tx(bar, TILE_BYTES);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(tile),
                         "l"(rec), "r"(TILE_BYTES), "r"(bar)
                         : "memory");
        }
        const KdaIn cur = nxt;
        if (item + (int)gridDim.x < nitems) kda_fetch<HD>(p, item + gridDim.x, j, nxt);
        const float(&x)[3] = cur.x;
        const float(&sw)[3][3] = cur.sw;
        const uint2(&wbits)[3] = cur.wbits;
        const float graw = cur.graw, gate_v = cur.gate_v, dt = cur.dt;

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
            const float sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_f(__fmul_rn(-exp_f(cur.a_log), raw))));
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
        // 4. recurrence: this thread owns value column j of the head's state tile
        {
            const float beta = sigmoid_ref(cur.beta_raw);
            mbar_wait(bar, phase, err, KDA_ERR_TILE);                       // on giving up: carries on, the host reports the call as failed
            phase ^= 1;
            float *col = s_tile + j;
            float delta = s_v[j];
#pragma unroll 8
            for (int kk = 0; kk < HD; kk += 4) {
                const float4 e4 = *reinterpret_cast<const float4 *>(s_eg + kk), k4 = *reinterpret_cast<const float4 *>(s_k + kk);
                delta = __fsub_rn(delta, __fmul_rn(k4.x, __fmul_rn(col[(kk + 0) * HD], e4.x)));
                delta = __fsub_rn(delta, __fmul_rn(k4.y, __fmul_rn(col[(kk + 1) * HD], e4.y)));
                delta = __fsub_rn(delta, __fmul_rn(k4.z, __fmul_rn(col[(kk + 2) * HD], e4.z)));
                delta = __fsub_rn(delta, __fmul_rn(k4.w, __fmul_rn(col[(kk + 3) * HD], e4.w)));
            }
            float o = 0.f;
#pragma unroll 8
            for (int kk = 0; kk < HD; kk += 4) {
                const float4 e4 = *reinterpret_cast<const float4 *>(s_eg + kk), k4 = *reinterpret_cast<const float4 *>(s_k + kk);
                const float4 q4 = *reinterpret_cast<const float4 *>(s_q + kk);
                const float s0 = __fadd_rn(__fmul_rn(col[(kk + 0) * HD], e4.x), __fmul_rn(__fmul_rn(beta, k4.x), delta));
                const float s1 = __fadd_rn(__fmul_rn(col[(kk + 1) * HD], e4.y), __fmul_rn(__fmul_rn(beta, k4.y), delta));
                const float s2 = __fadd_rn(__fmul_rn(col[(kk + 2) * HD], e4.z), __fmul_rn(__fmul_rn(beta, k4.z), delta));
                const float s3 = __fadd_rn(__fmul_rn(col[(kk + 3) * HD], e4.w), __fmul_rn(__fmul_rn(beta, k4.w), delta));
                col[(kk + 0) * HD] = s0; col[(kk + 1) * HD] = s1; col[(kk + 2) * HD] = s2; col[(kk + 3) * HD] = s3;
                o = __fadd_rn(o, __fmul_rn(q4.x, s0));
                o = __fadd_rn(o, __fmul_rn(q4.y, s1));
                o = __fadd_rn(o, __fmul_rn(q4.z, s2));
                o = __fadd_rn(o, __fmul_rn(q4.w, s3));
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // the column, visible to the copy engine
            s_core[j] = o;
        }
        __syncthreads();
        if (j == COPIER) {                                                  // the tile goes back under the gated norm
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(rec), "r"(tile), "r"(TILE_BYTES) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
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
    if (j == COPIER) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
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
    const size_t smem = (size_t)hd * hd * sizeof(float);
    static int per_sm[16][3] = {{0}};                                   // resident blocks per SM, by device and head dim
    int &resident = per_sm[ctx->device & 15][hd == 128 ? 2 : hd == 64 ? 1 : 0];
    if (!resident) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(kda_step_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 128 * 4));
        int nb = 0;
        if (hd == 128) CWK_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kda_step_kernel<128>, 128, smem));
        else if (hd == 64) CWK_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kda_step_kernel<64>, 64, smem));
        else CWK_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kda_step_kernel<32>, 32, smem));
        resident = std::max(nb, 1);
    }
    const int grid = std::min(nitems, resident * ctx->sm_count);
    int es = cwk_ensure_err_word(ctx);
    if (es != CWK_OK) return es;
    CwkKernelTimer timer(ctx);
    if (hd == 128) kda_step_kernel<128><<<grid, 128, smem, ctx->stream>>>(p, nitems, ctx->dev_err);
    else if (hd == 64) kda_step_kernel<64><<<grid, 64, smem, ctx->stream>>>(p, nitems, ctx->dev_err);
    else kda_step_kernel<32><<<grid, 32, smem, ctx->stream>>>(p, nitems, ctx->dev_err);
    CWK_LAUNCH_CHECK(ctx, "kda_step_kernel");
    return CWK_OK;
}
