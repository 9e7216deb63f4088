// gdn.cu -- the Gated DeltaNet scan of the Qwen3.5 linear-attention layers: lin_rec_heads
// (src/q35_model.c:1177-1264) for n positions of B slots, after the projections, the convolution and the q/k
// normalisation (which are GEMMs and elementwise passes on the caller's side, :1277-1372).
//
// One work item per (value head, slot), one thread per VALUE row of the head's [head_v][head_k] state; blocks are
// persistent, and the next item's state tile streams into shared memory (16-byte asynchronous copies, padded rows)
// while the current item is scanned. A thread keeps
// its row (head_k floats) in registers over all n positions, so the state is read once and written once per call;
// per position the block shares q and k of the head's key head through shared memory. A row's two passes -- decay
// and dot with k; update with k delta and dot with q -- are sequential over the key dimension, in the
// reference's order; the head's RMS sum over the value rows is formed by one thread in index order (f32, as the
// reference forms it). Positions are a scan: they run one after the other (a decode step is n = 1).
// Products and sums that the reference rounds separately use the _rn intrinsics (fast-math build); exp and log1p go
// through double.
#include <algorithm>

#include "cwk_common.cuh"

namespace {

__device__ __forceinline__ float g_exp(float x) { return (float)exp((double)x); }

struct GdnParams {
    const float *up;       // [B][n][qkv_dim]: q heads | k heads | v heads
    const float *gdec;     // [B][n][nh]
    const float *beta;     // [B][n][nh]
    const float *gate;     // [B][n][val_dim]
    const float *a_log, *dt_bias;      // [nh]
    const float *norm;     // [head_v]
    float *S;              // [B][nh][head_v][head_k]
    float *out;            // [B][n][val_dim]
    int n, nh, kv_group;
    int n_stride;          // positions per slot in the arrays (>= n: a call's tail after the chunk-parallel part)
    float rms_eps;
};

// Row stride of the staged state tile in shared memory: 4 floats of padding make a thread's 16-byte reads of its own
// row conflict-free (eight lanes of a quarter warp then cover all 32 banks).
template <int HK> __host__ __device__ constexpr int gdn_ld() { return HK + 4; }

template <int HK>
__device__ __forceinline__ void gdn_prefetch(const GdnParams &p, int item, int hv, float *s_tile, int j, int nthreads) {
    const int vh = item % p.nh, b = item / p.nh;
    const float *src = p.S + (((int64_t)b * p.nh + vh) * hv) * HK;
    const uint32_t tb = (uint32_t)__cvta_generic_to_shared(s_tile);
    for (int ch = j; ch < hv * (HK / 4); ch += nthreads) {            // 16-byte chunks, coalesced
        const int row = ch / (HK / 4), c4 = ch % (HK / 4);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(tb + (uint32_t)(row * gdn_ld<HK>() + c4 * 4) * 4u), "l"(src + (int64_t)ch * 4) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// Persistent blocks: block g works on items g, g + G, ... (item = slot * nh + value head). While an item's positions
// are scanned with the state in registers, the next item's state tile streams into shared memory.
template <int HK>
__global__ void __launch_bounds__(128) gdn_scan_kernel(const GdnParams p, int nitems) {
    extern __shared__ float4 s_dyn4[];
    float *s_tile = reinterpret_cast<float *>(s_dyn4);                // [hv][HK + 4], the NEXT item's state
    __shared__ float s_q[HK], s_k[HK], s_tmp[128];
    __shared__ float s_rstd;
    const int j = threadIdx.x, hv = blockDim.x;
    const int key_dim = (p.nh / p.kv_group) * HK, val_dim = p.nh * hv, qkv_dim = 2 * key_dim + val_dim;
    const bool single = nitems <= (int)gridDim.x;                     // one item per block: nothing to overlap with
    const float nw = p.norm[j];
    if (!single) gdn_prefetch<HK>(p, blockIdx.x, hv, s_tile, j, hv);
    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int vh = item % p.nh, b = item / p.nh;
        const int kh = vh / p.kv_group;
        float *Srow = p.S + ((((int64_t)b * p.nh + vh) * hv) + j) * HK;
        float sj[HK];
        if (single) {
#pragma unroll
            for (int i = 0; i < HK; i += 4) {
                const float4 v = *reinterpret_cast<const float4 *>(Srow + i);
                sj[i] = v.x; sj[i + 1] = v.y; sj[i + 2] = v.z; sj[i + 3] = v.w;
            }
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
#pragma unroll
            for (int i = 0; i < HK; i += 4) {
                const float4 v = *reinterpret_cast<const float4 *>(s_tile + j * gdn_ld<HK>() + i);
                sj[i] = v.x; sj[i + 1] = v.y; sj[i + 2] = v.z; sj[i + 3] = v.w;
            }
            __syncthreads();
            if (item + (int)gridDim.x < nitems) gdn_prefetch<HK>(p, item + gridDim.x, hv, s_tile, j, hv);
        }
        const float ea = g_exp(p.a_log[vh]), dtb = p.dt_bias[vh];
        for (int t = 0; t < p.n; t++) {
            const float *row = p.up + ((int64_t)b * p.n_stride + t) * qkv_dim;
            for (int i = j; i < HK; i += hv) {
                s_q[i] = row[(int64_t)kh * HK + i];
                s_k[i] = row[key_dim + (int64_t)kh * HK + i];
            }
            const float vj = row[2 * key_dim + (int64_t)vh * hv + j];
            const float zj = p.gate[((int64_t)b * p.n_stride + t) * val_dim + (int64_t)vh * hv + j];
            const float x = __fadd_rn(p.gdec[((int64_t)b * p.n_stride + t) * p.nh + vh], dtb);
            const float sp = x > 20.0f ? x : (float)log1p((double)g_exp(x));
            const float decay = g_exp(__fmul_rn(-ea, sp));
            const float bet = __fdiv_rn(1.0f, __fadd_rn(1.0f, g_exp(-p.beta[((int64_t)b * p.n_stride + t) * p.nh + vh])));
            __syncthreads();
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < HK; i++) {
                sj[i] = __fmul_rn(sj[i], decay);
                dot = __fadd_rn(dot, __fmul_rn(sj[i], s_k[i]));
            }
            const float delta = __fmul_rn(bet, __fsub_rn(vj, dot));
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < HK; i++) {
                sj[i] = __fadd_rn(sj[i], __fmul_rn(s_k[i], delta));
                acc = __fadd_rn(acc, __fmul_rn(sj[i], s_q[i]));
            }
            s_tmp[j] = acc;
            __syncthreads();
            if (j == 0) {
                float ss = 0.f;
                for (int r = 0; r < hv; r++) ss = __fadd_rn(ss, __fmul_rn(s_tmp[r], s_tmp[r]));
                s_rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)hv), p.rms_eps)));
            }
            __syncthreads();
            float o = __fmul_rn(acc, s_rstd);
            o = __fmul_rn(o, nw);
            o = __fmul_rn(o, __fdiv_rn(zj, __fadd_rn(1.0f, g_exp(-zj))));
            p.out[((int64_t)b * p.n_stride + t) * val_dim + (int64_t)vh * hv + j] = o;
        }
#pragma unroll
        for (int i = 0; i < HK; i += 4) *reinterpret_cast<float4 *>(Srow + i) = make_float4(sj[i], sj[i + 1], sj[i + 2], sj[i + 3]);
    }
}

}  // namespace

int cwk_gdn_scan_chunked(cwk_ctx *ctx, int B, int n_stride, int nchunks, int nh, int kv_group, const float *up, const float *gdec,
                         const float *beta, const float *gate, const float *a_log, const float *dt_bias, const float *norm,
                         float rms_eps, float *S, float *out);

extern "C" int cwk_gdn_scan(cwk_ctx *ctx, int B, int n, int nh, int head_k, int head_v, int kv_group, const float *up,
                            const float *gdec, const float *beta, const float *gate, const float *a_log, const float *dt_bias,
                            const float *norm, float rms_eps, float *S, float *out) {
    if (!ctx || !up || !gdec || !beta || !gate || !a_log || !dt_bias || !norm || !S || !out || B <= 0 || n <= 0 || nh <= 0 ||
        kv_group <= 0 || nh % kv_group)
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "gdn_scan: bad argument");
    if ((head_k != 64 && head_k != 128) || head_v < 32 || head_v > 128 || (head_v & 31))
        return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "gdn_scan is built for key dims 64, 128 and value dims 32..128 (got %d, %d)", head_k, head_v);
    if (reinterpret_cast<uintptr_t>(S) & 15) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "gdn_scan: the state must be 16-byte aligned");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    // A prompt (at least two chunks of 64 positions, head dims 128 x 128) goes through the chunk-parallel form; its last
    // n % 64 positions, decode steps and every other shape through the position-serial kernel, which keeps the
    // reference's summation order. cwk_ctx_force_mla_path(ctx, 0) keeps everything on the serial kernel.
    int done = 0;
    if (head_k == 128 && head_v == 128 && n >= 128 && ctx->force_mla_path != 0 && (reinterpret_cast<uintptr_t>(up) & 15) == 0) {
        const int nchunks = n / 64;
        int s = cwk_gdn_scan_chunked(ctx, B, n, nchunks, nh, kv_group, up, gdec, beta, gate, a_log, dt_bias, norm, rms_eps, S, out);
        if (s != CWK_OK) return s;
        done = nchunks * 64;
        if (done == n) return CWK_OK;
    }
    const int key_dim_h = (nh / kv_group) * head_k, val_dim_h = nh * head_v;
    GdnParams p;
    p.up = up + (int64_t)done * (2 * key_dim_h + val_dim_h); p.gdec = gdec + (int64_t)done * nh; p.beta = beta + (int64_t)done * nh;
    p.gate = gate + (int64_t)done * val_dim_h; p.a_log = a_log; p.dt_bias = dt_bias; p.norm = norm; p.S = S;
    p.out = out + (int64_t)done * val_dim_h;
    p.n = n - done; p.n_stride = n; p.nh = nh; p.kv_group = kv_group; p.rms_eps = rms_eps;
    const int nitems = B * nh;
    const int grid = std::min(nitems, 2 * ctx->sm_count);
    const size_t smem = (size_t)head_v * (head_k + 4) * sizeof(float);
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(gdn_scan_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 132 * 4));
        CWK_CUDA(ctx, cudaFuncSetAttribute(gdn_scan_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 68 * 4));
        attr_set[ctx->device & 15] = true;
    }
    CwkKernelTimer timer(ctx);
    if (head_k == 128) gdn_scan_kernel<128><<<grid, head_v, smem, ctx->stream>>>(p, nitems);
    else gdn_scan_kernel<64><<<grid, head_v, smem, ctx->stream>>>(p, nitems);
    CWK_LAUNCH_CHECK(ctx, "gdn_scan_kernel");
    return CWK_OK;
}
