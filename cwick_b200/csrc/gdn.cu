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

#include "tc_common.cuh"

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

constexpr int GDN_ERR_TILE = 0x6d01;

// Byte offset, inside an item's state tile in shared memory, of the 16-byte piece `m` (key entries 4m .. 4m + 3) of value
// row `j`. The tile arrives by one TMA copy as hk / 32 column blocks of [hv rows][32 floats] under the 128-byte swizzle:
// a row of a block is 128 bytes, its 16-byte pieces permuted by the row's low three bits -- which also makes a
// thread-per-row access conflict-free (the eight lanes of a quarter warp cover all 32 banks).
__device__ __forceinline__ uint32_t gdn_piece(int j, int m, int hv) {
    return (uint32_t)((m >> 3) * hv * 128 + j * 128 + (((m & 7) ^ (j & 7)) << 4));
}

// One position's inputs of one item, as thread j holds them: its value row's v and gate entry, the head's decay and beta
// logits, and the entries j, j + hv, ... of the key head's q and k (the block shares those through shared memory).
template <int HK> struct GdnPos {
    static constexpr int PER = HK / 32;                                     // hv >= 32
    float q[PER], k[PER], v, z, gdec, beta, a_log, dt_bias;
};
template <int HK> __device__ __forceinline__ void gdn_fetch(const GdnParams &p, int item, int t, int j, int hv, GdnPos<HK> &r) {
    const int vh = item % p.nh, b = item / p.nh, kh = vh / p.kv_group;
    const int key_dim = (p.nh / p.kv_group) * HK, val_dim = p.nh * hv;
    const float *row = p.up + ((int64_t)b * p.n_stride + t) * (2 * key_dim + val_dim);
#pragma unroll
    for (int u = 0; u < GdnPos<HK>::PER; u++)
        if (j + u * hv < HK) {
            r.q[u] = __ldg(row + (int64_t)kh * HK + j + u * hv);
            r.k[u] = __ldg(row + key_dim + (int64_t)kh * HK + j + u * hv);
        }
    r.v = __ldg(row + 2 * key_dim + (int64_t)vh * hv + j);
    r.z = __ldg(p.gate + ((int64_t)b * p.n_stride + t) * val_dim + (int64_t)vh * hv + j);
    r.gdec = __ldg(p.gdec + ((int64_t)b * p.n_stride + t) * p.nh + vh);
    r.beta = __ldg(p.beta + ((int64_t)b * p.n_stride + t) * p.nh + vh);
    r.a_log = __ldg(p.a_log + vh);
    r.dt_bias = __ldg(p.dt_bias + vh);
}

// Persistent blocks: block g works on items g, g + G, ... (item = slot * nh + value head). An item's [hv][hk] state
// comes into shared memory by one TMA copy, is scanned there over the call's positions (a thread owns one value row:
// no other thread touches it), and goes back by one TMA copy. Few registers and one tile per block leave room for
// three blocks per SM, which is what overlaps one item's copies with another's arithmetic.
template <int HK>
__global__ void __launch_bounds__(128) gdn_scan_kernel(const __grid_constant__ CUtensorMap tm_s, const GdnParams p, int nitems, int *err) {
    extern __shared__ uint8_t s_dyn[];
    __shared__ __align__(16) float s_q[HK], s_k[HK], s_tmp[128];
    __shared__ float s_rstd;
    __shared__ __align__(8) uint64_t s_bar;
    const int j = threadIdx.x, hv = blockDim.x;
    const int val_dim = p.nh * hv;
    const float nw = p.norm[j];
    const uint32_t bar = smem_u32(&s_bar);
    const uint32_t tile = (smem_u32(s_dyn) + 1023u) & ~1023u;               // the swizzle pattern repeats every 1024 bytes
    uint8_t *tile_g = s_dyn + (tile - smem_u32(s_dyn));
    const int copier = hv > 32 ? 32 : 0;                                    // the thread that issues the tile copies
    if (j == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    uint32_t phase = 0;
    GdnPos<HK> nxt;
    if ((int)blockIdx.x < nitems) gdn_fetch<HK>(p, blockIdx.x, 0, j, hv, nxt);
    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int vh = item % p.nh, b = item / p.nh;
        if (j == copier) {
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the last write-back has left the tile
            mbar_expect_tx(bar, (uint32_t)(hv * HK * 4));
            tma_load_3d(tile, &tm_s, 0, item * hv, 0, bar);
        }
        for (int t = 0; t < p.n; t++) {
            const GdnPos<HK> cur = nxt;
            {                                                               // the next position's inputs, a position ahead
                const bool more = t + 1 < p.n;
                const int nitem = more ? item : item + (int)gridDim.x;
                if (nitem < nitems) gdn_fetch<HK>(p, nitem, more ? t + 1 : 0, j, hv, nxt);
            }
#pragma unroll
            for (int u = 0; u < GdnPos<HK>::PER; u++)
                if (j + u * hv < HK) { s_q[j + u * hv] = cur.q[u]; s_k[j + u * hv] = cur.k[u]; }
            const float vj = cur.v, zj = cur.z;
            const float ea = g_exp(cur.a_log);
            const float x = __fadd_rn(cur.gdec, cur.dt_bias);
            const float sp = x > 20.0f ? x : (float)log1p((double)g_exp(x));
            const float decay = g_exp(__fmul_rn(-ea, sp));
            const float bet = __fdiv_rn(1.0f, __fadd_rn(1.0f, g_exp(-cur.beta)));
            const float silu = __fdiv_rn(zj, __fadd_rn(1.0f, g_exp(-zj)));
            if (t == 0) {                                                   // the tile, under the loads and exps above
                mbar_wait(bar, phase, err, GDN_ERR_TILE);                   // on giving up: carries on, the host reports the call as failed
                phase ^= 1;
            }
            __syncthreads();
            float dot = 0.f;
#pragma unroll 8
            for (int m = 0; m < HK / 4; m++) {
                const float4 s4 = *reinterpret_cast<const float4 *>(tile_g + gdn_piece(j, m, hv));
                const float4 k4 = *reinterpret_cast<const float4 *>(s_k + 4 * m);
                dot = __fadd_rn(dot, __fmul_rn(__fmul_rn(s4.x, decay), k4.x));
                dot = __fadd_rn(dot, __fmul_rn(__fmul_rn(s4.y, decay), k4.y));
                dot = __fadd_rn(dot, __fmul_rn(__fmul_rn(s4.z, decay), k4.z));
                dot = __fadd_rn(dot, __fmul_rn(__fmul_rn(s4.w, decay), k4.w));
            }
            const float delta = __fmul_rn(bet, __fsub_rn(vj, dot));
            float acc = 0.f;
#pragma unroll 8
            for (int m = 0; m < HK / 4; m++) {
                float4 *sp4 = reinterpret_cast<float4 *>(tile_g + gdn_piece(j, m, hv));
                float4 s4 = *sp4;
                const float4 k4 = *reinterpret_cast<const float4 *>(s_k + 4 * m);
                const float4 q4 = *reinterpret_cast<const float4 *>(s_q + 4 * m);
                s4.x = __fadd_rn(__fmul_rn(s4.x, decay), __fmul_rn(k4.x, delta));
                s4.y = __fadd_rn(__fmul_rn(s4.y, decay), __fmul_rn(k4.y, delta));
                s4.z = __fadd_rn(__fmul_rn(s4.z, decay), __fmul_rn(k4.z, delta));
                s4.w = __fadd_rn(__fmul_rn(s4.w, decay), __fmul_rn(k4.w, delta));
                acc = __fadd_rn(acc, __fmul_rn(s4.x, q4.x));
                acc = __fadd_rn(acc, __fmul_rn(s4.y, q4.y));
                acc = __fadd_rn(acc, __fmul_rn(s4.z, q4.z));
                acc = __fadd_rn(acc, __fmul_rn(s4.w, q4.w));
                *sp4 = s4;
            }
            const bool last = t == p.n - 1;
            if (last) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the row, visible to the copy engine
            s_tmp[j] = acc;
            __syncthreads();
            if (last && j == copier) {                                      // the tile goes back under the output's arithmetic
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(&tm_s), "r"(0),
                             "r"(item * hv), "r"(0), "r"(tile)
                             : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            if (j == 0) {
                float ss = 0.f;
                for (int r = 0; r < hv; r += 4) {
                    const float4 a4 = *reinterpret_cast<const float4 *>(s_tmp + r);
                    ss = __fadd_rn(ss, __fmul_rn(a4.x, a4.x));
                    ss = __fadd_rn(ss, __fmul_rn(a4.y, a4.y));
                    ss = __fadd_rn(ss, __fmul_rn(a4.z, a4.z));
                    ss = __fadd_rn(ss, __fmul_rn(a4.w, a4.w));
                }
                s_rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)hv), p.rms_eps)));
            }
            __syncthreads();
            float o = __fmul_rn(acc, s_rstd);
            o = __fmul_rn(o, nw);
            o = __fmul_rn(o, silu);
            p.out[((int64_t)b * p.n_stride + t) * val_dim + (int64_t)vh * hv + j] = o;
        }
    }
    if (j == copier) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
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
    if ((int64_t)nitems * head_v > 0x7fffffffLL) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "gdn_scan: more than 2^31 state rows");
    const size_t smem = (size_t)head_v * head_k * sizeof(float) + 1024;   // + slack to align the tile to the swizzle period
    static int per_sm[16][2] = {{0}};                                   // resident blocks per SM, by device and key dim
    int &resident = per_sm[ctx->device & 15][head_k == 128];
    if (!resident) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(gdn_scan_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 128 * 4 + 1024));
        CWK_CUDA(ctx, cudaFuncSetAttribute(gdn_scan_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 64 * 4 + 1024));
        int nb = 0;
        if (head_k == 128) CWK_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, gdn_scan_kernel<128>, 128, 128 * 128 * 4 + 1024));
        else CWK_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, gdn_scan_kernel<64>, 128, 128 * 64 * 4 + 1024));
        resident = std::max(nb, 1);
    }
    const int grid = std::min(nitems, resident * ctx->sm_count);
    int es = cwk_ensure_err_word(ctx);
    if (es != CWK_OK) return es;
    // The state as [32 floats][rows = slot, head, value row][hk / 32 column blocks]; one box is one item's whole tile.
    CwkEncodeTiledFn enc = cwk_encode_tiled_fn();
    if (!enc) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled not available");
    CUtensorMap tm_s;
    {
        cuuint64_t dims[3] = {32, (cuuint64_t)nitems * head_v, (cuuint64_t)(head_k / 32)};
        cuuint64_t strides[2] = {(cuuint64_t)head_k * 4, 128};
        cuuint32_t box[3] = {32, (cuuint32_t)head_v, (cuuint32_t)(head_k / 32)};
        cuuint32_t es3[3] = {1, 1, 1};
        CUresult r = enc(&tm_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, S, dims, strides, box, es3, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled(state) failed: %d", (int)r);
    }
    CwkKernelTimer timer(ctx);
    if (head_k == 128) gdn_scan_kernel<128><<<grid, head_v, smem, ctx->stream>>>(tm_s, p, nitems, ctx->dev_err);
    else gdn_scan_kernel<64><<<grid, head_v, smem, ctx->stream>>>(tm_s, p, nitems, ctx->dev_err);
    CWK_LAUNCH_CHECK(ctx, "gdn_scan_kernel");
    return CWK_OK;
}
