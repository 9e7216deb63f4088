// gdn_chunk.cu -- the Gated DeltaNet scan of a PROMPT, chunk-parallel (head dims 128 x 128).
//
// lin_rec_heads (src/q35_model.c:1177-1264) walks the positions one after the other: per position and value
// head, S <- d S;  u = beta (v - S k);  S <- S + u k^T;  o = S q.  gdn.cu does the same, which is the right form
// for a decode step and the wrong one for a prompt: 4096 positions x two dependent 128-term sums each is
// 5 ms per layer on 32 of the 148 SMs. The recurrence is linear in S, so 64 positions can be taken at once:
// with G_t the running sum of log d inside the chunk and r(t, s) = exp(G_t - G_s),
//
//   A[t][s] = beta_t r(t, s) (k_t . k_s)  (s < t),      T = (I + A)^-1          (64 x 64, unit lower triangular)
//   W = T diag(beta e^G) K,    U~ = T diag(beta) V,     M[t][s] = r(t, s) (q_t . k_s)  (s <= t)
//
// depend on the chunk's inputs only (phase 1: every chunk of every head at the same time), and then per chunk,
// in order, with S0 the state at the chunk's start,
//
//   U = U~ - W S0^T,      O = diag(e^G) Q S0^T + M U,      S0^T <- e^(G_64) S0^T + K^T diag(e^(G_64 - G)) U
//
// (phase 2) are small matrix products. A value row of S never meets another one, so phase 2 runs one block per
// (head, 32 value columns): 4 x heads x slots blocks. Everything is f32 on the CUDA cores: the sums are formed in
// another order than the reference's, so results agree to rounding (a few 1e-6 relative), not bit for bit;
// the position-serial kernel stays the form for decode steps, short calls and a call's last n % 64 positions.
// A third pass applies the gated RMS norm over a head's 128 outputs.
#include <algorithm>

#include "cwk_common.cuh"

namespace {

constexpr int GC = 64;            // positions per chunk
constexpr int GD = 128;           // head_k = head_v
constexpr int GLD = GD + 4;       // padded rows of the [64][128] tiles: float4 reads of 8 rows cover all banks
constexpr int GJ = 32;            // value columns per phase-2 block

__device__ __forceinline__ float gc_exp(float x) { return (float)exp((double)x); }

struct GdnChunkParams {
    const float *up, *gdec, *beta, *gate, *a_log, *dt_bias, *norm;
    float *S, *out;
    float *ws;                    // per (slot, head, chunk): W [64][128] | U~ [64][128] | M [64][64] | G [64]
    int n_stride;                 // positions per slot in the caller's arrays
    int nchunks, nh, kv_group;
    float rms_eps;
};
constexpr int64_t WS_PER = (int64_t)GC * GD * 2 + GC * GC + GC;

__device__ __forceinline__ float *ws_of(const GdnChunkParams &p, int b, int vh, int c) {
    return p.ws + (((int64_t)b * p.nh + vh) * p.nchunks + c) * WS_PER;
}

// ---- phase 1: grid (chunk, value head, slot), 256 threads
__global__ void __launch_bounds__(256) gdn_chunk_prep_kernel(const GdnChunkParams p) {
    extern __shared__ float4 gsm4[];
    float *sK = reinterpret_cast<float *>(gsm4), *sQ = sK + GC * GLD, *sV = sQ;      // V takes Q's place once M is formed
    float *sA = sQ + GC * GLD, *sT = sA + GC * (GC + 1), *sG = sT + GC * (GC + 1), *sB = sG + GC;
    const int c = blockIdx.x, vh = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
    const int kh = vh / p.kv_group;
    const int key_dim = (p.nh / p.kv_group) * GD, val_dim = p.nh * GD, qkv_dim = 2 * key_dim + val_dim;
    const int64_t pos0 = (int64_t)b * p.n_stride + (int64_t)c * GC;
    for (int x = tid; x < GC * (GD / 4); x += 256) {
        const int t = x / (GD / 4), i4 = x % (GD / 4);
        const float *row = p.up + (pos0 + t) * qkv_dim;
        *reinterpret_cast<float4 *>(sQ + t * GLD + i4 * 4) = *reinterpret_cast<const float4 *>(row + (int64_t)kh * GD + i4 * 4);
        *reinterpret_cast<float4 *>(sK + t * GLD + i4 * 4) = *reinterpret_cast<const float4 *>(row + key_dim + (int64_t)kh * GD + i4 * 4);
    }
    if (tid < GC) {
        const float ea = gc_exp(p.a_log[vh]);
        const float x = p.gdec[(pos0 + tid) * p.nh + vh] + p.dt_bias[vh];
        const float sp = x > 20.0f ? x : (float)log1p((double)gc_exp(x));
        sG[tid] = -ea * sp;                                          // log of the position's decay
        sB[tid] = 1.0f / (1.0f + gc_exp(-p.beta[(pos0 + tid) * p.nh + vh]));
    }
    __syncthreads();
    if (tid == 0) {
        float g = 0.f;
        for (int t = 0; t < GC; t++) { g += sG[t]; sG[t] = g; }      // running sum inside the chunk
    }
    __syncthreads();
    float *w = ws_of(p, b, vh, c);
    float *wW = w, *wU = w + GC * GD, *wM = wU + GC * GD, *wG = wM + GC * GC;
    if (tid < GC) wG[tid] = sG[tid];
    // A (strictly lower) and M (lower, with the diagonal)
    for (int e = 0; e < 16; e++) {
        const int t = (tid >> 6) + 4 * e, s = tid & 63;
        float a = 0.f, m = 0.f;
        if (s <= t) {
            const float4 *kt = reinterpret_cast<const float4 *>(sK + t * GLD), *ks = reinterpret_cast<const float4 *>(sK + s * GLD);
            const float4 *qt = reinterpret_cast<const float4 *>(sQ + t * GLD);
            float kk = 0.f, qk = 0.f;
#pragma unroll 8
            for (int i = 0; i < GD / 4; i++) {
                const float4 x = ks[i], y = kt[i], z = qt[i];
                kk += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
                qk += x.x * z.x + x.y * z.y + x.z * z.z + x.w * z.w;
            }
            const float r = expf(sG[t] - sG[s]);
            m = r * qk;
            if (s < t) a = sB[t] * r * kk;
        }
        sA[t * (GC + 1) + s] = a;
        wM[t * GC + s] = m;
    }
    __syncthreads();
    // T = (I + A)^-1 by forward substitution: one thread per column, the column in registers (both loops unrolled, so every
    // index is a constant and the only chain is a row's sum). The other warps fetch V (times beta) into Q's place and
    // scale K by beta e^G meanwhile.
    if (tid < GC) {
        const int col = tid;
        float tc[GC];
#pragma unroll
        for (int t = 0; t < GC; t++) {
            float v = (t == col) ? 1.f : 0.f;
#pragma unroll
            for (int s = 0; s < t; s++) v -= sA[t * (GC + 1) + s] * tc[s];       // tc[s] = 0 above the diagonal
            tc[t] = (t < col) ? 0.f : v;
        }
#pragma unroll
        for (int t = 0; t < GC; t++) sT[t * (GC + 1) + col] = tc[t];
    } else {
        for (int x = tid - GC; x < GC * (GD / 4); x += 256 - GC) {
            const int t = x / (GD / 4), i4 = x % (GD / 4);
            const float bt = sB[t], be = bt * expf(sG[t]);
            float4 v = *reinterpret_cast<const float4 *>(p.up + (pos0 + t) * qkv_dim + 2 * key_dim + (int64_t)vh * GD + i4 * 4);
            v.x *= bt; v.y *= bt; v.z *= bt; v.w *= bt;
            *reinterpret_cast<float4 *>(sV + t * GLD + i4 * 4) = v;
            float4 k = *reinterpret_cast<float4 *>(sK + t * GLD + i4 * 4);
            k.x *= be; k.y *= be; k.z *= be; k.w *= be;
            *reinterpret_cast<float4 *>(sK + t * GLD + i4 * 4) = k;
        }
    }
    __syncthreads();
    // W = T K', U~ = T V' (lower-triangular T): thread = one column, 32 rows
    {
        const int i = tid & 127, tg = tid >> 7;
        for (int tt = 0; tt < 32; tt++) {
            const int t = tg * 32 + tt;
            float aw = 0.f, au = 0.f;
            for (int s = 0; s <= t; s++) {
                const float tv = sT[t * (GC + 1) + s];
                aw += tv * sK[s * GLD + i];
                au += tv * sV[s * GLD + i];
            }
            wW[t * GD + i] = aw;
            wU[t * GD + i] = au;
        }
    }
}

// ---- phase 2: grid (32-column block of the value dimension, value head, slot), 512 threads; chunks in order.
// The chunk's operands arrive by 16-byte asynchronous copies issued as soon as their buffer is free: W, Q, U~ and G of
// the next chunk after this chunk's first step, M after the second, K after the third; so a chunk's copies run under
// the arithmetic of the chunk before.
constexpr int GUL = GJ + 4;       // row stride of the U tiles (16-byte aligned rows)
constexpr int GML = GC + 4;       // row stride of M
constexpr int GT2 = 512;          // threads of a phase-2 block

__device__ __forceinline__ void gc_cp16(float *dst, const float *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void gc_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

__global__ void __launch_bounds__(GT2) gdn_chunk_scan_kernel(const GdnChunkParams p) {
    extern __shared__ float4 gsm4[];
    float *sS = reinterpret_cast<float *>(gsm4);          // S0^T block [128 key][33]
    float *sW = sS + GD * (GJ + 1);                       // [64][132]
    float *sQ = sW + GC * GLD, *sK = sQ + GC * GLD;       // [64][132] each
    float *sU0 = sK + GC * GLD;                           // two [64][36] tiles: U~ of this chunk (then U, then U scaled) and of the next
    float *sM = sU0 + 2 * GC * GUL;                       // [64][68]
    float *sG = sM + GC * GML;                            // [64] running log decay, then [64] e^G, [64] e^(G_last - G)
    float *sE = sG + GC, *sF = sE + GC;
    const int jb = blockIdx.x, vh = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
    const int kh = vh / p.kv_group;
    const int key_dim = (p.nh / p.kv_group) * GD, val_dim = p.nh * GD, qkv_dim = 2 * key_dim + val_dim;
    float *Sh = p.S + (((int64_t)b * p.nh + vh) * GD + (int64_t)jb * GJ) * GD;       // rows jb*32 .. +31 of the head's [value][key] state
    auto issue_wqug = [&](int c) {
        if (c < p.nchunks) {
            const int64_t pos0 = (int64_t)b * p.n_stride + (int64_t)c * GC;
            const float *w = ws_of(p, b, vh, c);
            float *su = sU0 + (c & 1) * GC * GUL;
            for (int x = tid; x < GC * (GD / 4); x += GT2) {
                const int t = x / (GD / 4), i4 = x % (GD / 4);
                gc_cp16(sW + t * GLD + i4 * 4, w + t * GD + i4 * 4);
                gc_cp16(sQ + t * GLD + i4 * 4, p.up + (pos0 + t) * qkv_dim + (int64_t)kh * GD + i4 * 4);
            }
            for (int x = tid; x < GC * (GJ / 4); x += GT2)
                gc_cp16(su + (x / (GJ / 4)) * GUL + (x % (GJ / 4)) * 4, w + GC * GD + (x / (GJ / 4)) * GD + jb * GJ + (x % (GJ / 4)) * 4);
            if (tid < GC / 4) gc_cp16(sG + tid * 4, w + 2 * GC * GD + GC * GC + tid * 4);
        }
        gc_commit();
    };
    auto issue_m = [&](int c) {
        if (c < p.nchunks) {
            const float *wM = ws_of(p, b, vh, c) + 2 * GC * GD;
            for (int x = tid; x < GC * (GC / 4); x += GT2) gc_cp16(sM + (x / (GC / 4)) * GML + (x % (GC / 4)) * 4, wM + (x / (GC / 4)) * GC + (x % (GC / 4)) * 4);
        }
        gc_commit();
    };
    auto issue_k = [&](int c) {
        if (c < p.nchunks) {
            const int64_t pos0 = (int64_t)b * p.n_stride + (int64_t)c * GC;
            for (int x = tid; x < GC * (GD / 4); x += GT2) {
                const int t = x / (GD / 4), i4 = x % (GD / 4);
                gc_cp16(sK + t * GLD + i4 * 4, p.up + (pos0 + t) * qkv_dim + key_dim + (int64_t)kh * GD + i4 * 4);
            }
        }
        gc_commit();
    };
    issue_wqug(0);
    issue_m(0);
    issue_k(0);
    for (int x = tid; x < GJ * GD; x += GT2) {
        const int jj = x / GD, i = x % GD;
        sS[i * (GJ + 1) + jj] = Sh[(int64_t)jj * GD + i];
    }
    const int jj = tid & 31, grp = tid >> 5;               // 16 warps: two per scheduler would leave shared-memory latency exposed
    for (int c = 0; c < p.nchunks; c++) {
        const int64_t pos0 = (int64_t)b * p.n_stride + (int64_t)c * GC;
        float *sU = sU0 + (c & 1) * GC * GUL;
        asm volatile("cp.async.wait_group 1;" ::: "memory");      // W, Q, U~, G and M of this chunk (K may still be on its way)
        __syncthreads();
        if (tid < GC) {
            const float gt = sG[tid], gl = sG[GC - 1];
            sE[tid] = expf(gt);
            sF[tid] = expf(gl - gt);
        }
        // step 1: W S0^T and Q S0^T, rows t = grp + 16 e, column jj
        float u[4], o[4];
#pragma unroll
        for (int e = 0; e < 4; e++) { u[e] = 0.f; o[e] = 0.f; }
        for (int i = 0; i < GD; i += 4) {
            const float s0 = sS[(i + 0) * (GJ + 1) + jj], s1 = sS[(i + 1) * (GJ + 1) + jj], s2 = sS[(i + 2) * (GJ + 1) + jj],
                        s3 = sS[(i + 3) * (GJ + 1) + jj];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int t = grp + 16 * e;
                const float4 wv = *reinterpret_cast<const float4 *>(sW + t * GLD + i), qv = *reinterpret_cast<const float4 *>(sQ + t * GLD + i);
                u[e] += wv.x * s0 + wv.y * s1 + wv.z * s2 + wv.w * s3;
                o[e] += qv.x * s0 + qv.y * s1 + qv.z * s2 + qv.w * s3;
            }
        }
#pragma unroll
        for (int e = 0; e < 4; e++) {                      // U = U~ - W S0^T (a thread rewrites only what it alone reads)
            const int t = grp + 16 * e;
            u[e] = sU[t * GUL + jj] - u[e];
            sU[t * GUL + jj] = u[e];
        }
        __syncthreads();                                   // U complete; W, Q, G are free
        issue_wqug(c + 1);
        // step 2: O = e^G (Q S0^T) + M U
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int t = grp + 16 * e;
            float acc = sE[t] * o[e];
            for (int s = 0; s <= t; s++) acc += sM[t * GML + s] * sU[s * GUL + jj];
            p.out[(pos0 + t) * val_dim + (int64_t)vh * GD + jb * GJ + jj] = acc;
        }
        const float dl = sE[GC - 1];
        __syncthreads();                                   // U has been read in its plain form; M is free
        issue_m(c + 1);
        // step 3: S0^T <- e^(G_last) S0^T + K^T diag(e^(G_last - G)) U: scale U's rows once, then key rows i = grp * 8 .. + 7
        for (int x = tid; x < GC * GJ; x += GT2) sU[(x / GJ) * GUL + (x % GJ)] *= sF[x / GJ];
        asm volatile("cp.async.wait_group 2;" ::: "memory");      // K of this chunk (the next chunk's two groups may be pending)
        __syncthreads();
        float sacc[8];
#pragma unroll
        for (int e = 0; e < 8; e++) sacc[e] = dl * sS[(grp * 8 + e) * (GJ + 1) + jj];
#pragma unroll 4
        for (int s = 0; s < GC; s++) {
            const float us = sU[s * GUL + jj];
#pragma unroll
            for (int e4 = 0; e4 < 2; e4++) {
                const float4 kv = *reinterpret_cast<const float4 *>(sK + s * GLD + grp * 8 + e4 * 4);
                sacc[e4 * 4 + 0] += kv.x * us; sacc[e4 * 4 + 1] += kv.y * us; sacc[e4 * 4 + 2] += kv.z * us; sacc[e4 * 4 + 3] += kv.w * us;
            }
        }
#pragma unroll
        for (int e = 0; e < 8; e++) sS[(grp * 8 + e) * (GJ + 1) + jj] = sacc[e];      // (a thread rewrites only what it read)
        __syncthreads();                                   // K is free; the new state is in place
        issue_k(c + 1);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    for (int x = tid; x < GJ * GD; x += GT2) {
        const int j2 = x / GD, i = x % GD;
        Sh[(int64_t)j2 * GD + i] = sS[i * (GJ + 1) + j2];
    }
}

// ---- gated RMS norm over a head's 128 outputs, in place: grid (position, head, slot), 128 threads
__global__ void __launch_bounds__(128) gdn_chunk_norm_kernel(const GdnChunkParams p, int npos) {
    const int t = blockIdx.x, vh = blockIdx.y, b = blockIdx.z, j = threadIdx.x;
    const int val_dim = p.nh * GD;
    const int64_t at = ((int64_t)b * p.n_stride + t) * val_dim + (int64_t)vh * GD + j;
    const float o = p.out[at];
    __shared__ float red[4];
    float ss = o * o;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if ((j & 31) == 0) red[j >> 5] = ss;
    __syncthreads();
    ss = (red[0] + red[1]) + (red[2] + red[3]);
    const float rstd = 1.0f / sqrtf(ss / (float)GD + p.rms_eps);
    const float z = p.gate[at];
    p.out[at] = o * rstd * p.norm[j] * (z / (1.0f + gc_exp(-z)));
    (void)npos;
}

constexpr size_t PREP_SMEM = (size_t)(2 * GC * GLD + 2 * GC * (GC + 1) + 2 * GC) * sizeof(float);
constexpr size_t SCAN_SMEM = (size_t)(GD * (GJ + 1) + 3 * GC * GLD + 2 * GC * GUL + GC * GML + 3 * GC) * sizeof(float);

}  // namespace

// The first nchunks * 64 positions of every slot; the caller runs the position-serial kernel on the rest.
int cwk_gdn_scan_chunked(cwk_ctx *ctx, int B, int n_stride, int nchunks, int nh, int kv_group, const float *up, const float *gdec,
                         const float *beta, const float *gate, const float *a_log, const float *dt_bias, const float *norm,
                         float rms_eps, float *S, float *out) {
    const size_t ws_bytes = (size_t)B * nh * nchunks * WS_PER * sizeof(float);
    int s = cwk_reserve_work(ctx, ws_bytes);
    if (s != CWK_OK) return s;
    static bool attr_set[16] = {false};
    if (!attr_set[ctx->device & 15]) {
        CWK_CUDA(ctx, cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PREP_SMEM));
        CWK_CUDA(ctx, cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SCAN_SMEM));
        attr_set[ctx->device & 15] = true;
    }
    GdnChunkParams p;
    p.up = up; p.gdec = gdec; p.beta = beta; p.gate = gate; p.a_log = a_log; p.dt_bias = dt_bias; p.norm = norm; p.S = S; p.out = out;
    p.ws = (float *)ctx->work; p.n_stride = n_stride; p.nchunks = nchunks; p.nh = nh; p.kv_group = kv_group; p.rms_eps = rms_eps;
    gdn_chunk_prep_kernel<<<dim3(nchunks, nh, B), 256, PREP_SMEM, ctx->stream>>>(p);
    CWK_LAUNCH_CHECK(ctx, "gdn_chunk_prep_kernel");
    {
        CwkKernelTimer timer(ctx);
        gdn_chunk_scan_kernel<<<dim3(GD / GJ, nh, B), GT2, SCAN_SMEM, ctx->stream>>>(p);
        CWK_LAUNCH_CHECK(ctx, "gdn_chunk_scan_kernel");
    }
    gdn_chunk_norm_kernel<<<dim3(nchunks * GC, nh, B), 128, 0, ctx->stream>>>(p, nchunks * GC);
    CWK_LAUNCH_CHECK(ctx, "gdn_chunk_norm_kernel");
    return CWK_OK;
}
