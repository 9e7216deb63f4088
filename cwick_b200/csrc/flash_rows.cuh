// flash_rows.cuh -- one streaming-softmax kernel over "a block of query rows
// that share a key stream", written on mma.sync m16n8k16 (bf16 in, f32
// accumulate). It is the general-shape workhorse behind three entry points:
//
//   MODE_MLA      rows = the heads of one sequence; key = a [L|R] latent row,
//                 value = its first L elements (same shared-memory tile).
//   MODE_GQA_DEC  rows = the `group` query heads of one KV head (padded to 16).
//   MODE_GQA_PRE  rows = (query tokens x group heads) of one KV head, causal.
//
// Shared-memory tiles are rows of 16-byte chunks with chunk' = chunk ^ (row&7),
// which makes every ldmatrix phase bank-conflict free. K/V tiles arrive by
// cp.async into a ring of NSTAGE tile buffers (2, or 3 where the kernel has nothing
// but memory latency to hide: NSTAGE - 1 tiles are in flight while one is in use);
// a split of the key range ends in an un-normalised partial {m, l, o} per row, or
// (direct mode) in normalised bf16 rows.
#pragma once
#include "cwk_common.cuh"

enum { MODE_MLA = 0, MODE_GQA_DEC = 1, MODE_GQA_PRE = 2 };

struct FlashRowsParams {
    const uint16_t *q;
    const uint16_t *k;
    const uint16_t *v;        // == k for MODE_MLA
    int64_t seq_stride;       // elements between sequences in k / v
    int64_t ld;               // elements per cached row
    const int32_t *kv_len;    // [B] device (MLA, GQA_DEC); NULL -> kv_len_imm for every sequence
    int kv_len_imm;
    const int32_t *sel;       // optional row gather (MLA)
    int64_t sel_ld;
    int nh, nkv, group;
    float scale_log2;         // softmax scale * log2(e)
    float *partial;           // [B][nsplit][nh*(DV+2)]
    uint16_t *out;            // direct mode: bf16 rows
    int nsplit;
    int direct;
    int64_t pos;              // GQA_PRE
    int nq;                   // GQA_PRE
};

template <int HB, int DK, int DV, int TK, int NWARPS, bool SEP_V, int NSTAGE = 2>
struct FlashRowsSmem {
    static constexpr int KC = DK / 8, VC = DV / 8, PC = TK / 8;
    static constexpr int Q_BYTES = HB * DK * 2;
    static constexpr int K_BYTES = TK * DK * 2;
    static constexpr int V_BYTES = SEP_V ? TK * DV * 2 : 0;
    static constexpr int P_BYTES = HB * TK * 2;
    static constexpr int WM = HB / 16, WN = NWARPS / WM;
    static constexpr int STAT_BYTES = 2 * 2 * WN * HB * 4;   // [parity][max|sum][WN][HB]
    static constexpr int TOTAL = Q_BYTES + NSTAGE * (K_BYTES + V_BYTES) + P_BYTES + STAT_BYTES;
};

template <int MODE, int HB, int DK, int DV, int TK, int NWARPS, bool SEP_V, int NSTAGE = 2>
__global__ void __launch_bounds__(NWARPS * 32, 1) flash_rows_kernel(const FlashRowsParams p) {
    using SM = FlashRowsSmem<HB, DK, DV, TK, NWARPS, SEP_V, NSTAGE>;
    static_assert(NSTAGE >= 2 && NSTAGE <= 4, "ring of 2 to 4 tile buffers");
    constexpr int KC = SM::KC, VC = SM::VC, PC = SM::PC;
    constexpr int WM = SM::WM, WN = SM::WN;
    constexpr int NT_S = TK / WN / 8;      // score n-tiles per warp
    constexpr int NT_O = DV / WN / 8;      // output n-tiles per warp
    constexpr int NTHREADS = NWARPS * 32;
    static_assert((NT_S % 2 == 0 || NT_S == 1) && NT_O % 2 == 0, "n-tiles are consumed in pairs (a warp may own one score tile)");
    static_assert(KC % 8 == 0 && VC % 8 == 0 && PC % 8 == 0, "swizzle needs 8-chunk groups");

    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *sQ = smem;
    uint8_t *sK0 = sQ + SM::Q_BYTES;
    uint8_t *sP = sK0 + NSTAGE * (SM::K_BYTES + SM::V_BYTES);
    float *sStat = reinterpret_cast<float *>(sP + SM::P_BYTES);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp % WM, wn = warp / WM;
    const int split = blockIdx.x, by = blockIdx.y, b = blockIdx.z;

    // ---- what this block covers -------------------------------------------
    int limit_uniform = 0;          // keys visible to every row (MLA / GQA_DEC)
    int tile_begin = 0, tile_end = 0;
    int QT = 1;                     // query tokens per block (GQA_PRE)
    if (MODE == MODE_GQA_PRE) {
        QT = HB / p.group;
        int q_last = min(p.nq, (split + 1) * QT) - 1;         // last query token in block
        int kmax = (int)p.pos + q_last + 1;
        tile_begin = 0;
        tile_end = (kmax + TK - 1) / TK;
    } else {
        limit_uniform = p.kv_len ? p.kv_len[b] : p.kv_len_imm;
        int ntiles = (limit_uniform + TK - 1) / TK;
        tile_begin = (int)((int64_t)ntiles * split / p.nsplit);
        tile_end = (int)((int64_t)ntiles * (split + 1) / p.nsplit);
    }

    // ---- Q rows -> shared ----------------------------------------------------
    for (int idx = tid; idx < HB * KC; idx += NTHREADS) {
        int r = idx / KC, c = idx % KC;
        const uint16_t *src = nullptr;
        if (MODE == MODE_MLA) {
            int head = by * HB + r;
            if (head < p.nh) src = p.q + ((int64_t)b * p.nh + head) * DK;
        } else if (MODE == MODE_GQA_DEC) {
            if (r < p.group) src = p.q + ((int64_t)b * p.nh + by * p.group + r) * DK;
        } else {
            int qt = split * QT + r / p.group;
            if (qt < p.nq) src = p.q + ((int64_t)qt * p.nh + by * p.group + r % p.group) * DK;
        }
        uint32_t dst = smem_u32(sQ + r * (DK * 2) + ((c ^ (r & 7)) << 4));
        cp_async16(dst, src ? (const void *)(src + c * 8) : (const void *)p.q, src != nullptr);
    }

    const uint16_t *kbase = p.k + (int64_t)b * p.seq_stride;
    const uint16_t *vbase = p.v + (int64_t)b * p.seq_stride;
    const int head_off = (MODE == MODE_MLA) ? 0 : by * DK;   // GQA: this KV head's slice of the row
    const int key_limit_block = (MODE == MODE_GQA_PRE) ? tile_end * TK : limit_uniform;
    const int kmax_block = (MODE == MODE_GQA_PRE)
                               ? (int)p.pos + min(p.nq, (split + 1) * QT)
                               : limit_uniform;
    (void)key_limit_block;

    auto load_tile = [&](int t, int buf) {
        uint8_t *dK = sK0 + buf * (SM::K_BYTES + SM::V_BYTES);
        uint8_t *dV = dK + SM::K_BYTES;
        constexpr int TPR = NTHREADS / TK;          // threads per row
        const int r = tid / TPR, c0 = tid % TPR;
        const int j = t * TK + r;                   // position in the key list
        const bool valid = j < kmax_block;
        int64_t row = j;
        if ((MODE == MODE_MLA || MODE == MODE_GQA_DEC) && p.sel != nullptr && valid) row = p.sel[(int64_t)b * p.sel_ld + j];
        const uint16_t *ksrc = kbase + row * p.ld + head_off;
        for (int c = c0; c < KC; c += TPR)
            cp_async16(smem_u32(dK + r * (DK * 2) + ((c ^ (r & 7)) << 4)),
                       valid ? (const void *)(ksrc + c * 8) : (const void *)p.k, valid);
        if (SEP_V) {
            const uint16_t *vsrc = vbase + row * p.ld + by * DV;
            for (int c = c0; c < VC; c += TPR)
                cp_async16(smem_u32(dV + r * (DV * 2) + ((c ^ (r & 7)) << 4)),
                           valid ? (const void *)(vsrc + c * 8) : (const void *)p.k, valid);
        }
    };

#pragma unroll
    for (int i = 0; i < NSTAGE - 1; i++) {          // one commit group per tile, empty ones included, so that the counts line up
        if (tile_begin + i < tile_end) load_tile(tile_begin + i, i);
        cp_async_commit();
    }

    // ---- running state for this thread's two rows -----------------------------
    const int r0 = wm * 16 + (lane >> 2), r1 = r0 + 8;
    int lim0 = limit_uniform, lim1 = limit_uniform;
    if (MODE == MODE_GQA_PRE) {
        lim0 = (int)p.pos + split * QT + r0 / p.group + 1;
        lim1 = (int)p.pos + split * QT + r1 / p.group + 1;
    }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float acc[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    for (int t = tile_begin; t < tile_end; t++) {
        const int buf = (t - tile_begin) % NSTAGE, par = (t - tile_begin) & 1;
        cp_async_wait<NSTAGE - 2>();
        __syncthreads();                 // tile t landed; everyone is done with tile t-1, whose buffer takes tile t+NSTAGE-1
        if (t + NSTAGE - 1 < tile_end) load_tile(t + NSTAGE - 1, (buf + NSTAGE - 1) % NSTAGE);
        cp_async_commit();

        const uint8_t *tK = sK0 + buf * (SM::K_BYTES + SM::V_BYTES);
        const uint8_t *tV = SEP_V ? tK + SM::K_BYTES : tK;
        constexpr int VROW = SEP_V ? DV * 2 : DK * 2;

        // ---- S = Q K^T for rows wm*16.., tokens wn*(TK/WN).. -----------------
        float s[NT_S][4];
#pragma unroll
        for (int i = 0; i < NT_S; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        {
            const int arow = wm * 16 + (lane & 15);
            const uint32_t abase = smem_u32(sQ + arow * (DK * 2));
            const int axor = arow & 7;
#pragma unroll 4
            for (int ks = 0; ks < DK / 16; ks++) {
                uint32_t a[4];
                ldmatrix_x4(a[0], a[1], a[2], a[3], abase + (((ks * 2 + (lane >> 4)) ^ axor) << 4));
                if constexpr (NT_S == 1) {          // eight keys per warp: one n-tile, two 8 x 8 matrices per k-step
                    const int brow = wn * 8 + (lane & 7);
                    uint32_t b0, b1;
                    ldmatrix_x2(b0, b1, smem_u32(tK + brow * (DK * 2)) + (((ks * 2 + ((lane >> 3) & 1)) ^ (brow & 7)) << 4));
                    mma_bf16_16816(s[0], a, b0, b1);
                }
#pragma unroll
                for (int np = 0; np < NT_S / 2; np++) {
                    const int brow = wn * (TK / WN) + np * 16 + (lane & 7) + ((lane >> 4) << 3);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3,
                                smem_u32(tK + brow * (DK * 2)) +
                                    (((ks * 2 + ((lane >> 3) & 1)) ^ (brow & 7)) << 4));
                    mma_bf16_16816(s[np * 2], a, b0, b1);
                    mma_bf16_16816(s[np * 2 + 1], a, b2, b3);
                }
            }
        }

        // ---- scale, mask, tile row max -----------------------------------------
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < NT_S; nt++) {
            const int j = t * TK + wn * (TK / WN) + nt * 8 + (lane & 3) * 2;
            s[nt][0] = (j < lim0) ? s[nt][0] * p.scale_log2 : -INFINITY;
            s[nt][1] = (j + 1 < lim0) ? s[nt][1] * p.scale_log2 : -INFINITY;
            s[nt][2] = (j < lim1) ? s[nt][2] * p.scale_log2 : -INFINITY;
            s[nt][3] = (j + 1 < lim1) ? s[nt][3] * p.scale_log2 : -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        float *stMax = sStat + par * (2 * WN * HB);
        float *stSum = stMax + WN * HB;
        if ((lane & 3) == 0) {
            stMax[wn * HB + r0] = mx0;
            stMax[wn * HB + r1] = mx1;
        }
        __syncthreads();
        float mn0 = m0, mn1 = m1;
#pragma unroll
        for (int w = 0; w < WN; w++) {
            mn0 = fmaxf(mn0, stMax[w * HB + r0]);
            mn1 = fmaxf(mn1, stMax[w * HB + r1]);
        }
        const float alpha0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - mn0);
        const float alpha1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - mn1);
        const float sub0 = (mn0 == -INFINITY) ? 0.f : mn0;
        const float sub1 = (mn1 == -INFINITY) ? 0.f : mn1;

        // ---- P = exp2(S - m), row sums, P -> shared (bf16) ---------------------
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT_S; nt++) {
            const float p0 = exp2f(s[nt][0] - sub0), p1 = exp2f(s[nt][1] - sub0);
            const float p2 = exp2f(s[nt][2] - sub1), p3 = exp2f(s[nt][3] - sub1);
            sum0 += p0 + p1;
            sum1 += p2 + p3;
            const int tok = wn * (TK / WN) + nt * 8 + (lane & 3) * 2;
            *reinterpret_cast<uint32_t *>(sP + r0 * (TK * 2) + (((tok >> 3) ^ (r0 & 7)) << 4) +
                                          (tok & 7) * 2) = pack_bf16x2(p0, p1);
            *reinterpret_cast<uint32_t *>(sP + r1 * (TK * 2) + (((tok >> 3) ^ (r1 & 7)) << 4) +
                                          (tok & 7) * 2) = pack_bf16x2(p2, p3);
        }
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        if ((lane & 3) == 0) {
            stSum[wn * HB + r0] = sum0;
            stSum[wn * HB + r1] = sum1;
        }
        __syncthreads();
        float ts0 = 0.f, ts1 = 0.f;
#pragma unroll
        for (int w = 0; w < WN; w++) {
            ts0 += stSum[w * HB + r0];
            ts1 += stSum[w * HB + r1];
        }
        l0 = l0 * alpha0 + ts0;
        l1 = l1 * alpha1 + ts1;
        m0 = mn0;
        m1 = mn1;

        // ---- O = alpha*O + P V for rows wm*16.., dims wn*(DV/WN).. ------------
#pragma unroll
        for (int i = 0; i < NT_O; i++) {
            acc[i][0] *= alpha0; acc[i][1] *= alpha0;
            acc[i][2] *= alpha1; acc[i][3] *= alpha1;
        }
        {
            const int arow = wm * 16 + (lane & 15);
            const uint32_t pbase = smem_u32(sP + arow * (TK * 2));
            const int axor = arow & 7;
#pragma unroll
            for (int kt = 0; kt < TK / 16; kt++) {
                uint32_t a[4];
                ldmatrix_x4(a[0], a[1], a[2], a[3], pbase + (((kt * 2 + (lane >> 4)) ^ axor) << 4));
                const int vrow = kt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                const uint32_t vbase_s = smem_u32(tV + vrow * VROW);
                const int vxor = vrow & 7;
#pragma unroll
                for (int np = 0; np < NT_O / 2; np++) {
                    const int chunk = wn * (DV / WN / 8) + np * 2 + (lane >> 4);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, vbase_s + ((chunk ^ vxor) << 4));
                    mma_bf16_16816(acc[np * 2], a, b0, b1);
                    mma_bf16_16816(acc[np * 2 + 1], a, b2, b3);
                }
            }
        }
    }
    cp_async_wait<0>();

    // ---- epilogue ----------------------------------------------------------------
    const float LN2 = 0.6931471805599453f;
    auto row_target = [&](int r, int &head, int64_t &orow) -> bool {
        if (MODE == MODE_MLA) {
            head = by * HB + r;
            orow = (int64_t)b * p.nh + head;
            return head < p.nh;
        } else if (MODE == MODE_GQA_DEC) {
            head = by * p.group + r;
            orow = (int64_t)b * p.nh + head;
            return r < p.group;
        } else {
            int qt = split * QT + r / p.group;
            head = by * p.group + r % p.group;
            orow = (int64_t)qt * p.nh + head;
            return qt < p.nq;
        }
    };
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int r = half ? r1 : r0;
        const float m = half ? m1 : m0, l = half ? l1 : l0;
        int head;
        int64_t orow;
        if (!row_target(r, head, orow)) continue;
        if (p.direct) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            uint16_t *o = p.out + orow * DV + wn * (DV / WN) + (lane & 3) * 2;
#pragma unroll
            for (int nt = 0; nt < NT_O; nt++)
                *reinterpret_cast<uint32_t *>(o + nt * 8) =
                    pack_bf16x2(acc[nt][half * 2] * inv, acc[nt][half * 2 + 1] * inv);
        } else {
            float *rec = p.partial + ((int64_t)b * p.nsplit + split) * ((int64_t)p.nh * (DV + 2));
            if (wn == 0 && (lane & 3) == 0) {
                rec[head] = (m == -INFINITY) ? -INFINITY : m * LN2;
                rec[p.nh + head] = l;
            }
            float *o = rec + 2 * p.nh + (int64_t)head * DV + wn * (DV / WN) + (lane & 3) * 2;
#pragma unroll
            for (int nt = 0; nt < NT_O; nt++)
                *reinterpret_cast<float2 *>(o + nt * 8) =
                    make_float2(acc[nt][half * 2], acc[nt][half * 2 + 1]);
        }
    }
}

// ---------------------------------------------------------------------------
// Split merge. grid (nh, B, ceil(D/128)), 128 threads, one output column per thread. A short call
// is a chain of latencies, so the loads of the first 64 records' values go out before anything
// else: the weights e^(m_s-M) (two warp-shuffle reductions, one block barrier each) are computed
// while they are in flight. FOLD = false: normalised bf16 rows out[b][h][D].
// FOLD = true: one un-normalised record (same layout as the inputs) at rec_out.
// ---------------------------------------------------------------------------
constexpr int CWK_MAX_SPLITS = 512;

// CWK_MERGE_AHEAD: records whose values a thread loads before it needs the weights (a load from L2 outlasts everything
// else here): 64 for one sequence in many splits, 8 for many sequences in few (registers, hence blocks per SM).
template <bool FOLD, int CWK_MERGE_AHEAD>
static __global__ void __launch_bounds__(128) lse_merge_kernel(const float *partial, int nsplit, int nh, int D,
                                                               uint16_t *out, float *rec_out) {
    const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t rec_sz = (int64_t)nh * (D + 2);
    const float *base = partial + (int64_t)b * nsplit * rec_sz;
    __shared__ float sw[CWK_MAX_SPLITS];
    __shared__ float red[8];
    // value pass, part one: blockIdx.z picks a 128-column chunk of the row
    const float *orow = base + 2 * nh + (int64_t)h * D;
    const int i = blockIdx.z * 128 + tid;
    float v[CWK_MERGE_AHEAD];
#pragma unroll
    for (int s = 0; s < CWK_MERGE_AHEAD; s++) v[s] = (i < D && s < nsplit) ? orow[(int64_t)s * rec_sz + i] : 0.f;

    float mloc = -INFINITY;
    for (int s = tid; s < nsplit; s += 128) {
        const float l = base[s * rec_sz + nh + h];
        const float m = base[s * rec_sz + h];
        sw[s] = (l > 0.f) ? m : -INFINITY;
        if (l > 0.f) mloc = fmaxf(mloc, m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
    if (lane == 0) red[warp] = mloc;
    __syncthreads();
    const float M = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    float dloc = 0.f;
    for (int s = tid; s < nsplit; s += 128) {
        const float m = sw[s];
        const float w = (m == -INFINITY) ? 0.f : __expf(m - M);
        sw[s] = w;
        dloc += w * base[s * rec_sz + nh + h];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dloc += __shfl_xor_sync(0xffffffffu, dloc, o);
    if (lane == 0) red[4 + warp] = dloc;
    __syncthreads();
    const float den = (red[4] + red[5]) + (red[6] + red[7]);
    const float inv = FOLD ? 1.f : (den > 0.f ? 1.f / den : 0.f);
    if (FOLD && tid == 0 && blockIdx.z == 0) {
        rec_out[h] = M;
        rec_out[nh + h] = den;
    }
    if (i < D) {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < CWK_MERGE_AHEAD; s++)
            if (s < nsplit) a[s & 3] += sw[s] * v[s];
        for (int s0 = CWK_MERGE_AHEAD; s0 < nsplit; s0 += 16) {
            float u[16];
#pragma unroll
            for (int j = 0; j < 16; j++) u[j] = (s0 + j < nsplit) ? orow[(int64_t)(s0 + j) * rec_sz + i] : 0.f;
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (s0 + j < nsplit) a[j & 3] += sw[s0 + j] * u[j];
        }
        const float r = (a[0] + a[1]) + (a[2] + a[3]);
        if (FOLD) rec_out[2 * nh + (int64_t)h * D + i] = r;
        else out[((int64_t)b * nh + h) * D + i] = (uint16_t)(pack_bf16x2(r * inv, 0.f) & 0xffffu);
    }
}

static inline void lse_combine_launch(cudaStream_t st, const float *partial, int nsplit, int nh, int D, int B,
                                      uint16_t *out) {
    const dim3 grid(nh, B, (D + 127) / 128);
    if (nsplit > 32) lse_merge_kernel<false, 64><<<grid, 128, 0, st>>>(partial, nsplit, nh, D, out, nullptr);
    else if (nsplit > 8) lse_merge_kernel<false, 32><<<grid, 128, 0, st>>>(partial, nsplit, nh, D, out, nullptr);
    else lse_merge_kernel<false, 8><<<grid, 128, 0, st>>>(partial, nsplit, nh, D, out, nullptr);
}
static inline void lse_fold_launch(cudaStream_t st, const float *partial, int nsplit, int nh, int D, float *rec_out) {
    const dim3 grid(nh, 1, (D + 127) / 128);
    if (nsplit > 32) lse_merge_kernel<true, 64><<<grid, 128, 0, st>>>(partial, nsplit, nh, D, nullptr, rec_out);
    else lse_merge_kernel<true, 32><<<grid, 128, 0, st>>>(partial, nsplit, nh, D, nullptr, rec_out);
}
