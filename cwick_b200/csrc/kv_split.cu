// kv_split.cu -- one long context split by KV range across the GPUs of a node, with the
// partial-softmax exchange done by the kernels themselves over peer memory (NVLink): no
// collective library call in the step.
//
// Every rank owns a "window": for each of two epoch parities, `world` record slots
// {m[nh], l[nh], o[nh][L]} and `world` epoch words. A step on rank r is two launches:
//   1. the split-KV decode over the local rows -> split records in local scratch;
//   2. xchg_step_kernel, one block per (head, 128-column chunk): folds the splits into ONE
//      un-normalised record and stores its part of it into slot r of EVERY rank's window (plain
//      stores through peer pointers); the last block to have done so publishes the step's epoch
//      number in word r of every window (release, system scope); every block then waits
//      (bounded) until all `world` words of the OWN window carry the epoch and merges its part of
//      the `world` records -> bf16 output. All blocks of the launch are resident at once (256
//      blocks of 128 threads), so the block that publishes never waits for a block that waits.
// The records land in the consumer's own memory before it reads them; nothing reads remote
// memory, nothing is multicast. Kernels of different GPUs wait on each other, kernels on one
// GPU never do. A rank can be at most one step ahead of a peer (its next merge needs the peer's
// next push, which is ordered after the peer's current merge), hence two parities.
#include "flash_rows.cuh"

int cwk_mla_launch_splits(cwk_ctx *ctx, const void *q, const void *cache, int64_t ld, int rows, int nh, int L, int R,
                          float scale, float **partial_out, int *nsplit_out);

namespace {

constexpr int MAX_WORLD = 8;
struct PeerWindows {
    float *win[MAX_WORLD];
};

__host__ __device__ inline size_t window_rec_floats(int nh, int L) { return (size_t)nh * (L + 2); }
__host__ __device__ inline size_t window_half_bytes(int nh, int L, int world) {
    return (((size_t)world * window_rec_floats(nh, L) * 4 + 255) & ~(size_t)255) + 256;   // records + epoch words
}
__device__ __forceinline__ float *slot_ptr(float *win, int parity, int nh, int L, int world, int slot) {
    return reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(win) + parity * window_half_bytes(nh, L, world)) +
           (size_t)slot * window_rec_floats(nh, L);
}
__device__ __forceinline__ uint32_t *flag_ptr(float *win, int parity, int nh, int L, int world) {
    uint8_t *b = reinterpret_cast<uint8_t *>(win) + parity * window_half_bytes(nh, L, world);
    return reinterpret_cast<uint32_t *>(b + (((size_t)world * window_rec_floats(nh, L) * 4 + 255) & ~(size_t)255));
}

// grid (nh, D / 128), 128 threads: thread = one column of one head. AHEAD: split records whose values a thread loads
// before it needs their weights (a load from L2 outlasts everything else here).
template <int AHEAD>
__global__ void __launch_bounds__(128) xchg_step_kernel(const float *partial, int nsplit, int nh, int D, PeerWindows pw, int rank,
                                                        int world, uint32_t epoch, unsigned int *ticket, uint16_t *out, int *err,
                                                        unsigned int wait_limit) {
    const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int i = blockIdx.y * 128 + tid;
    const int64_t rec_sz = (int64_t)nh * (D + 2);
    __shared__ float sw[CWK_MAX_SPLITS];
    __shared__ float red[8];
    __shared__ int s_ok;
    // ---- fold the local splits: this thread's column of every record, the head's weights
    const float *orow = partial + 2 * nh + (int64_t)h * D;
    float v[AHEAD];
#pragma unroll
    for (int s = 0; s < AHEAD; s++) v[s] = (i < D && s < nsplit) ? orow[(int64_t)s * rec_sz + i] : 0.f;
    float mloc = -INFINITY;
    for (int s = tid; s < nsplit; s += 128) {
        const float l = partial[s * rec_sz + nh + h], m = partial[s * rec_sz + h];
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
        const float w = (sw[s] == -INFINITY) ? 0.f : __expf(sw[s] - M);
        sw[s] = w;
        dloc += w * partial[s * rec_sz + nh + h];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dloc += __shfl_xor_sync(0xffffffffu, dloc, o);
    if (lane == 0) red[4 + warp] = dloc;
    __syncthreads();
    const float den = (red[4] + red[5]) + (red[6] + red[7]);
    float r = 0.f;
    if (i < D) {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < AHEAD; s++)
            if (s < nsplit) a[s & 3] += sw[s] * v[s];
        for (int s0 = AHEAD; s0 < nsplit; s0 += 16) {
            float u[16];
#pragma unroll
            for (int j = 0; j < 16; j++) u[j] = (s0 + j < nsplit) ? orow[(int64_t)(s0 + j) * rec_sz + i] : 0.f;
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (s0 + j < nsplit) a[j & 3] += sw[s0 + j] * u[j];
        }
        r = (a[0] + a[1]) + (a[2] + a[3]);
    }
    // ---- this block's part of the folded record into every rank's window
    const int parity = (int)(epoch & 1u);
    for (int g = 0; g < world; g++) {
        float *dst = slot_ptr(pw.win[g], parity, nh, D, world, rank);
        if (i < D) dst[2 * nh + (int64_t)h * D + i] = r;
        if (blockIdx.y == 0 && tid == 0) {
            dst[h] = M;
            dst[nh + h] = den;
        }
    }
    // ---- publish once every block's stores are out
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        const unsigned int t = atomicAdd(ticket, 1u);
        if (t == gridDim.x * gridDim.y - 1) {
            *ticket = 0;
            __threadfence_system();
            for (int g = 0; g < world; g++) {
                uint32_t *f = flag_ptr(pw.win[g], parity, nh, D, world) + rank;
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
            }
        }
        // ---- wait (bounded) for every rank's record in the OWN window
        const uint32_t *f = flag_ptr(pw.win[rank], parity, nh, D, world);
        int ok = 1;
        for (int g = 0; g < world && ok; g++) {
            uint32_t fv = 0;
            unsigned int spins = 0;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(fv) : "l"(f + g) : "memory");
                if (fv == epoch) break;
                if (++spins > wait_limit) { ok = 0; break; }      // default ~1 s: a peer never published
                __nanosleep(100);
            }
        }
        if (!ok) atomicCAS(err, 0, 701);
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
    // ---- merge the ranks' records: this thread's column
    const float *base = slot_ptr(pw.win[rank], parity, nh, D, world, 0);
    float ov[MAX_WORLD], mv[MAX_WORLD], lv[MAX_WORLD];
#pragma unroll
    for (int g = 0; g < MAX_WORLD; g++) {
        const bool in = g < world && i < D;
        ov[g] = in ? __ldcg(base + g * rec_sz + 2 * nh + (int64_t)h * D + i) : 0.f;
        mv[g] = in ? __ldcg(base + g * rec_sz + h) : -INFINITY;
        lv[g] = in ? __ldcg(base + g * rec_sz + nh + h) : 0.f;
    }
    float M2 = -INFINITY;
#pragma unroll
    for (int g = 0; g < MAX_WORLD; g++)
        if (lv[g] > 0.f) M2 = fmaxf(M2, mv[g]);
    float den2 = 0.f, acc = 0.f;
#pragma unroll
    for (int g = 0; g < MAX_WORLD; g++) {
        const float w = lv[g] > 0.f ? __expf(mv[g] - M2) : 0.f;
        den2 += w * lv[g];
        acc += w * ov[g];
    }
    const float res = den2 > 0.f ? acc / den2 : 0.f;
    // two columns per store
    const float nb = __shfl_down_sync(0xffffffffu, res, 1);
    if ((lane & 1) == 0 && i < D) *reinterpret_cast<uint32_t *>(out + (int64_t)h * D + i) = pack_bf16x2(res, nb);      // D is even
}

}  // namespace

extern "C" {

int cwk_xchg_create(cwk_ctx *ctx, int nh, int L, int world, void **window, size_t *bytes) {
    if (!ctx || !window || nh <= 0 || L <= 0 || world <= 0 || world > MAX_WORLD) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "xchg_create: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t b = 2 * window_half_bytes(nh, L, world);
    CWK_CUDA(ctx, cudaMalloc(window, b));
    CWK_CUDA(ctx, cudaMemset(*window, 0, b));
    if (bytes) *bytes = b;
    if (!ctx->ticket) {
        CWK_CUDA(ctx, cudaMalloc(&ctx->ticket, sizeof(unsigned int)));
        CWK_CUDA(ctx, cudaMemset(ctx->ticket, 0, sizeof(unsigned int)));
    }
    return CWK_OK;
}

int cwk_xchg_export(cwk_ctx *ctx, void *window, void *handle64) {
    if (!ctx || !window || !handle64) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "xchg_export: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    CWK_CUDA(ctx, cudaIpcGetMemHandle((cudaIpcMemHandle_t *)handle64, window));
    return CWK_OK;
}

int cwk_xchg_open(cwk_ctx *ctx, const void *handle64, void **peer_window) {
    if (!ctx || !handle64 || !peer_window) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "xchg_open: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    CWK_CUDA(ctx, cudaIpcOpenMemHandle(peer_window, h, cudaIpcMemLazyEnablePeerAccess));
    return CWK_OK;
}

int cwk_xchg_close(cwk_ctx *ctx, void *peer_window) {
    if (!ctx || !peer_window) return CWK_ERR_ARGUMENT;
    CWK_CUDA(ctx, cudaIpcCloseMemHandle(peer_window));
    return CWK_OK;
}

int cwk_xchg_destroy(cwk_ctx *ctx, void *window) {
    if (!ctx || !window) return CWK_ERR_ARGUMENT;
    CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    CWK_CUDA(ctx, cudaFree(window));
    return CWK_OK;
}

int cwk_mla_decode_kv_split(cwk_ctx *ctx, const void *q, const void *cache, int64_t ld, int64_t rows, int nh, int L, int R,
                            float scale, void *const *windows, int rank, int world, uint32_t epoch, void *out) {
    if (!ctx || !q || !cache || !windows || !out || rows < 0 || world <= 0 || world > MAX_WORLD || rank < 0 || rank >= world ||
        epoch == 0 || (L & 1))
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "mla_decode_kv_split: bad argument (epoch counts from 1)");
    {
        int es = cwk_ensure_err_word(ctx);
        if (es != CWK_OK) return es;
        if (!ctx->ticket) return cwk_fail(ctx, CWK_ERR_STATE, "mla_decode_kv_split: create the exchange window first");
    }
    float *partial = nullptr;
    int ns = 0;
    int s = cwk_mla_launch_splits(ctx, q, cache, ld, (int)rows, nh, L, R, scale, &partial, &ns);
    if (s != CWK_OK) return s;
    PeerWindows pw;
    for (int g = 0; g < MAX_WORLD; g++) pw.win[g] = (g < world) ? (float *)windows[g] : nullptr;
    const dim3 grid(nh, (L + 127) / 128);
    if (ns > 32)
        xchg_step_kernel<64><<<grid, 128, 0, ctx->stream>>>(partial, ns, nh, L, pw, rank, world, epoch, (unsigned int *)ctx->ticket,
                                                          (uint16_t *)out, ctx->dev_err, ctx->wait_limit);
    else
        xchg_step_kernel<32><<<grid, 128, 0, ctx->stream>>>(partial, ns, nh, L, pw, rank, world, epoch, (unsigned int *)ctx->ticket,
                                                          (uint16_t *)out, ctx->dev_err, ctx->wait_limit);
    CWK_LAUNCH_CHECK(ctx, "xchg_step_kernel");
    return CWK_OK;
}

}  // extern "C"
