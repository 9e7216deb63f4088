// kv_split.cu -- one long context split by KV range across the GPUs of a node, with the
// partial-softmax exchange done by the kernels themselves over peer memory (NVLink): no
// collective library call in the step.
//
// Every rank owns a "window": for each of two epoch parities, `world` record slots
// {m[nh], l[nh], o[nh][L]} and `world` epoch words. A step on rank r is three launches:
//   1. the split-KV decode over the local rows -> split records in local scratch;
//   2. fold_push_kernel: folds the splits into ONE un-normalised record and stores it into
//      slot r of EVERY rank's window (plain stores through peer pointers), then publishes the
//      step's epoch number in word r of every window (release, system scope);
//   3. wait_merge_kernel: waits (bounded) until all `world` words of the OWN window carry the
//      epoch, then merges the `world` records -> bf16 output.
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

// grid (nh), 128 threads.
__global__ void __launch_bounds__(128) fold_push_kernel(const float *partial, int nsplit, int nh, int D, PeerWindows pw,
                                                        int rank, int world, uint32_t epoch, unsigned int *ticket) {
    const int h = blockIdx.x, tid = threadIdx.x;
    const int64_t rec_sz = (int64_t)nh * (D + 2);
    __shared__ float sw[CWK_MAX_SPLITS];
    __shared__ float red[128];
    float mloc = -INFINITY;
    for (int s = tid; s < nsplit; s += 128) {
        const float l = partial[s * rec_sz + nh + h], m = partial[s * rec_sz + h];
        sw[s] = (l > 0.f) ? m : -INFINITY;
        if (l > 0.f) mloc = fmaxf(mloc, m);
    }
    red[tid] = mloc;
    __syncthreads();
    for (int o = 64; o > 0; o >>= 1) { if (tid < o) red[tid] = fmaxf(red[tid], red[tid + o]); __syncthreads(); }
    const float M = red[0];
    __syncthreads();
    float dloc = 0.f;
    for (int s = tid; s < nsplit; s += 128) {
        const float w = (sw[s] == -INFINITY) ? 0.f : __expf(sw[s] - M);
        sw[s] = w;
        dloc += w * partial[s * rec_sz + nh + h];
    }
    red[tid] = dloc;
    __syncthreads();
    for (int o = 64; o > 0; o >>= 1) { if (tid < o) red[tid] += red[tid + o]; __syncthreads(); }
    const float den = red[0];
    const int parity = (int)(epoch & 1u);
    if (tid == 0)
        for (int g = 0; g < world; g++) {
            float *dst = slot_ptr(pw.win[g], parity, nh, D, world, rank);
            dst[h] = M;
            dst[nh + h] = den;
        }
    const float *orow = partial + 2 * nh + (int64_t)h * D;
    for (int i = tid * 2; i < D; i += 256) {
        float a0 = 0.f, a1 = 0.f;
        for (int s = 0; s < nsplit; s++) {
            const float2 o = *reinterpret_cast<const float2 *>(orow + s * rec_sz + i);
            a0 += sw[s] * o.x;
            a1 += sw[s] * o.y;
        }
        for (int g = 0; g < world; g++)
            *reinterpret_cast<float2 *>(slot_ptr(pw.win[g], parity, nh, D, world, rank) + 2 * nh + (int64_t)h * D + i) =
                make_float2(a0, a1);
    }
    // publish once every head's stores are out
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        const unsigned int t = atomicAdd(ticket, 1u);
        if (t == (unsigned int)nh - 1) {
            *ticket = 0;
            __threadfence_system();
            for (int g = 0; g < world; g++) {
                uint32_t *f = flag_ptr(pw.win[g], parity, nh, D, world) + rank;
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
            }
        }
    }
}

// grid (nh), 128 threads. Waits on the OWN window only.
__global__ void __launch_bounds__(128) wait_merge_kernel(float *own, int nh, int D, int world, uint32_t epoch, uint16_t *out,
                                                         int *err, unsigned int wait_limit) {
    const int h = blockIdx.x, tid = threadIdx.x;
    const int parity = (int)(epoch & 1u);
    __shared__ int s_ok;
    if (tid == 0) {
        const uint32_t *f = flag_ptr(own, parity, nh, D, world);
        int ok = 1;
        for (int g = 0; g < world && ok; g++) {
            uint32_t v = 0;
            unsigned int spins = 0;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f + g) : "memory");
                if (v == epoch) break;
                if (++spins > wait_limit) { ok = 0; break; }      // default ~1 s: a peer never published
                __nanosleep(200);
            }
        }
        if (!ok) atomicCAS(err, 0, 701);
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
    const float *base = slot_ptr(own, parity, nh, D, world, 0);
    const int64_t rec_sz = (int64_t)nh * (D + 2);
    float M = -INFINITY;
    for (int g = 0; g < world; g++)
        if (base[g * rec_sz + nh + h] > 0.f) M = fmaxf(M, base[g * rec_sz + h]);
    float w[MAX_WORLD], den = 0.f;
    for (int g = 0; g < world; g++) {
        const float l = base[g * rec_sz + nh + h];
        w[g] = l > 0.f ? __expf(base[g * rec_sz + h] - M) : 0.f;
        den += w[g] * l;
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    for (int i = tid * 2; i < D; i += 256) {
        float a0 = 0.f, a1 = 0.f;
        for (int g = 0; g < world; g++) {
            const float2 o = *reinterpret_cast<const float2 *>(base + g * rec_sz + 2 * nh + (int64_t)h * D + i);
            a0 += w[g] * o.x;
            a1 += w[g] * o.y;
        }
        *reinterpret_cast<uint32_t *>(out + (int64_t)h * D + i) = pack_bf16x2(a0 * inv, a1 * inv);
    }
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
    if (ns > 4) {
        // Many split records (a long local range): fold them with the wide merge kernel first (a block per head and
        // 128-column chunk, loads in flight 32 deep), so that the push kernel below, whose blocks walk the splits one
        // after another, has a single record left to send.
        float *folded = partial + (size_t)ns * window_rec_floats(nh, L);        // room behind the splits (reserved by the launch below)
        lse_fold_launch(ctx->stream, partial, ns, nh, L, folded);
        CWK_LAUNCH_CHECK(ctx, "lse_merge_kernel<fold>");
        partial = folded;
        ns = 1;
    }
    fold_push_kernel<<<nh, 128, 0, ctx->stream>>>(partial, ns, nh, L, pw, rank, world, epoch, (unsigned int *)ctx->ticket);
    CWK_LAUNCH_CHECK(ctx, "fold_push_kernel");
    wait_merge_kernel<<<nh, 128, 0, ctx->stream>>>((float *)windows[rank], nh, L, world, epoch, (uint16_t *)out, ctx->dev_err,
                                                 ctx->wait_limit);
    CWK_LAUNCH_CHECK(ctx, "wait_merge_kernel");
    return CWK_OK;
}

}  // extern "C"
