// cwk_common.cuh -- shared device helpers and the context object.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstring>
#include <vector>

#include "../../include/cwk_attn.h"

struct cwk_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    // split-KV scratch: [B*heads_blocks][n_splits] partials, grown on demand
    float *scratch = nullptr;
    size_t scratch_bytes = 0;
    // workspace of the composite entry points (prefill): separate from the split scratch
    void *work = nullptr;
    size_t work_bytes = 0;
    // FP8 weights widened to bf16 for the tensor-core projection
    void *wbf16 = nullptr;
    size_t wbf16_bytes = 0;
    // ... and the widened copies kept across calls (fp8_linear_tc.cu), with their byte budget
    void *wide_cache = nullptr;
    size_t wide_cache_budget = 0;             // off until the caller says its weights are immutable (cwk_ctx_weight_cache)
    // staging for the *_host entry points
    void *stage_dev = nullptr;
    size_t stage_dev_bytes = 0;
    void *stage_pin = nullptr;
    size_t stage_pin_bytes = 0;
    uint64_t launches = 0;
    int force_mla_path = -1;
    bool keep_splits = false;   // internal: leave split records in scratch (no merge, no fold)
    int last_nsplit = 0;
    // optional event pairs around main kernels (cwk_ctx_profile)
    bool profiling = false;
    std::vector<cudaEvent_t> ev;      // pool, pairs (2i, 2i+1)
    size_t ev_used = 0;
    // device word written by kernels whose bounded waits gave up (0 = fine)
    int *dev_err = nullptr;
    // block ticket of the KV-split push kernel
    void *ticket = nullptr;
    // optional device buffer for the tcgen05 kernel's phase stamps (only in a -DCWK_TRACE build)
    void *tc_trace = nullptr;
    // persistent MLA decode kernel: accumulators + parked records + control words (one allocation, fixed size),
    // and its cache of encoded tensor maps
    void *sk_acc = nullptr;
    size_t sk_bytes = 0;
    void *sk_tmaps = nullptr;
    // iteration limit of the bounded device-side waits on a peer's flag (cwk_ctx_set_wait_limit)
    unsigned int wait_limit = 1u << 22;
    char err[512] = {0};
};

int cwk_fail(cwk_ctx *ctx, int status, const char *fmt, ...);
int cwk_check_cuda(cwk_ctx *ctx, cudaError_t e, const char *what);
int cwk_reserve_scratch(cwk_ctx *ctx, size_t bytes);
int cwk_reserve_stage(cwk_ctx *ctx, size_t dev_bytes, size_t pin_bytes);
int cwk_reserve_work(cwk_ctx *ctx, size_t bytes);
// After a stream synchronise: turn a kernel-side give-up code into CWK_ERR_STATE.
int cwk_check_device_error(cwk_ctx *ctx);
// Allocate the error word on first use: pinned, mapped host memory, so the host reads it without a copy.
int cwk_ensure_err_word(cwk_ctx *ctx);
// persistent MLA decode kernel (mla_decode_sk.cu): release its buffers; zero them after a failed step
void cwk_sk_free(cwk_ctx *ctx);
void cwk_fp8_weight_cache_free(cwk_ctx *ctx);
void cwk_sk_reset(cwk_ctx *ctx);

// Brackets a main-kernel launch with events when profiling is on.
struct CwkKernelTimer {
    cwk_ctx *ctx;
    explicit CwkKernelTimer(cwk_ctx *c) : ctx(c) {
        if (!ctx->profiling) return;
        if (ctx->ev_used + 2 > ctx->ev.size()) {
            cudaEvent_t a, b;
            cudaEventCreate(&a);
            cudaEventCreate(&b);
            ctx->ev.push_back(a);
            ctx->ev.push_back(b);
        }
        record(ctx->ev[ctx->ev_used]);
    }
    ~CwkKernelTimer() {
        if (!ctx->profiling) return;
        record(ctx->ev[ctx->ev_used + 1]);
        ctx->ev_used += 2;
    }
    // Inside a stream capture the record becomes an event-record node of the graph (the "external" form, whose time can
    // be read after a replay): a caller can time the kernels in the graph it actually replays.
    void record(cudaEvent_t e) {
        cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(ctx->stream, &st);
        cudaEventRecordWithFlags(e, ctx->stream, st == cudaStreamCaptureStatusActive ? cudaEventRecordExternal : cudaEventRecordDefault);
    }
};

#define CWK_CUDA(ctx, call)                                            \
    do {                                                               \
        int _s = cwk_check_cuda((ctx), (call), #call);                 \
        if (_s != CWK_OK) return _s;                                   \
    } while (0)

#define CWK_LAUNCH_CHECK(ctx, name)                                    \
    do {                                                               \
        (ctx)->launches++;                                             \
        int _s = cwk_check_cuda((ctx), cudaGetLastError(), name);      \
        if (_s != CWK_OK) return _s;                                   \
    } while (0)

// ---- device helpers ---------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) {
    return __uint_as_float(((uint32_t)b) << 16);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
    int sz = valid ? 16 : 0;   // src-size 0 -> the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3,
                                            uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t &r0, uint32_t &r1, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                                  uint32_t &r3, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
