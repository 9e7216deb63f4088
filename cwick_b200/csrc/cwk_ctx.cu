// cwk_ctx.cu -- context lifecycle, error text, scratch and staging buffers.
#include <cstdarg>

#include "cwk_common.cuh"

int cwk_fail(cwk_ctx *ctx, int status, const char *fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return status;
}

int cwk_check_cuda(cwk_ctx *ctx, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return CWK_OK;
    return cwk_fail(ctx, e == cudaErrorMemoryAllocation ? CWK_ERR_MEMORY : CWK_ERR_CUDA,
                    "%s: %s", what, cudaGetErrorString(e));
}

int cwk_reserve_scratch(cwk_ctx *ctx, size_t bytes) {
    if (bytes <= ctx->scratch_bytes) return CWK_OK;
    if (ctx->scratch) {
        CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        CWK_CUDA(ctx, cudaFree(ctx->scratch));
        ctx->scratch = nullptr;
        ctx->scratch_bytes = 0;
    }
    size_t want = bytes + (bytes >> 2);
    CWK_CUDA(ctx, cudaMalloc(&ctx->scratch, want));
    ctx->scratch_bytes = want;
    return CWK_OK;
}

int cwk_reserve_work(cwk_ctx *ctx, size_t bytes) {
    if (bytes <= ctx->work_bytes) return CWK_OK;
    if (ctx->work) {
        CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        CWK_CUDA(ctx, cudaFree(ctx->work));
        ctx->work = nullptr;
        ctx->work_bytes = 0;
    }
    CWK_CUDA(ctx, cudaMalloc(&ctx->work, bytes));
    ctx->work_bytes = bytes;
    return CWK_OK;
}

int cwk_reserve_stage(cwk_ctx *ctx, size_t dev_bytes, size_t pin_bytes) {
    if (dev_bytes > ctx->stage_dev_bytes) {
        if (ctx->stage_dev) {
            CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            CWK_CUDA(ctx, cudaFree(ctx->stage_dev));
            ctx->stage_dev = nullptr;
            ctx->stage_dev_bytes = 0;
        }
        CWK_CUDA(ctx, cudaMalloc(&ctx->stage_dev, dev_bytes));
        ctx->stage_dev_bytes = dev_bytes;
    }
    if (pin_bytes > ctx->stage_pin_bytes) {
        if (ctx->stage_pin) {
            CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            CWK_CUDA(ctx, cudaFreeHost(ctx->stage_pin));
            ctx->stage_pin = nullptr;
            ctx->stage_pin_bytes = 0;
        }
        CWK_CUDA(ctx, cudaMallocHost(&ctx->stage_pin, pin_bytes));
        ctx->stage_pin_bytes = pin_bytes;
    }
    return CWK_OK;
}

int cwk_ensure_err_word(cwk_ctx *ctx) {
    if (ctx->dev_err) return CWK_OK;
    CWK_CUDA(ctx, cudaHostAlloc((void **)&ctx->dev_err, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable));
    *ctx->dev_err = 0;
    return CWK_OK;
}

int cwk_check_device_error(cwk_ctx *ctx) {
    if (!ctx->dev_err) return CWK_OK;
    const int code = *(volatile int *)ctx->dev_err;      // call after a stream synchronise
    if (code == 0) return CWK_OK;
    *(volatile int *)ctx->dev_err = 0;
    cwk_sk_reset(ctx);          // accumulators and tickets of the persistent decode kernel may hold a half-finished step
    cudaStreamSynchronize(ctx->stream);
    return cwk_fail(ctx, CWK_ERR_STATE, "a kernel gave up a bounded wait (code %d); its results are invalid", code);
}

extern "C" {

int cwk_ctx_create(int device, cwk_ctx **out) {
    if (!out) return CWK_ERR_ARGUMENT;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) return CWK_ERR_STATE;
    if (device < 0 || device >= n) return CWK_ERR_ARGUMENT;
    if (cudaSetDevice(device) != cudaSuccess) return CWK_ERR_CUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return CWK_ERR_CUDA;
    if (prop.major != 10) return CWK_ERR_UNSUPPORTED;   // built for sm_100a only
    cwk_ctx *c = new cwk_ctx();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete c;
        return CWK_ERR_CUDA;
    }
    c->own_stream = true;
    *out = c;
    return CWK_OK;
}

void cwk_ctx_destroy(cwk_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->stage_dev) cudaFree(ctx->stage_dev);
    if (ctx->work) cudaFree(ctx->work);
    if (ctx->wbf16) cudaFree(ctx->wbf16);
    if (ctx->stage_pin) cudaFreeHost(ctx->stage_pin);
    if (ctx->dev_err) cudaFreeHost(ctx->dev_err);
    if (ctx->ticket) cudaFree(ctx->ticket);
    cwk_sk_free(ctx);
    cwk_fp8_weight_cache_free(ctx);
    for (cudaEvent_t e : ctx->ev) cudaEventDestroy(e);
    if (ctx->own_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

int cwk_ctx_set_stream(cwk_ctx *ctx, void *cuda_stream) {
    if (!ctx) return CWK_ERR_ARGUMENT;
    if (ctx->own_stream && ctx->stream) {
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
    }
    ctx->stream = (cudaStream_t)cuda_stream;
    ctx->own_stream = false;
    return CWK_OK;
}

int cwk_ctx_sync(cwk_ctx *ctx) {
    if (!ctx) return CWK_ERR_ARGUMENT;
    CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return cwk_check_device_error(ctx);
}

const char *cwk_last_error(const cwk_ctx *ctx) { return ctx ? ctx->err : "no context"; }
uint64_t cwk_ctx_launch_count(const cwk_ctx *ctx) { return ctx ? ctx->launches : 0; }
int cwk_ctx_sm_count(const cwk_ctx *ctx) { return ctx ? ctx->sm_count : 0; }

int cwk_ctx_profile(cwk_ctx *ctx, int on) {
    if (!ctx) return CWK_ERR_ARGUMENT;
    ctx->profiling = on != 0;
    return CWK_OK;
}

int cwk_ctx_profile_read(cwk_ctx *ctx, double *total_ms, int *launches) {
    if (!ctx || !total_ms || !launches) return CWK_ERR_ARGUMENT;
    CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    double t = 0.0;
    for (size_t i = 0; i + 1 < ctx->ev_used; i += 2) {
        float ms = 0.f;
        CWK_CUDA(ctx, cudaEventElapsedTime(&ms, ctx->ev[i], ctx->ev[i + 1]));
        t += ms;
    }
    *total_ms = t;
    *launches = (int)(ctx->ev_used / 2);
    ctx->ev_used = 0;
    return CWK_OK;
}

#ifdef CWK_TRACE
// Developer builds only (-DCWK_TRACE; not declared in the public header): a device buffer of at least 4096 bytes that
// block (0,0) of the split-record tcgen05 MLA decode kernel fills with clock64() stamps of its pipeline phases
// ([role 0..2][tile 0..15][event 0..7] as int64). NULL turns it off.
CWK_API int cwk_ctx_debug_trace(cwk_ctx *ctx, void *device_buffer);
int cwk_ctx_debug_trace(cwk_ctx *ctx, void *device_buffer) {
    if (!ctx) return CWK_ERR_ARGUMENT;
    ctx->tc_trace = device_buffer;
    return CWK_OK;
}
#endif

int cwk_ctx_weight_cache(cwk_ctx *ctx, size_t budget_bytes) {
    if (!ctx) return CWK_ERR_ARGUMENT;
    CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    cwk_fp8_weight_cache_free(ctx);
    ctx->wide_cache_budget = budget_bytes;
    return CWK_OK;
}

int cwk_ctx_set_wait_limit(cwk_ctx *ctx, unsigned int polls) {
    if (!ctx || polls == 0) return CWK_ERR_ARGUMENT;
    ctx->wait_limit = polls;
    return CWK_OK;
}

int cwk_ctx_force_mla_path(cwk_ctx *ctx, int path) {
    if (!ctx || path < -1 || path > 4) return CWK_ERR_ARGUMENT;     // 3: exact form of the prefill attention (cwk_mla_prefill only)
    ctx->force_mla_path = path;
    return CWK_OK;
}

}  // extern "C"
