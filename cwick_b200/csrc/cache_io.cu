// cache_io.cu -- the device-resident caches in the reference's prefix-state layouts. The server's prefix cache
// stores a prefix as f32 rows per KV slot (cwick_prefix_state.keys [nslots][pos][lat_stride], src/pfx.h:40-60,
// written and read by src/pfx.c:561, :681); the Qwen3.5 snapshot stores bf16 rows per layer
// (q35_prefix_pack / _apply, src/q35_model.c:591-665). A bf16 cache on the device exports to and imports from
// both: widening is exact, narrowing follows either the reference's cache-row write (cwick_f32_to_bf16,
// src/util.c:202-210, which the latent path uses at src/attention.c:703-705) or round-to-nearest-even
// (q35_narrow_rows, src/q35_model.c:1558-1575). bf16 rows to bf16 rows is a strided copy.
// Rows travel through a device staging buffer in chunks of 16 MB, so the caller's host buffer may be pageable.
#include <algorithm>

#include "cwk_common.cuh"

namespace {

constexpr size_t IO_CHUNK = 16u << 20;

__global__ void widen_rows_kernel(const uint16_t *cache, int64_t ld, int64_t rows, int width, float *out) {
    const int64_t n = rows * width;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = bf16_bits_to_f32(cache[(i / width) * ld + (i % width)]);
}

__global__ void narrow_rows_kernel(const float *in, int64_t rows, int width, uint16_t *cache, int64_t ld, int rounding) {
    const int64_t n = rows * width;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t u = __float_as_uint(in[i]);
        const uint32_t odd = (u >> 16) & 1u;
        // rounding 1: the reference's increment bit15 + lsb (a truncation in effect); 0: 0x7fff + lsb (nearest even)
        const uint32_t inc = rounding ? (((u >> 15) & 1u) + odd) : (0x7FFFu + odd);
        cache[(i / width) * ld + (i % width)] = (uint16_t)((u + inc) >> 16);
    }
}

}  // namespace

extern "C" {

int cwk_cache_export_f32(cwk_ctx *ctx, const void *cache, int64_t ld, int64_t rows, int width, float *out_host) {
    if (!ctx || !cache || !out_host || rows < 0 || width <= 0 || ld < width) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "cache_export_f32: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const int64_t per = std::max<int64_t>(1, (int64_t)(IO_CHUNK / ((size_t)width * 4)));
    int s = cwk_reserve_work(ctx, (size_t)std::min(rows, per) * width * 4 + 16);
    if (s != CWK_OK) return s;
    for (int64_t r0 = 0; r0 < rows; r0 += per) {
        const int64_t nr = std::min(per, rows - r0);
        widen_rows_kernel<<<(unsigned)std::min<int64_t>((nr * width + 255) / 256, 4 * ctx->sm_count), 256, 0, ctx->stream>>>(
            (const uint16_t *)cache + r0 * ld, ld, nr, width, (float *)ctx->work);
        CWK_LAUNCH_CHECK(ctx, "widen_rows_kernel");
        CWK_CUDA(ctx, cudaMemcpyAsync(out_host + r0 * width, ctx->work, (size_t)nr * width * 4, cudaMemcpyDeviceToHost, ctx->stream));
        CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return CWK_OK;
}

int cwk_cache_import_f32(cwk_ctx *ctx, const float *in_host, int64_t rows, int width, void *cache, int64_t ld, int rounding) {
    if (!ctx || !cache || !in_host || rows < 0 || width <= 0 || ld < width || (rounding != 0 && rounding != 1))
        return cwk_fail(ctx, CWK_ERR_ARGUMENT, "cache_import_f32: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    const int64_t per = std::max<int64_t>(1, (int64_t)(IO_CHUNK / ((size_t)width * 4)));
    int s = cwk_reserve_work(ctx, (size_t)std::min(rows, per) * width * 4 + 16);
    if (s != CWK_OK) return s;
    for (int64_t r0 = 0; r0 < rows; r0 += per) {
        const int64_t nr = std::min(per, rows - r0);
        CWK_CUDA(ctx, cudaMemcpyAsync(ctx->work, in_host + r0 * width, (size_t)nr * width * 4, cudaMemcpyHostToDevice, ctx->stream));
        narrow_rows_kernel<<<(unsigned)std::min<int64_t>((nr * width + 255) / 256, 4 * ctx->sm_count), 256, 0, ctx->stream>>>(
            (const float *)ctx->work, nr, width, (uint16_t *)cache + r0 * ld, ld, rounding);
        CWK_LAUNCH_CHECK(ctx, "narrow_rows_kernel");
        CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));       // the staging buffer is reused by the next chunk
    }
    return CWK_OK;
}

int cwk_cache_copy_bf16(cwk_ctx *ctx, int to_device, void *host, void *cache, int64_t ld, int64_t rows, int width) {
    if (!ctx || !cache || !host || rows < 0 || width <= 0 || ld < width) return cwk_fail(ctx, CWK_ERR_ARGUMENT, "cache_copy_bf16: bad argument");
    CWK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (rows == 0) return CWK_OK;
    if (to_device)
        CWK_CUDA(ctx, cudaMemcpy2DAsync(cache, (size_t)ld * 2, host, (size_t)width * 2, (size_t)width * 2, (size_t)rows, cudaMemcpyHostToDevice, ctx->stream));
    else
        CWK_CUDA(ctx, cudaMemcpy2DAsync(host, (size_t)width * 2, cache, (size_t)ld * 2, (size_t)width * 2, (size_t)rows, cudaMemcpyDeviceToHost, ctx->stream));
    CWK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return CWK_OK;
}

}  // extern "C"
