// mla_decode_noalloc.cu -- MLA absorbed decode for callers that must not allocate.
//
// Some hosts of this library cannot reach cudaMalloc at the moment they need
// attention: an inference server that hands the whole device to its own arena
// at start-up and forbids later driver allocations, a request thread with a
// latency budget that a cudaMalloc's implicit device synchronisation would
// blow, or code running where allocation calls are simply not permitted. The
// regular entry point keeps its split-KV records in a buffer it grows with
// cudaMalloc on demand; this one keeps them in a fixed array that is part of
// the library image, so the call allocates nothing, ever.
//
// The price is a fixed ceiling (CWK_NOALLOC_SCRATCH_BYTES, held by every GPU
// that loads the library until the process exits) and no isolation between
// calls: all calls on a device share the one array.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <mutex>

#include "flash_rows.cuh"

#define CWK_NOALLOC_SCRATCH_BYTES (16u << 20)   // 16 MiB = 127 split records of 64 heads x (512+2) f32

// The split records live here. In HOST code this name is only a handle for
// cudaGetSymbolAddress -- it is not a device address and must never be passed
// to a kernel as a pointer.
static __device__ __align__(256) float g_noalloc_scratch[CWK_NOALLOC_SCRATCH_BYTES / sizeof(float)];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mu;
float *g_scratch_ptr[kMaxDevices] = {nullptr};   // device address of g_noalloc_scratch, per device
int g_sm_count[kMaxDevices] = {0};

int fail(char *err, size_t cap, int status, const char *fmt, ...) {
    if (err && cap) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, cap, fmt, ap);
        va_end(ap);
    }
    return status;
}

using Smem = FlashRowsSmem<64, 576, 512, 64, 8, false>;

// Once per device, with that device current: resolve the array's device address
// and raise the kernel's dynamic shared-memory limit. Neither call allocates.
int setup_device(int dev, char *err, size_t cap) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_scratch_ptr[dev]) return CWK_OK;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return fail(err, cap, CWK_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10) return fail(err, cap, CWK_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a", dev, prop.major, prop.minor);
    float *ptr = nullptr;
    e = cudaGetSymbolAddress((void **)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) return fail(err, cap, CWK_ERR_CUDA, "cudaGetSymbolAddress(g_noalloc_scratch): %s", cudaGetErrorString(e));
    e = cudaFuncSetAttribute(flash_rows_kernel<MODE_MLA, 64, 576, 512, 64, 8, false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::TOTAL);
    if (e != cudaSuccess) return fail(err, cap, CWK_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    g_sm_count[dev] = prop.multiProcessorCount;
    g_scratch_ptr[dev] = ptr;
    return CWK_OK;
}
}  // namespace

extern "C" int cwk_mla_decode_noalloc(void *cuda_stream, const void *q, const void *cache, int64_t seq_stride,
                                      int64_t ld, const int32_t *kv_len, int max_kv_len, int B, int nh,
                                      float scale, void *out, char *err, size_t err_cap) {
    constexpr int L = 512, R = 64;
    if (!q || !cache || !kv_len || !out || B <= 0 || nh <= 0 || max_kv_len < 0 || ld < L + R)
        return fail(err, err_cap, CWK_ERR_ARGUMENT, "mla_decode_noalloc: null pointer or bad dimension");
    if ((ld % 8) != 0 || (seq_stride % 8) != 0 || ((uintptr_t)cache % 16) != 0 || ((uintptr_t)q % 16) != 0)
        return fail(err, err_cap, CWK_ERR_ARGUMENT, "mla_decode_noalloc: q, cache, ld and seq_stride must be 16-byte aligned");
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return fail(err, err_cap, CWK_ERR_STATE, "mla_decode_noalloc: no current CUDA device");
    int s = setup_device(dev, err, err_cap);
    if (s != CWK_OK) return s;

    // How many split records fit, and how many splits that allows per sequence.
    const size_t rec_bytes = (size_t)nh * (L + 2) * sizeof(float);
    const int64_t max_records = (int64_t)(CWK_NOALLOC_SCRATCH_BYTES / rec_bytes);
    if (B > max_records)
        return fail(err, err_cap, CWK_ERR_ARGUMENT,
                    "mla_decode_noalloc: %d sequences x %d heads need %d split records of %zu bytes; the "
                    "static scratch holds %lld (%u bytes). Use cwk_mla_decode, or fewer sequences per call.",
                    B, nh, B, rec_bytes, (long long)max_records, CWK_NOALLOC_SCRATCH_BYTES);
    const int hblocks = (nh + 63) / 64;
    const int max_tiles = std::max(1, (max_kv_len + 63) / 64);
    const int ns_cap = (int)std::min<int64_t>(std::min(max_tiles, 256), max_records / B);
    int ns = 1;
    double best = 1e30;
    for (int c = 1; c <= ns_cap; c++) {
        const double waves = std::ceil((double)B * hblocks * c / g_sm_count[dev]);
        const double cost = waves * (std::ceil((double)max_tiles / c) + 1.5) + 0.02 * c;
        if (cost < best - 1e-9) { best = cost; ns = c; }
    }

    float *scratch = g_scratch_ptr[dev];          // the address cudaGetSymbolAddress returned
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    FlashRowsParams p{};
    p.q = (const uint16_t *)q; p.k = (const uint16_t *)cache; p.v = p.k;
    p.seq_stride = seq_stride; p.ld = ld; p.kv_len = kv_len; p.kv_len_imm = max_kv_len;
    p.sel = nullptr; p.sel_ld = 0; p.nh = nh; p.nkv = 1; p.group = nh;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.partial = scratch; p.out = nullptr; p.nsplit = ns; p.direct = 0;
    // Every record the merge reads is written in full by this launch (empty splits write
    // m = -inf, l = 0, o = 0), so nothing in the array has to be cleared first.
    flash_rows_kernel<MODE_MLA, 64, 576, 512, 64, 8, false><<<dim3(ns, hblocks, B), 256, Smem::TOTAL, stream>>>(p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(err, err_cap, CWK_ERR_CUDA, "flash_rows_kernel launch: %s", cudaGetErrorString(e));
    lse_combine_launch(stream, scratch, ns, nh, L, B, (uint16_t *)out);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(err, err_cap, CWK_ERR_CUDA, "lse_merge_kernel launch: %s", cudaGetErrorString(e));
    return CWK_OK;
}
