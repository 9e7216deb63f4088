// tc_common.cuh -- helpers shared by the tcgen05/TMA kernels: bounded mbarrier waits, TMA tile
// loads, shared-memory and instruction descriptors, MMA issue/commit, TMEM load/store macros,
// and the driver entry point that encodes tensor maps.
#pragma once
#include <cuda.h>

#include "cwk_common.cuh"

namespace {

constexpr uint32_t WAIT_LIMIT = 1u << 22;   // try_wait iterations before a wait gives up

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait. Returns false (and records `code`) when it gives up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int *err, int code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++)
        if (mbar_try(bar, parity)) return true;
    atomicCAS(err, 0, code);
    return false;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *tm, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *tm, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst), "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tm, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(tm), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (Blackwell).
// addr / lbo / sbo in bytes. bits [0,14) addr>>4, [16,30) lbo>>4, [32,46) sbo>>4,
// [46,48) version = 1, [61,64) layout = 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor for kind::f16: f32 accumulate, bf16 A and B.
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, int a_mn, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}
// the same with the A operand in tensor memory (rows = lanes, two 16-bit elements per 32-bit column)
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

#define TMEM_LD16(arr, off, taddr)                                                                          \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];" \
                 : "=r"(arr[off + 0]), "=r"(arr[off + 1]), "=r"(arr[off + 2]), "=r"(arr[off + 3]),          \
                   "=r"(arr[off + 4]), "=r"(arr[off + 5]), "=r"(arr[off + 6]), "=r"(arr[off + 7]),          \
                   "=r"(arr[off + 8]), "=r"(arr[off + 9]), "=r"(arr[off + 10]), "=r"(arr[off + 11]),        \
                   "=r"(arr[off + 12]), "=r"(arr[off + 13]), "=r"(arr[off + 14]), "=r"(arr[off + 15])       \
                 : "r"(taddr))
#define TMEM_ST16(arr, off, taddr)                                                                          \
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};" \
                 ::"r"(arr[off + 0]), "r"(arr[off + 1]), "r"(arr[off + 2]), "r"(arr[off + 3]),              \
                   "r"(arr[off + 4]), "r"(arr[off + 5]), "r"(arr[off + 6]), "r"(arr[off + 7]),              \
                   "r"(arr[off + 8]), "r"(arr[off + 9]), "r"(arr[off + 10]), "r"(arr[off + 11]),            \
                   "r"(arr[off + 12]), "r"(arr[off + 13]), "r"(arr[off + 14]), "r"(arr[off + 15]),          \
                   "r"(taddr)                                                                               \
                 : "memory")


typedef CUresult (*CwkEncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                     const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver-entry-point lookup, so the library has no
// link-time dependency on libcuda.
inline CwkEncodeTiledFn cwk_encode_tiled_fn() {
    static CwkEncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (CwkEncodeTiledFn)p;
    }
    return fn;
}

// 2-D bf16 row-major tensor [rows][cols] (row stride ld elements), box [box_rows][64 cols], 128-byte swizzle.
inline bool cwk_make_tmap_bf16_2d(CUtensorMap *tm, const void *ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                                  uint32_t box_rows) {
    CwkEncodeTiledFn enc = cwk_encode_tiled_fn();
    if (!enc) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t es[2] = {1, 1};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims, strides, box, es,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace
