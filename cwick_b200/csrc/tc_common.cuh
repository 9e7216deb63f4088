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
// one thread standing in for `count` arrivals
__device__ __forceinline__ void mbar_arrive_n(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(count) : "memory");
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

// ---- tensor maps of the MLA decode kernels, cached per context ------------------------------------------------
// Encoding a tensor map costs about a microsecond of host time and a decode call needs three; a serving loop calls
// with the same few (pointer, shape) combinations over and over, so each context keeps the last 64 of each kind.
struct CwkMlaTmapKey {
    const void *ptr;
    int64_t a, b, c;
    int d;
    bool operator==(const CwkMlaTmapKey &o) const { return ptr == o.ptr && a == o.a && b == o.b && c == o.c && d == o.d; }
};
struct CwkMlaTmapEntry {
    CwkMlaTmapKey key;
    CUtensorMap m[2];
    bool used;
};
struct CwkMlaTmapCache {
    static constexpr int SLOTS = 64;
    CwkMlaTmapEntry q[SLOTS], kv[SLOTS];
    int next_q = 0, next_kv = 0;
    CwkMlaTmapCache() {
        for (int i = 0; i < SLOTS; i++) q[i].used = kv[i].used = false;
    }
};

// q as [64][B*64 heads][blocks] (one box = all column blocks of a sequence's 64 heads); the cache as
// [64][rows][blocks][sequences] with boxes of two column blocks (tm_kv) or three (tm_kr: blocks 6, 7 and the rope block).
// width = 576, or 512 for a rope-free latent (its ninth block is then out of range and reads as zeros).
inline int cwk_mla_tensor_maps(cwk_ctx *ctx, const void *q, const void *cache, int64_t seq_stride, int64_t ld, int max_kv_len,
                               int B, int width, const CUtensorMap **tm_q, const CUtensorMap **tm_kv, const CUtensorMap **tm_kr) {
    constexpr int NH_ = 64, NBLK_ = 9, TILE_ = 128;
    CwkEncodeTiledFn enc = cwk_encode_tiled_fn();
    if (!enc) return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled not available");
    if (!ctx->sk_tmaps) ctx->sk_tmaps = new CwkMlaTmapCache();
    CwkMlaTmapCache *tc = (CwkMlaTmapCache *)ctx->sk_tmaps;
    const cuuint64_t nblk = (cuuint64_t)(width / 64);
    {
        const CwkMlaTmapKey key{q, B, width, 0, 0};
        CwkMlaTmapEntry *e = nullptr;
        for (int i = 0; i < CwkMlaTmapCache::SLOTS; i++)
            if (tc->q[i].used && tc->q[i].key == key) { e = &tc->q[i]; break; }
        if (!e) {
            e = &tc->q[tc->next_q];
            tc->next_q = (tc->next_q + 1) % CwkMlaTmapCache::SLOTS;
            e->used = false;
            cuuint64_t dims[3] = {64, (cuuint64_t)B * NH_, nblk};
            cuuint64_t strides[2] = {(cuuint64_t)width * 2, 128};
            cuuint32_t box[3] = {64, NH_, NBLK_};
            cuuint32_t es[3] = {1, 1, 1};
            CUresult r = enc(&e->m[0], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(q), dims, strides, box, es,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled(q) failed: %d", (int)r);
            e->key = key;
            e->used = true;
        }
        *tm_q = &e->m[0];
    }
    const bool shared_cache = (seq_stride == 0);
    {
        const CwkMlaTmapKey key{cache, seq_stride, ld, max_kv_len, shared_cache ? -width : B * 1024 + width};
        CwkMlaTmapEntry *e = nullptr;
        for (int i = 0; i < CwkMlaTmapCache::SLOTS; i++)
            if (tc->kv[i].used && tc->kv[i].key == key) { e = &tc->kv[i]; break; }
        if (!e) {
            e = &tc->kv[tc->next_kv];
            tc->next_kv = (tc->next_kv + 1) % CwkMlaTmapCache::SLOTS;
            e->used = false;
            for (int pass = 0; pass < 2; pass++) {
                const cuuint64_t nb = shared_cache ? 1 : (cuuint64_t)B;
                cuuint64_t dims[4] = {64, (cuuint64_t)max_kv_len, nblk, nb};
                cuuint64_t strides[3] = {(cuuint64_t)ld * 2, 128,
                                         shared_cache ? (cuuint64_t)ld * 2 * (cuuint64_t)max_kv_len : (cuuint64_t)seq_stride * 2};
                cuuint32_t box[4] = {64, TILE_, pass == 0 ? 2u : 3u, 1};
                cuuint32_t es[4] = {1, 1, 1, 1};
                CUresult r = enc(&e->m[pass], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(cache), dims, strides, box, es,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                if (r != CUDA_SUCCESS) return cwk_fail(ctx, CWK_ERR_CUDA, "cuTensorMapEncodeTiled(cache) failed: %d", (int)r);
            }
            e->key = key;
            e->used = true;
        }
        *tm_kv = &e->m[0];
        *tm_kr = &e->m[1];
    }
    return CWK_OK;
}
