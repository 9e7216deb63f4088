/* arm_neon.h -- stand-in for the ARM header, so that the reference's model files, which use NEON
 * intrinsics without a portable alternative, compile on this x86-64 host into oracle/_ref.
 * TEST INFRASTRUCTURE ONLY. Each intrinsic does, lane by lane, what the Arm C Language Extensions
 * define for it; the two whose rounding matters are vfmaq_f32 (one rounding per lane: fmaf) and
 * vaddvq_f32 (pairwise: (a0 + a1) + (a2 + a3), the FADDP, FADDP sequence). Nothing here is
 * arithmetic of this project's own choosing. Only the intrinsics those files use are defined. */
#ifndef CWK_ORACLE_ARM_NEON_SHIM_H
#define CWK_ORACLE_ARM_NEON_SHIM_H
#include <math.h>
#include <stdatomic.h>
#include <stdint.h>
#include <string.h>

/* GCC's atomic_fetch_add does not take floating types (clang's does, and the reference only uses it on
 * wall-clock profiling totals): an atomic compound assignment does the same job here. */
#undef atomic_fetch_add_explicit
#define atomic_fetch_add_explicit(p, v, order) __extension__({ __typeof__(+(v)) old_ = *(p); *(p) += (v); old_; })

typedef float float32x4_t __attribute__((vector_size(16)));
typedef uint32_t uint32x4_t __attribute__((vector_size(16)));
typedef uint16_t uint16x8_t __attribute__((vector_size(16)));
typedef uint16_t uint16x4_t __attribute__((vector_size(8)));
typedef uint8_t uint8x16_t __attribute__((vector_size(16)));
typedef uint8_t uint8x8_t __attribute__((vector_size(8)));
typedef struct { uint16_t h[4]; } float16x4_t;        /* IEEE half bit patterns */

#define NEON_FN static inline __attribute__((always_inline, unused))

NEON_FN float32x4_t vld1q_f32(const float *p) { float32x4_t v; memcpy(&v, p, 16); return v; }
NEON_FN void vst1q_f32(float *p, float32x4_t v) { memcpy(p, &v, 16); }
NEON_FN float32x4_t vdupq_n_f32(float x) { return (float32x4_t){x, x, x, x}; }
NEON_FN float32x4_t vaddq_f32(float32x4_t a, float32x4_t b) { return a + b; }
NEON_FN float32x4_t vmulq_f32(float32x4_t a, float32x4_t b) { return a * b; }
NEON_FN float32x4_t vmulq_n_f32(float32x4_t a, float b) { return a * (float32x4_t){b, b, b, b}; }
NEON_FN float32x4_t vfmaq_f32(float32x4_t a, float32x4_t b, float32x4_t c) {
    return (float32x4_t){fmaf(b[0], c[0], a[0]), fmaf(b[1], c[1], a[1]), fmaf(b[2], c[2], a[2]), fmaf(b[3], c[3], a[3])};
}
NEON_FN float32x4_t vfmaq_n_f32(float32x4_t a, float32x4_t b, float c) {
    return (float32x4_t){fmaf(b[0], c, a[0]), fmaf(b[1], c, a[1]), fmaf(b[2], c, a[2]), fmaf(b[3], c, a[3])};
}
NEON_FN float vaddvq_f32(float32x4_t a) { return (a[0] + a[1]) + (a[2] + a[3]); }

NEON_FN uint32x4_t vdupq_n_u32(uint32_t x) { return (uint32x4_t){x, x, x, x}; }
NEON_FN uint32x4_t vaddq_u32(uint32x4_t a, uint32x4_t b) { return a + b; }
NEON_FN uint32x4_t vandq_u32(uint32x4_t a, uint32x4_t b) { return a & b; }
#define vshrq_n_u32(a, n) ((a) >> (n))
NEON_FN uint32x4_t vreinterpretq_u32_f32(float32x4_t a) { uint32x4_t r; memcpy(&r, &a, 16); return r; }
NEON_FN float32x4_t vreinterpretq_f32_u32(uint32x4_t a) { float32x4_t r; memcpy(&r, &a, 16); return r; }
NEON_FN uint16x4_t vmovn_u32(uint32x4_t a) { return (uint16x4_t){(uint16_t)a[0], (uint16_t)a[1], (uint16_t)a[2], (uint16_t)a[3]}; }

NEON_FN uint16x8_t vld1q_u16(const uint16_t *p) { uint16x8_t v; memcpy(&v, p, 16); return v; }
NEON_FN uint16x4_t vld1_u16(const uint16_t *p) { uint16x4_t v; memcpy(&v, p, 8); return v; }
NEON_FN void vst1_u16(uint16_t *p, uint16x4_t v) { memcpy(p, &v, 8); }
NEON_FN uint16x8_t vdupq_n_u16(uint16_t x) { return (uint16x8_t){x, x, x, x, x, x, x, x}; }
NEON_FN uint16x8_t vaddq_u16(uint16x8_t a, uint16x8_t b) { return a + b; }
NEON_FN uint16x8_t vandq_u16(uint16x8_t a, uint16x8_t b) { return a & b; }
NEON_FN uint16x8_t vorrq_u16(uint16x8_t a, uint16x8_t b) { return a | b; }
#define vshlq_n_u16(a, n) ((a) << (n))
NEON_FN uint16x4_t vget_low_u16(uint16x8_t a) { return (uint16x4_t){a[0], a[1], a[2], a[3]}; }
NEON_FN uint16x4_t vget_high_u16(uint16x8_t a) { return (uint16x4_t){a[4], a[5], a[6], a[7]}; }
#define vshll_n_u16(a, n) ((uint32x4_t){(uint32_t)(a)[0] << (n), (uint32_t)(a)[1] << (n), (uint32_t)(a)[2] << (n), (uint32_t)(a)[3] << (n)})

NEON_FN uint8x8_t vld1_u8(const uint8_t *p) { uint8x8_t v; memcpy(&v, p, 8); return v; }
NEON_FN uint8x16_t vld1q_u8(const uint8_t *p) { uint8x16_t v; memcpy(&v, p, 16); return v; }
NEON_FN uint8x8_t vdup_n_u8(uint8_t x) { return (uint8x8_t){x, x, x, x, x, x, x, x}; }
NEON_FN uint8x8_t vand_u8(uint8x8_t a, uint8x8_t b) { return a & b; }
#define vshr_n_u8(a, n) ((a) >> (n))
NEON_FN uint16x8_t vmovl_u8(uint8x8_t a) { return (uint16x8_t){a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7]}; }
#define vshll_n_u8(a, n) ((uint16x8_t){(uint16_t)((uint16_t)(a)[0] << (n)), (uint16_t)((uint16_t)(a)[1] << (n)), (uint16_t)((uint16_t)(a)[2] << (n)), (uint16_t)((uint16_t)(a)[3] << (n)), \
                                      (uint16_t)((uint16_t)(a)[4] << (n)), (uint16_t)((uint16_t)(a)[5] << (n)), (uint16_t)((uint16_t)(a)[6] << (n)), (uint16_t)((uint16_t)(a)[7] << (n))})
NEON_FN uint8x8_t vqtbl1_u8(uint8x16_t t, uint8x8_t idx) {
    uint8x8_t r;
    for (int i = 0; i < 8; i++) r[i] = idx[i] < 16 ? t[idx[i]] : 0;
    return r;
}

NEON_FN float16x4_t vreinterpret_f16_u16(uint16x4_t a) { float16x4_t r; memcpy(&r, &a, 8); return r; }
NEON_FN float neon_shim_half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else { float f = ldexpf((float)man, -24); memcpy(&u, &f, 4); u |= sign; }
    } else if (exp == 31) u = sign | 0x7F800000u | (man << 13);
    else u = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}
NEON_FN float32x4_t vcvt_f32_f16(float16x4_t a) {
    return (float32x4_t){neon_shim_half_to_float(a.h[0]), neon_shim_half_to_float(a.h[1]), neon_shim_half_to_float(a.h[2]), neon_shim_half_to_float(a.h[3])};
}
#endif
