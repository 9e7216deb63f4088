// ds_codec.cuh -- scalar codecs of the DeepSeek path shared by its kernels: E4M3 decode, bf16 rounding,
// and the reference encoder's E4M3 round trip (with its subnormal quirk).
#pragma once
#include "cwk_common.cuh"

__device__ __forceinline__ float e4m3f(uint32_t b) {
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    float mag;
    if (e == 0) mag = (float)m * 0.001953125f;
    else if (e == 15 && m == 7) mag = __int_as_float(0x7fc00000);
    else mag = __uint_as_float(((e + 120u) << 23) | (m << 20));
    return (b & 0x80u) ? -mag : mag;
}
__device__ __forceinline__ float bf16_round_rne(float v) {       // ds_bf16_round, src/ds_ops.c:89-96
    uint32_t u = __float_as_uint(v);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return __uint_as_float(u & 0xFFFF0000u);
}
// E4M3 round trip of a clamped value with the reference encoder's behaviour (src/ds_quant.c:102-128):
// round to nearest even; a subnormal whose mantissa carries to 8 comes back as zero.
__device__ __forceinline__ float e4m3_quantise_dequantise_ref(float v) {
    if (v == 0.f) return 0.f;
    const float a = fabsf(v);
    int ex;
    (void)frexpf(a, &ex);
    int e = ex - 1;
    float r;
    if (e < -6) {
        if (e < -10) return copysignf(0.f, v);
        const float qv = rintf(a * 512.f);
        r = (qv >= 8.f) ? 0.f : qv * 0.001953125f;      // the reference masks a carried mantissa to zero
    } else {
        float qv = rintf(ldexpf(a, 3 - e));
        if (qv == 16.f) { qv = 8.f; e++; }
        if (e > 8) { e = 8; qv = 14.f; }
        r = ldexpf(qv, e - 3);
    }
    return copysignf(r, v);
}
