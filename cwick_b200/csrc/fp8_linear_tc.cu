// fp8_linear_tc.cu -- tcgen05 block-scaled FP8 GEMM (placeholder until the kernel lands).
#include "cwk_common.cuh"

bool cwk_fp8_linear_tc_available() { return false; }

int cwk_fp8_linear_tc_launch(cwk_ctx *ctx, const void *, const void *, const float *, int64_t, int64_t,
                             int64_t, void *, int) {
    return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "tcgen05 FP8 GEMM not built");
}
