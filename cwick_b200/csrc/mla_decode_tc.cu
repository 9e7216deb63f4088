// mla_decode_tc.cu -- tcgen05/TMA MLA decode (placeholder until the kernel lands).
#include "cwk_common.cuh"

bool cwk_mla_decode_tc_available() { return false; }

int cwk_mla_decode_tc_launch(cwk_ctx *ctx, const void *, const void *, int64_t, int64_t, const int32_t *,
                             int, int, int, float, float *, int) {
    return cwk_fail(ctx, CWK_ERR_UNSUPPORTED, "tcgen05 MLA decode not built");
}
