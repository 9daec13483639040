#include "common.cuh"
cq_status launch_gemm(cq_ctx *ctx, int, int, int, const float *, int64_t, int64_t, int64_t, const void *, int64_t, float *, int64_t) {
    return cq_fail(ctx, CQ_ERR_UNSUPPORTED, "prefill GEMM not built yet");
}
