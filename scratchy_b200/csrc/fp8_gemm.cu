// fp8-dynamic-per-channel: prefill GEMM on tcgen05 tensor cores (kind::f8f6f4).
// (placeholder: the dispatcher uses token tiles through the matvec kernel until enabled)
#include "fp8.cuh"

bool fp8_gemm_tc_enabled() { return false; }
size_t fp8_gemm_tc_workspace(int, int, int) { return 0; }
int32_t fp8_gemm_tc_launch(scr_ctx* ctx, const uint8_t*, const uint8_t*, uint16_t*, int, int, int, void*, size_t,
                           cudaStream_t) {
    return scr_fail(ctx, SCR_E_UNSUPPORTED, "tensor-core fp8 GEMM not built");
}
