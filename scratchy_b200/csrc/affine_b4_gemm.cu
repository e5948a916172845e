// MLX affine int4 (group 64): prefill GEMM on tcgen05 tensor cores.  (placeholder: the
// dispatcher uses token tiles through the matvec kernel until this is enabled)
#include "affine_b4.cuh"

bool affine_b4_gemm_tc_enabled() { return false; }
size_t affine_b4_gemm_tc_workspace(int, int, int) { return 0; }
int32_t affine_b4_gemm_tc_launch(scr_ctx* ctx, const uint8_t*, const uint16_t*, uint16_t*, int, int, int, void*, size_t,
                                 cudaStream_t) {
    return scr_fail(ctx, SCR_E_UNSUPPORTED, "tensor-core int4 GEMM not built");
}
