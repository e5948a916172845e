// Shared host/device helpers for the sm_100a quantized-linear library.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <atomic>

#include "../../include/scratchy_cuda.h"

// What a forward call asks of a linear's epilogue, passed down as an argument (never parked in the context: a
// context may serve two streams).
struct LinearEnds {
    int out_f32 = 0;                         // unrounded f32 partial sums instead of bf16 (row-parallel linears)
    const uint16_t* bias = nullptr;          // the linear's own bias [N] (bf16), added in f32 before the one rounding
};

struct scr_ctx {
    int device = 0;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    std::atomic<long long> launches{0};
    int* dev_status = nullptr;      // device word: first bounded wait that ran out (0 = none)
    char err[256] = {0};
};

static inline int32_t scr_fail(scr_ctx* ctx, int32_t code, const char* fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

// Checks the launch that was just issued (configuration errors surface here; execution
// errors surface at the caller's next synchronisation).
static inline int32_t scr_check_launch(scr_ctx* ctx, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
    if (ctx) ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return SCR_OK;
}

static inline bool scr_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define SCR_REQUIRE_CTX(ctx) do { if (!(ctx)) return SCR_E_ARG; (ctx)->err[0] = 0; } while (0)

static inline int scr_ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- device-side load helpers -------------------------------------------------------
// Streaming 128-bit / 64-bit loads for weights that are read exactly once per call:
// read-only path, no L1 allocation.
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_v2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
// Activations: an ordinary (coherent, L1-allocating) 128-bit load.  They are written by the preceding kernel of the
// stream, and under programmatic dependent launch the reading kernel is alive before that kernel has finished, so
// the read-only path (whose contract is data constant for the kernel's lifetime) is not used for them.
__device__ __forceinline__ uint4 ld_act_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// Cached read-only 128-bit load: load-time constants only (norm gains, tables).
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
