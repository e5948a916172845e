// Device helpers of the int4 decode matvec kernels (affine_b4.cu: the matvec and the matvec tape):
// mbarrier / bulk-copy / shared-memory PTX wrappers, the bf16 MMA, one packed block against
// pre-loaded activations, and the output modes of the epilogue.
#pragma once

#include "affine_b4.cuh"

// ---- small PTX helpers for the matvec kernels ------------------------------------------
__device__ __forceinline__ uint32_t gemv_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gemv_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void gemv_fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void gemv_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gemv_bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Bounded wait on a stage barrier: gives up after 2^20 polls (or as soon as another waiter has
// recorded a failure), records code 6 in the status word and lets the kernel run to its end.
__device__ __forceinline__ void gemv_wait(uint32_t bar, uint32_t parity, int* status) {
#pragma unroll 1
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return;
        if ((i & 255u) == 255u && *reinterpret_cast<volatile int*>(status) != 0) return;
    }
    atomicCAS(status, 0, 6);
}
__device__ __forceinline__ uint4 gemv_lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 gemv_lds_v2(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t gemv_cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void gemv_cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void gemv_st_cluster_rank0_f32(const float* local_ptr, float v) {
    const uint32_t local = (uint32_t)__cvta_generic_to_shared(local_ptr);
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

__device__ __forceinline__ void mma_bf16_16816(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void gemv_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void gemv_consumer_sync() {          // the 8 consumer warps only
    asm volatile("bar.sync 1, 256;" ::: "memory");
}

#define GEMV_CWARPS 8
#define GEMV_THREADS ((GEMV_CWARPS + 1) * 32)
#define GEMV_STAGES 4
#define GEMV_STAGE_BYTES (GEMV_CWARPS * AFF_BLOCK_BYTES)
#define GEMV_MAX_SPLIT 8

// One 1152-byte block from shared memory against pre-loaded activations (xv: this lane's 32
// activations per token tile, in k order).
// GS: log2 of the (scale, bias) entries per row and block (1: groups of 64 or 128, 2: groups of 32).
template <int MT, bool CHECK, int GS = 1>
__device__ __forceinline__ void gemv_block_compute(uint32_t blk, float acc[2][MT][4], const uint4 xv[MT][4], int lane) {
    const uint4 p0 = gemv_lds_v4(blk + lane * 16);
    const uint4 p1 = gemv_lds_v4(blk + 512 + lane * 16);
    const uint2 sb = gemv_lds_v2(blk + 1024 + (((lane >> 2) << GS) + ((lane & 3) >> (2 - GS))) * 8);
    const uint32_t wa[4] = {p0.x, p0.y, p0.z, p0.w};
    const uint32_t wb[4] = {p1.x, p1.y, p1.z, p1.w};
    if (CHECK) {
        // generic variant: per-group test for the exact path; weights unscaled
        const uint32_t s2a = __byte_perm(sb.x, sb.x, 0x1010), b2a = __byte_perm(sb.x, sb.x, 0x3232);
        const uint32_t s2b = __byte_perm(sb.y, sb.y, 0x1010), b2b = __byte_perm(sb.y, sb.y, 0x3232);
        const bool slow_a = affine_slow_group(sb.x);
        const bool slow_b = affine_slow_group(sb.y);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t w0[4], w1[4];
            affine_dequant_word<true>(wa[i], sb.x, s2a, b2a, slow_a, w0);
            affine_dequant_word<true>(wb[i], sb.y, s2b, b2b, slow_b, w1);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_bf16_16816(acc[0][mt], w0[0], w1[0], w0[1], w1[1], xv[mt][i].x, xv[mt][i].y);
                mma_bf16_16816(acc[1][mt], w0[2], w1[2], w0[3], w1[3], xv[mt][i].z, xv[mt][i].w);
            }
        }
    } else {
        // scaled variant: weights carry a factor 2^-7 that the caller removes from the accumulators
        const AffineScaled ca = affine_scaled_consts(sb.x);
        const AffineScaled cb = affine_scaled_consts(sb.y);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t w0[4], w1[4];
            affine_dequant_word_scaled(wa[i], ca, w0);
            affine_dequant_word_scaled(wb[i], cb, w1);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                // two independent accumulator sets halve the dependent-MMA chain
                mma_bf16_16816(acc[0][mt], w0[0], w1[0], w0[1], w1[1], xv[mt][i].x, xv[mt][i].y);
                mma_bf16_16816(acc[1][mt], w0[2], w1[2], w0[3], w1[3], xv[mt][i].z, xv[mt][i].w);
            }
        }
    }
}

// Output modes of the matvec epilogue (the `out_f32` argument): bf16, unrounded f32 partials, or the
// gate/up pairing: the matrix holds, per 16-row block, 8 gate rows then the 8 up rows of the same
// channels (the loader's `load_rows_interleave8`), so gate_i and up_i end up in the same lane two
// accumulator slots apart; the lane holding the gate sum takes the up sum by shuffle and stores
// bf16(silu(bf16(gate)) * bf16(up)) — the value the separate silu*up kernel computes from the two
// bf16 outputs (crates/targets/metal/src/cpu_golden.rs:211-219), one launch saved.
#define GEMV_OUT_BF16 0
#define GEMV_OUT_F32 1
#define GEMV_OUT_SILU_PAIRS 2

// Called by all 32 lanes of a warp.  `total` is this lane's (row, token) sum; bit 1 of `idx` says
// whether the row is a gate row (0) or the up row 8 below it (1).
__device__ __forceinline__ void gemv_store_silu_pair(float total, int idx, int tok, int M, int channel, int channels,
                                                     uint16_t* __restrict__ y) {
    const float other = __shfl_xor_sync(0xffffffffu, total, 2);
    if ((idx & 2) == 0 && tok < M && channel < channels) {
        const float g = __bfloat162float(__float2bfloat16_rn(total));
        const float u = __bfloat162float(__float2bfloat16_rn(other));
        const __nv_bfloat16 v = __float2bfloat16_rn(__fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u));
        y[(size_t)tok * channels + channel] = *reinterpret_cast<const uint16_t*>(&v);
    }
}

