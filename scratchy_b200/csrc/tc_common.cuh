// Blackwell (sm_100a) tensor-core plumbing shared by the prefill GEMMs: mbarriers with
// bounded waits, 1-D bulk (TMA) copies, TMEM allocation, tcgen05.mma / commit / ld and the
// shared-memory and instruction descriptors.  Inline PTX only; no multicast anywhere.
#pragma once

#include <cuda.h>

#include "common.cuh"

// Every wait in these kernels is bounded: after TC_WAIT_LIMIT failed polls the waiter records
// a code in the kernel's status word and carries on, and from then on every other wait gives
// up as soon as it sees the word set, so a broken pipeline drains quickly with garbage
// results and an error status instead of hanging the GPU.
#define TC_WAIT_LIMIT (1u << 20)

#define TC_ERR_FULL_WAIT   1
#define TC_ERR_EMPTY_WAIT  2
#define TC_ERR_ACC_FULL    3
#define TC_ERR_ACC_EMPTY   4
#define TC_ERR_DEQ_WAIT    5

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and records `code`) when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        // once any wait anywhere in the grid has run out, every later wait gives up at once
        if ((i & 255u) == 255u && *reinterpret_cast<volatile int*>(status) != 0) return false;
    }
    atomicCAS(status, 0, code);
    return false;
}

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// ---- TMEM ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {     // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {      // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, one CTA.  `accumulate` = 0 overwrites D.
__device__ __forceinline__ void umma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive f32 columns -> 32 registers per thread (thread = TMEM lane).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t r[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- descriptors --------------------------------------------------------------------
// Shared-memory matrix descriptor, K-major operand with 128-byte swizzle: rows of 128 bytes,
// 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1 (sm_100),
// layout type 2 (SWIZZLE_128B).  Advancing along K inside the 128-byte row adds the byte
// offset >> 4 to the start-address field.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
    d |= (uint64_t)1u << 16;                 // leading byte offset (ignored for swizzled K-major)
    d |= (uint64_t)(1024u >> 4) << 32;       // stride byte offset between 8-row groups
    d |= (uint64_t)1u << 46;                 // descriptor version
    d |= (uint64_t)2u << 61;                 // SWIZZLE_128B
    return d;
}
// Instruction descriptor: f32 accumulate, both operands K-major, M x N tile.
//   a_fmt/b_fmt: kind::f16 -> 0 = f16, 1 = bf16 ; kind::f8f6f4 -> 0 = e4m3, 1 = e5m2
__host__ __device__ __forceinline__ uint32_t umma_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t M, uint32_t N) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// Work units of a persistent GEMM with `tiles` output tiles of `k_steps` k-steps on `sms` SMs.  Candidates: whole
// tiles only; every tile split ks ways along k; or whole tiles round by round with only the last, partial round
// split (units [0, full) are whole tiles, the other tiles - full are split ks_tail ways).  The estimate is in
// tile-times.  A split unit costs 1/ks of a tile plus a fixed ~3 us (its own accumulator drain and f32 slab
// write), and split work needs the finishing kernel (~4 us); `us_per_kstep` (how long one k-step of one tile
// takes, measured per kernel) turns those into tile-times.  Returns the estimate.
static inline float tc_plan_units(int tiles, int k_steps, int sms, float us_per_kstep, int* full, int* ks_tail) {
    *full = tiles;
    *ks_tail = 1;
    const int max_ks = k_steps / 4 < 8 ? k_steps / 4 : 8;
    const float tile_us = k_steps * us_per_kstep;
    const float unit_ovh = 3.0f / tile_us, finish = 4.0f / tile_us;
    float best = (float)((tiles + sms - 1) / sms);
    for (int ks = 2; ks <= max_ks; ++ks) {
        const float all = (float)((tiles * ks + sms - 1) / sms) * (1.0f / ks + unit_ovh) + finish;
        // splitting everything only pays clearly when the tiles do not fill one round; beyond that it has to win by 10 %
        if (all < best * (tiles <= sms ? 0.97f : 0.90f)) {
            best = all;
            *full = 0;
            *ks_tail = ks;
        }
        const int rem = tiles % sms;
        if (tiles > sms && rem > 0 && rem * ks <= sms) {
            const float tail = (float)(tiles / sms) + 1.0f / ks + unit_ovh + finish;
            if (tail < best * 0.97f) {
                best = tail;
                *full = tiles - rem;
                *ks_tail = ks;
            }
        }
    }
    return best;
}
// Unit -> (tile, k range) for such a plan.
__device__ __forceinline__ void tc_unit(int unit, int full, int ks_tail, int k_steps, int& tile, int& ks, int& k_lo, int& k_hi) {
    if (unit < full) {
        tile = unit;
        ks = 0;
        k_lo = 0;
        k_hi = k_steps;
        return;
    }
    const int v = unit - full;
    tile = full + v / ks_tail;
    ks = v - (v / ks_tail) * ks_tail;
    const int per = (k_steps + ks_tail - 1) / ks_tail;
    k_lo = ks * per;
    k_hi = min(k_steps, k_lo + per);
}
static inline int tc_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
            sms = v;
        else
            return 148;        // no device (size queries on a CPU-only host): a B200's count
    }
    return sms;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

// ---- tensor maps ----------------------------------------------------------------------------
// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
typedef CUresult (*tc_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                       const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static inline tc_encode_tiled_fn tc_tensor_map_encoder() {
    static tc_encode_tiled_fn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (tc_encode_tiled_fn)p;
    }
    return fn;
}
