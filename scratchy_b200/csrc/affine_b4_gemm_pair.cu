// MLX affine int4: prefill GEMM on a CTA PAIR (tcgen05.mma.cta_group::2), a 256-token x 256-channel tile per pair of SMs.
//
//   y[m,n] = bf16( sum_k x[m,k] * w[n,k] (+ bias[n]) ),  w = the bit-exact bf16 dequantisation of the codes
//
// Why a pair.  The one-CTA kernel (affine_b4_gemm.cu: 256 tokens x 128 channels per CTA) pulls 64 KB of activations per
// 128-k chunk for 256 x 128 x 128 MACs, about what one SM can take from L2 at the rate the tensor core wants them, and
// its two 32 KB stages of dequantised weights are too shallow for the dequantise -> MMA hand-off: an instrumented build
// showed the MMA thread waiting 430 cycles per chunk for activations and 375 for dequantised weights beside 1040 of MMA.
// In a pair each CTA loads the activations of ITS 128 tokens (32 KB per chunk) and dequantises ITS 128 of the tile's 256
// channels; one `tcgen05.mma.cta_group::2` of shape 256 x 256 x 16, issued by the pair's leader CTA, reads the token rows
// and the channel rows from both SMs' shared memory and leaves each CTA's 128 accumulator rows in that CTA's own TMEM.
// Same MACs and the same dequantise work per SM and chunk, 44 % less L2 traffic, and room for three stages of each ring.
// Measured: the same bits as the one-CTA kernel at the same speed (see `affine_b4_gemm_pair_applies`), so it is opt-in.
//
// Per CTA (704 threads), both CTAs of a pair run the same code:
//   warp 0       producer: per chunk 2 tiled TMA loads of this CTA's activations (`.cta_group::2`, completing on the
//                LEADER's barrier; no multicast) and 8 bulk copies of this CTA's packed weight blocks
//   warp 1       leader CTA only: one thread waits for both CTAs' activations and dequantised weights, issues 8 MMAs
//                (2 atoms of 64 k x 4 steps of K = 16) and commits to the stages' `empty` barriers of both CTAs
//   warps 2-17   dequantise this CTA's 128 channels into the K-major 128-byte-swizzled operand image; lane 0 of each warp
//                arrives on the leader's `dfull` barrier (the peer's warps with a remote arrive)
//   warps 18-21  epilogue of this CTA's 128 rows x 256 columns
// Every wait is bounded; the pair meets at a cluster barrier before either CTA frees its TMEM or exits.
#include <cuda.h>

#include <cstdlib>

#include "affine_b4.cuh"
#include "tc_common.cuh"

namespace {

constexpr int A4P_THREADS = 704;
constexpr int A4P_DQ_WARPS = 16;
constexpr int A4P_SX = 3, A4P_SP = 3, A4P_SD = 3;          // activation, packed-weight, dequantised-weight stages
constexpr int A4P_BN = 256;                                 // channels per pair tile (128 per CTA)
constexpr uint32_t A4P_XSTAGE = 32768u;                     // 128 tokens x 128 k bf16: 2 atoms of 128 rows x 128 B
constexpr uint32_t A4P_DSTAGE = 32768u;                     // 128 channels x 128 k bf16: 2 atoms of 128 rows x 128 B
constexpr uint32_t A4P_PSTAGE = 8u * (uint32_t)aff_block_bytes(2);   // 8 row-blocks, sized for the largest block
constexpr uint32_t A4P_XOFF = 0;
constexpr uint32_t A4P_DOFF = A4P_XOFF + A4P_SX * A4P_XSTAGE;
constexpr uint32_t A4P_POFF = A4P_DOFF + A4P_SD * A4P_DSTAGE;
constexpr uint32_t A4P_BAROFF = (A4P_POFF + A4P_SP * A4P_PSTAGE + 127u) & ~127u;
constexpr uint32_t A4P_SMEM_TOTAL = A4P_BAROFF + 256u + 1024u;

__device__ __forceinline__ uint32_t a4p_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void a4p_pair_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t a4p_map(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
// Arrive on a barrier of the other CTA of the pair (default semantics, as for the pair's other barrier operations:
// `.release.cluster` here measured 28 % slower for the same bits).
__device__ __forceinline__ void a4p_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void a4p_umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on the barrier at `bar`'s offset in BOTH CTAs once every MMA this thread has issued is complete (a signal; no data).
__device__ __forceinline__ void a4p_commit(uint32_t bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(both) : "memory");
}
// Tiled TMA load into this CTA's shared memory whose completion is counted on `bar_cluster_addr`, which may be a
// barrier of the other CTA of the pair.
__device__ __forceinline__ void a4p_tma_2d(uint32_t dst_smem, const CUtensorMap* tmap, int c0, int c1, uint32_t bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst_smem), "l"(tmap), "r"(c0), "r"(c1), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void a4p_st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 a4p_ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t a4p_ld_shared_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__global__ void __launch_bounds__(A4P_THREADS, 1)
affine_b4_gemm_pair_kernel(const __grid_constant__ CUtensorMap x_map, const uint8_t* __restrict__ packed, uint16_t* __restrict__ y,
                           int M, int N, int RB, int KC, int gs, int MTP, int out_f32, const uint16_t* __restrict__ bias,
                           int* __restrict__ status) {
    const uint32_t block_bytes = (uint32_t)aff_block_bytes(gs);       // 1152 (groups of 64, 128) or 1280 (groups of 32)
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + A4P_BAROFF;
    // barrier slots: xfull[SX] (leader) xempty[SX] pfull[SP] pempty[SP] dfull[SD] (leader) dempty[SD] accf[2] acce[2] (leader)
    auto xfull = [&](int s) { return bar_base + 8u * s; };
    auto xempty = [&](int s) { return bar_base + 8u * (A4P_SX + s); };
    auto pfull = [&](int s) { return bar_base + 8u * (2 * A4P_SX + s); };
    auto pempty = [&](int s) { return bar_base + 8u * (2 * A4P_SX + A4P_SP + s); };
    auto dfull = [&](int s) { return bar_base + 8u * (2 * A4P_SX + 2 * A4P_SP + s); };
    auto dempty = [&](int s) { return bar_base + 8u * (2 * A4P_SX + 2 * A4P_SP + A4P_SD + s); };
    constexpr int kAccSlot = 2 * A4P_SX + 2 * A4P_SP + 2 * A4P_SD;
    auto accf = [&](int b) { return bar_base + 8u * (kAccSlot + b); };
    auto acce = [&](int b) { return bar_base + 8u * (kAccSlot + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + A4P_BAROFF + 8 * (kAccSlot + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = a4p_cta_rank();                 // 0 = the pair's leader
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int NTP = RB * 16 / A4P_BN;                     // pair tiles along the channels (RB is a multiple of 16 here)
    const int tiles = MTP * NTP;

    if (threadIdx.x == 0) {
        for (int s = 0; s < A4P_SX; ++s) { mbar_init(xfull(s), 1); mbar_init(xempty(s), 1); }
        for (int s = 0; s < A4P_SP; ++s) { mbar_init(pfull(s), 1); mbar_init(pempty(s), A4P_DQ_WARPS / 2); }
        for (int s = 0; s < A4P_SD; ++s) { mbar_init(dfull(s), A4P_DQ_WARPS); mbar_init(dempty(s), 1); }       // 8 warps of each CTA per chunk
        for (int b = 0; b < 2; ++b) { mbar_init(accf(b), 1); mbar_init(acce(b), 256); }                          // both CTAs' epilogue threads
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_slot), 2 * A4P_BN);    // each CTA allocates its own columns; both get the same base
        tmem_relinquish();
    }
    tc_fence_before();
    a4p_pair_sync();                                      // both CTAs' barriers and TMEM exist before anything crosses over
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ producers (both CTAs)
        // Two lanes, one ring each: the packed-weight ring follows the dequantise warps, the activation ring follows the
        // MMA; one lane serving both would hold the activation loads back whenever the dequantise warps are behind.
        if (lane == 0) {
            int sp = 0;
            uint32_t php = 0;
            for (int t = pair; t < tiles; t += npairs) {
                const int nb = t / MTP;
                const int rb0 = (2 * nb + (int)rank) * 8;                 // this CTA's 8 row-blocks (128 channels)
                for (int kc = 0; kc < KC; ++kc) {
                    mbar_wait(pempty(sp), php ^ 1u, status, TC_ERR_EMPTY_WAIT);
                    mbar_arrive_expect_tx(pfull(sp), 8u * block_bytes);
                    for (int j = 0; j < 8; ++j)
                        bulk_g2s(smem_base + A4P_POFF + sp * A4P_PSTAGE + j * block_bytes,
                                 packed + ((size_t)(rb0 + j) * KC + kc) * block_bytes, block_bytes, pfull(sp));
                    if (++sp == A4P_SP) { sp = 0; php ^= 1u; }
                }
            }
        } else if (lane == 1) {
            int sx = 0;
            uint32_t phx = 0;
            for (int t = pair; t < tiles; t += npairs) {
                const int mb = t % MTP;
                const int row0 = (2 * mb + (int)rank) * 128;              // this CTA's tokens
                for (int kc = 0; kc < KC; ++kc) {
                    mbar_wait(xempty(sx), phx ^ 1u, status, TC_ERR_EMPTY_WAIT);
                    // both CTAs' activation loads of the stage complete on the LEADER's barrier
                    const uint32_t lead_xfull = a4p_map(xfull(sx), 0);
                    if (rank == 0) mbar_arrive_expect_tx(xfull(sx), 2u * A4P_XSTAGE);
                    const uint32_t xs = smem_base + A4P_XOFF + sx * A4P_XSTAGE;
                    a4p_tma_2d(xs, &x_map, kc * 128, row0, lead_xfull);
                    a4p_tma_2d(xs + 16384u, &x_map, kc * 128 + 64, row0, lead_xfull);
                    if (++sx == A4P_SX) { sx = 0; phx ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA)
        if (lane == 0 && rank == 0) {
            int sx = 0, sd = 0;
            uint32_t phx = 0, phd = 0;
            int it = 0;
            const uint32_t idesc = umma_idesc(1, 1, 256, A4P_BN);
            for (int t = pair; t < tiles; t += npairs, ++it) {
                const int buf = it & 1;
                mbar_wait(acce(buf), ((uint32_t)(it >> 1) & 1u) ^ 1u, status, TC_ERR_ACC_EMPTY);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * A4P_BN);
                for (int kc = 0; kc < KC; ++kc) {
                    mbar_wait(xfull(sx), phx, status, TC_ERR_FULL_WAIT);
                    mbar_wait(dfull(sd), phd, status, TC_ERR_DEQ_WAIT);
                    tc_fence_after();
                    const uint32_t xs = smem_base + A4P_XOFF + sx * A4P_XSTAGE;
                    const uint32_t ds = smem_base + A4P_DOFF + sd * A4P_DSTAGE;
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        const uint64_t adesc = umma_desc_k_sw128(xs + a * 16384u);
                        const uint64_t bdesc = umma_desc_k_sw128(ds + a * 16384u);
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4)
                            a4p_umma_f16(d_tmem, adesc + (uint64_t)(2 * k4), bdesc + (uint64_t)(2 * k4), idesc, (kc | a | k4) != 0);
                    }
                    a4p_commit(xempty(sx));
                    a4p_commit(dempty(sd));
                    if (++sx == A4P_SX) { sx = 0; phx ^= 1u; }
                    if (++sd == A4P_SD) { sd = 0; phd ^= 1u; }
                }
                a4p_commit(accf(buf));
            }
        }
    } else if (warp < 2 + A4P_DQ_WARPS) {
        // ------------------------------------------------------------------ dequantise (warps 2..17, both CTAs)
        const int dw = warp - 2;
        // Lane -> piece of a (row-block, half) pair, arranged so that the eight lanes of a quarter-warp
        // hold four rows and one k-quarter pair: their 16-byte stores then hit eight distinct bank groups.
        const int g = ((lane >> 3) & 1) * 4 + ((lane & 7) >> 1);
        const int t4 = (lane >> 4) * 2 + (lane & 1);
        const bool check = *reinterpret_cast<const unsigned int*>(packed + (size_t)RB * KC * block_bytes) != 0;
        const uint32_t entry = (uint32_t)(((g << gs) + (t4 >> (2 - gs))) * 8);    // this lane's (scale, bias) entry in a block
        // Two groups of 8 warps take alternate chunks (two (row-block, half) pairs per warp and chunk): a warp's chunk is a
        // serial chain (shared load -> dequantise -> stores -> proxy fence -> arrive) of well over a thousand cycles, so
        // with every warp on every chunk that chain, not the work, set the rate; two chains in flight nearly double it.
        const int grp = dw >> 3, lw = dw & 7;
        int c = 0;                                        // chunk counter over the whole kernel
        for (int t = pair; t < tiles; t += npairs) {
            for (int kc = 0; kc < KC; ++kc, ++c) {
                if ((c & 1) != grp) continue;
                const int sp = c % A4P_SP, sd = c % A4P_SD;
                const uint32_t php = (uint32_t)(c / A4P_SP) & 1u, phd = (uint32_t)(c / A4P_SD) & 1u;
                mbar_wait(pfull(sp), php, status, TC_ERR_FULL_WAIT);
                mbar_wait(dempty(sd), phd ^ 1u, status, TC_ERR_EMPTY_WAIT);
                const uint32_t ps = smem_base + A4P_POFF + sp * A4P_PSTAGE;
                const uint32_t ds = smem_base + A4P_DOFF + sd * A4P_DSTAGE;
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int pr = lw + 8 * u;
                    const int rbl = pr >> 1, half = pr & 1;
                    const uint32_t blk = ps + (uint32_t)rbl * block_bytes;
                    const uint4 piece = a4p_ld_shared_v4(blk + half * 512 + (4 * g + t4) * 16);
                    const uint32_t sb = a4p_ld_shared_u32(blk + 1024 + entry + half * 4);
                    uint32_t w[16];
                    if (check) {
                        affine_dequant_piece<true>(piece, sb, w);
                    } else {
                        // scaled variant (w * 2^-7); the epilogue multiplies the accumulators by 2^7
                        const AffineScaled cs = affine_scaled_consts(sb);
                        affine_dequant_word_scaled(piece.x, cs, w + 0);
                        affine_dequant_word_scaled(piece.y, cs, w + 4);
                        affine_dequant_word_scaled(piece.z, cs, w + 8);
                        affine_dequant_word_scaled(piece.w, cs, w + 12);
                    }
                    // row = 16 rbl + 8 half + g -> 8-row group (2 rbl + half), row-in-group g;
                    // k = 32 t4 + [0,32) -> atom t4>>1, 16-byte chunks (t4&1)*4 + [0,4), swizzled with g
                    const uint32_t rowbase = ds + (uint32_t)(t4 >> 1) * 16384u + (uint32_t)(2 * rbl + half) * 1024u + (uint32_t)g * 128u;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t chunk = (uint32_t)(((t4 & 1) * 4 + j) ^ g);
                        a4p_st_shared_v4(rowbase + chunk * 16u, w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
                    }
                }
                fence_proxy_async_smem();              // generic-proxy stores -> visible to the tensor cores
                __syncwarp();                          // every lane has stored (and fenced) and is done with the packed stage
                if (lane == 0) {
                    if (rank == 0) mbar_arrive(dfull(sd));
                    else a4p_arrive_remote(a4p_map(dfull(sd), 0));
                    mbar_arrive(pempty(sp));
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 18..21, both CTAs)
        const int q = warp & 3;                        // TMEM lane quadrant this warp may read
        const bool vec_ok = (N % 8) == 0;
        const bool f32mode = out_f32 != 0;
        float* fbase = reinterpret_cast<float*>(y);
        const float out_scale =
            (*reinterpret_cast<const unsigned int*>(packed + (size_t)RB * KC * block_bytes) != 0) ? 1.0f : AFF_SCALED_FACTOR;
        int it = 0;
        for (int t = pair; t < tiles; t += npairs, ++it) {
            const int mb = t % MTP, nb = t / MTP;
            const int n0 = nb * A4P_BN;
            const int buf = it & 1;
            mbar_wait(accf(buf), (uint32_t)(it >> 1) & 1u, status, TC_ERR_ACC_FULL);
            tc_fence_after();
            const int m = (2 * mb + (int)rank) * 128 + q * 32 + lane;
            uint16_t* yrow = y + (size_t)m * N;
            for (int c = 0; c < A4P_BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * A4P_BN + c * 32), r);
                tmem_ld_wait();
                const int nc = n0 + c * 32;
                if (m >= M || nc >= N) continue;
                if (f32mode) {
                    float* frow = fbase + (size_t)m * N + nc;
                    const bool v4 = (N % 4) == 0 && nc + 32 <= N;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 v = make_float4(__uint_as_float(r[4 * j]) * out_scale, __uint_as_float(r[4 * j + 1]) * out_scale,
                                                     __uint_as_float(r[4 * j + 2]) * out_scale, __uint_as_float(r[4 * j + 3]) * out_scale);
                        if (v4) {
                            reinterpret_cast<float4*>(frow)[j] = v;
                        } else {
                            if (nc + 4 * j + 0 < N) frow[4 * j + 0] = v.x;
                            if (nc + 4 * j + 1 < N) frow[4 * j + 1] = v.y;
                            if (nc + 4 * j + 2 < N) frow[4 * j + 2] = v.z;
                            if (nc + 4 * j + 3 < N) frow[4 * j + 3] = v.w;
                        }
                    }
                } else {
                    uint32_t o[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float lo = __uint_as_float(r[2 * j]) * out_scale, hi = __uint_as_float(r[2 * j + 1]) * out_scale;
                        if (bias) {                // the linear's own bias, added in f32 before the one rounding
                            const int n2 = nc + 2 * j;
                            if (n2 < N) lo += __uint_as_float(uint32_t(bias[n2]) << 16);
                            if (n2 + 1 < N) hi += __uint_as_float(uint32_t(bias[n2 + 1]) << 16);
                        }
                        const __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);
                        o[j] = *reinterpret_cast<const uint32_t*>(&pk);
                    }
                    if (vec_ok && nc + 32 <= N) {
                        uint4* dst = reinterpret_cast<uint4*>(yrow + nc);
#pragma unroll
                        for (int j = 0; j < 4; ++j) dst[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (nc + j < N) yrow[nc + j] = (uint16_t)((o[j >> 1] >> ((j & 1) * 16)) & 0xFFFFu);
                    }
                }
            }
            tc_fence_before();
            if (rank == 0) mbar_arrive(acce(buf));
            else a4p_arrive_remote(a4p_map(acce(buf), 0));
        }
    }

    tc_fence_before();
    a4p_pair_sync();                                      // nobody frees TMEM or leaves while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * A4P_BN);
    }
}

}  // namespace


// Whether the pair kernel takes this GEMM.  It is OFF unless `SCR_AFFINE_GEMM_PAIR=1` is in the environment (read once):
// on the Llama-3.2-3B gate shape at 2048 tokens it gives the same bits in 100.1 us against the one-CTA kernel's 99.3 us —
// with the dequantise warps' serial chain per chunk as the limiter of both, halving the activation traffic buys nothing
// yet.  When on: whole 256-channel pair tiles, at least one full round of pairs, and rounds that are at least 85 % full
// (the one-CTA kernel splits its tail along k instead).
bool affine_b4_gemm_pair_applies(int M, int N, int K, int sms) {
    static const bool enabled = [] {
        const char* e = std::getenv("SCR_AFFINE_GEMM_PAIR");
        return e && e[0] == '1';
    }();
    if (!enabled) return false;
    const AffineGeom g = affine_geom(N, K, 64);
    if ((g.RB % 16) != 0 || g.KC < 1 || M <= 128) return false;
    const int pairs = sms / 2, tiles = scr_ceil_div(M, 256) * (g.RB / 16);
    if (pairs < 1 || tiles < pairs) return false;
    const int rounds = (tiles + pairs - 1) / pairs;
    return (float)tiles >= 0.85f * (float)(rounds * pairs);
}

int32_t affine_b4_gemm_pair_launch(scr_ctx* ctx, const CUtensorMap& x_map, const uint8_t* packed, uint16_t* y, int M, int N, int K,
                                   int gs, int out_f32, const uint16_t* bias, cudaStream_t stream, bool* launched) {
    *launched = false;
    const AffineGeom g = affine_geom(N, K, 64);          // RB / KC only: the same for every group size
    cudaError_t e = cudaFuncSetAttribute(affine_b4_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)A4P_SMEM_TOTAL);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "affine gemm pair smem attribute: %s", cudaGetErrorString(e));
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(A4P_THREADS);
    cfg.dynamicSmemBytes = A4P_SMEM_TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(2 * (ctx->sm_count / 2));
    // how many pairs fit at once (the pairing may leave an SM of a GPC unused; the grid is persistent): asked once per device
    static int pairs_of_device[64] = {0};
    int max_pairs = (ctx->device >= 0 && ctx->device < 64) ? pairs_of_device[ctx->device] : 0;
    if (max_pairs == 0) {
        e = cudaOccupancyMaxActiveClusters(&max_pairs, affine_b4_gemm_pair_kernel, &cfg);
        if (e != cudaSuccess || max_pairs < 1) {
            (void)cudaGetLastError();
            max_pairs = -1;
        }
        if (ctx->device >= 0 && ctx->device < 64) pairs_of_device[ctx->device] = max_pairs;
    }
    if (max_pairs < 1) return SCR_OK;                     // not launched: the caller runs the one-CTA kernel
    const int MTP = scr_ceil_div(M, 256);
    const int tiles = MTP * (g.RB / 16);
    cfg.gridDim = dim3(2 * std::min(tiles, max_pairs));
    e = cudaLaunchKernelEx(&cfg, affine_b4_gemm_pair_kernel, x_map, packed, y, M, N, g.RB, g.KC, gs, MTP, out_f32, bias,
                           ctx->dev_status);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "affine gemm pair launch: %s", cudaGetErrorString(e));
    *launched = true;
    return scr_check_launch(ctx, "affine_b4_gemm_pair");
}
