// MLX affine int4 (group 64): prefill GEMM on tcgen05 tensor cores, M > 16.
//
//   y[m,n] = bf16( sum_k x[m,k] * w[n,k] ),  w = the bit-exact bf16 dequantisation of the codes
//
// Persistent, warp-specialised CTA (704 threads), one per SM; a tile is TM x 128 tokens by 128
// channels (TM = 2 when M > 128, so every dequantised weight tile feeds two MMAs):
//   warp 0       producer: per 128-k chunk, 2 x TM TMA tile loads of the activations (tensor map over
//                x[M,K], 64 x 128 box, 128-byte swizzle; out-of-range rows/k read as zero) and one
//                1-D bulk copy per row-block of the packed weight blocks (8 x 1152 bytes)
//   warp 1       owns TMEM; one elected thread issues tcgen05.mma kind::f16 (A = 128 tokens,
//                B = 128 channels, 8 x K=16 per chunk and token half) and commits the barriers
//   warps 2-17   dequantise: packed codes (shared) -> bf16 -> the K-major 128-byte-swizzled operand
//                image the MMA reads (bank-conflict-free 16-byte stores)
//   warps 18-21  epilogue: tcgen05.ld the 128 x 128 f32 accumulators (thread = token row), round to
//                bf16 (or keep f32 partials), 16-byte stores
// TMEM holds 2 buffers x TM accumulators of 128 columns, so the epilogue of tile i overlaps the
// main loop of tile i+1.  No multicast: every CTA issues its own loads.
#include <cuda.h>

#include "affine_b4.cuh"
#include "tc_common.cuh"

bool affine_b4_gemm_tc_enabled() { return true; }
// Defined in affine_b4_gemm_pair.cu
bool affine_b4_gemm_pair_applies(int M, int N, int K, int sms);
int32_t affine_b4_gemm_pair_launch(scr_ctx* ctx, const CUtensorMap& x_map, const uint8_t* packed, uint16_t* y, int M, int N, int K,
                                   int gs, int out_f32, const uint16_t* bias, cudaStream_t stream, bool* launched);
size_t affine_b4_gemm_tc_workspace_plan(int M, int N, int K);
size_t affine_b4_gemm_tc_workspace(int M, int N, int K) { return affine_b4_gemm_tc_workspace_plan(M, N, K); }

#define A4G_THREADS 704
#define A4G_DQ_WARPS 16
#define A4G_SP 3          // packed-weight stages
#define A4G_SD 2          // dequantised-weight stages
#define A4G_BN 128

template <int TM>
struct A4GSmem {
    static constexpr int kSX = (TM == 1) ? 3 : 2;                       // activation stages
    static constexpr uint32_t kXStage = 32768u * TM;                    // TM x 2 atoms of 128 rows x 128 B
    static constexpr uint32_t kDStage = 2u * A4G_BN * 128u;             // 2 atoms of 128 rows x 128 B
    static constexpr uint32_t kPStage = (uint32_t)(A4G_BN / 16) * aff_block_bytes(2);   // sized for the largest block (groups of 32)
    static constexpr uint32_t kXOff = 0;
    static constexpr uint32_t kDOff = kXOff + kSX * kXStage;
    static constexpr uint32_t kPOff = kDOff + A4G_SD * kDStage;
    static constexpr uint32_t kBarOff = (kPOff + A4G_SP * kPStage + 127u) & ~127u;
    static constexpr uint32_t kTotal = kBarOff + 256u + 1024u;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* tmap, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst_smem), "l"(tmap), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t ld_shared_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Finishes the split tiles: sums a tile's ks_tail partial tiles in slab order (deterministic) and stores the
// result, rounded once (or as f32 partials).  One CTA per (tail tile, 8 rows), one float4 per thread.
__global__ void __launch_bounds__(256) affine_b4_gemm_tail_finish_kernel(const float* __restrict__ slabs, int ks_tail, int n_tail,
                                                                         int full, int MT, int tile_rows, int M, int N,
                                                                         uint16_t* __restrict__ y, int out_f32,
                                                                         const uint16_t* __restrict__ bias) {
    const int groups = tile_rows / 8;
    const int tt = blockIdx.x / groups, grp = blockIdx.x - tt * groups;
    const int tile = full + tt;
    const int mt = tile % MT, nb = tile / MT;
    const size_t tile_elems = (size_t)tile_rows * A4G_BN;
    const int rl = grp * 8 + threadIdx.x / (A4G_BN / 4), c4 = (threadIdx.x % (A4G_BN / 4)) * 4;
    const int m = mt * tile_rows + rl, n = nb * A4G_BN + c4;
    if (m >= M || n >= N) return;
    const float* p = slabs + (size_t)tt * tile_elems + (size_t)rl * A4G_BN + c4;
    float4 a = *reinterpret_cast<const float4*>(p);
    for (int k = 1; k < ks_tail; ++k) {
        const float4 b = *reinterpret_cast<const float4*>(p + (size_t)k * n_tail * tile_elems);
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    const float v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (n + j >= N) break;
        if (out_f32) {
            reinterpret_cast<float*>(y)[(size_t)m * N + n + j] = v[j];
        } else {
            const __nv_bfloat16 o = __float2bfloat16_rn(bias ? v[j] + __uint_as_float(uint32_t(bias[n + j]) << 16) : v[j]);
            y[(size_t)m * N + n + j] = *reinterpret_cast<const uint16_t*>(&o);
        }
    }
}

template <int TM>
__global__ void __launch_bounds__(A4G_THREADS, 1)
affine_b4_gemm_tc_kernel(const __grid_constant__ CUtensorMap x_map, const uint8_t* __restrict__ packed,
                         uint16_t* __restrict__ y, int M, int N, int RB, int KC, int gs, int MT, int out_f32,
                         const uint16_t* __restrict__ bias, int full, int ks_tail, float* __restrict__ slabs,
                         int* __restrict__ status) {
    using S = A4GSmem<TM>;
    const uint32_t block_bytes = (uint32_t)aff_block_bytes(gs);       // 1152 (groups of 64, 128) or 1280 (groups of 32)
    constexpr int SX = S::kSX;
    constexpr int BN = A4G_BN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + S::kBarOff;
    // barrier slots: xfull[SX] xempty[SX] pfull[SP] pempty[SP] dfull[SD] dempty[SD] accf[2] acce[2]
    auto xfull = [&](int s) { return bar_base + 8u * s; };
    auto xempty = [&](int s) { return bar_base + 8u * (SX + s); };
    auto pfull = [&](int s) { return bar_base + 8u * (2 * SX + s); };
    auto pempty = [&](int s) { return bar_base + 8u * (2 * SX + A4G_SP + s); };
    auto dfull = [&](int s) { return bar_base + 8u * (2 * SX + 2 * A4G_SP + s); };
    auto dempty = [&](int s) { return bar_base + 8u * (2 * SX + 2 * A4G_SP + A4G_SD + s); };
    constexpr int kAccSlot = 2 * SX + 2 * A4G_SP + 2 * A4G_SD;
    auto accf = [&](int b) { return bar_base + 8u * (kAccSlot + b); };
    auto acce = [&](int b) { return bar_base + 8u * (kAccSlot + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + S::kBarOff + 8 * (kAccSlot + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NTB = RB * 16 / BN;                        // RB is a multiple of 8 (N padded to 128)
    // Work units: the first `full` tiles whole; each of the remaining (tail) tiles as ks_tail units that share its k
    // extent and leave f32 partial tiles in `slabs` for the finishing kernel (MT = token tiles of 128 * TM).
    const int n_tail = MT * NTB - full;
    const int tiles = full + n_tail * ks_tail;
    constexpr uint32_t kAccCols = (uint32_t)(TM * BN);   // TMEM columns per accumulator buffer

    if (threadIdx.x == 0) {
        for (int s = 0; s < SX; ++s) { mbar_init(xfull(s), 1); mbar_init(xempty(s), 1); }
        // one arrival per dequantise WARP (its lane 0, after the warp has synchronised): 512 thread arrivals per stage on
        // one barrier serialise in the barrier unit and cost more than the dequantisation itself (measured)
        for (int s = 0; s < A4G_SP; ++s) { mbar_init(pfull(s), 1); mbar_init(pempty(s), A4G_DQ_WARPS); }
        for (int s = 0; s < A4G_SD; ++s) { mbar_init(dfull(s), A4G_DQ_WARPS); mbar_init(dempty(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf(b), 1); mbar_init(acce(b), 128); }
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_slot), 2 * kAccCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            int sx = 0, sp = 0;
            uint32_t phx = 0, php = 0;
            for (int unit = blockIdx.x; unit < tiles; unit += gridDim.x) {
                int t2, ks, kc_lo, kc_hi;
                tc_unit(unit, full, ks_tail, KC, t2, ks, kc_lo, kc_hi);
                const int mt = t2 % MT, nb = t2 / MT;
                const int rb0 = nb * (BN / 16);
                for (int kc = kc_lo; kc < kc_hi; ++kc) {
                    mbar_wait(pempty(sp), php ^ 1u, status, TC_ERR_EMPTY_WAIT);
                    mbar_arrive_expect_tx(pfull(sp), (BN / 16) * block_bytes);
                    for (int j = 0; j < BN / 16; ++j)   // row-block-major packing: one block per row-block
                        bulk_g2s(smem_base + S::kPOff + sp * S::kPStage + j * block_bytes,
                                 packed + ((size_t)(rb0 + j) * KC + kc) * block_bytes, block_bytes, pfull(sp));
                    if (++sp == A4G_SP) { sp = 0; php ^= 1u; }

                    mbar_wait(xempty(sx), phx ^ 1u, status, TC_ERR_EMPTY_WAIT);
                    mbar_arrive_expect_tx(xfull(sx), S::kXStage);
                    const uint32_t xs = smem_base + S::kXOff + sx * S::kXStage;
#pragma unroll
                    for (int h = 0; h < TM; ++h) {
                        tma_load_2d(xs + h * 32768u, &x_map, kc * 128, (mt * TM + h) * 128, xfull(sx));
                        tma_load_2d(xs + h * 32768u + 16384u, &x_map, kc * 128 + 64, (mt * TM + h) * 128, xfull(sx));
                    }
                    if (++sx == SX) { sx = 0; phx ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int sx = 0, sd = 0;
            uint32_t phx = 0, phd = 0;
            int it = 0;
            const uint32_t idesc = umma_idesc(1, 1, 128, BN);
            for (int unit = blockIdx.x; unit < tiles; unit += gridDim.x, ++it) {
                const int buf = it & 1;
                mbar_wait(acce(buf), ((uint32_t)(it >> 1) & 1u) ^ 1u, status, TC_ERR_ACC_EMPTY);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)buf * kAccCols;
                int t2, ks, kc_lo, kc_hi;
                tc_unit(unit, full, ks_tail, KC, t2, ks, kc_lo, kc_hi);
                for (int kc = kc_lo; kc < kc_hi; ++kc) {
                    mbar_wait(xfull(sx), phx, status, TC_ERR_FULL_WAIT);
                    mbar_wait(dfull(sd), phd, status, TC_ERR_DEQ_WAIT);
                    tc_fence_after();
                    const uint32_t xs = smem_base + S::kXOff + sx * S::kXStage;
                    const uint32_t ds = smem_base + S::kDOff + sd * S::kDStage;
#pragma unroll
                    for (int h = 0; h < TM; ++h) {
#pragma unroll
                        for (int a = 0; a < 2; ++a) {
                            const uint64_t adesc = umma_desc_k_sw128(xs + h * 32768u + a * 16384u);
                            const uint64_t bdesc = umma_desc_k_sw128(ds + a * (uint32_t)(BN * 128));
#pragma unroll
                            for (int k4 = 0; k4 < 4; ++k4)
                                umma_f16(d_tmem + (uint32_t)(h * BN), adesc + (uint64_t)(2 * k4), bdesc + (uint64_t)(2 * k4), idesc,
                                         ((kc - kc_lo) | a | k4) != 0);
                        }
                    }
                    umma_commit(xempty(sx));
                    umma_commit(dempty(sd));
                    if (++sx == SX) { sx = 0; phx ^= 1u; }
                    if (++sd == A4G_SD) { sd = 0; phd ^= 1u; }
                }
                umma_commit(accf(buf));
            }
        }
    }
    else if (warp < 2 + A4G_DQ_WARPS) {
        // ------------------------------------------------------------------ dequantise (warps 2..17)
        const int dw = warp - 2;
        // Lane -> piece of a (row-block, half) pair, arranged so that the eight lanes of a quarter-warp
        // hold four rows and one k-quarter pair: their 16-byte stores then hit eight distinct bank groups.
        const int g = ((lane >> 3) & 1) * 4 + ((lane & 7) >> 1);
        const int t = (lane >> 4) * 2 + (lane & 1);
        const bool check = *reinterpret_cast<const unsigned int*>(packed + (size_t)RB * KC * block_bytes) != 0;
        const uint32_t entry = (uint32_t)(((g << gs) + (t >> (2 - gs))) * 8);     // this lane's (scale, bias) entry in a block
        int sp = 0, sd = 0;
        uint32_t php = 0, phd = 0;
        for (int unit = blockIdx.x; unit < tiles; unit += gridDim.x) {
            int t2, ks, kc_lo, kc_hi;
            tc_unit(unit, full, ks_tail, KC, t2, ks, kc_lo, kc_hi);
            for (int kc = kc_lo; kc < kc_hi; ++kc) {
                mbar_wait(pfull(sp), php, status, TC_ERR_FULL_WAIT);
                mbar_wait(dempty(sd), phd ^ 1u, status, TC_ERR_EMPTY_WAIT);
                const uint32_t ps = smem_base + S::kPOff + sp * S::kPStage;
                const uint32_t ds = smem_base + S::kDOff + sd * S::kDStage;
                // 16 (row-block, half) pairs per stage, one per warp
#pragma unroll
                for (int u = 0; u < 2 * (BN / 16) / A4G_DQ_WARPS; ++u) {
                    const int pr = dw + u * A4G_DQ_WARPS;
                    const int rbl = pr >> 1, half = pr & 1;
                    const uint32_t blk = ps + (uint32_t)rbl * block_bytes;
                    const uint4 piece = ld_shared_v4(blk + half * 512 + (4 * g + t) * 16);
                    const uint32_t sb = ld_shared_u32(blk + 1024 + entry + half * 4);
                    uint32_t w[16];
                    if (check) {
                        affine_dequant_piece<true>(piece, sb, w);
                    } else {
                        // scaled variant (w * 2^-7); the epilogue multiplies the accumulators by 2^7
                        const AffineScaled c = affine_scaled_consts(sb);
                        affine_dequant_word_scaled(piece.x, c, w + 0);
                        affine_dequant_word_scaled(piece.y, c, w + 4);
                        affine_dequant_word_scaled(piece.z, c, w + 8);
                        affine_dequant_word_scaled(piece.w, c, w + 12);
                    }
                    // row = 16 rbl + 8 half + g -> 8-row group (2 rbl + half), row-in-group g;
                    // k = 32 t + [0,32) -> atom t>>1, 16-byte chunks (t&1)*4 + [0,4), swizzled with g
                    const uint32_t rowbase = ds + (uint32_t)(t >> 1) * (uint32_t)(BN * 128) + (uint32_t)(2 * rbl + half) * 1024u +
                                             (uint32_t)g * 128u;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t chunk = (uint32_t)(((t & 1) * 4 + j) ^ g);
                        st_shared_v4(rowbase + chunk * 16u, w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
                    }
                }
                fence_proxy_async_smem();              // generic-proxy stores -> visible to the tensor core
                __syncwarp();                          // every lane has stored (and fenced) and is done with the packed stage
                if (lane == 0) {
                    mbar_arrive(dfull(sd));
                    mbar_arrive(pempty(sp));
                }
                if (++sp == A4G_SP) { sp = 0; php ^= 1u; }
                if (++sd == A4G_SD) { sd = 0; phd ^= 1u; }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 18..21)
        const int q = warp & 3;                        // TMEM lane quadrant this warp may read
        const bool vec_ok = (N % 8) == 0;
        const float out_scale =
            (*reinterpret_cast<const unsigned int*>(packed + (size_t)RB * KC * block_bytes) != 0) ? 1.0f : AFF_SCALED_FACTOR;
        int it = 0;
        for (int unit = blockIdx.x; unit < tiles; unit += gridDim.x, ++it) {
            int t2, ks, kc_lo, kc_hi;
            tc_unit(unit, full, ks_tail, KC, t2, ks, kc_lo, kc_hi);
            const int mt = t2 % MT, nb = t2 / MT;
            const int n0 = nb * BN;
            const int buf = it & 1;
            // a split unit writes its f32 partial tile (TM*128 x 128, padding included) into its own slab
            const bool split = unit >= full && ks_tail > 1;
            const bool f32mode = out_f32 != 0;
            float* fbase = reinterpret_cast<float*>(y);
            float* slab = split ? slabs + ((size_t)ks * n_tail + (t2 - full)) * (size_t)(TM * 128 * BN) : nullptr;
            mbar_wait(accf(buf), (uint32_t)(it >> 1) & 1u, status, TC_ERR_ACC_FULL);
            tc_fence_after();
#pragma unroll 1
            for (int h = 0; h < TM; ++h) {
                const int m = (mt * TM + h) * 128 + q * 32 + lane;
                uint16_t* yrow = y + (size_t)m * N;
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)buf * kAccCols + (uint32_t)(h * BN + c * 32), r);
                    tmem_ld_wait();
                    const int nc = n0 + c * 32;
                    if (split) {
                        if (m >= M) continue;          // rows of padding are never read back
                        float4* dst = reinterpret_cast<float4*>(slab + (size_t)(h * 128 + q * 32 + lane) * BN + c * 32);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            dst[j] = make_float4(__uint_as_float(r[4 * j]) * out_scale, __uint_as_float(r[4 * j + 1]) * out_scale,
                                                 __uint_as_float(r[4 * j + 2]) * out_scale, __uint_as_float(r[4 * j + 3]) * out_scale);
                    } else if (m < M && nc < N && f32mode) {
                        // unrounded f32 (row-parallel partials, or a split-K slab)
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
                    } else if (m < M && nc < N) {
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
            }
            tc_fence_before();
            mbar_arrive(acce(buf));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * kAccCols);
    }
}

// ---- host --------------------------------------------------------------------------------
static int affine_gemm_tm(int M, int N, int K, int sms) {
    // 256-token tiles reuse every dequantised weight tile twice; below 129 tokens they would be half
    // empty, and they need enough tiles to fill the machine.
    const AffineGeom g = affine_geom(N, K, 64);
    const int tiles2 = scr_ceil_div(M, 256) * (g.RB * 16 / A4G_BN);
    return (M > 128 && tiles2 >= sms / 2) ? 2 : 1;
}
// How the tiles are cut into work units.  Few tiles (less than half the SMs): every tile is split along k.
// Otherwise the persistent CTAs take whole tiles round by round, and when the last round would leave more than
// half the machine idle its tiles (the tail) are split along k so that the round is about full again.
struct AffineGemmPlan {
    int tm, mt, tiles, full, ks_tail;
    int n_tail() const { return tiles - full; }
    size_t slab_floats() const { return ks_tail > 1 ? (size_t)ks_tail * n_tail() * (size_t)(tm * 128 * A4G_BN) : 0; }
};
static AffineGemmPlan affine_gemm_plan(int M, int N, int K, int sms) {
    const AffineGeom g = affine_geom(N, K, 64);
    AffineGemmPlan p;
    p.tm = affine_gemm_tm(M, N, K, sms);
    p.mt = scr_ceil_div(M, 128 * p.tm);
    p.tiles = p.mt * (g.RB * 16 / A4G_BN);
    tc_plan_units(p.tiles, g.KC, sms, 1.0f * p.tm, &p.full, &p.ks_tail);      // ~1 us per 128-k step and 128 tokens (measured)
    return p;
}
size_t affine_b4_gemm_tc_workspace_plan(int M, int N, int K) { return affine_gemm_plan(M, N, K, tc_sm_count()).slab_floats() * sizeof(float); }

template <int TM>
static int32_t affine_gemm_launch_tm(scr_ctx* ctx, const CUtensorMap& map, const uint8_t* packed, uint16_t* y, int M, int N,
                                     int K, int gs, int out_f32, const uint16_t* bias, const AffineGemmPlan& p, float* slabs,
                                     cudaStream_t stream) {
    const AffineGeom g = affine_geom(N, K, 64);
    const int units = p.full + p.n_tail() * p.ks_tail;
    const int grid = std::min(units, ctx->sm_count);
    cudaError_t e = cudaFuncSetAttribute(affine_b4_gemm_tc_kernel<TM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)A4GSmem<TM>::kTotal);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "affine gemm smem attribute: %s", cudaGetErrorString(e));
    affine_b4_gemm_tc_kernel<TM><<<grid, A4G_THREADS, A4GSmem<TM>::kTotal, stream>>>(map, packed, y, M, N, g.RB, g.KC, gs, p.mt,
                                                                                    out_f32, bias, p.full, p.ks_tail, slabs,
                                                                                    ctx->dev_status);
    int32_t st = scr_check_launch(ctx, "affine_b4_gemm_tc");
    if (st || p.ks_tail == 1) return st;
    affine_b4_gemm_tail_finish_kernel<<<p.n_tail() * (TM * 128 / 8), 256, 0, stream>>>(slabs, p.ks_tail, p.n_tail(), p.full, p.mt,
                                                                                       TM * 128, M, N, y, out_f32, bias);
    return scr_check_launch(ctx, "affine_b4_gemm_tail_finish");
}

int32_t affine_b4_gemm_tc_launch(scr_ctx* ctx, const uint8_t* packed, const uint16_t* x, uint16_t* y, int M, int N, int K,
                                 int gs, int out_f32, const uint16_t* bias, void* workspace, size_t, cudaStream_t stream) {
    if (((uintptr_t)packed & 127u) != 0) return scr_fail(ctx, SCR_E_ALIGN, "packed weights must be 128-byte aligned for the GEMM path");
    if (!scr_aligned16(y)) return scr_fail(ctx, SCR_E_ALIGN, "y must be 16-byte aligned");
    tc_encode_tiled_fn enc = tc_tensor_map_encoder();
    if (!enc) return scr_fail(ctx, SCR_E_CUDA, "cuTensorMapEncodeTiled entry point not available");
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)x, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return scr_fail(ctx, SCR_E_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    if (affine_b4_gemm_pair_applies(M, N, K, ctx->sm_count)) {     // large, evenly tiled GEMMs: the two-CTA kernel (affine_b4_gemm_pair.cu)
        bool launched = false;
        const int32_t st = affine_b4_gemm_pair_launch(ctx, map, packed, y, M, N, K, gs, out_f32, bias, stream, &launched);
        if (st || launched) return st;
    }
    const AffineGemmPlan plan = affine_gemm_plan(M, N, K, ctx->sm_count);
    float* slabs = reinterpret_cast<float*>(workspace);
    if (plan.ks_tail > 1 && (!slabs || !scr_aligned16(slabs))) return scr_fail(ctx, SCR_E_WORKSPACE, "split-K needs an aligned workspace");
    if (plan.tm == 2) return affine_gemm_launch_tm<2>(ctx, map, packed, y, M, N, K, gs, out_f32, bias, plan, slabs, stream);
    return affine_gemm_launch_tm<1>(ctx, map, packed, y, M, N, K, gs, out_f32, bias, plan, slabs, stream);
}
