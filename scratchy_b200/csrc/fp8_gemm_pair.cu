// fp8-dynamic-per-channel prefill GEMM on a CTA PAIR: tcgen05.mma.cta_group::2, a 256-token x 256-channel tile
// per pair of SMs.
//
//   y[m,n] = bf16( (sum_k x_q[m,k] * w_q[n,k]) * a_scale[m] * w_scale[n] (+ bias[n]) )
//
// Why a pair.  With one CTA per tile (fp8_gemm.cu: 128 tokens x 256 channels) a 128-byte k-tile costs that SM 48 KB of
// L2 -> shared-memory traffic for 2 * 128 * 256 * 128 flops; at the rate the tensor core wants them that is close to
// what one SM can pull from L2, and the 4 stages of 48 KB that fit run dry.  In a pair each CTA stages its own 128 tokens
// of A and only ITS HALF (128 channels) of B: 32 KB per k-tile for the same flops per SM.  One
// `tcgen05.mma.cta_group::2` of shape 256 x 256 x 32, issued by the pair's leader CTA, reads A rows and B columns
// from both SMs' shared memory and writes each CTA's 128 accumulator rows into that CTA's own TMEM.
//
// Per CTA (192 threads), both CTAs of a pair run the same code:
//   warp 0     producer: tiled TMA loads (`.cta_group::2`, no multicast) of this CTA's pre-swizzled 16 KB A and B
//              tiles into a 3-stage ring of 2 k-tiles per stage in ITS OWN shared memory; both CTAs' loads of a stage
//              complete on the LEADER's `full` barrier
//   warp 1     leader CTA only: one thread waits for a stage, issues 8 MMAs (K = 32 each) and commits to the stage's
//              `empty` barrier of both CTAs (one commit per two k-tiles: a commit per k-tile measured 8 % slower)
//   warps 2-5  epilogue of this CTA's 128 rows x 256 columns (tcgen05.ld, scales, bias, bf16 or f32 stores); they
//              release the accumulator buffer to the leader (the peer's warps with remote mbarrier arrives)
// Two accumulator buffers (2 x 256 TMEM columns) overlap the epilogue of tile i with the main loop of tile i + 1.
// Every wait is bounded (tc_common.cuh); the pair meets at a cluster barrier before either CTA frees its TMEM or
// exits, so no remote arrive can reach a CTA that has left.
//
// Measured against the one-CTA kernel on Qwen2.5-7B shapes (same bits): gate M = 8192 2667 against 2387 TFLOP/s, gate
// M = 2048 2414 against 2229, q M = 8192 1790 against 1607, down M = 8192 1985 against 1935.  An instrumented build
// showed the tensor pipe about 93 % busy in cycles; what remains is the clock under the power cap.  Variants measured
// and dropped: the peer's "stage full" relayed to the leader by a thread of the peer with a remote arrive instead of
// `.cta_group::2` loads (5 % slower); `.acquire.cluster` / `.release.cluster` on the cross-CTA barrier operations (2x
// slower: the default scopes are what the pair's barriers need); 6 or 7 stages of one k-tile.
#include "fp8.cuh"
#include "tc_common.cuh"

#include <cstdlib>

namespace {

constexpr int F8P_STAGES = 3;
constexpr int F8P_THREADS = 192;
constexpr int F8P_KSTEP = 2;                                 // k-tiles per ring stage (one commit per stage)
constexpr uint32_t F8P_STAGE_BYTES = 32768u * F8P_KSTEP;     // per k-tile: A tile + this CTA's B tile
constexpr uint32_t F8P_BAR_OFFSET = F8P_STAGES * F8P_STAGE_BYTES;
constexpr uint32_t F8P_SMEM_TOTAL = F8P_BAR_OFFSET + 256u + 1024u;
constexpr int F8P_BN = 256;                                   // channels per pair tile (128 per CTA)

__device__ __forceinline__ uint32_t pair_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void pair_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of `local` (a shared::cta address of this CTA) inside CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t pair_map(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ void pair_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// D[tmem of both CTAs] (+)= A[both CTAs' smem] * B[both CTAs' smem]^T: 256 x N x 32, issued by the leader CTA.
__device__ __forceinline__ void umma_f8f6f4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on the barrier at `bar`'s offset in BOTH CTAs of the pair once every MMA this thread has issued is complete
// (a barrier signal sent to two CTAs; no data moves).
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(both) : "memory");
}

// One pre-swizzled 16 KB tile as a tiled TMA load of 64 rows x 256 bytes of a byte tensor [bytes / 256][256].  With
// `.cta_group::2` the completion may be counted on a barrier of the OTHER CTA of the pair: both CTAs' loads of a stage
// complete on the leader's `full` barrier, so the MMA thread learns "the stage is full in both CTAs" from one wait.  The
// destination is this CTA's own shared memory; nothing is multicast.
__device__ __forceinline__ void pair_tma_tile(uint32_t dst_smem, const CUtensorMap* map, int row, uint32_t bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst_smem), "l"(map), "r"(0), "r"(row), "r"(bar_cluster_addr) : "memory");
}

__global__ void __launch_bounds__(F8P_THREADS, 1)
fp8_gemm_pair_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                     const uint8_t* __restrict__ wpack, const float* __restrict__ w_scale, const uint8_t* __restrict__ xq,
                     const float* __restrict__ a_scale, uint16_t* __restrict__ y, int M, int N, int KT, int NT, int MT,
                     int M_pad, int out_f32, const uint16_t* __restrict__ bias, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + F8P_BAR_OFFSET;
    // barrier slots (8 bytes each): full[S] (used on the leader), empty[S], acc_full[2], acc_empty[2] (used on the leader)
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (F8P_STAGES + s); };
    auto accf_bar = [&](int b) { return bar_base + 8u * (2 * F8P_STAGES + b); };
    auto acce_bar = [&](int b) { return bar_base + 8u * (2 * F8P_STAGES + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + F8P_BAR_OFFSET + 8 * (2 * F8P_STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = pair_cta_rank();               // 0 = the pair's leader
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int MTP = MT >> 1, NTP = NT >> 1;              // pair tiles: 256 tokens x 256 channels
    const int tiles = MTP * NTP;

    if (threadIdx.x == 0) {
        for (int s = 0; s < F8P_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), 256); }   // 128 epilogue threads of each CTA
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_slot), 2 * F8P_BN);     // each CTA allocates its own columns; both get the same base
        tmem_relinquish();
    }
    tc_fence_before();
    pair_sync();                                          // both CTAs' barriers and TMEM exist before anything crosses over
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (both CTAs)
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            for (int t = pair; t < tiles; t += npairs) {
                const int mb = t % MTP, nb = t / MTP;
                const int mt = 2 * mb + (int)rank, nt = 2 * nb + (int)rank;
                for (int kt = 0; kt < KT; kt += F8P_KSTEP) {
                    mbar_wait(empty_bar(s), ph ^ 1u, status, TC_ERR_EMPTY_WAIT);
                    const int nk = min(F8P_KSTEP, KT - kt);
                    // both CTAs' loads of the stage complete on the LEADER's barrier: it expects both CTAs' bytes
                    const uint32_t lead_full = pair_map(full_bar(s), 0);
                    if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2u * 32768u * nk);
                    for (int j = 0; j < nk; ++j) {
                        const uint32_t sa = smem_base + s * F8P_STAGE_BYTES + j * 32768u;
                        pair_tma_tile(sa, &x_map, (kt + j) * (M_pad / 2) + mt * 64, lead_full);              // tile offset / 256 bytes
                        pair_tma_tile(sa + 16384u, &w_map, (nt * KT + kt + j) * 64, lead_full);
                    }
                    if (++s == F8P_STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // -------------------------------------------------------------- MMA issuer (leader CTA)
            const uint32_t idesc = umma_idesc(0, 0, 256, F8P_BN);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            for (int t = pair; t < tiles; t += npairs, ++it) {
                const int buf = it & 1;
                mbar_wait(acce_bar(buf), ((uint32_t)(it >> 1) & 1u) ^ 1u, status, TC_ERR_ACC_EMPTY);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * F8P_BN);
                for (int kt = 0; kt < KT; kt += F8P_KSTEP) {
                    mbar_wait(full_bar(s), ph, status, TC_ERR_FULL_WAIT);
                    tc_fence_after();
                    const int nk = min(F8P_KSTEP, KT - kt);
                    for (int j = 0; j < nk; ++j) {
                        const uint32_t sa = smem_base + s * F8P_STAGE_BYTES + j * 32768u;
                        const uint64_t adesc = umma_desc_k_sw128(sa);
                        const uint64_t bdesc = umma_desc_k_sw128(sa + 16384u);
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4)
                            umma_f8f6f4_pair(d_tmem, adesc + (uint64_t)(2 * k4), bdesc + (uint64_t)(2 * k4), idesc, ((kt + j) | k4) != 0);
                    }
                    umma_commit_pair(empty_bar(s));
                    if (++s == F8P_STAGES) { s = 0; ph ^= 1u; }
                }
                umma_commit_pair(accf_bar(buf));
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
        const int q = warp & 3;                                   // TMEM lane quadrant this warp may read
        const bool vec_ok = (N % 8) == 0;
        const bool f32mode = out_f32 != 0;
        float* fbase = reinterpret_cast<float*>(y);
        int it = 0;
        for (int t = pair; t < tiles; t += npairs, ++it) {
            const int mb = t % MTP, nb = t / MTP;
            const int n0 = nb * F8P_BN;
            const int buf = it & 1;
            mbar_wait(accf_bar(buf), (uint32_t)(it >> 1) & 1u, status, TC_ERR_ACC_FULL);
            tc_fence_after();
            const int m = (2 * mb + (int)rank) * 128 + q * 32 + lane;
            const float as = (m < M) ? a_scale[m] : 0.f;
            uint16_t* yrow = y + (size_t)m * N;
            for (int c = 0; c < F8P_BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * F8P_BN + c * 32), r);
                tmem_ld_wait();
                const int nc = n0 + c * 32;
                if (m >= M || nc >= N) continue;
                if (f32mode) {
                    float* frow = fbase + (size_t)m * N + nc;
                    const bool v4 = (N % 4) == 0 && nc + 32 <= N;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 ws = __ldg(reinterpret_cast<const float4*>(w_scale + nc) + j);
                        float4 v;
                        v.x = __fmul_rn(__fmul_rn(__uint_as_float(r[4 * j + 0]), as), ws.x);
                        v.y = __fmul_rn(__fmul_rn(__uint_as_float(r[4 * j + 1]), as), ws.y);
                        v.z = __fmul_rn(__fmul_rn(__uint_as_float(r[4 * j + 2]), as), ws.z);
                        v.w = __fmul_rn(__fmul_rn(__uint_as_float(r[4 * j + 3]), as), ws.w);
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
                    for (int j = 0; j < 8; ++j) {
                        const float4 ws = __ldg(reinterpret_cast<const float4*>(w_scale + nc) + j);   // scales are padded to NT*128
                        float v0 = __fmul_rn(__fmul_rn(__uint_as_float(r[4 * j + 0]), as), ws.x);
                        float v1 = __fmul_rn(__fmul_rn(__uint_as_float(r[4 * j + 1]), as), ws.y);
                        float v2 = __fmul_rn(__fmul_rn(__uint_as_float(r[4 * j + 2]), as), ws.z);
                        float v3 = __fmul_rn(__fmul_rn(__uint_as_float(r[4 * j + 3]), as), ws.w);
                        if (bias) {                    // the linear's own bias, added in f32 before the one rounding
                            const int n4 = nc + 4 * j;
                            if (n4 + 0 < N) v0 += __uint_as_float(uint32_t(bias[n4 + 0]) << 16);
                            if (n4 + 1 < N) v1 += __uint_as_float(uint32_t(bias[n4 + 1]) << 16);
                            if (n4 + 2 < N) v2 += __uint_as_float(uint32_t(bias[n4 + 2]) << 16);
                            if (n4 + 3 < N) v3 += __uint_as_float(uint32_t(bias[n4 + 3]) << 16);
                        }
                        const __nv_bfloat162 p0 = __floats2bfloat162_rn(v0, v1);
                        const __nv_bfloat162 p1 = __floats2bfloat162_rn(v2, v3);
                        o[2 * j] = *reinterpret_cast<const uint32_t*>(&p0);
                        o[2 * j + 1] = *reinterpret_cast<const uint32_t*>(&p1);
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
            if (rank == 0) mbar_arrive(acce_bar(buf));
            else pair_arrive_remote(pair_map(acce_bar(buf), 0));
        }
    }

    tc_fence_before();
    pair_sync();                                          // nobody frees TMEM or leaves while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * F8P_BN);
    }
}

}  // namespace


// Whether the pair kernel takes this GEMM: whole pair tiles in both directions, at least one full round of pairs and
// rounds that are at least 70 % full (measured: at 76 % full, q and down of Qwen2.5-7B at 2048 tokens, the pair kernel is
// still 5 and 9 % ahead of the one-CTA kernel, which splits its tail along k instead).  `SCR_FP8_GEMM_PAIR=0` in the
// environment switches the pair kernel off (read once).
bool fp8_gemm_pair_applies(int M, int N, int K, int sms) {
    static const bool enabled = [] {
        const char* e = std::getenv("SCR_FP8_GEMM_PAIR");
        return !(e && e[0] == '0');
    }();
    if (!enabled) return false;
    const Fp8Geom g = fp8_geom(N, K);
    const int MT = scr_ceil_div(M, 128);
    if ((MT & 1) || (g.NT & 1) || g.KT < 1) return false;
    const int pairs = sms / 2, tiles = (MT / 2) * (g.NT / 2);
    if (pairs < 1 || tiles < pairs) return false;
    const int rounds = (tiles + pairs - 1) / pairs;
    return (float)tiles >= 0.70f * (float)(rounds * pairs);
}

int32_t fp8_gemm_pair_launch(scr_ctx* ctx, const uint8_t* wpack, const uint8_t* act, uint16_t* y, int M, int N, int K,
                             const LinearEnds& ends, cudaStream_t stream, bool* launched) {
    *launched = false;
    const Fp8Geom g = fp8_geom(N, K);
    const int MT = scr_ceil_div(M, 128);
    const float* w_scale = reinterpret_cast<const float*>(wpack + (size_t)g.NT * g.KT * FP8_TILE_BYTES);
    const float* a_scale = reinterpret_cast<const float*>(act);
    const uint8_t* xq = act + fp8_act_scale_bytes(M);
    cudaError_t e = cudaFuncSetAttribute(fp8_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F8P_SMEM_TOTAL);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "fp8_gemm_pair smem attribute: %s", cudaGetErrorString(e));
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(F8P_THREADS);
    cfg.dynamicSmemBytes = F8P_SMEM_TOTAL;
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
        e = cudaOccupancyMaxActiveClusters(&max_pairs, fp8_gemm_pair_kernel, &cfg);
        if (e != cudaSuccess || max_pairs < 1) {
            (void)cudaGetLastError();
            max_pairs = -1;
        }
        if (ctx->device >= 0 && ctx->device < 64) pairs_of_device[ctx->device] = max_pairs;
    }
    if (max_pairs < 1) return SCR_OK;                     // not launched: the caller runs the one-CTA kernel
    const int tiles = (MT / 2) * (g.NT / 2);
    cfg.gridDim = dim3(2 * std::min(tiles, max_pairs));
    // the pre-swizzled 16 KB tiles of both operands as byte tensors [bytes / 256][256]: a tile is a box of 64 rows
    tc_encode_tiled_fn enc = tc_tensor_map_encoder();
    if (!enc) return SCR_OK;
    CUtensorMap maps[2];
    const void* bases[2] = {wpack, xq};
    const unsigned long long bytes[2] = {(unsigned long long)g.NT * g.KT * FP8_TILE_BYTES, (unsigned long long)g.KT * MT * 16384ull};
    for (int i = 0; i < 2; ++i) {
        const cuuint64_t dims[2] = {256, (cuuint64_t)(bytes[i] / 256)};
        const cuuint64_t strides[1] = {256};
        const cuuint32_t box[2] = {256, 64};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult r = enc(&maps[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(bases[i]), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return SCR_OK;               // not launched: the caller runs the one-CTA kernel
    }
    e = cudaLaunchKernelEx(&cfg, fp8_gemm_pair_kernel, maps[0], maps[1], wpack, w_scale, xq, a_scale, y, M, N, g.KT, g.NT, MT, MT * 128,
                           ends.out_f32, ends.bias, ctx->dev_status);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "fp8_gemm_pair launch: %s", cudaGetErrorString(e));
    *launched = true;
    return scr_check_launch(ctx, "fp8_gemm_pair");
}
