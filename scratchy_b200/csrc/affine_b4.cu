// MLX affine int4 (group 64): load-time repack, dequant dump hook and the decode matvec.
#include "affine_b4.cuh"

// ------------------------------------------------------------------------------------
// Repack: checkpoint layout -> streaming blocks (layout in affine_b4.cuh).
// One thread per 16-byte piece plus one thread per 8-byte scale entry.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t affine_interleave_word(uint32_t src) {
    // src: code i at bits [4i, 4i+4).  dst: e_{2j} at [4j,4j+4), e_{2j+1} at [16+4j, ...).
    uint32_t dst = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        dst |= ((src >> (8 * j)) & 0xFu) << (4 * j);
        dst |= ((src >> (8 * j + 4)) & 0xFu) << (16 + 4 * j);
    }
    return dst;
}

__global__ void affine_b4_repack_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ scales,
                                        const uint16_t* __restrict__ biases, int N, int K, int RB, int KC,
                                        uint8_t* __restrict__ dst, unsigned int* __restrict__ slow_flag) {
    const long long nblocks = (long long)RB * KC;
    const long long items = nblocks * 80;               // 64 pieces + 16 scale entries per block
    for (long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x; it < items;
         it += (long long)gridDim.x * blockDim.x) {
        const long long blk = it / 80;
        const int sub = int(it % 80);
        const int kc = int(blk / RB), rb = int(blk % RB);
        uint8_t* out = dst + blk * AFF_BLOCK_BYTES;
        if (sub < 64) {
            const int half = sub >> 5, lane = sub & 31, g = lane >> 2, t = lane & 3;
            const int row = rb * 16 + half * 8 + g;
            const int k0 = kc * 128 + t * 32;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < N && k0 < K) {
                const uint4 s = *reinterpret_cast<const uint4*>(w + (size_t)row * (K / 8) + k0 / 8);
                v.x = affine_interleave_word(s.x);
                v.y = affine_interleave_word(s.y);
                v.z = affine_interleave_word(s.z);
                v.w = affine_interleave_word(s.w);
            }
            *reinterpret_cast<uint4*>(out + half * 512 + lane * 16) = v;
        } else {
            const int e = sub - 64, g = e >> 1, h = e & 1;
            const int grp = kc * 2 + h;
            uint2 v = make_uint2(0, 0);
            if (grp * 64 < K) {
                const int G = K / 64;
                const int r0 = rb * 16 + g, r1 = r0 + 8;
                if (r0 < N) v.x = uint32_t(scales[(size_t)r0 * G + grp]) | (uint32_t(biases[(size_t)r0 * G + grp]) << 16);
                if (r1 < N) v.y = uint32_t(scales[(size_t)r1 * G + grp]) | (uint32_t(biases[(size_t)r1 * G + grp]) << 16);
            }
            *reinterpret_cast<uint2*>(out + 1024 + e * 8) = v;
            if (affine_slow_group(v.x) || affine_slow_group(v.y)) atomicOr(slow_flag, 1u);
        }
    }
}

// ------------------------------------------------------------------------------------
// Dump hook: streaming blocks -> dense bf16 [N, K], through affine_dequant_piece.
// ------------------------------------------------------------------------------------
__global__ void affine_b4_dump_kernel(const uint8_t* __restrict__ packed, int N, int K, int RB, int KC,
                                      uint16_t* __restrict__ out) {
    const long long items = (long long)RB * KC * 64;
    const bool check = *reinterpret_cast<const unsigned int*>(packed + (size_t)RB * KC * AFF_BLOCK_BYTES) != 0;
    for (long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x; it < items;
         it += (long long)gridDim.x * blockDim.x) {
        const long long blk = it / 64;
        const int sub = int(it % 64);
        const int kc = int(blk / RB), rb = int(blk % RB);
        const int half = sub >> 5, lane = sub & 31, g = lane >> 2, t = lane & 3;
        const int row = rb * 16 + half * 8 + g;
        const int k0 = kc * 128 + t * 32;
        if (row >= N || k0 >= K) continue;
        const uint8_t* b = packed + blk * AFF_BLOCK_BYTES;
        const uint4 piece = *reinterpret_cast<const uint4*>(b + half * 512 + lane * 16);
        const uint2 sb2 = *reinterpret_cast<const uint2*>(b + 1024 + (g * 2 + (t >> 1)) * 8);
        uint32_t regs[16];
        if (check) affine_dequant_piece<true>(piece, half ? sb2.y : sb2.x, regs);
        else affine_dequant_piece<false>(piece, half ? sb2.y : sb2.x, regs);
        uint4* o = reinterpret_cast<uint4*>(out + (size_t)row * K + k0);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = make_uint4(regs[4 * i], regs[4 * i + 1], regs[4 * i + 2], regs[4 * i + 3]);
    }
}

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

// ------------------------------------------------------------------------------------
// Decode matvec, M <= 16.
//
// Persistent CTAs of 8 warps.  A CTA walks row-blocks (16 weight rows) rb = blockIdx.x,
// += gridDim.x; its warps interleave the row-block's k-chunks (warp w takes kc = w, w+8, ...),
// so the cross-warp reduction stays inside the CTA: partial accumulators go through
// double-buffered shared memory once per row-block, in fixed warp order (deterministic).
//
// Weights stream HBM -> shared memory through per-warp rings of 1-D bulk (TMA) copies, one
// 1152-byte block per stage, each stage with its own mbarrier; the ring runs ahead across
// row-block boundaries, so GEMV_STAGES-1 blocks per warp are always in flight.  A stage is read
// back with two conflict-free 16-byte loads per lane and dequantised in registers; the
// dequantised bf16 weights are the A operand of mma.sync.m16n8k16 and the tokens the 8 columns
// of B (MT = 1: up to 8 tokens, MT = 2: up to 16).  Lane (g, t) holds codes of rows g and g+8
// at k = 128kc + 32t + [0,32) and the activations of token g (and g+8) at the same k, so the
// contraction index is permuted identically on both operands.
//
// When there are too few row-blocks to fill the machine, gridDim.y = SPLIT CTAs form a
// thread-block cluster that splits the k-chunks and reduces through distributed shared memory
// in rank order.  Every wait is bounded (see gemv_wait).
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16_16816(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#define GEMV_WARPS 8
#define GEMV_STAGES 6
#define GEMV_MAX_SPLIT 8

// One 1152-byte block from shared memory against the activations.  Tokens beyond M and k beyond K
// read clamped (valid) activation addresses instead of zeros: a column of B only reaches the
// same column of D, which is discarded for tokens >= M, and padded k meets zero weights.
template <int MT, bool CHECK>
__device__ __forceinline__ void gemv_block_compute(uint32_t stage, float acc[2][MT][4], const uint16_t* const xrow[MT],
                                                   int k0, int lane) {
    const uint4 p0 = gemv_lds_v4(stage + lane * 16);
    const uint4 p1 = gemv_lds_v4(stage + 512 + lane * 16);
    const uint2 sb = gemv_lds_v2(stage + 1024 + ((lane >> 2) * 2 + ((lane & 3) >> 1)) * 8);
    uint4 xv[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) xv[mt][i] = ld_nc_v4(xrow[mt] + k0 + 8 * i);
    uint32_t w0[16], w1[16];
    affine_dequant_piece<CHECK>(p0, sb.x, w0);
    affine_dequant_piece<CHECK>(p1, sb.y, w1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            // two independent accumulator sets halve the dependent-MMA chain
            mma_bf16_16816(acc[0][mt], w0[4 * i + 0], w1[4 * i + 0], w0[4 * i + 1], w1[4 * i + 1], xv[mt][i].x, xv[mt][i].y);
            mma_bf16_16816(acc[1][mt], w0[4 * i + 2], w1[4 * i + 2], w0[4 * i + 3], w1[4 * i + 3], xv[mt][i].z, xv[mt][i].w);
        }
    }
}

template <int MT, int SPLIT_CLUSTER, bool CHECK>
__device__ __forceinline__ void gemv_main(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ x,
                                          uint16_t* __restrict__ y, int M, int N, int K, int RB, int KC, int rb_real,
                                          int split, int* __restrict__ status, uint8_t* ring_gen,
                                          uint64_t (*bars)[GEMV_STAGES], float (*red)[GEMV_WARPS][32][MT * 4],
                                          float (*cl_part)[16][MT * 8]) {
    const int sp = SPLIT_CLUSTER ? int(gemv_cluster_ctarank()) : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    // k-chunks of this CTA: [kc_lo, kc_hi); warp w takes kc_lo + w, + GEMV_WARPS, ...
    const int per = (KC + split - 1) / split;
    const int kc_lo = sp * per;
    const int kc_hi = min(KC, kc_lo + per);
    const int kc_first = kc_lo + warp;
    const bool has_work = kc_first < kc_hi;

    const size_t chunk_stride = (size_t)RB * AFF_BLOCK_BYTES;
    const uint32_t ring_base = gemv_smem_u32(ring_gen) + (uint32_t)warp * (GEMV_STAGES * AFF_BLOCK_BYTES);
    const uint32_t bar_base = gemv_smem_u32(&bars[warp][0]);

    // producer cursor (only lane 0 uses it): next block to request, in consumption order
    int prb = blockIdx.x, pkc = kc_first, pslot = 0;
    auto issue = [&]() {
        if (has_work && prb < rb_real) {
            const uint32_t bar = bar_base + 8u * pslot;
            gemv_arrive_expect_tx(bar, AFF_BLOCK_BYTES);
            gemv_bulk_g2s(ring_base + pslot * AFF_BLOCK_BYTES, packed + (size_t)pkc * chunk_stride + (size_t)prb * AFF_BLOCK_BYTES,
                          AFF_BLOCK_BYTES, bar);
            pkc += GEMV_WARPS;
            if (pkc >= kc_hi) { pkc = kc_first; prb += gridDim.x; }
        }
        pslot = (pslot + 1 == GEMV_STAGES) ? 0 : pslot + 1;
    };
    if (lane == 0) {
#pragma unroll 1
        for (int d = 0; d < GEMV_STAGES; ++d) issue();
    }

    // activation rows this lane feeds into the B operand (clamped to a valid token)
    const uint16_t* xrow[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) xrow[mt] = x + (size_t)min(mt * 8 + g, M - 1) * K;
    const int kt_off = t * 32;

    int slot = 0;
    uint32_t phases = 0;                       // bit d = parity the next wait on stage d expects
    int it = 0;

    for (int rb = blockIdx.x; rb < rb_real; rb += gridDim.x, ++it) {
        float acc[2][MT][4];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[a][mt][i] = 0.f;

#pragma unroll 1
        for (int kc = kc_first; kc < kc_hi; kc += GEMV_WARPS) {
            gemv_wait(bar_base + 8u * slot, (phases >> slot) & 1u, status);
            int k0 = kc * 128 + kt_off;
            if (k0 >= K) k0 = 0;               // padded k: the weights there are zero
            gemv_block_compute<MT, CHECK>(ring_base + slot * AFF_BLOCK_BYTES, acc, xrow, k0, lane);
            phases ^= 1u << slot;
            __syncwarp();                      // every lane has consumed the stage: refill it
            if (lane == 0) issue();
            slot = (slot + 1 == GEMV_STAGES) ? 0 : slot + 1;
        }

        // cross-warp reduction of this row-block, fixed warp order, double-buffered
        const int buf = it & 1;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) red[buf][warp][lane][mt * 4 + i] = acc[0][mt][i] + acc[1][mt][i];
        __syncthreads();

        // thread e owns accumulator slot (ln, idx): c0,c1 -> row g, tokens 2t,2t+1 ; c2,c3 -> row g+8
        constexpr int SLOTS = 32 * MT * 4;     // <= 256 = blockDim.x
        const int e = threadIdx.x;
        const int ln = e / (MT * 4), idx = e % (MT * 4);
        const int row = (ln >> 2) + (((idx & 3) >> 1) ? 8 : 0);
        const int tok = (idx >> 2) * 8 + (ln & 3) * 2 + (idx & 1);
        const int n = rb * 16 + row;
        if (e < SLOTS && tok < M) {
            float total = 0.f;
#pragma unroll
            for (int wdx = 0; wdx < GEMV_WARPS; ++wdx) total += red[buf][wdx][ln][idx];
            if (SPLIT_CLUSTER) {
                gemv_st_cluster_rank0_f32(&cl_part[sp][row][tok], total);
            } else if (n < N) {
                const __nv_bfloat16 v = __float2bfloat16_rn(total);
                y[(size_t)tok * N + n] = *reinterpret_cast<const uint16_t*>(&v);
            }
        }
        if (SPLIT_CLUSTER) {
            // one row-block per CTA in cluster mode (gridDim.x == rb_real): exchange once
            gemv_cluster_sync_all();
            if (sp == 0 && e < SLOTS && tok < M && n < N) {
                float s = 0.f;
                for (int r = 0; r < split; ++r) s += cl_part[r][row][tok];   // rank order
                const __nv_bfloat16 v = __float2bfloat16_rn(s);
                y[(size_t)tok * N + n] = *reinterpret_cast<const uint16_t*>(&v);
            }
        }
    }
}

template <int MT, int SPLIT_CLUSTER>
__global__ void __launch_bounds__(GEMV_WARPS * 32, 2)
affine_b4_gemv_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                      int M, int N, int K, int RB, int KC, int rb_real, int split, int* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t gemv_ring[];          // [GEMV_WARPS][GEMV_STAGES][AFF_BLOCK_BYTES]
    __shared__ __align__(8) uint64_t bars[GEMV_WARPS][GEMV_STAGES];
    __shared__ float red[2][GEMV_WARPS][32][MT * 4];
    __shared__ float cl_part[SPLIT_CLUSTER ? GEMV_MAX_SPLIT : 1][16][MT * 8];

    if ((threadIdx.x & 31) == 0) {
#pragma unroll
        for (int d = 0; d < GEMV_STAGES; ++d) gemv_mbar_init(gemv_smem_u32(&bars[threadIdx.x >> 5][d]), 1);
    }
    gemv_fence_mbar_init();
    __syncthreads();

    // one word per matrix says whether any group needs the exact (two-step rounding) path
    const bool check = *reinterpret_cast<const unsigned int*>(packed + (size_t)RB * KC * AFF_BLOCK_BYTES) != 0;
    if (check) gemv_main<MT, SPLIT_CLUSTER, true>(packed, x, y, M, N, K, RB, KC, rb_real, split, status, gemv_ring, bars, red, cl_part);
    else gemv_main<MT, SPLIT_CLUSTER, false>(packed, x, y, M, N, K, RB, KC, rb_real, split, status, gemv_ring, bars, red, cl_part);
}

// ------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------
static int32_t affine_check_shape(scr_ctx* ctx, int N, int K, int group) {
    if (N <= 0 || K <= 0) return scr_fail(ctx, SCR_E_SHAPE, "N=%d K=%d must be positive", N, K);
    if (group != 64) return scr_fail(ctx, SCR_E_DTYPE, "group_size=%d: this build implements group 64 only", group);
    if (K % group != 0) return scr_fail(ctx, SCR_E_SHAPE, "K=%d not divisible by group_size=%d", K, group);
    return SCR_OK;
}

extern "C" int32_t scr_affine_b4_repack_size(int32_t N, int32_t K, int32_t group, size_t* bytes) {
    if (!bytes) return SCR_E_ARG;
    if (N <= 0 || K <= 0) return SCR_E_SHAPE;
    if (group != 64) return SCR_E_DTYPE;
    if (K % group != 0) return SCR_E_SHAPE;
    const AffineGeom g = affine_geom(N, K);
    *bytes = affine_packed_bytes(g);
    return SCR_OK;
}

extern "C" int32_t scr_affine_b4_repack(scr_ctx* ctx, const uint32_t* w, const uint16_t* scales, const uint16_t* biases,
                                        int32_t N, int32_t K, int32_t group, void* dst, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!w || !scales || !biases || !dst) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    int32_t st = affine_check_shape(ctx, N, K, group);
    if (st) return st;
    if (!scr_aligned16(w) || !scr_aligned16(dst)) return scr_fail(ctx, SCR_E_ALIGN, "w/dst must be 16-byte aligned");
    const AffineGeom g = affine_geom(N, K);
    const long long items = (long long)g.RB * g.KC * 80;
    const int threads = 256;
    const int blocks = (int)std::min<long long>((items + threads - 1) / threads, (long long)ctx->sm_count * 32);
    unsigned int* flag = reinterpret_cast<unsigned int*>((uint8_t*)dst + affine_blocks_bytes(g));
    cudaError_t e = cudaMemsetAsync(flag, 0, AFF_TRAILER_BYTES, (cudaStream_t)stream);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "affine_b4_repack memset: %s", cudaGetErrorString(e));
    affine_b4_repack_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>(w, scales, biases, N, K, g.RB, g.KC,
                                                                         (uint8_t*)dst, flag);
    return scr_check_launch(ctx, "affine_b4_repack");
}

extern "C" int32_t scr_affine_b4_dequant_dump(scr_ctx* ctx, const void* packed, int32_t N, int32_t K, int32_t group,
                                              uint16_t* w_bf16, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!packed || !w_bf16) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    int32_t st = affine_check_shape(ctx, N, K, group);
    if (st) return st;
    if (!scr_aligned16(packed) || !scr_aligned16(w_bf16)) return scr_fail(ctx, SCR_E_ALIGN, "pointers must be 16-byte aligned");
    const AffineGeom g = affine_geom(N, K);
    const long long items = (long long)g.RB * g.KC * 64;
    const int threads = 256;
    const int blocks = (int)std::min<long long>((items + threads - 1) / threads, (long long)ctx->sm_count * 32);
    affine_b4_dump_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>((const uint8_t*)packed, N, K, g.RB, g.KC, w_bf16);
    return scr_check_launch(ctx, "affine_b4_dequant_dump");
}

// Launch shape.  With enough row-blocks the grid is persistent (two CTAs per SM) and nothing
// is split; with few row-blocks each CTA takes one row-block and a cluster of `split` CTAs
// shares its k-chunks so that about one CTA per SM is busy.
static void affine_gemv_shape(int rb_real, int KC, int sms, int* grid_x, int* split) {
    if (rb_real >= sms) {
        *grid_x = std::min(rb_real, 2 * sms);
        *split = 1;
        return;
    }
    int s = 1;
    while (s * 2 <= GEMV_MAX_SPLIT && rb_real * s * 2 <= 2 * sms && KC / (s * 2) >= GEMV_WARPS / 2) s *= 2;
    *grid_x = rb_real;
    *split = s;
}

template <int MT>
static int32_t affine_gemv_launch(scr_ctx* ctx, const uint8_t* packed, const uint16_t* x, uint16_t* y, int M, int N,
                                  int K, cudaStream_t stream) {
    const AffineGeom g = affine_geom(N, K);
    const int rb_real = scr_ceil_div(N, 16);
    int grid_x = 1, split = 1;
    affine_gemv_shape(rb_real, g.KC, ctx->sm_count, &grid_x, &split);
    constexpr int kRingBytes = GEMV_WARPS * GEMV_STAGES * AFF_BLOCK_BYTES;
    if (split == 1) {
        cudaError_t e0 = cudaFuncSetAttribute(affine_b4_gemv_kernel<MT, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes);
        if (e0 != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "affine_b4_gemv smem attribute: %s", cudaGetErrorString(e0));
        affine_b4_gemv_kernel<MT, 0><<<dim3(grid_x, 1), GEMV_WARPS * 32, kRingBytes, stream>>>(packed, x, y, M, N, K, g.RB, g.KC,
                                                                                              rb_real, 1, ctx->dev_status);
        return scr_check_launch(ctx, "affine_b4_gemv");
    }
    cudaError_t e1 = cudaFuncSetAttribute(affine_b4_gemv_kernel<MT, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes);
    if (e1 != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "affine_b4_gemv smem attribute: %s", cudaGetErrorString(e1));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid_x, split, 1);
    cfg.blockDim = dim3(GEMV_WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = kRingBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = split;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, affine_b4_gemv_kernel<MT, 1>, packed, x, y, M, N, K, g.RB, g.KC, rb_real, split,
                                       ctx->dev_status);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "affine_b4_gemv cluster launch: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "affine_b4_gemv(cluster)");
}

// Defined in affine_b4_gemm.cu
int32_t affine_b4_gemm_tc_launch(scr_ctx* ctx, const uint8_t* packed, const uint16_t* x, uint16_t* y, int M, int N,
                                 int K, void* workspace, size_t workspace_bytes, cudaStream_t stream);
size_t affine_b4_gemm_tc_workspace(int M, int N, int K);
bool affine_b4_gemm_tc_enabled();

size_t affine_workspace_bytes(int M, int N, int K) {
    if (M <= 16 || !affine_b4_gemm_tc_enabled()) return 0;
    return affine_b4_gemm_tc_workspace(M, N, K);
}

extern "C" int32_t scr_linear_affine_b4(scr_ctx* ctx, const void* packed, const uint16_t* x, int32_t M, int32_t N,
                                        int32_t K, int32_t group, uint16_t* y, void* workspace, size_t workspace_bytes,
                                        void* stream_) {
    SCR_REQUIRE_CTX(ctx);
    if (!packed || !x || !y) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    int32_t st = affine_check_shape(ctx, N, K, group);
    if (st) return st;
    if (M <= 0) return scr_fail(ctx, SCR_E_SHAPE, "M=%d must be positive", M);
    if (!scr_aligned16(packed) || !scr_aligned16(x)) return scr_fail(ctx, SCR_E_ALIGN, "packed/x must be 16-byte aligned");
    cudaStream_t stream = (cudaStream_t)stream_;
    const uint8_t* pk = (const uint8_t*)packed;
    if (M <= 8) return affine_gemv_launch<1>(ctx, pk, x, y, M, N, K, stream);
    if (M <= 16) return affine_gemv_launch<2>(ctx, pk, x, y, M, N, K, stream);
    if (affine_b4_gemm_tc_enabled()) {
        const size_t need = affine_b4_gemm_tc_workspace(M, N, K);
        if (need > 0 && (!workspace || workspace_bytes < need))
            return scr_fail(ctx, SCR_E_WORKSPACE, "workspace %zu bytes < required %zu", workspace_bytes, need);
        return affine_b4_gemm_tc_launch(ctx, pk, x, y, M, N, K, workspace, workspace_bytes, stream);
    }
    // Token tiles of 16 through the matvec kernel (weights re-streamed per tile).
    for (int m0 = 0; m0 < M; m0 += 16) {
        const int mt = std::min(16, M - m0);
        st = (mt <= 8) ? affine_gemv_launch<1>(ctx, pk, x + (size_t)m0 * K, y + (size_t)m0 * N, mt, N, K, stream)
                       : affine_gemv_launch<2>(ctx, pk, x + (size_t)m0 * K, y + (size_t)m0 * N, mt, N, K, stream);
        if (st) return st;
    }
    return SCR_OK;
}
