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
                                        uint8_t* __restrict__ dst) {
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
        }
    }
}

// ------------------------------------------------------------------------------------
// Dump hook: streaming blocks -> dense bf16 [N, K], through affine_dequant_piece.
// ------------------------------------------------------------------------------------
__global__ void affine_b4_dump_kernel(const uint8_t* __restrict__ packed, int N, int K, int RB, int KC,
                                      uint16_t* __restrict__ out) {
    const long long items = (long long)RB * KC * 64;
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
        affine_dequant_piece(piece, half ? sb2.y : sb2.x, regs);
        uint4* o = reinterpret_cast<uint4*>(out + (size_t)row * K + k0);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = make_uint4(regs[4 * i], regs[4 * i + 1], regs[4 * i + 2], regs[4 * i + 3]);
    }
}

// ------------------------------------------------------------------------------------
// Decode matvec, M <= 16.
//
// A warp owns one row-block (16 weight rows) over a set of k-chunks and feeds
// mma.sync.m16n8k16 (bf16 x bf16 -> f32) with the dequantised weights as the A operand
// straight from registers; the tokens are the 8 columns of the B operand (MT = 1: up to 8
// tokens, MT = 2: up to 16).  Lane (g, t) holds codes of rows g and g+8 at
// k = 128kc + 32t + [0,32) and the activations of token g (and g+8) at the same k, so the
// contraction index is permuted identically on both operands.
//
// Grid: (RB_real, SPLIT).  The 8 warps of a CTA interleave the CTA's k-chunks; partial
// sums are reduced through shared memory in warp order, and, when SPLIT > 1, across the
// SPLIT CTAs of a thread-block cluster through distributed shared memory in rank order
// (deterministic; no global scratch).
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16_16816(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cluster_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

#define GEMV_WARPS 4
#define GEMV_STAGES 4
#define GEMV_MAX_SPLIT 8

struct GemvStage {
    uint4 p0, p1;   // codes of rows g / g+8
    uint2 sb;       // (scale, bias) of rows g / g+8
};

__device__ __forceinline__ void gemv_stage_load(GemvStage& s, const uint8_t* blk, int lane) {
    s.p0 = ld_stream_v4(blk + lane * 16);
    s.p1 = ld_stream_v4(blk + 512 + lane * 16);
    s.sb = ld_stream_v2(blk + 1024 + ((lane >> 2) * 2 + ((lane & 3) >> 1)) * 8);
}

template <int MT>
__device__ __forceinline__ void gemv_stage_compute(const GemvStage& s, float acc[MT][4], const uint16_t* __restrict__ x,
                                                   int kc, int K, int g, int t, bool tok_ok0, bool tok_ok1) {
    const int k0 = kc * 128 + t * 32;
    uint32_t xr[MT][16];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const bool ok = (mt == 0 ? tok_ok0 : tok_ok1) && (k0 < K);
        const uint16_t* xp = x + (size_t)(mt * 8 + g) * K + k0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (ok) v = ld_nc_v4(xp + 8 * i);
            xr[mt][4 * i + 0] = v.x; xr[mt][4 * i + 1] = v.y; xr[mt][4 * i + 2] = v.z; xr[mt][4 * i + 3] = v.w;
        }
    }
    uint32_t w0[16], w1[16];
    affine_dequant_piece(s.p0, s.sb.x, w0);
    affine_dequant_piece(s.p1, s.sb.y, w1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            mma_bf16_16816(acc[mt], w0[4 * i + 0], w1[4 * i + 0], w0[4 * i + 1], w1[4 * i + 1],
                           xr[mt][4 * i + 0], xr[mt][4 * i + 1]);
            mma_bf16_16816(acc[mt], w0[4 * i + 2], w1[4 * i + 2], w0[4 * i + 3], w1[4 * i + 3],
                           xr[mt][4 * i + 2], xr[mt][4 * i + 3]);
        }
    }
}

template <int MT, int SPLIT_CLUSTER>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
affine_b4_gemv_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                      int M, int N, int K, int RB, int KC, int split) {
    // [warp][lane][MT*4] partials, then (cluster) [rank][16 rows][MT*8 tokens]
    __shared__ float red[GEMV_WARPS][32][MT * 4];
    __shared__ float cl_part[SPLIT_CLUSTER ? GEMV_MAX_SPLIT : 1][16][MT * 8];

    const int rb = blockIdx.x;
    const int sp = SPLIT_CLUSTER ? int(cluster_ctarank()) : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    // k-chunks of this CTA: [kc_lo, kc_hi), interleaved over the warps
    const int per = (KC + split - 1) / split;
    const int kc_lo = sp * per;
    const int kc_hi = min(KC, kc_lo + per);

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;

    const size_t chunk_stride = (size_t)RB * AFF_BLOCK_BYTES;
    const uint8_t* base = packed + (size_t)rb * AFF_BLOCK_BYTES;
    const bool tok_ok0 = g < M;
    const bool tok_ok1 = (MT > 1) && (g + 8 < M);

    // register ring of GEMV_STAGES chunks in flight per warp
    GemvStage st[GEMV_STAGES];
    int kc = kc_lo + warp;
#pragma unroll
    for (int d = 0; d < GEMV_STAGES; ++d) {
        const int k = kc + d * GEMV_WARPS;
        if (k < kc_hi) gemv_stage_load(st[d], base + (size_t)k * chunk_stride, lane);
    }
    for (; kc < kc_hi; kc += GEMV_STAGES * GEMV_WARPS) {
#pragma unroll
        for (int d = 0; d < GEMV_STAGES; ++d) {
            const int kcur = kc + d * GEMV_WARPS;
            if (kcur < kc_hi) {
                const GemvStage cur = st[d];
                const int knext = kcur + GEMV_STAGES * GEMV_WARPS;
                if (knext < kc_hi) gemv_stage_load(st[d], base + (size_t)knext * chunk_stride, lane);
                gemv_stage_compute<MT>(cur, acc, x, kcur, K, g, t, tok_ok0, tok_ok1);
            }
        }
    }

    // cross-warp reduction, fixed warp order
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][lane][mt * 4 + i] = acc[mt][i];
    __syncthreads();

    // MT*4 accumulator slots per lane: thread e sums slot (ln, idx) over the warps
    constexpr int SLOTS = 32 * MT * 4;
    static_assert(SLOTS % (GEMV_WARPS * 32) == 0 || SLOTS <= GEMV_WARPS * 32, "slot mapping");
    constexpr int PER_THREAD = (SLOTS + GEMV_WARPS * 32 - 1) / (GEMV_WARPS * 32);
    float total[PER_THREAD];
    int row[PER_THREAD], tok[PER_THREAD];
#pragma unroll
    for (int u = 0; u < PER_THREAD; ++u) {
        const int e = threadIdx.x + u * GEMV_WARPS * 32;
        total[u] = 0.f; row[u] = 0; tok[u] = 0;
        if (e < SLOTS) {
            const int ln = e / (MT * 4), idx = e % (MT * 4);
            const int mt = idx >> 2, i = idx & 3;
#pragma unroll
            for (int wdx = 0; wdx < GEMV_WARPS; ++wdx) total[u] += red[wdx][ln][idx];
            // accumulator fragment: c0,c1 -> row g, tokens 2t,2t+1 ; c2,c3 -> row g+8
            row[u] = (ln >> 2) + ((i >> 1) ? 8 : 0);
            tok[u] = mt * 8 + (ln & 3) * 2 + (i & 1);
        }
    }

    if (SPLIT_CLUSTER) {
        // every CTA of the cluster deposits its partials in rank 0's shared memory
#pragma unroll
        for (int u = 0; u < PER_THREAD; ++u) {
            const int e = threadIdx.x + u * GEMV_WARPS * 32;
            if (e < SLOTS) {
                const uint32_t local = (uint32_t)__cvta_generic_to_shared(&cl_part[sp][row[u]][tok[u]]);
                st_cluster_f32(map_to_cluster_rank(local, 0), total[u]);
            }
        }
        cluster_sync_all();
        if (sp != 0) return;
#pragma unroll
        for (int u = 0; u < PER_THREAD; ++u) {
            const int e = threadIdx.x + u * GEMV_WARPS * 32;
            if (e < SLOTS) {
                float s = 0.f;
                for (int r = 0; r < split; ++r) s += cl_part[r][row[u]][tok[u]];   // rank order
                total[u] = s;
            }
        }
    }
#pragma unroll
    for (int u = 0; u < PER_THREAD; ++u) {
        const int e = threadIdx.x + u * GEMV_WARPS * 32;
        if (e < SLOTS) {
            const int n = rb * 16 + row[u];
            if (n < N && tok[u] < M) {
                const __nv_bfloat16 v = __float2bfloat16_rn(total[u]);
                y[(size_t)tok[u] * N + n] = *reinterpret_cast<const uint16_t*>(&v);
            }
        }
    }
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
    *bytes = (size_t)g.RB * g.KC * AFF_BLOCK_BYTES;
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
    affine_b4_repack_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>(w, scales, biases, N, K, g.RB, g.KC,
                                                                         (uint8_t*)dst);
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

// Split of a row-block's k-chunks over the CTAs of a cluster.  Cost model: the busiest
// SM runs ceil(ctas / sms) CTAs back to back, each as long as its busiest warp
// (ceil(chunks_per_cta / warps) chunks); a split adds the cluster exchange.
static int affine_gemv_pick_split(int rb_real, int KC, int sms) {
    int best = 1;
    long long best_cost = -1;
    for (int s = 1; s <= GEMV_MAX_SPLIT && s <= KC; ++s) {
        const long long ctas = (long long)rb_real * s;
        const long long per_sm = (ctas + sms - 1) / sms;
        const int cpc = (KC + s - 1) / s;
        const int cpw = (cpc + GEMV_WARPS - 1) / GEMV_WARPS;
        const long long cost = per_sm * cpw * 8 + (s > 1 ? per_sm * 2 : 0);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
    }
    return best;
}

template <int MT>
static int32_t affine_gemv_launch(scr_ctx* ctx, const uint8_t* packed, const uint16_t* x, uint16_t* y, int M, int N,
                                  int K, cudaStream_t stream) {
    const AffineGeom g = affine_geom(N, K);
    const int rb_real = scr_ceil_div(N, 16);
    const int split = affine_gemv_pick_split(rb_real, g.KC, ctx->sm_count);
    if (split == 1) {
        affine_b4_gemv_kernel<MT, 0><<<dim3(rb_real, 1), GEMV_WARPS * 32, 0, stream>>>(packed, x, y, M, N, K, g.RB, g.KC, 1);
        return scr_check_launch(ctx, "affine_b4_gemv");
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rb_real, split, 1);
    cfg.blockDim = dim3(GEMV_WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = split;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, affine_b4_gemv_kernel<MT, 1>, packed, x, y, M, N, K, g.RB, g.KC, split);
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
