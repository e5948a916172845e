// fp8-dynamic-per-channel: weight repack, per-token activation quantisation, test hooks and
// the decode matvec (M <= 16).  Layouts are described in fp8.cuh.
#include "fp8.cuh"

// ------------------------------------------------------------------------------------
// Weight repack: [N, K] e4m3 row-major -> swizzled 128x128 tiles + padded scales.
// One thread per 16-byte chunk of the destination.
// ------------------------------------------------------------------------------------
__global__ void fp8_repack_kernel(const uint8_t* __restrict__ w, const float* __restrict__ w_scale, int N, int K,
                                  int NT, int KT, uint8_t* __restrict__ dst) {
    const long long chunks = (long long)NT * KT * (FP8_TILE_BYTES / 16);
    const bool vec_ok = (K % 16) == 0;
    for (long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x; it < chunks;
         it += (long long)gridDim.x * blockDim.x) {
        const long long tile = it / 1024;
        const int ch = int(it % 1024);
        const int nt = int(tile / KT), kt = int(tile % KT);
        const int r = ch >> 3, c16 = ch & 7;                  // logical row / 16-byte column chunk
        const int n = nt * 128 + r, k0 = kt * 128 + c16 * 16;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (n < N && k0 < K) {
            if (vec_ok) {
                v = *reinterpret_cast<const uint4*>(w + (size_t)n * K + k0);
            } else {
                uint8_t tmp[16];
                for (int i = 0; i < 16; ++i) tmp[i] = (k0 + i < K) ? w[(size_t)n * K + k0 + i] : 0;
                v = *reinterpret_cast<const uint4*>(tmp);
            }
        }
        *reinterpret_cast<uint4*>(dst + tile * FP8_TILE_BYTES + fp8_swizzled_offset(r, c16 * 16)) = v;
    }
    float* sc = reinterpret_cast<float*>(dst + (size_t)NT * KT * FP8_TILE_BYTES);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)NT * 128;
         i += (long long)gridDim.x * blockDim.x)
        sc[i] = (i < N) ? w_scale[i] : 0.f;
}

// ------------------------------------------------------------------------------------
// Per-token dynamic quantisation.  One CTA per token row: absmax, then encode.
//   a_scale = min(max(absmax * (1/448), 1/448/448), 448); inv = 1 / a_scale (IEEE division);
//   x_q = e4m3(min(max(x * inv, -448), 448))
// (ktir_matmul_fp8.rs:300-322,430-480,517-531 / superdsc_opspec.rs:1998-2009 of the reference,
//  in f32).
// ------------------------------------------------------------------------------------
#define QUANT_THREADS 256

__global__ void __launch_bounds__(QUANT_THREADS)
fp8_quant_per_token_kernel(const uint16_t* __restrict__ x, int M, int K, int tiled, int M_pad, uint8_t* __restrict__ act) {
    __shared__ float warp_max[QUANT_THREADS / 32];
    __shared__ float s_inv;
    const int m = blockIdx.x;
    const uint16_t* xr = x + (size_t)m * K;
    const int nvec = K / 8;                                   // 16-byte vectors of bf16 (K % 8 == 0 checked on host)

    float amax = 0.f;
    for (int v = threadIdx.x; v < nvec; v += QUANT_THREADS) {
        const uint4 q = ld_nc_v4(xr + v * 8);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            amax = fmaxf(amax, fabsf(__uint_as_float(w[i] << 16)));
            amax = fmaxf(amax, fabsf(__uint_as_float(w[i] & 0xFFFF0000u)));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < QUANT_THREADS / 32; ++i) a = fmaxf(a, warp_max[i]);
        const float mul_const = 1.0f / 448.0f;
        const float clip_min = 1.0f / 448.0f / 448.0f;
        const float s = fminf(fmaxf(__fmul_rn(a, mul_const), clip_min), 448.0f);
        reinterpret_cast<float*>(act)[m] = s;
        s_inv = __fdiv_rn(1.0f, s);
    }
    __syncthreads();
    const float inv = s_inv;

    const size_t scale_bytes = ((size_t)M * 4 + 127) / 128 * 128;
    uint8_t* xq = act + scale_bytes;
    const int K16 = (K + 15) / 16 * 16;
    const int kspan = tiled ? (K + 127) / 128 * 128 : K16;    // columns this row must write (zero padded)
    for (int c = threadIdx.x; c < kspan / 16; c += QUANT_THREADS) {
        const int k0 = c * 16;
        uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int kk = k0 + h * 8;
            if (kk < K) {                                     // K % 8 == 0: a vector is all in or all out
                const uint4 q = ld_nc_v4(xr + kk);
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float lo = fminf(fmaxf(__fmul_rn(__uint_as_float(w[i] << 16), inv), -448.0f), 448.0f);
                    const float hi = fminf(fmaxf(__fmul_rn(__uint_as_float(w[i] & 0xFFFF0000u), inv), -448.0f), 448.0f);
                    const uint32_t two = e4m3_encode_ref(lo) | (e4m3_encode_ref(hi) << 8);
                    out[h * 2 + (i >> 1)] |= two << ((i & 1) * 16);
                }
            }
        }
        size_t off;
        if (tiled) off = (size_t)(k0 >> 7) * ((size_t)M_pad * 128) + fp8_swizzled_offset(m, k0 & 127);
        else off = (size_t)m * K16 + k0;
        *reinterpret_cast<uint4*>(xq + off) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

__global__ void fp8_act_unpack_kernel(const uint8_t* __restrict__ act, int M, int K, int tiled, int M_pad,
                                      uint8_t* __restrict__ xq_out, float* __restrict__ a_scale) {
    const size_t scale_bytes = ((size_t)M * 4 + 127) / 128 * 128;
    const uint8_t* xq = act + scale_bytes;
    const int K16 = (K + 15) / 16 * 16;
    const long long total = (long long)M * K;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int m = int(i / K), k = int(i % K);
        size_t off;
        if (tiled) off = (size_t)(k >> 7) * ((size_t)M_pad * 128) + fp8_swizzled_offset(m, k & 127);
        else off = (size_t)m * K16 + k;
        xq_out[i] = xq[off];
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < M; i += gridDim.x * blockDim.x)
        a_scale[i] = reinterpret_cast<const float*>(act)[i];
}

__global__ void e4m3_encode_kernel(const float* __restrict__ v, long long count, uint8_t* __restrict__ out) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
        out[i] = (uint8_t)e4m3_encode_ref(v[i]);
}

// ------------------------------------------------------------------------------------
// Decode matvec, M <= 16: weights go from HBM straight into the A operand of
// mma.sync.m16n8k32 (e4m3 x e4m3 -> f32); no dequantisation arithmetic at all.
// A warp owns 16 weight rows (two 8-row swizzle groups of a tile) over a set of k-tiles;
// lane (g, t) loads the 16-byte chunks t and t+4 of rows g and g+8 and the same chunks of
// token g's quantised activations, so both operands see the same permutation of k.
// Grid (ceil(N/16), split); split > 1 runs as a thread-block cluster and reduces over
// distributed shared memory in rank order.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_e4m3_16832(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t fp8_cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void fp8_cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void fp8_st_cluster_rank0_f32(const float* local_ptr, float v) {
    const uint32_t local = (uint32_t)__cvta_generic_to_shared(local_ptr);
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

#define F8V_WARPS 4
#define F8V_STAGES 4
#define F8V_MAX_SPLIT 8

struct F8Stage {
    uint4 a_lo, a_hi;     // row g: chunks t, t+4
    uint4 b_lo, b_hi;     // row g+8
};

__device__ __forceinline__ void f8_stage_load(F8Stage& s, const uint8_t* rowblk, int g, int t) {
    const uint8_t* r0 = rowblk + g * 128;
    s.a_lo = ld_stream_v4(r0 + ((t ^ g) << 4));
    s.a_hi = ld_stream_v4(r0 + (((t + 4) ^ g) << 4));
    s.b_lo = ld_stream_v4(r0 + 1024 + ((t ^ g) << 4));
    s.b_hi = ld_stream_v4(r0 + 1024 + (((t + 4) ^ g) << 4));
}

template <int MT>
__device__ __forceinline__ void f8_stage_compute(const F8Stage& s, float acc[MT][4], const uint8_t* __restrict__ xq,
                                                 int kt, int K16, int g, int t, bool ok0, bool ok1) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const bool ok = (mt == 0) ? ok0 : ok1;
        const uint8_t* xr = xq + (size_t)(mt * 8 + g) * K16 + kt * 128;
        uint4 xlo = make_uint4(0, 0, 0, 0), xhi = make_uint4(0, 0, 0, 0);
        if (ok && kt * 128 + t * 16 < K16) xlo = ld_nc_v4(xr + t * 16);
        if (ok && kt * 128 + (t + 4) * 16 < K16) xhi = ld_nc_v4(xr + (t + 4) * 16);
        mma_e4m3_16832(acc[mt], s.a_lo.x, s.b_lo.x, s.a_lo.y, s.b_lo.y, xlo.x, xlo.y);
        mma_e4m3_16832(acc[mt], s.a_lo.z, s.b_lo.z, s.a_lo.w, s.b_lo.w, xlo.z, xlo.w);
        mma_e4m3_16832(acc[mt], s.a_hi.x, s.b_hi.x, s.a_hi.y, s.b_hi.y, xhi.x, xhi.y);
        mma_e4m3_16832(acc[mt], s.a_hi.z, s.b_hi.z, s.a_hi.w, s.b_hi.w, xhi.z, xhi.w);
    }
}

template <int MT, int SPLIT_CLUSTER>
__global__ void __launch_bounds__(F8V_WARPS * 32)
fp8_gemv_kernel(const uint8_t* __restrict__ wpack, const float* __restrict__ w_scale, const uint8_t* __restrict__ xq,
                const float* __restrict__ a_scale, uint16_t* __restrict__ y, int M, int N, int K16, int KT, int split) {
    __shared__ float red[F8V_WARPS][32][MT * 4];
    __shared__ float cl_part[SPLIT_CLUSTER ? F8V_MAX_SPLIT : 1][16][MT * 8];

    const int rb = blockIdx.x;
    const int sp = SPLIT_CLUSTER ? int(fp8_cluster_ctarank()) : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const int per = (KT + split - 1) / split;
    const int kt_lo = sp * per;
    const int kt_hi = min(KT, kt_lo + per);

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;

    // row-block rb = rows [16rb, 16rb+16) = swizzle groups 2j, 2j+1 of tile row nt
    const uint8_t* base = wpack + (size_t)(rb >> 3) * KT * FP8_TILE_BYTES + (size_t)(rb & 7) * 2048;
    const bool ok0 = g < M;
    const bool ok1 = (MT > 1) && (g + 8 < M);

    F8Stage st[F8V_STAGES];
    int kt = kt_lo + warp;
#pragma unroll
    for (int d = 0; d < F8V_STAGES; ++d) {
        const int k = kt + d * F8V_WARPS;
        if (k < kt_hi) f8_stage_load(st[d], base + (size_t)k * FP8_TILE_BYTES, g, t);
    }
    for (; kt < kt_hi; kt += F8V_STAGES * F8V_WARPS) {
#pragma unroll
        for (int d = 0; d < F8V_STAGES; ++d) {
            const int kcur = kt + d * F8V_WARPS;
            if (kcur < kt_hi) {
                const F8Stage cur = st[d];
                const int knext = kcur + F8V_STAGES * F8V_WARPS;
                if (knext < kt_hi) f8_stage_load(st[d], base + (size_t)knext * FP8_TILE_BYTES, g, t);
                f8_stage_compute<MT>(cur, acc, xq, kcur, K16, g, t, ok0, ok1);
            }
        }
    }

#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][lane][mt * 4 + i] = acc[mt][i];
    __syncthreads();

    constexpr int SLOTS = 32 * MT * 4;
    constexpr int PER_THREAD = (SLOTS + F8V_WARPS * 32 - 1) / (F8V_WARPS * 32);
    float total[PER_THREAD];
    int row[PER_THREAD], tok[PER_THREAD];
#pragma unroll
    for (int u = 0; u < PER_THREAD; ++u) {
        const int e = threadIdx.x + u * F8V_WARPS * 32;
        total[u] = 0.f; row[u] = 0; tok[u] = 0;
        if (e < SLOTS) {
            const int ln = e / (MT * 4), idx = e % (MT * 4);
            const int mt = idx >> 2, i = idx & 3;
#pragma unroll
            for (int wdx = 0; wdx < F8V_WARPS; ++wdx) total[u] += red[wdx][ln][idx];
            row[u] = (ln >> 2) + ((i >> 1) ? 8 : 0);
            tok[u] = mt * 8 + (ln & 3) * 2 + (i & 1);
        }
    }
    if (SPLIT_CLUSTER) {
#pragma unroll
        for (int u = 0; u < PER_THREAD; ++u) {
            const int e = threadIdx.x + u * F8V_WARPS * 32;
            if (e < SLOTS) fp8_st_cluster_rank0_f32(&cl_part[sp][row[u]][tok[u]], total[u]);
        }
        fp8_cluster_sync_all();
        if (sp != 0) return;
#pragma unroll
        for (int u = 0; u < PER_THREAD; ++u) {
            const int e = threadIdx.x + u * F8V_WARPS * 32;
            if (e < SLOTS) {
                float s = 0.f;
                for (int r = 0; r < split; ++r) s += cl_part[r][row[u]][tok[u]];
                total[u] = s;
            }
        }
    }
#pragma unroll
    for (int u = 0; u < PER_THREAD; ++u) {
        const int e = threadIdx.x + u * F8V_WARPS * 32;
        if (e < SLOTS) {
            const int n = rb * 16 + row[u];
            if (n < N && tok[u] < M) {
                // (raw * a_scale[m]) * w_scale[n], in that order (ktir_matmul_fp8.rs:676-712)
                const float o = __fmul_rn(__fmul_rn(total[u], a_scale[tok[u]]), w_scale[n]);
                const __nv_bfloat16 v = __float2bfloat16_rn(o);
                y[(size_t)tok[u] * N + n] = *reinterpret_cast<const uint16_t*>(&v);
            }
        }
    }
}

// ------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------
// Defined in fp8_gemm.cu
int32_t fp8_gemm_tc_launch(scr_ctx* ctx, const uint8_t* wpack, const uint8_t* act, uint16_t* y, int M, int N, int K,
                           void* workspace, size_t workspace_bytes, cudaStream_t stream);
size_t fp8_gemm_tc_workspace(int M, int N, int K);

static int32_t fp8_check_shape(scr_ctx* ctx, int N, int K) {
    if (N <= 0 || K <= 0) return scr_fail(ctx, SCR_E_SHAPE, "N=%d K=%d must be positive", N, K);
    return SCR_OK;
}

extern "C" int32_t scr_fp8_repack_size(int32_t N, int32_t K, size_t* bytes) {
    if (!bytes) return SCR_E_ARG;
    if (N <= 0 || K <= 0) return SCR_E_SHAPE;
    *bytes = fp8_weight_bytes(N, K);
    return SCR_OK;
}

extern "C" int32_t scr_fp8_repack(scr_ctx* ctx, const uint8_t* w, const float* w_scale, int32_t N, int32_t K, void* dst,
                                  void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!w || !w_scale || !dst) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    int32_t st = fp8_check_shape(ctx, N, K);
    if (st) return st;
    if (!scr_aligned16(dst) || ((K % 16) == 0 && !scr_aligned16(w)))
        return scr_fail(ctx, SCR_E_ALIGN, "w/dst must be 16-byte aligned");
    const Fp8Geom g = fp8_geom(N, K);
    const long long chunks = (long long)g.NT * g.KT * 1024;
    const int threads = 256;
    const int blocks = (int)std::min<long long>((chunks + threads - 1) / threads, (long long)ctx->sm_count * 32);
    fp8_repack_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>(w, w_scale, N, K, g.NT, g.KT, (uint8_t*)dst);
    return scr_check_launch(ctx, "fp8_repack");
}

extern "C" int32_t scr_fp8_act_size(int32_t M, int32_t K, size_t* bytes) {
    if (!bytes) return SCR_E_ARG;
    if (M <= 0 || K <= 0) return SCR_E_SHAPE;
    *bytes = fp8_act_bytes(M, K);
    return SCR_OK;
}

extern "C" int32_t scr_fp8_quant_per_token(scr_ctx* ctx, const uint16_t* x, int32_t M, int32_t K, void* act, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!x || !act) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    if (M <= 0 || K <= 0) return scr_fail(ctx, SCR_E_SHAPE, "M=%d K=%d must be positive", M, K);
    if (K % 8 != 0) return scr_fail(ctx, SCR_E_SHAPE, "K=%d must be a multiple of 8", K);
    if (!scr_aligned16(x) || !scr_aligned16(act)) return scr_fail(ctx, SCR_E_ALIGN, "x/act must be 16-byte aligned");
    const int tiled = fp8_act_tiled(M) ? 1 : 0;
    const int M_pad = scr_ceil_div(M, FP8_TILE) * FP8_TILE;
    fp8_quant_per_token_kernel<<<M, QUANT_THREADS, 0, (cudaStream_t)stream>>>(x, M, K, tiled, M_pad, (uint8_t*)act);
    return scr_check_launch(ctx, "fp8_quant_per_token");
}

extern "C" int32_t scr_fp8_act_unpack(scr_ctx* ctx, const void* act, int32_t M, int32_t K, uint8_t* xq, float* a_scale,
                                      void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!act || !xq || !a_scale) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    if (M <= 0 || K <= 0) return scr_fail(ctx, SCR_E_SHAPE, "M=%d K=%d must be positive", M, K);
    const int tiled = fp8_act_tiled(M) ? 1 : 0;
    const int M_pad = scr_ceil_div(M, FP8_TILE) * FP8_TILE;
    fp8_act_unpack_kernel<<<ctx->sm_count * 4, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)act, M, K, tiled, M_pad, xq,
                                                                            a_scale);
    return scr_check_launch(ctx, "fp8_act_unpack");
}

extern "C" int32_t scr_e4m3_encode(scr_ctx* ctx, const float* v, int64_t count, uint8_t* out, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!v || !out) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    if (count <= 0) return SCR_OK;
    e4m3_encode_kernel<<<ctx->sm_count * 4, 256, 0, (cudaStream_t)stream>>>(v, (long long)count, out);
    return scr_check_launch(ctx, "e4m3_encode");
}

static int fp8_gemv_pick_split(int rb_real, int KT, int sms) {
    int best = 1;
    long long best_cost = -1;
    for (int s = 1; s <= F8V_MAX_SPLIT && s <= KT; ++s) {
        const long long ctas = (long long)rb_real * s;
        const long long per_sm = (ctas + sms - 1) / sms;
        const int cpc = (KT + s - 1) / s;
        const int cpw = (cpc + F8V_WARPS - 1) / F8V_WARPS;
        const long long cost = per_sm * cpw * 8 + (s > 1 ? per_sm * 2 : 0);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
    }
    return best;
}

template <int MT>
static int32_t fp8_gemv_launch(scr_ctx* ctx, const uint8_t* wpack, const uint8_t* xq, const float* a_scale, uint16_t* y,
                               int M, int N, int K, cudaStream_t stream) {
    const Fp8Geom g = fp8_geom(N, K);
    const float* w_scale = reinterpret_cast<const float*>(wpack + (size_t)g.NT * g.KT * FP8_TILE_BYTES);
    const int K16 = scr_ceil_div(K, 16) * 16;
    const int rb_real = scr_ceil_div(N, 16);
    const int split = fp8_gemv_pick_split(rb_real, g.KT, ctx->sm_count);
    if (split == 1) {
        fp8_gemv_kernel<MT, 0><<<dim3(rb_real, 1), F8V_WARPS * 32, 0, stream>>>(wpack, w_scale, xq, a_scale, y, M, N, K16,
                                                                               g.KT, 1);
        return scr_check_launch(ctx, "fp8_gemv");
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rb_real, split, 1);
    cfg.blockDim = dim3(F8V_WARPS * 32, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = split;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, fp8_gemv_kernel<MT, 1>, wpack, w_scale, xq, a_scale, y, M, N, K16, g.KT, split);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "fp8_gemv cluster launch: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "fp8_gemv(cluster)");
}

size_t fp8_workspace_bytes(int M, int N, int K) {
    // the dynamic entry point keeps its activation pack in the workspace
    size_t b = (fp8_act_bytes(M, K) + 127) / 128 * 128;
    if (fp8_act_tiled(M)) b += fp8_gemm_tc_workspace(M, N, K);
    return (b + 127) / 128 * 128;
}

static int32_t fp8_linear_from_pack(scr_ctx* ctx, const uint8_t* wpack, const uint8_t* act, int M, int N, int K,
                                    uint16_t* y, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    const float* a_scale = reinterpret_cast<const float*>(act);
    const uint8_t* xq = act + fp8_act_scale_bytes(M);
    if (M <= 8) return fp8_gemv_launch<1>(ctx, wpack, xq, a_scale, y, M, N, K, stream);
    if (M <= 16) return fp8_gemv_launch<2>(ctx, wpack, xq, a_scale, y, M, N, K, stream);
    if (fp8_act_tiled(M)) return fp8_gemm_tc_launch(ctx, wpack, act, y, M, N, K, workspace, workspace_bytes, stream);
    const int K16 = scr_ceil_div(K, 16) * 16;
    for (int m0 = 0; m0 < M; m0 += 16) {
        const int mt = std::min(16, M - m0);
        int32_t st = (mt <= 8)
            ? fp8_gemv_launch<1>(ctx, wpack, xq + (size_t)m0 * K16, a_scale + m0, y + (size_t)m0 * N, mt, N, K, stream)
            : fp8_gemv_launch<2>(ctx, wpack, xq + (size_t)m0 * K16, a_scale + m0, y + (size_t)m0 * N, mt, N, K, stream);
        if (st) return st;
    }
    return SCR_OK;
}

extern "C" int32_t scr_linear_fp8(scr_ctx* ctx, const void* packed, const void* act, int32_t M, int32_t N, int32_t K,
                                  uint16_t* y, void* workspace, size_t workspace_bytes, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!packed || !act || !y) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    int32_t st = fp8_check_shape(ctx, N, K);
    if (st) return st;
    if (M <= 0) return scr_fail(ctx, SCR_E_SHAPE, "M=%d must be positive", M);
    if (!scr_aligned16(packed) || !scr_aligned16(act)) return scr_fail(ctx, SCR_E_ALIGN, "packed/act must be 16-byte aligned");
    if (fp8_act_tiled(M)) {
        const size_t need = fp8_gemm_tc_workspace(M, N, K);
        if (need > 0 && (!workspace || workspace_bytes < need))
            return scr_fail(ctx, SCR_E_WORKSPACE, "workspace %zu bytes < required %zu", workspace_bytes, need);
    }
    return fp8_linear_from_pack(ctx, (const uint8_t*)packed, (const uint8_t*)act, M, N, K, y, workspace, workspace_bytes,
                                (cudaStream_t)stream);
}

extern "C" int32_t scr_linear_fp8_dynamic(scr_ctx* ctx, const void* packed, const uint16_t* x, int32_t M, int32_t N,
                                          int32_t K, uint16_t* y, void* workspace, size_t workspace_bytes, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!packed || !x || !y) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    int32_t st = fp8_check_shape(ctx, N, K);
    if (st) return st;
    if (M <= 0) return scr_fail(ctx, SCR_E_SHAPE, "M=%d must be positive", M);
    const size_t need = fp8_workspace_bytes(M, N, K);
    if (!workspace || workspace_bytes < need)
        return scr_fail(ctx, SCR_E_WORKSPACE, "workspace %zu bytes < required %zu", workspace_bytes, need);
    if (!scr_aligned16(workspace)) return scr_fail(ctx, SCR_E_ALIGN, "workspace must be 16-byte aligned");
    st = scr_fp8_quant_per_token(ctx, x, M, K, workspace, stream);
    if (st) return st;
    const size_t act_bytes = (fp8_act_bytes(M, K) + 127) / 128 * 128;
    return fp8_linear_from_pack(ctx, (const uint8_t*)packed, (const uint8_t*)workspace, M, N, K, y,
                                (uint8_t*)workspace + act_bytes, workspace_bytes - act_bytes, (cudaStream_t)stream);
}
