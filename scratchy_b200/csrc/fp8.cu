// fp8-dynamic-per-channel: weight repack, per-token activation quantisation, test hooks and
// the decode matvec (M <= 16).  Layouts are described in fp8.cuh.
#include "fp8.cuh"
#include "tp_comm.cuh"

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

__global__ void fp8_repack_fence_kernel() {}

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
        const uint4 q = ld_act_v4(xr + v * 8);
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
                const uint4 q = ld_act_v4(xr + kk);
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

// RMSNorm fused with the per-token quantisation: the producer of a W8A8 linear's activation pack straight from
// the residual stream (the reference quantises on the norm side for its W4A8 path,
// crates/targets/metal/src/shaders/norm_w4a8_quant.h:1-12; golden of the norm crates/targets/metal/src/cpu_golden.rs:25-37).
// Per token: inv_rms from the sum of squares, normed = bf16((x * inv_rms) * gain) — the value the stand-alone norm
// kernel would have stored — then absmax, a_scale and the e4m3 codes exactly as the quantise kernel computes them
// from those bf16 values.  One CTA per token; the normed row lives in shared memory between the passes.
__global__ void __launch_bounds__(QUANT_THREADS)
fp8_rmsnorm_quant_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gain, float eps, int M, int K, int tiled,
                         int M_pad, uint8_t* __restrict__ act, uint16_t* __restrict__ normed_out) {
    extern __shared__ float nrow[];                       // K floats: the bf16-rounded normed row
    __shared__ float warp_red[QUANT_THREADS / 32];
    __shared__ float s_bcast;
    const int m = blockIdx.x;
    const uint16_t* xr = x + (size_t)m * K;
    const int nvec = K / 8;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    float sq = 0.f;
    for (int v = threadIdx.x; v < nvec; v += QUANT_THREADS) {
        const uint4 q = ld_act_v4(xr + v * 8);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xFFFF0000u);
            sq = __fadd_rn(sq, __fmul_rn(lo, lo));
            sq = __fadd_rn(sq, __fmul_rn(hi, hi));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, o);
    if (lane == 0) warp_red[warp] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < QUANT_THREADS / 32; ++i) t += warp_red[i];
        s_bcast = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)K), eps)));
    }
    __syncthreads();
    const float inv_rms = s_bcast;

    float amax = 0.f;
    for (int v = threadIdx.x; v < nvec; v += QUANT_THREADS) {
        const uint4 q = ld_act_v4(xr + v * 8);
        const uint4 gq = ld_nc_v4(gain + v * 8);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w}, gw[4] = {gq.x, gq.y, gq.z, gq.w};
        uint32_t ow[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float lo = __fmul_rn(__fmul_rn(__uint_as_float(w[i] << 16), inv_rms), __uint_as_float(gw[i] << 16));
            const float hi = __fmul_rn(__fmul_rn(__uint_as_float(w[i] & 0xFFFF0000u), inv_rms), __uint_as_float(gw[i] & 0xFFFF0000u));
            const __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);
            ow[i] = *reinterpret_cast<const uint32_t*>(&pk);
            const float rlo = __uint_as_float(ow[i] << 16), rhi = __uint_as_float(ow[i] & 0xFFFF0000u);
            nrow[v * 8 + 2 * i] = rlo;
            nrow[v * 8 + 2 * i + 1] = rhi;
            amax = fmaxf(amax, fmaxf(fabsf(rlo), fabsf(rhi)));
        }
        if (normed_out) *reinterpret_cast<uint4*>(normed_out + (size_t)m * K + v * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    __syncthreads();                                      // s_bcast and warp_red are reused
    if (lane == 0) warp_red[warp] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < QUANT_THREADS / 32; ++i) a = fmaxf(a, warp_red[i]);
        const float sc = fminf(fmaxf(__fmul_rn(a, 1.0f / 448.0f), 1.0f / 448.0f / 448.0f), 448.0f);
        reinterpret_cast<float*>(act)[m] = sc;
        s_bcast = __fdiv_rn(1.0f, sc);
    }
    __syncthreads();
    const float inv = s_bcast;

    const size_t scale_bytes = ((size_t)M * 4 + 127) / 128 * 128;
    uint8_t* xq = act + scale_bytes;
    const int K16 = (K + 15) / 16 * 16;
    const int kspan = tiled ? (K + 127) / 128 * 128 : K16;
    for (int c = threadIdx.x; c < kspan / 16; c += QUANT_THREADS) {
        const int k0 = c * 16;
        uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int kk = k0 + j;
            if (kk < K) {
                const float v = fminf(fmaxf(__fmul_rn(nrow[kk], inv), -448.0f), 448.0f);
                out[j >> 2] |= e4m3_encode_ref(v) << ((j & 3) * 8);
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
// Decode matvec, M <= 16: e4m3 weights are the A operand of mma.sync.m16n8k32
// (e4m3 x e4m3 -> f32) exactly as stored; there is no dequantisation arithmetic.
//
// Persistent CTAs of 8 consumer warps + 1 producer warp walk row-blocks (16 weight rows = two
// 8-row swizzle groups of a 128 x 128 tile, 2 KB per k-tile) rb = blockIdx.x, += gridDim.x.
// The producer streams 8 k-tiles (8 x 2 KB 1-D bulk copies) per stage of a 4-stage ring with
// full/empty mbarriers, running ahead across row-blocks; consumer warp w takes k-tile w of every
// stage.  Lane (g, t) reads the 16-byte chunks t and t+4 of rows g and g+8 and the same chunks
// of token g's quantised activations, so both operands see the same permutation of k.  The 8
// warps' partial sums meet once per row-block in double-buffered shared memory (warp order).
// With few row-blocks, gridDim.y = SPLIT CTAs form a cluster that splits the k-tiles and
// reduces over distributed shared memory in rank order.  Launched with programmatic stream
// serialisation: the weight prefetch starts before the preceding kernel has finished, the
// consumers wait for it (griddepcontrol.wait) before they touch the activations.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_e4m3_16832(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t f8v_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
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
// Bounded wait: gives up after 2^20 polls (or once another waiter recorded a failure), records
// code 7 in the status word and lets the kernel run to its end.
__device__ __forceinline__ void f8v_wait(uint32_t bar, uint32_t parity, int* status) {
#pragma unroll 1
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return;
        if ((i & 255u) == 255u && *reinterpret_cast<volatile int*>(status) != 0) return;
    }
    atomicCAS(status, 0, 7);
}
__device__ __forceinline__ uint4 f8v_lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

#define F8V_CWARPS 8
#define F8V_THREADS ((F8V_CWARPS + 1) * 32)
// 3 stages of 16 KB: with the static shared memory that is 61 KB per CTA, so three CTAs share an SM (four
// stages made it two, and the 3-per-SM grid ran as one and a half waves) and a fused x_q of up to 14 KB still fits
#define F8V_STAGES 3
#define F8V_BLOCK_BYTES 2048
#define F8V_STAGE_BYTES (F8V_CWARPS * F8V_BLOCK_BYTES)
#define F8V_MAX_SPLIT 8

// One 2 KB block (16 rows x 128 k) from shared memory against the quantised activations.  Tokens
// beyond M read a clamped (valid) row: a column of B only reaches the same, discarded, column of D.
template <int MT>
__device__ __forceinline__ void f8_block_compute(uint32_t blk, float acc[2][MT][4], const uint4 xlo[MT], const uint4 xhi[MT],
                                                 int g, int t) {
    const uint32_t r0 = blk + g * 128;
    const uint4 a_lo = f8v_lds_v4(r0 + ((t ^ g) << 4));
    const uint4 a_hi = f8v_lds_v4(r0 + (((t + 4) ^ g) << 4));
    const uint4 b_lo = f8v_lds_v4(r0 + 1024 + ((t ^ g) << 4));
    const uint4 b_hi = f8v_lds_v4(r0 + 1024 + (((t + 4) ^ g) << 4));
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        mma_e4m3_16832(acc[0][mt], a_lo.x, b_lo.x, a_lo.y, b_lo.y, xlo[mt].x, xlo[mt].y);
        mma_e4m3_16832(acc[1][mt], a_lo.z, b_lo.z, a_lo.w, b_lo.w, xlo[mt].z, xlo[mt].w);
        mma_e4m3_16832(acc[0][mt], a_hi.x, b_hi.x, a_hi.y, b_hi.y, xhi[mt].x, xhi[mt].y);
        mma_e4m3_16832(acc[1][mt], a_hi.z, b_hi.z, a_hi.w, b_hi.w, xhi[mt].z, xhi[mt].w);
    }
}

// FUSE_Q: the kernel takes the bf16 activations and quantises them itself (every CTA repeats the
// per-token absmax and the encode into its own shared memory: a few KB from L2, one launch saved);
// the arithmetic is the quantise kernel's, statement for statement, so x_q and a_scale are the same bits.
//
// EXCH: a row-parallel linear under tensor parallelism.  The f32 partial sums do not go to y: the epilogue stores
// them straight into this rank's slot of EVERY rank's receive buffer (plain peer stores over NVLink) as 8-byte
// {value, call number} packets; at its end each CTA reads — bounded polls — the W ranks' packets of its own rows,
// sums them in rank order and rounds once: matvec and all-reduce in one launch, no flag array and no system-scope
// fence, the same bits as the partial matvec followed by the stand-alone exchange.
template <int MT, int SPLIT_CLUSTER, int FUSE_Q, int EXCH>
__global__ void __launch_bounds__(F8V_THREADS, (MT == 1 ? 3 : 2))
fp8_gemv_kernel(const uint8_t* __restrict__ wpack, const float* __restrict__ w_scale, const uint8_t* __restrict__ xq,
                const float* __restrict__ a_scale, const uint16_t* __restrict__ x_bf16, int K, uint16_t* __restrict__ y, int M,
                int N, int K16, int KT, int rb_real, int split, int out_f32, const uint16_t* __restrict__ bias,
                int* __restrict__ status, TpcExchange ex) {
    extern __shared__ __align__(128) uint8_t f8v_ring[];           // [F8V_STAGES][8 blocks of 2 KB] (+ x_q [M][K16] when FUSE_Q)
    __shared__ __align__(8) uint64_t full_bar[F8V_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[F8V_STAGES];
    __shared__ float red[2][F8V_CWARPS][32][MT * 4];
    __shared__ float cl_part[SPLIT_CLUSTER ? F8V_MAX_SPLIT : 1][16][MT * 8];
    __shared__ float q_wmax[F8V_CWARPS];
    __shared__ float q_scale[8];
    __shared__ unsigned int s_epoch;                               // EXCH: the call number of this exchange

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int d = 0; d < F8V_STAGES; ++d) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(f8v_smem_u32(&full_bar[d])), "r"(1) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(f8v_smem_u32(&empty_bar[d])), "r"(F8V_CWARPS) : "memory");
        }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int sp = SPLIT_CLUSTER ? int(fp8_cluster_ctarank()) : 0;
    // cluster mode stores row-block blockIdx.x at the very end: fetch that row's (constant, cold) output
    // scale now instead of at the tail
    float ws_final = 0.f;
    if (SPLIT_CLUSTER && sp == 0) {
        const int e0 = threadIdx.x, ln0 = e0 / (MT * 4), idx0 = e0 % (MT * 4);
        const int n0 = blockIdx.x * 16 + (ln0 >> 2) + (((idx0 & 3) >> 1) ? 8 : 0);
        if (e0 < 32 * MT * 4 && n0 < N) ws_final = w_scale[n0];
    }
    const int per = (KT + split - 1) / split;
    const int kt_lo = sp * per;
    const int kt_hi = min(KT, kt_lo + per);
    const int nstage = (max(kt_hi - kt_lo, 0) + F8V_CWARPS - 1) / F8V_CWARPS;
    const uint32_t ring_base = f8v_smem_u32(f8v_ring);
    const uint32_t full_base = f8v_smem_u32(&full_bar[0]);
    const uint32_t empty_base = f8v_smem_u32(&empty_bar[0]);

    if (warp == F8V_CWARPS) {
        // ---- producer: weights are load-time constants, so it never waits for the previous kernel
        if (lane == 0) {
            uint32_t n_it = 0;
            for (int rb = blockIdx.x; rb < rb_real; rb += gridDim.x) {
                // row-block rb = swizzle groups 2j, 2j+1 (j = rb % 8) of tile row rb / 8
                const uint8_t* src = wpack + ((size_t)(rb >> 3) * KT + kt_lo) * FP8_TILE_BYTES + (size_t)(rb & 7) * F8V_BLOCK_BYTES;
                for (int j = 0; j < nstage; ++j, ++n_it) {
                    const uint32_t slot = n_it % F8V_STAGES;
                    f8v_wait(empty_base + 8u * slot, ((n_it / F8V_STAGES) & 1u) ^ 1u, status);
                    const int nblk = min(F8V_CWARPS, kt_hi - kt_lo - j * F8V_CWARPS);
                    const uint32_t bar = full_base + 8u * slot;
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(nblk * F8V_BLOCK_BYTES) : "memory");
                    for (int b = 0; b < nblk; ++b)
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(ring_base + slot * F8V_STAGE_BYTES + b * F8V_BLOCK_BYTES),
                                       "l"(src + (size_t)(j * F8V_CWARPS + b) * FP8_TILE_BYTES), "r"(F8V_BLOCK_BYTES), "r"(bar) : "memory");
                }
            }
        }
        __syncwarp();
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");        // the activations are settled
        // (read by the other threads after the consumer barriers of the quantise / the first cross-warp sum)
        if (EXCH && threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile unsigned int*>(&ex.state[0]) + 1u;
        const uint32_t xs_base = ring_base + F8V_STAGES * F8V_STAGE_BYTES;
        if (FUSE_Q) {
            uint8_t* xs = f8v_ring + F8V_STAGES * F8V_STAGE_BYTES;
            const int tid = threadIdx.x;                          // 0..255: the consumer warps
            for (int m = 0; m < M; ++m) {
                const uint16_t* xr = x_bf16 + (size_t)m * K;
                float amax = 0.f;
                for (int v = tid; v < K / 8; v += F8V_CWARPS * 32) {
                    const uint4 q = ld_act_v4(xr + v * 8);
                    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        amax = fmaxf(amax, fabsf(__uint_as_float(w[i] << 16)));
                        amax = fmaxf(amax, fabsf(__uint_as_float(w[i] & 0xFFFF0000u)));
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
                if (lane == 0) q_wmax[warp] = amax;
                asm volatile("bar.sync 1, 256;" ::: "memory");
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < F8V_CWARPS; ++i) a = fmaxf(a, q_wmax[i]);
                const float sc = fminf(fmaxf(__fmul_rn(a, 1.0f / 448.0f), 1.0f / 448.0f / 448.0f), 448.0f);
                const float inv = __fdiv_rn(1.0f, sc);
                if (tid == 0) q_scale[m] = sc;
                for (int c = tid; c < K16 / 16; c += F8V_CWARPS * 32) {
                    const int k0 = c * 16;
                    uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int kk = k0 + h * 8;
                        if (kk < K) {
                            const uint4 q = ld_act_v4(xr + kk);
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
                    *reinterpret_cast<uint4*>(xs + (size_t)m * K16 + k0) = make_uint4(out[0], out[1], out[2], out[3]);
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");    // q_wmax is reused; x_q of this token is complete
            }
        }
        const float* a_scale_eff = FUSE_Q ? q_scale : a_scale;
        const uint8_t* xrow[MT];
        uint32_t xrow_s[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            xrow[mt] = xq + (size_t)min(mt * 8 + g, M - 1) * K16;
            xrow_s[mt] = xs_base + (uint32_t)(min(mt * 8 + g, M - 1) * K16);
        }
        uint32_t n_it = 0;
        int it = 0;
        for (int rb = blockIdx.x; rb < rb_real; rb += gridDim.x, ++it) {
            float acc[2][MT][4];
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[a][mt][i] = 0.f;
            // the output scale of the row this thread will store: a load-time constant, cold in HBM; fetch it
            // now so that its latency hides under the k loop instead of sitting at the tail
            float ws_mine = 0.f;
            {
                const int e0 = threadIdx.x, ln0 = e0 / (MT * 4), idx0 = e0 % (MT * 4);
                const int n0 = rb * 16 + (ln0 >> 2) + (((idx0 & 3) >> 1) ? 8 : 0);
                if (e0 < 32 * MT * 4 && n0 < N) ws_mine = w_scale[n0];
            }

#pragma unroll 1
            for (int j = 0; j < nstage; ++j, ++n_it) {
                const int kt = kt_lo + j * F8V_CWARPS + warp;
                const bool active = kt < kt_hi;                   // warp-uniform
                const uint32_t slot = n_it % F8V_STAGES;
                // k beyond the row (K16 not a multiple of 128, or an idle warp) meets zero weights
                // or is not used: read offset 0 instead
                int klo = kt * 128 + t * 16, khi = klo + 64;
                if (klo >= K16) klo = 0;
                if (khi >= K16) khi = 0;
                uint4 xlo[MT], xhi[MT];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    if (FUSE_Q) {
                        xlo[mt] = f8v_lds_v4(xrow_s[mt] + klo);
                        xhi[mt] = f8v_lds_v4(xrow_s[mt] + khi);
                    } else {
                        xlo[mt] = ld_act_v4(xrow[mt] + klo);
                        xhi[mt] = ld_act_v4(xrow[mt] + khi);
                    }
                }
                f8v_wait(full_base + 8u * slot, (n_it / F8V_STAGES) & 1u, status);
                if (active) f8_block_compute<MT>(ring_base + slot * F8V_STAGE_BYTES + warp * F8V_BLOCK_BYTES, acc, xlo, xhi, g, t);
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_base + 8u * slot) : "memory");
            }

            const int buf = it & 1;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int i = 0; i < 4; ++i) red[buf][warp][lane][mt * 4 + i] = acc[0][mt][i] + acc[1][mt][i];
            asm volatile("bar.sync 1, 256;" ::: "memory");        // the 8 consumer warps

            constexpr int SLOTS = 32 * MT * 4;
            const int e = threadIdx.x;
            const int ln = e / (MT * 4), idx = e % (MT * 4);
            const int row = (ln >> 2) + (((idx & 3) >> 1) ? 8 : 0);
            const int tok = (idx >> 2) * 8 + (ln & 3) * 2 + (idx & 1);
            const int n = rb * 16 + row;
            if (e < SLOTS && tok < M) {
                float total = 0.f;
#pragma unroll
                for (int wdx = 0; wdx < F8V_CWARPS; ++wdx) total += red[buf][wdx][ln][idx];
                if (SPLIT_CLUSTER) {
                    fp8_st_cluster_rank0_f32(&cl_part[sp][row][tok], total);
                } else if (n < N) {
                    // (raw * a_scale[m]) * w_scale[n], in that order (ktir_matmul_fp8.rs:676-712)
                    float o = __fmul_rn(__fmul_rn(total, a_scale_eff[tok]), ws_mine);
                    if (!EXCH && bias) o += __uint_as_float(uint32_t(bias[n]) << 16);      // the linear's own bias, before the one rounding
                    if (EXCH) {
                        const unsigned int e_call = s_epoch;
                        const long long at = tpc_slot(e_call, ex.world, ex.rank, ex.max_elems, (long long)tok * N + n);
                        for (int p = 0; p < ex.world; ++p) tpc_ll_store(ex.peers.ll[p] + at, o, e_call);
                    } else if (out_f32) {
                        reinterpret_cast<float*>(y)[(size_t)tok * N + n] = o;
                    } else {
                        const __nv_bfloat16 v = __float2bfloat16_rn(o);
                        y[(size_t)tok * N + n] = *reinterpret_cast<const uint16_t*>(&v);
                    }
                }
            }
        }
    }

    if (SPLIT_CLUSTER) {
        // one row-block per CTA in cluster mode (gridDim.x == rb_real): exchange once, rank order
        fp8_cluster_sync_all();
        constexpr int SLOTS = 32 * MT * 4;
        const int e = threadIdx.x;
        const int ln = e / (MT * 4), idx = e % (MT * 4);
        const int row = (ln >> 2) + (((idx & 3) >> 1) ? 8 : 0);
        const int tok = (idx >> 2) * 8 + (ln & 3) * 2 + (idx & 1);
        const int n = blockIdx.x * 16 + row;
        if (sp == 0 && e < SLOTS && tok < M && n < N) {
            float s = 0.f;
            for (int r = 0; r < split; ++r) s += cl_part[r][row][tok];
            float o = __fmul_rn(__fmul_rn(s, (FUSE_Q ? q_scale : a_scale)[tok]), ws_final);
            if (!EXCH && bias) o += __uint_as_float(uint32_t(bias[n]) << 16);
            if (EXCH) {
                const unsigned int e_call = s_epoch;
                const long long at = tpc_slot(e_call, ex.world, ex.rank, ex.max_elems, (long long)tok * N + n);
                for (int p = 0; p < ex.world; ++p) tpc_ll_store(ex.peers.ll[p] + at, o, e_call);
            } else if (out_f32) {
                reinterpret_cast<float*>(y)[(size_t)tok * N + n] = o;
            } else {
                const __nv_bfloat16 v = __float2bfloat16_rn(o);
                y[(size_t)tok * N + n] = *reinterpret_cast<const uint16_t*>(&v);
            }
        }
    }

    if (EXCH) {
        if (SPLIT_CLUSTER && sp != 0) return;                      // the cluster's CTA 0 owns the row-block (block-uniform exit)
        __syncthreads();                                           // (the producer warp learns the call number)
        const unsigned int e_call = s_epoch;
        constexpr int SLOTS = 32 * MT * 4;
        const int e = threadIdx.x;
        const int ln = e / (MT * 4), idx = e % (MT * 4);
        const int row = (ln >> 2) + (((idx & 3) >> 1) ? 8 : 0);
        const int tok = (idx >> 2) * 8 + (ln & 3) * 2 + (idx & 1);
        const uint2* mine = ex.peers.ll[ex.rank];
        for (int rb = blockIdx.x; rb < rb_real; rb += (SPLIT_CLUSTER ? rb_real : int(gridDim.x))) {
            const int n = rb * 16 + row;
            if (e < SLOTS && tok < M && n < N) {
                const long long at = (long long)tok * N + n;
                float s = tpc_ll_wait(mine + tpc_slot(e_call, ex.world, 0, ex.max_elems, at), e_call, status, ex.wait_limit);
                for (int q = 1; q < ex.world; ++q)
                    s = __fadd_rn(s, tpc_ll_wait(mine + tpc_slot(e_call, ex.world, q, ex.max_elems, at), e_call, status, ex.wait_limit));
                const __nv_bfloat16 v = __float2bfloat16_rn(s);
                ex.y_bf16[at] = *reinterpret_cast<const uint16_t*>(&v);
            }
        }
        tpc_finish_call(ex.state, e_call, gridDim.x);
    }
}

// ------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------
// Defined in fp8_gemm.cu
int32_t fp8_gemm_tc_launch(scr_ctx* ctx, const uint8_t* wpack, const uint8_t* act, uint16_t* y, int M, int N, int K,
                           const LinearEnds& ends, void* workspace, size_t workspace_bytes, cudaStream_t stream);
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
    int32_t st2 = scr_check_launch(ctx, "fp8_repack");
    if (st2) return st2;
    // a plain launch after the repack: kernels that prefetch weights ahead of their stream
    // dependency (programmatic dependent launch) must never follow the repack directly
    fp8_repack_fence_kernel<<<1, 32, 0, (cudaStream_t)stream>>>();
    return scr_check_launch(ctx, "fp8_repack_fence");
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

extern "C" int32_t scr_rmsnorm_fp8_quant(scr_ctx* ctx, const uint16_t* x, const uint16_t* gain, float eps, int32_t M, int32_t K,
                                         void* act, uint16_t* normed_out, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!x || !gain || !act) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    if (M <= 0 || K <= 0) return scr_fail(ctx, SCR_E_SHAPE, "M=%d K=%d must be positive", M, K);
    if (K % 8 != 0) return scr_fail(ctx, SCR_E_SHAPE, "K=%d must be a multiple of 8", K);
    if (!scr_aligned16(x) || !scr_aligned16(gain) || !scr_aligned16(act) || (normed_out && !scr_aligned16(normed_out)))
        return scr_fail(ctx, SCR_E_ALIGN, "x/gain/act/normed must be 16-byte aligned");
    const size_t smem = (size_t)K * sizeof(float);
    if (smem > 200 * 1024) return scr_fail(ctx, SCR_E_UNSUPPORTED, "K=%d exceeds the shared-memory row buffer", K);
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(fp8_rmsnorm_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "rmsnorm_fp8_quant smem attribute: %s", cudaGetErrorString(e));
    }
    const int tiled = fp8_act_tiled(M) ? 1 : 0;
    const int M_pad = scr_ceil_div(M, FP8_TILE) * FP8_TILE;
    fp8_rmsnorm_quant_kernel<<<M, QUANT_THREADS, smem, (cudaStream_t)stream>>>(x, gain, eps, M, K, tiled, M_pad, (uint8_t*)act,
                                                                              normed_out);
    return scr_check_launch(ctx, "rmsnorm_fp8_quant");
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

static void fp8_gemv_shape(int rb_real, int KC, int sms, int* grid_x, int* split) {
    // Enough row-blocks: persistent CTAs (3 per SM) walk them, nothing is split.
    const int slots = 3 * sms;
    if (rb_real >= slots) {
        *grid_x = slots;
        *split = 1;
        return;
    }
    // Fewer: one row-block per CTA and a cluster of `s` CTAs shares its k extent, chosen so that
    // everything is resident at once and the longest CTA runs the fewest ring stages.
    int best = 1, best_stages = (KC + F8V_CWARPS - 1) / F8V_CWARPS;
    for (int s = 2; s <= F8V_MAX_SPLIT && rb_real * s <= slots; ++s) {
        const int per = (KC + s - 1) / s;
        const int stages = (per + F8V_CWARPS - 1) / F8V_CWARPS;
        if (stages < best_stages) { best_stages = stages; best = s; }
    }
    *grid_x = rb_real;
    *split = best;
}

// Largest M and x_q footprint the matvec quantises by itself (beyond it the separate quantise kernel runs once).
#define F8V_FUSE_MAX_M 4
#define F8V_FUSE_MAX_BYTES (14 * 1024)
static bool fp8_gemv_fuses_quant(int M, int K) {
    return M <= F8V_FUSE_MAX_M && K % 8 == 0 && (size_t)M * (scr_ceil_div(K, 16) * 16) <= F8V_FUSE_MAX_BYTES;
}

template <int MT>
static int32_t fp8_gemv_launch(scr_ctx* ctx, const uint8_t* wpack, const uint8_t* xq, const float* a_scale, uint16_t* y,
                               int M, int N, int K, const LinearEnds& ends, cudaStream_t stream, const uint16_t* x_bf16 = nullptr,
                               const TpcExchange* exchange = nullptr) {
    const Fp8Geom g = fp8_geom(N, K);
    const float* w_scale = reinterpret_cast<const float*>(wpack + (size_t)g.NT * g.KT * FP8_TILE_BYTES);
    const int K16 = scr_ceil_div(K, 16) * 16;
    const int rb_real = scr_ceil_div(N, 16);
    int grid_x = 1, split = 1;
    fp8_gemv_shape(rb_real, g.KT, ctx->sm_count, &grid_x, &split);
    const bool fuse = (MT == 1) && x_bf16 != nullptr;
    const int kRingBytes = F8V_STAGES * F8V_STAGE_BYTES + (fuse ? M * K16 : 0);
    if (exchange && !fuse) return scr_fail(ctx, SCR_E_UNSUPPORTED, "fp8 matvec + exchange: needs the self-quantising matvec");
    auto kernel = exchange ? ((split == 1) ? fp8_gemv_kernel<1, 0, 1, 1> : fp8_gemv_kernel<1, 1, 1, 1>)
                  : fuse   ? ((split == 1) ? fp8_gemv_kernel<1, 0, 1, 0> : fp8_gemv_kernel<1, 1, 1, 0>)
                           : ((split == 1) ? fp8_gemv_kernel<MT, 0, 0, 0> : fp8_gemv_kernel<MT, 1, 0, 0>);
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "fp8_gemv smem attribute: %s", cudaGetErrorString(e));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid_x, split, 1);
    cfg.blockDim = dim3(F8V_THREADS, 1, 1);
    cfg.dynamicSmemBytes = kRingBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
    if (split > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = split;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    TpcExchange ex = {};
    if (exchange) {
        // CTAs of this launch wait for their peers on the other ranks: every one of them has to be resident
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, F8V_THREADS, kRingBytes);
        if (e != cudaSuccess || (long long)per_sm * ctx->sm_count < (long long)grid_x * split)
            return scr_fail(ctx, SCR_E_UNSUPPORTED, "fp8 matvec + exchange: %d CTAs cannot all be resident", grid_x * split);
        ex = *exchange;
    }
    e = cudaLaunchKernelEx(&cfg, kernel, wpack, w_scale, xq, a_scale, x_bf16, K, y, M, N, K16, g.KT, rb_real, split, ends.out_f32,
                           ends.bias, ctx->dev_status, ex);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "fp8_gemv launch: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "fp8_gemv");
}

size_t fp8_workspace_bytes(int M, int N, int K) {
    // the dynamic entry point keeps its activation pack in the workspace
    size_t b = (fp8_act_bytes(M, K) + 127) / 128 * 128;
    if (fp8_act_tiled(M)) b += fp8_gemm_tc_workspace(M, N, K);
    return (b + 127) / 128 * 128;
}

static int32_t fp8_linear_from_pack(scr_ctx* ctx, const uint8_t* wpack, const uint8_t* act, int M, int N, int K,
                                    uint16_t* y, const LinearEnds& ends, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    // every path below streams the weight pack with bulk copies and reads the activation pack 16 bytes at a time: a
    // misaligned pointer is refused here, on the host, and never reaches a kernel
    if (!scr_aligned16(wpack) || !scr_aligned16(act)) return scr_fail(ctx, SCR_E_ALIGN, "weight pack and activation pack must be 16-byte aligned");
    if (ends.bias && ends.out_f32) return scr_fail(ctx, SCR_E_ARG, "a bias is added after the partial sums have been reduced, not to a partial");
    const float* a_scale = reinterpret_cast<const float*>(act);
    const uint8_t* xq = act + fp8_act_scale_bytes(M);
    if (M <= 8) return fp8_gemv_launch<1>(ctx, wpack, xq, a_scale, y, M, N, K, ends, stream);
    if (M <= 16) return fp8_gemv_launch<2>(ctx, wpack, xq, a_scale, y, M, N, K, ends, stream);
    if (fp8_act_tiled(M)) return fp8_gemm_tc_launch(ctx, wpack, act, y, M, N, K, ends, workspace, workspace_bytes, stream);
    const int K16 = scr_ceil_div(K, 16) * 16;
    const size_t ystride = ends.out_f32 ? 2 : 1;
    for (int m0 = 0; m0 < M; m0 += 16) {
        const int mt = std::min(16, M - m0);
        uint16_t* yt = y + (size_t)m0 * N * ystride;
        int32_t st = (mt <= 8)
            ? fp8_gemv_launch<1>(ctx, wpack, xq + (size_t)m0 * K16, a_scale + m0, yt, mt, N, K, ends, stream)
            : fp8_gemv_launch<2>(ctx, wpack, xq + (size_t)m0 * K16, a_scale + m0, yt, mt, N, K, ends, stream);
        if (st) return st;
    }
    return SCR_OK;
}

static int32_t fp8_linear(scr_ctx* ctx, const void* packed, const void* act, int M, int N, int K, void* y, const LinearEnds& ends,
                          void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (!packed || !act || !y) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    int32_t st = fp8_check_shape(ctx, N, K);
    if (st) return st;
    if (M <= 0) return scr_fail(ctx, SCR_E_SHAPE, "M=%d must be positive", M);
    if (fp8_act_tiled(M)) {
        const size_t need = fp8_gemm_tc_workspace(M, N, K);
        if (need > 0 && (!workspace || workspace_bytes < need))
            return scr_fail(ctx, SCR_E_WORKSPACE, "workspace %zu bytes < required %zu", workspace_bytes, need);
    }
    return fp8_linear_from_pack(ctx, (const uint8_t*)packed, (const uint8_t*)act, M, N, K, static_cast<uint16_t*>(y), ends, workspace,
                                workspace_bytes, stream);
}

static int32_t fp8_linear_dynamic(scr_ctx* ctx, const void* packed, const uint16_t* x, int M, int N, int K, void* y,
                                  const LinearEnds& ends, void* workspace, size_t workspace_bytes, void* stream) {
    if (!packed || !x || !y) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    int32_t st = fp8_check_shape(ctx, N, K);
    if (st) return st;
    if (M <= 0) return scr_fail(ctx, SCR_E_SHAPE, "M=%d must be positive", M);
    if (!scr_aligned16(packed) || !scr_aligned16(x)) return scr_fail(ctx, SCR_E_ALIGN, "packed/x must be 16-byte aligned");
    if (ends.bias && ends.out_f32) return scr_fail(ctx, SCR_E_ARG, "a bias is added after the partial sums have been reduced, not to a partial");
    if (fp8_gemv_fuses_quant(M, K)) {
        // few tokens: the matvec quantises the activations itself, no pack and no second launch
        return fp8_gemv_launch<1>(ctx, (const uint8_t*)packed, nullptr, nullptr, static_cast<uint16_t*>(y), M, N, K, ends,
                                  (cudaStream_t)stream, x);
    }
    const size_t need = fp8_workspace_bytes(M, N, K);
    if (!workspace || workspace_bytes < need)
        return scr_fail(ctx, SCR_E_WORKSPACE, "workspace %zu bytes < required %zu", workspace_bytes, need);
    if (!scr_aligned16(workspace)) return scr_fail(ctx, SCR_E_ALIGN, "workspace must be 16-byte aligned");
    st = scr_fp8_quant_per_token(ctx, x, M, K, workspace, stream);
    if (st) return st;
    const size_t act_bytes = (fp8_act_bytes(M, K) + 127) / 128 * 128;
    return fp8_linear_from_pack(ctx, (const uint8_t*)packed, (const uint8_t*)workspace, M, N, K, static_cast<uint16_t*>(y), ends,
                                (uint8_t*)workspace + act_bytes, workspace_bytes - act_bytes, (cudaStream_t)stream);
}

extern "C" int32_t scr_linear_fp8(scr_ctx* ctx, const void* packed, const void* act, int32_t M, int32_t N, int32_t K,
                                  const uint16_t* bias, uint16_t* y, void* workspace, size_t workspace_bytes, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    LinearEnds ends;
    ends.bias = bias;
    return fp8_linear(ctx, packed, act, M, N, K, y, ends, workspace, workspace_bytes, (cudaStream_t)stream);
}

extern "C" int32_t scr_linear_fp8_dynamic(scr_ctx* ctx, const void* packed, const uint16_t* x, int32_t M, int32_t N,
                                          int32_t K, const uint16_t* bias, uint16_t* y, void* workspace, size_t workspace_bytes,
                                          void* stream) {
    SCR_REQUIRE_CTX(ctx);
    LinearEnds ends;
    ends.bias = bias;
    return fp8_linear_dynamic(ctx, packed, x, M, N, K, y, ends, workspace, workspace_bytes, stream);
}

// Row-parallel partials (crates/compiler/subtile/src/tensor_parallel.rs:1-63): the UNROUNDED f32 sums over this
// rank's K-slice; the all-reduce sums them over the ranks and rounds once.
extern "C" int32_t scr_linear_fp8_partial(scr_ctx* ctx, const void* packed, const void* act, int32_t M, int32_t N, int32_t K,
                                          float* y_f32, void* workspace, size_t workspace_bytes, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    LinearEnds ends;
    ends.out_f32 = 1;
    return fp8_linear(ctx, packed, act, M, N, K, y_f32, ends, workspace, workspace_bytes, (cudaStream_t)stream);
}

extern "C" int32_t scr_linear_fp8_dynamic_partial(scr_ctx* ctx, const void* packed, const uint16_t* x, int32_t M, int32_t N,
                                                  int32_t K, float* y_f32, void* workspace, size_t workspace_bytes,
                                                  void* stream) {
    SCR_REQUIRE_CTX(ctx);
    LinearEnds ends;
    ends.out_f32 = 1;
    return fp8_linear_dynamic(ctx, packed, x, M, N, K, y_f32, ends, workspace, workspace_bytes, stream);
}

// Row-parallel fp8 linear + all-reduce in one launch (decode sizes): see EXCH above.
extern "C" int32_t scr_linear_fp8_dynamic_allreduce(scr_tp_comm* comm, const void* packed, const uint16_t* x, int32_t M,
                                                    int32_t N, int32_t K, uint16_t* y, void* stream) {
    if (!comm) return SCR_E_ARG;
    scr_ctx* ctx = comm->ctx;
    SCR_REQUIRE_CTX(ctx);
    if (!packed || !x || !y) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    if (!comm->connected) return scr_fail(ctx, SCR_E_COMM, "fp8 matvec + exchange: peers are not connected");
    int32_t st = fp8_check_shape(ctx, N, K);
    if (st) return st;
    if (M <= 0) return scr_fail(ctx, SCR_E_SHAPE, "M=%d must be positive", M);
    if ((long long)M * N > comm->one_elems)
        return scr_fail(ctx, SCR_E_SHAPE, "fp8 matvec + exchange: %lld outputs exceed the communicator's %lld", (long long)M * N,
                        comm->one_elems);
    if (!fp8_gemv_fuses_quant(M, K))
        return scr_fail(ctx, SCR_E_UNSUPPORTED,
                        "fp8 matvec + exchange: M=%d K=%d is beyond the self-quantising matvec (use scr_linear_fp8_dynamic_partial "
                        "and scr_tp_allreduce_partial)", M, K);
    if (!scr_aligned16(packed) || !scr_aligned16(x)) return scr_fail(ctx, SCR_E_ALIGN, "packed/x must be 16-byte aligned");
    TpcExchange ex = {};
    ex.peers = tpc_peer_table(comm);
    ex.world = comm->world;
    ex.rank = comm->rank;
    ex.max_elems = comm->one_elems;
    ex.state = comm->state;
    ex.y_bf16 = y;
    ex.wait_limit = comm->wait_limit;
    return fp8_gemv_launch<1>(ctx, (const uint8_t*)packed, nullptr, nullptr, y, M, N, K, LinearEnds(), (cudaStream_t)stream, x, &ex);
}

// ------------------------------------------------------------------------------------
// scr_linear_fp8_dynamic_static: the fp8 dynamic linear for callers that cannot allocate.
//
// The per-token quantised activations (x_q and a_scale) normally live in a workspace the caller
// allocates.  Some callers have no allocator at hand when they run a step: a runtime that has
// handed all device memory to its own arena and must not grow it, code running inside a
// region where the CUDA allocator is forbidden, or a thin FFI shim that only owns the input
// and output tensors.  For them this variant keeps the activation pack in the fixed device
// array below, which every GPU that loads this library reserves until the process exits.
//
//  * It allocates nothing: no cudaMalloc / cudaFree and no allocating library routine.
//  * Limit: the activation pack for (M, K) must fit SCR_STATIC_SCRATCH_BYTES (8 MiB); larger
//    requests are refused with SCR_E_WORKSPACE and a message that states both sizes.
//  * The first call on a device looks the array's device address up (the name `scratch` is only
//    a host-side handle, never a pointer a kernel may use) and caches it; make that first call
//    outside any stream capture, with the context's device current.
//  * All calls share the one array and it keeps the last call's contents.  Nothing in it has
//    to start at zero: the quantise kernel rewrites every byte the contraction reads for the
//    tokens it is given.  Calls that overlap on the GPU (different streams, or several host
//    threads on one device) race on it — serialise them, or use scr_linear_fp8_dynamic with
//    separate workspaces.
// ------------------------------------------------------------------------------------
#define SCR_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char scr_static_scratch[SCR_STATIC_SCRATCH_BYTES];

#define SCR_MAX_DEVICES 64
static void* g_static_scratch_ptr[SCR_MAX_DEVICES] = {nullptr};
static std::atomic<int> g_static_scratch_state[SCR_MAX_DEVICES];     // 0 = not looked up, 2 = ready

static int32_t static_scratch_for(scr_ctx* ctx, void** out) {
    const int dev = ctx->device;
    if (dev < 0 || dev >= SCR_MAX_DEVICES) return scr_fail(ctx, SCR_E_ARG, "device %d out of range", dev);
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != dev)
        return scr_fail(ctx, SCR_E_ARG, "device %d must be current (current is %d)", dev, cur);
    if (g_static_scratch_state[dev].load(std::memory_order_acquire) != 2) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, scr_static_scratch);
        if (e != cudaSuccess || !p)
            return scr_fail(ctx, SCR_E_CUDA, "cudaGetSymbolAddress(scr_static_scratch): %s", cudaGetErrorString(e));
        g_static_scratch_ptr[dev] = p;                       // the same value from every thread: a benign race
        g_static_scratch_state[dev].store(2, std::memory_order_release);
    }
    *out = g_static_scratch_ptr[dev];
    return SCR_OK;
}

extern "C" int32_t scr_linear_fp8_dynamic_static(scr_ctx* ctx, const void* packed, const uint16_t* x, int32_t M, int32_t N,
                                                 int32_t K, uint16_t* y, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!packed || !x || !y) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    int32_t st = fp8_check_shape(ctx, N, K);
    if (st) return st;
    if (M <= 0) return scr_fail(ctx, SCR_E_SHAPE, "M=%d must be positive", M);
    if (!scr_aligned16(packed) || !scr_aligned16(x)) return scr_fail(ctx, SCR_E_ALIGN, "packed/x must be 16-byte aligned");
    const size_t need = fp8_workspace_bytes(M, N, K);
    if (need > (size_t)SCR_STATIC_SCRATCH_BYTES)
        return scr_fail(ctx, SCR_E_WORKSPACE,
                        "M=%d K=%d needs %zu bytes of scratch, the built-in array holds %u; use scr_linear_fp8_dynamic "
                        "with a caller workspace", M, K, need, (unsigned)SCR_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    st = static_scratch_for(ctx, &scratch);
    if (st) return st;
    st = scr_fp8_quant_per_token(ctx, x, M, K, scratch, stream);
    if (st) return st;
    const size_t act_bytes = (fp8_act_bytes(M, K) + 127) / 128 * 128;
    return fp8_linear_from_pack(ctx, (const uint8_t*)packed, (const uint8_t*)scratch, M, N, K, y, LinearEnds(),
                                (uint8_t*)scratch + act_bytes, (size_t)SCR_STATIC_SCRATCH_BYTES - act_bytes, (cudaStream_t)stream);
}
