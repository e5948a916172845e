// fp8-dynamic-per-channel: prefill GEMM on tcgen05 tensor cores (kind::f8f6f4, e4m3 x e4m3,
// f32 accumulators in TMEM), M > 16.
//
//   y[m,n] = bf16( (sum_k x_q[m,k] * w_q[n,k]) * a_scale[m] * w_scale[n] )
//
// Persistent, warp-specialised CTA (192 threads), one per SM:
//   warp 0     producer: 1-D bulk (TMA) copies of pre-swizzled 16 KB tiles into a 4-stage ring
//   warp 1     owns TMEM; one elected thread issues tcgen05.mma (A = 128 tokens, B = BN channels,
//              4 x K=32 per 128-byte k-tile) and commits stage/accumulator barriers
//   warps 2-5  epilogue: tcgen05.ld the 128 x BN f32 accumulator (thread = token row), apply
//              (acc * a_scale[m]) * w_scale[n], round to bf16, 16-byte stores
// Two accumulator buffers in TMEM (2 x BN columns) let the epilogue of tile i overlap the
// main loop of tile i+1.  Both operands arrive in the exact K-major / 128-byte-swizzle image
// the MMA reads (weights repacked at load time, activations written that way by the
// quantisation kernel), so no tensor map and no multicast is involved.
#include "fp8.cuh"
#include "tc_common.cuh"

bool fp8_gemm_tc_enabled() { return true; }
// Defined in fp8_gemm_pair.cu
bool fp8_gemm_pair_applies(int M, int N, int K, int sms);
int32_t fp8_gemm_pair_launch(scr_ctx* ctx, const uint8_t* wpack, const uint8_t* act, uint16_t* y, int M, int N, int K,
                             const LinearEnds& ends, cudaStream_t stream, bool* launched);
// Channel-tile width and work units.  Wide (256-channel) tiles reuse every activation tile twice and are preferred;
// a 128-channel tile does half the work in about three quarters of the time (measured), which can still win
// when it quantises better over the SMs.  Units as in `tc_plan_units`.
struct Fp8GemmPlan {
    int bn, mt, tiles, full, ks_tail;
    int n_tail() const { return tiles - full; }
    size_t slab_floats() const { return ks_tail > 1 ? (size_t)ks_tail * n_tail() * (size_t)(128 * bn) : 0; }
};
static Fp8GemmPlan fp8_gemm_plan(int M, int N, int K, int sms) {
    const Fp8Geom g = fp8_geom(N, K);
    Fp8GemmPlan best{};
    float best_est = 0.f;
    for (int bn = 256; bn >= 128; bn -= 128) {
        Fp8GemmPlan p;
        p.bn = bn;
        p.mt = scr_ceil_div(M, 128);
        p.tiles = p.mt * ((g.NT * 128 + bn - 1) / bn);
        // one k-step of a 128 x 256 tile takes ~0.5 us, of a 128 x 128 tile ~0.37 us (measured)
        const float est = tc_plan_units(p.tiles, g.KT, sms, bn == 256 ? 0.5f : 0.37f, &p.full, &p.ks_tail) * (bn == 256 ? 1.0f : 0.75f);
        if (bn == 256 || est < best_est * 0.97f) {
            best = p;
            best_est = est;
        }
        if (g.NT < 2) break;                 // a single 128-channel tile row: nothing to widen
    }
    return best;
}
size_t fp8_gemm_tc_workspace(int M, int N, int K) { return fp8_gemm_plan(M, N, K, tc_sm_count()).slab_floats() * sizeof(float); }

// Finishes the split tiles: sums a tile's partial tiles in slab order (deterministic), one rounding (or f32 out).
// One CTA per (tail tile, 1024 / BN rows), one float4 per thread.
__global__ void __launch_bounds__(256) fp8_gemm_tail_finish_kernel(const float* __restrict__ slabs, int ks_tail, int n_tail, int full,
                                                                   int MT, int bn, int M, int N, uint16_t* __restrict__ y,
                                                                   int out_f32, const uint16_t* __restrict__ bias) {
    const int rows_per_cta = 1024 / bn;                  // 256 threads x 4 columns
    const int groups = 128 / rows_per_cta;
    const int tt = blockIdx.x / groups, grp = blockIdx.x - tt * groups;
    const int tile = full + tt;
    const int mt = tile % MT, nb = tile / MT;
    const size_t tile_elems = (size_t)128 * bn;
    const int rl = grp * rows_per_cta + threadIdx.x / (bn / 4), c4 = (threadIdx.x % (bn / 4)) * 4;
    const int m = mt * 128 + rl, n = nb * bn + c4;
    if (m >= M || n >= N) return;
    const float* p = slabs + (size_t)tt * tile_elems + (size_t)rl * bn + c4;
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

#define F8G_STAGES 4
#define F8G_THREADS 192

template <int BN>
struct F8GSmem {
    static constexpr uint32_t kStageBytes = 16384u + (uint32_t)BN * 128u;
    static constexpr uint32_t kBarOffset = F8G_STAGES * kStageBytes;
    static constexpr uint32_t kTotal = kBarOffset + 256u + 1024u;     // barriers + alignment slack
};

template <int BN>
__global__ void __launch_bounds__(F8G_THREADS, 1)
fp8_gemm_tc_kernel(const uint8_t* __restrict__ wpack, const float* __restrict__ w_scale, const uint8_t* __restrict__ xq,
                   const float* __restrict__ a_scale, uint16_t* __restrict__ y, int M, int N, int KT, int NT, int MT,
                   int M_pad, int out_f32, const uint16_t* __restrict__ bias, int full, int ks_tail, float* __restrict__ slabs,
                   int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + F8GSmem<BN>::kBarOffset;
    // barrier slots (8 bytes each): full[S], empty[S], acc_full[2], acc_empty[2]; then the TMEM pointer
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (F8G_STAGES + s); };
    auto accf_bar = [&](int b) { return bar_base + 8u * (2 * F8G_STAGES + b); };
    auto acce_bar = [&](int b) { return bar_base + 8u * (2 * F8G_STAGES + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + F8GSmem<BN>::kBarOffset + 8 * (2 * F8G_STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NTB = (NT * 128 + BN - 1) / BN;            // channel tiles of BN
    const int n_tail = MT * NTB - full;                  // tiles whose k extent is split ks_tail ways (see tc_plan_units)
    const int tiles = full + n_tail * ks_tail;

    if (threadIdx.x == 0) {
        for (int s = 0; s < F8G_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), 128); }
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_slot), 2 * BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            for (int unit = blockIdx.x; unit < tiles; unit += gridDim.x) {
                int t2, ks, kt_lo, kt_hi;
                tc_unit(unit, full, ks_tail, KT, t2, ks, kt_lo, kt_hi);
                const int mt = t2 % MT, nb = t2 / MT;
                const int nt0 = nb * (BN / 128);
                const int ntn = min(BN / 128, NT - nt0);                  // 128-row weight tiles in this channel tile
                for (int kt = kt_lo; kt < kt_hi; ++kt) {
                    mbar_wait(empty_bar(s), ph ^ 1u, status, TC_ERR_EMPTY_WAIT);
                    const uint32_t sa = smem_base + s * F8GSmem<BN>::kStageBytes;
                    const uint32_t sb = sa + 16384u;
                    mbar_arrive_expect_tx(full_bar(s), 16384u * (1 + ntn));
                    bulk_g2s(sa, xq + (size_t)kt * ((size_t)M_pad * 128) + (size_t)mt * 16384, 16384u, full_bar(s));
                    for (int j = 0; j < ntn; ++j)
                        bulk_g2s(sb + j * 16384u, wpack + ((size_t)(nt0 + j) * KT + kt) * FP8_TILE_BYTES, 16384u, full_bar(s));
                    if (++s == F8G_STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            for (int unit = blockIdx.x; unit < tiles; unit += gridDim.x, ++it) {
                int t2, ks, kt_lo, kt_hi;
                tc_unit(unit, full, ks_tail, KT, t2, ks, kt_lo, kt_hi);
                const int nb = t2 / MT;
                const int nt0 = nb * (BN / 128);
                const int ntn = min(BN / 128, NT - nt0);
                const uint32_t idesc = umma_idesc(0, 0, 128, 128u * ntn);
                const int buf = it & 1;
                mbar_wait(acce_bar(buf), ((uint32_t)(it >> 1) & 1u) ^ 1u, status, TC_ERR_ACC_EMPTY);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                for (int kt = kt_lo; kt < kt_hi; ++kt) {
                    mbar_wait(full_bar(s), ph, status, TC_ERR_FULL_WAIT);
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * F8GSmem<BN>::kStageBytes;
                    const uint64_t adesc = umma_desc_k_sw128(sa);
                    const uint64_t bdesc = umma_desc_k_sw128(sa + 16384u);
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4)
                        umma_f8f6f4(d_tmem, adesc + (uint64_t)(2 * k4), bdesc + (uint64_t)(2 * k4), idesc, ((kt - kt_lo) | k4) != 0);
                    umma_commit(empty_bar(s));
                    if (++s == F8G_STAGES) { s = 0; ph ^= 1u; }
                }
                umma_commit(accf_bar(buf));
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;                                   // TMEM lane quadrant this warp may read
        const bool vec_ok = (N % 8) == 0;
        int it = 0;
        for (int unit = blockIdx.x; unit < tiles; unit += gridDim.x, ++it) {
            int t2, ks, kt_lo, kt_hi;
            tc_unit(unit, full, ks_tail, KT, t2, ks, kt_lo, kt_hi);
            const int mt = t2 % MT, nb = t2 / MT;
            const int n0 = nb * BN;
            const int bn_cur = min(BN, NT * 128 - n0);
            const int buf = it & 1;
            // a split unit writes its scaled f32 partial tile (128 x BN, padding columns included) into its own slab
            const bool split = unit >= full && ks_tail > 1;
            const bool f32mode = out_f32 != 0;
            float* fbase = reinterpret_cast<float*>(y);
            float* slab = split ? slabs + ((size_t)ks * n_tail + (t2 - full)) * (size_t)(128 * BN) : nullptr;
            mbar_wait(accf_bar(buf), (uint32_t)(it >> 1) & 1u, status, TC_ERR_ACC_FULL);
            tc_fence_after();
            const int m = mt * 128 + q * 32 + lane;
            const float as = (m < M) ? a_scale[m] : 0.f;
            uint16_t* yrow = y + (size_t)m * N;
            for (int c = 0; c < bn_cur / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + c * 32), r);
                tmem_ld_wait();
                const int nc = n0 + c * 32;
                if (split) {
                    if (m >= M) continue;              // rows of padding are never read back
                    float4* dst = reinterpret_cast<float4*>(slab + (size_t)(q * 32 + lane) * BN + c * 32);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 ws = __ldg(reinterpret_cast<const float4*>(w_scale + nc) + j);
                        dst[j] = make_float4(__fmul_rn(__fmul_rn(__uint_as_float(r[4 * j + 0]), as), ws.x),
                                             __fmul_rn(__fmul_rn(__uint_as_float(r[4 * j + 1]), as), ws.y),
                                             __fmul_rn(__fmul_rn(__uint_as_float(r[4 * j + 2]), as), ws.z),
                                             __fmul_rn(__fmul_rn(__uint_as_float(r[4 * j + 3]), as), ws.w));
                    }
                } else if (m < M && nc < N && f32mode) {
                    // unrounded f32 (row-parallel partials, or a split-K slab)
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
                } else if (m < M && nc < N) {
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
            mbar_arrive(acce_bar(buf));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * BN);
    }
}

template <int BN>
static int32_t fp8_gemm_launch_bn(scr_ctx* ctx, const uint8_t* wpack, const uint8_t* act, uint16_t* y, int M, int N, int K,
                                  const LinearEnds& ends, const Fp8GemmPlan& p, float* slabs, cudaStream_t stream) {
    const Fp8Geom g = fp8_geom(N, K);
    const float* w_scale = reinterpret_cast<const float*>(wpack + (size_t)g.NT * g.KT * FP8_TILE_BYTES);
    const float* a_scale = reinterpret_cast<const float*>(act);
    const uint8_t* xq = act + fp8_act_scale_bytes(M);
    const int units = p.full + p.n_tail() * p.ks_tail;
    const int grid = std::min(units, ctx->sm_count);
    cudaError_t e = cudaFuncSetAttribute(fp8_gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)F8GSmem<BN>::kTotal);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "fp8_gemm smem attribute: %s", cudaGetErrorString(e));
    fp8_gemm_tc_kernel<BN><<<grid, F8G_THREADS, F8GSmem<BN>::kTotal, stream>>>(wpack, w_scale, xq, a_scale, y, M, N, g.KT,
                                                                              g.NT, p.mt, p.mt * 128, ends.out_f32, ends.bias, p.full,
                                                                              p.ks_tail, slabs, ctx->dev_status);
    int32_t st = scr_check_launch(ctx, "fp8_gemm_tc");
    if (st || p.ks_tail == 1) return st;
    fp8_gemm_tail_finish_kernel<<<p.n_tail() * (128 / (1024 / BN)), 256, 0, stream>>>(slabs, p.ks_tail, p.n_tail(), p.full, p.mt, BN,
                                                                                     M, N, y, ends.out_f32, ends.bias);
    return scr_check_launch(ctx, "fp8_gemm_tail_finish");
}

int32_t fp8_gemm_tc_launch(scr_ctx* ctx, const uint8_t* wpack, const uint8_t* act, uint16_t* y, int M, int N, int K,
                           const LinearEnds& ends, void* workspace, size_t, cudaStream_t stream) {
    if (((uintptr_t)(act + fp8_act_scale_bytes(M)) & 127u) != 0 || ((uintptr_t)wpack & 127u) != 0)
        return scr_fail(ctx, SCR_E_ALIGN, "weight pack and activation pack must be 128-byte aligned for the GEMM path");
    if (!scr_aligned16(y)) return scr_fail(ctx, SCR_E_ALIGN, "y must be 16-byte aligned");
    if (fp8_gemm_pair_applies(M, N, K, ctx->sm_count)) {        // large, evenly tiled GEMMs: the two-CTA kernel (fp8_gemm_pair.cu)
        bool launched = false;
        const int32_t st = fp8_gemm_pair_launch(ctx, wpack, act, y, M, N, K, ends, stream, &launched);
        if (st || launched) return st;
    }
    const Fp8GemmPlan plan = fp8_gemm_plan(M, N, K, ctx->sm_count);
    float* slabs = reinterpret_cast<float*>(workspace);
    if (plan.ks_tail > 1 && (!slabs || !scr_aligned16(slabs))) return scr_fail(ctx, SCR_E_WORKSPACE, "split-K needs an aligned workspace");
    if (plan.bn == 256) return fp8_gemm_launch_bn<256>(ctx, wpack, act, y, M, N, K, ends, plan, slabs, stream);
    return fp8_gemm_launch_bn<128>(ctx, wpack, act, y, M, N, K, ends, plan, slabs, stream);
}
