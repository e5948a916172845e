// MLX affine int4 (groups of 32, 64, 128): load-time repack, dequant dump hook and the decode matvec.
#include "affine_b4.cuh"
#include "gemv_common.cuh"

#include <cuda_fp16.h>

#include <algorithm>
#include <new>
#include <vector>

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

// A scale or bias as the kernels keep it: bf16 bits.  F16 storage (what every mlx-community 4-bit checkpoint ships)
// is narrowed to the bf16 activation type exactly as the reference does before it multiplies
// (`TAct::from_f32(scales[g].to_f32())`, crates/targets/metal/src/cpu_reference.rs:90-92): f16 -> f32 is exact, f32 -> bf16
// rounds to nearest even.
__device__ __forceinline__ uint32_t affine_scale_bits(uint16_t raw, int f16) {
    if (!f16) return raw;
    const float f = __half2float(__ushort_as_half(raw));
    const __nv_bfloat16 b = __float2bfloat16_rn(f);
    return *reinterpret_cast<const uint16_t*>(&b);
}

__global__ void affine_b4_repack_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ scales,
                                        const uint16_t* __restrict__ biases, int f16, int N, int K, int group, int gs, int RB, int KC,
                                        uint8_t* __restrict__ dst, unsigned int* __restrict__ slow_flag) {
    const long long nblocks = (long long)RB * KC;
    const int epr = 1 << gs;                            // entries per row and block
    const int per_block = 64 + 8 * epr;                 // 64 pieces + one 8-byte entry per row pair and k extent
    const int block_bytes = aff_block_bytes(gs);
    const long long items = nblocks * per_block;
    for (long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x; it < items;
         it += (long long)gridDim.x * blockDim.x) {
        const long long blk = it / per_block;
        const int sub = int(it % per_block);
        const int rb = int(blk / KC), kc = int(blk % KC);
        uint8_t* out = dst + blk * block_bytes;
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
            // entry e = g * epr + h covers k [kc * 128 + h * (128 / epr), +128 / epr) of rows g and g + 8; with groups of
            // 128 both entries of a row are the same group's
            const int e = sub - 64, g = e >> gs, h = e & (epr - 1);
            const int k0 = kc * 128 + h * (128 >> gs);
            uint2 v = make_uint2(0, 0);
            if (k0 < K) {
                const int G = K / group, grp = k0 / group;
                const int r0 = rb * 16 + g, r1 = r0 + 8;
                if (r0 < N) v.x = affine_scale_bits(scales[(size_t)r0 * G + grp], f16) | (affine_scale_bits(biases[(size_t)r0 * G + grp], f16) << 16);
                if (r1 < N) v.y = affine_scale_bits(scales[(size_t)r1 * G + grp], f16) | (affine_scale_bits(biases[(size_t)r1 * G + grp], f16) << 16);
            }
            *reinterpret_cast<uint2*>(out + 1024 + e * 8) = v;
            if (affine_group_needs_generic(v.x) || affine_group_needs_generic(v.y)) atomicOr(slow_flag, 1u);
        }
    }
}

// The matvec kernels prefetch weights before they wait for the preceding kernel of the stream
// (programmatic dependent launch), which is only sound if the weights are complete by then.
// A plain launch of this empty kernel after the repack puts a full stream-order dependency
// between the repack and anything launched later.
__global__ void affine_b4_repack_fence_kernel() {}

// ------------------------------------------------------------------------------------
// Dump hook: streaming blocks -> dense bf16 [N, K], through affine_dequant_piece.
// ------------------------------------------------------------------------------------
// One piece (32 weights of one row) of a block, dequantised the way the kernels do it: 16 words of two bf16 each.
__device__ __forceinline__ void affine_block_piece(const uint8_t* b, int half, int g, int t, int gs, bool check, uint32_t regs[16]) {
    const uint4 piece = *reinterpret_cast<const uint4*>(b + half * 512 + (4 * g + t) * 16);
    const uint2 sb2 = *reinterpret_cast<const uint2*>(b + 1024 + ((g << gs) + (t >> (2 - gs))) * 8);
    const uint32_t sb = half ? sb2.y : sb2.x;
    if (check) {
        affine_dequant_piece<true>(piece, sb, regs);
    } else {
        // the scaled variant the kernels use, brought back by the exact factor 2^7
        const AffineScaled c = affine_scaled_consts(sb);
        affine_dequant_word_scaled(piece.x, c, regs + 0);
        affine_dequant_word_scaled(piece.y, c, regs + 4);
        affine_dequant_word_scaled(piece.z, c, regs + 8);
        affine_dequant_word_scaled(piece.w, c, regs + 12);
        const uint32_t k128 = 0x43004300u;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&regs[i]),
                                             *reinterpret_cast<const __nv_bfloat162*>(&k128));
            regs[i] = *reinterpret_cast<const uint32_t*>(&v);
        }
    }
}

__global__ void affine_b4_dump_kernel(const uint8_t* __restrict__ packed, int N, int K, int gs, int RB, int KC,
                                      uint16_t* __restrict__ out) {
    const long long items = (long long)RB * KC * 64;
    const int block_bytes = aff_block_bytes(gs);
    const bool check = *reinterpret_cast<const unsigned int*>(packed + (size_t)RB * KC * block_bytes) != 0;
    for (long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x; it < items;
         it += (long long)gridDim.x * blockDim.x) {
        const long long blk = it / 64;
        const int sub = int(it % 64);
        const int rb = int(blk / KC), kc = int(blk % KC);
        const int half = sub >> 5, lane = sub & 31, g = lane >> 2, t = lane & 3;
        const int row = rb * 16 + half * 8 + g;
        const int k0 = kc * 128 + t * 32;
        if (row >= N || k0 >= K) continue;
        uint32_t regs[16];
        affine_block_piece(packed + blk * block_bytes, half, g, t, gs, check, regs);
        uint4* o = reinterpret_cast<uint4*>(out + (size_t)row * K + k0);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = make_uint4(regs[4 * i], regs[4 * i + 1], regs[4 * i + 2], regs[4 * i + 3]);
    }
}

// ------------------------------------------------------------------------------------
// Quantized token embedding (`AffineQuantEmbedding`, crates/models/quantization/src/layers_quant.rs:105-150; kernel
// `affine_embed_b4`, crates/targets/metal/shaders/quantized_dequantize.metal:82-157): out[i, :] = dequant(table[ids[i], :]),
// the gather and the dequantisation in one pass.  The table is a repacked matrix [vocab, hidden] — the same buffer a
// tied lm_head multiplies with, as in the reference, where both layers share one buffer triple.  One thread per
// 32-weight piece; an id beyond the vocabulary records a code and leaves a row of zeros.
// ------------------------------------------------------------------------------------
#define AFF_BAD_TOKEN_ID 0x0E000001
__global__ void affine_b4_embed_kernel(const uint8_t* __restrict__ packed, const uint32_t* __restrict__ ids, int n_ids, int vocab,
                                       int K, int gs, int RB, int KC, uint16_t* __restrict__ out, int* status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");                 // the ids may be the preceding kernel's output
    const int block_bytes = aff_block_bytes(gs);
    const bool check = *reinterpret_cast<const unsigned int*>(packed + (size_t)RB * KC * block_bytes) != 0;
    const int pieces = K / 32;                                         // per row
    const long long items = (long long)n_ids * pieces;
    for (long long it = blockIdx.x * (long long)blockDim.x + threadIdx.x; it < items; it += (long long)gridDim.x * blockDim.x) {
        const int i = int(it / pieces), p = int(it % pieces);
        const uint32_t id = ids[i];
        uint4* o = reinterpret_cast<uint4*>(out + (size_t)i * K + (size_t)p * 32);
        if (id >= (uint32_t)vocab) {
            if (p == 0) atomicCAS(status, 0, AFF_BAD_TOKEN_ID);
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = make_uint4(0, 0, 0, 0);
            continue;
        }
        const int rb = int(id >> 4), half = int(id >> 3) & 1, g = int(id) & 7;
        const int kc = p >> 2, t = p & 3;
        uint32_t regs[16];
        affine_block_piece(packed + ((size_t)rb * KC + kc) * block_bytes, half, g, t, gs, check, regs);
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = make_uint4(regs[4 * j], regs[4 * j + 1], regs[4 * j + 2], regs[4 * j + 3]);
    }
}

// ------------------------------------------------------------------------------------
// Decode matvec, M <= 16.
//
// Persistent CTAs of 8 consumer warps + 1 producer warp.  A CTA walks row-blocks (16 weight
// rows) rb = blockIdx.x, += gridDim.x.  The producer streams each row-block's contiguous
// k extent HBM -> shared memory with 1-D bulk (TMA) copies of up to 8 blocks (9216 bytes) per
// stage of a 4-stage ring (full/empty mbarriers), running ahead across row-block boundaries.
// Consumer warp w takes block w of every stage: two conflict-free 16-byte shared loads per
// lane, dequantisation in registers, and the dequantised bf16 weights as the A operand of
// mma.sync.m16n8k16 with the tokens as the 8 columns of B (MT = 1: up to 8 tokens, MT = 2: up
// to 16).  Lane (g, t) holds codes of rows g and g+8 at k = 128kc + 32t + [0,32) and the
// activations of token g (and g+8) at the same k, so the contraction index is permuted
// identically on both operands.  Partial sums of the 8 warps meet once per row-block in
// double-buffered shared memory, summed in warp order (deterministic).
//
// With too few row-blocks to fill the machine, gridDim.y = SPLIT CTAs form a thread-block
// cluster that splits the k extent and reduces through distributed shared memory in rank
// order.  Every wait is bounded (gemv_wait).
// ------------------------------------------------------------------------------------
// GEMV_OUT_RESIDUAL_NORM: the o / down projection with the ends the reference folds around its matvec
// (`QmvEnds`, crates/targets/metal/src/tape/step.rs:472-482), i.e. `fused_add_rmsnorm`
// (crates/targets/metal/src/cpu_golden.rs:171-200) without a kernel of its own:
//   residual[m,n] <- bf16(residual[m,n] + bf16(y[m,n]))          in the epilogue, element by element
//   normed[m,:]   <- rmsnorm(residual[m,:], gain, eps)           by the last CTA to finish
// Every CTA leaves the sum of squares of the residual values it stored (per token) in `scratch`, takes a
// ticket, and the CTA that draws the last ticket adds the partial sums in CTA order (deterministic),
// and normalises the rows.  `scratch` = the ticket counter (16 floats reserved), then [gridDim.x][16] f32; the
// counter must be zero before the first call and is left zero.
#define GEMV_OUT_RESIDUAL_NORM 3
#define GEMV_OUT_RESIDUAL_ADD 4
struct GemvEnds {
    uint16_t* residual;
    const uint16_t* gain;
    uint16_t* normed;
    float* scratch;         // [0] = ticket counter (as u32), [16 + cta*16 + token] = the CTAs' sums of squares
    float eps;
};

__device__ __forceinline__ float gemv_bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// The epilogue's element step: returns the square of the stored residual (0 outside the matrix).
__device__ __forceinline__ float gemv_residual_update(float total, int tok, int M, int n, int N, const GemvEnds& ends) {
    if (tok >= M || n >= N) return 0.f;
    uint16_t* p = ends.residual + (size_t)tok * N + n;
    const float r = gemv_bf16_round(__fadd_rn(__uint_as_float(uint32_t(*p) << 16), gemv_bf16_round(total)));
    const __nv_bfloat16 rb = __float2bfloat16_rn(r);
    *p = *reinterpret_cast<const uint16_t*>(&rb);
    return __fmul_rn(r, r);
}

// The tail: called by `nthreads` threads of the CTA (a multiple of 32, thread ids 0..nthreads-1), all of which
// reach every barrier `bar_id`.  `my_sq` = this CTA's sum of squares for token threadIdx.x (threads < M).
__device__ __forceinline__ void gemv_norm_tail(float my_sq, int M, int N, int ncta, int cta, const GemvEnds& ends, int bar_id,
                                               int nthreads) {
    __shared__ int s_last;
    __shared__ float s_inv[16];
    const int tid = threadIdx.x;
    if (tid < M) ends.scratch[16 + cta * 16 + tid] = my_sq;
    __threadfence();
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
    if (tid == 0) {
        unsigned int* counter = reinterpret_cast<unsigned int*>(ends.scratch);
        const unsigned int ticket = atomicAdd(counter, 1u);
        s_last = (ticket == (unsigned int)ncta - 1u);
        if (s_last) *counter = 0u;                   // every CTA has drawn: leave it ready for the next call
        __threadfence();
    }
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
    if (!s_last) return;
    // sum of squares per token, partials in CTA order: lane l adds CTAs l, l+32, ... then a fixed shuffle tree
    const int warp = tid >> 5, lane = tid & 31, nwarps = nthreads >> 5;
    for (int tok = warp; tok < M; tok += nwarps) {
        float a = 0.f;
        for (int c = lane; c < ncta; c += 32) a = __fadd_rn(a, __ldcg(ends.scratch + 16 + c * 16 + tok));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, o));
        if (lane == 0) s_inv[tok] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(a, float(N)), ends.eps)));
    }
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads) : "memory");
    const int nv = N >> 3;                           // N % 8 == 0 is checked on the host for this mode
    for (int i = tid; i < M * nv; i += nthreads) {
        const int tok = i / nv, v = i - tok * nv;
        const uint4 rv = __ldcg(reinterpret_cast<const uint4*>(ends.residual + (size_t)tok * N) + v);
        const uint4 gv = *reinterpret_cast<const uint4*>(ends.gain + v * 8);
        const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
        const float inv = s_inv[tok];
        uint32_t ow[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float lo = __fmul_rn(__fmul_rn(__uint_as_float(rw[j] << 16), inv), __uint_as_float(gw[j] << 16));
            const float hi = __fmul_rn(__fmul_rn(__uint_as_float(rw[j] & 0xFFFF0000u), inv), __uint_as_float(gw[j] & 0xFFFF0000u));
            const __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);
            ow[j] = *reinterpret_cast<const uint32_t*>(&pk);
        }
        reinterpret_cast<uint4*>(ends.normed + (size_t)tok * N)[v] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

// Activations the preceding kernel of the stream (or, in the tape, another CTA of this launch) has written: an ordinary
// (coherent, L1-allocating) load — never the read-only path, whose contract is data that stays constant for the
// kernel's lifetime, and this kernel is alive before its producer has finished.
__device__ __forceinline__ uint4 tape_ld_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// The ends of the reference's one-row matvec (`QmvEnds`, crates/targets/metal/src/tape/step.rs:472-498) that are not an
// output mode of their own: RMSNorm applied to the input as it is loaded, the projection's bias, a scale.
struct GemvExtra {
    const uint16_t* bias;        // [N] bf16 or null: added to the f32 sum
    const uint16_t* norm_gain;   // [K] bf16 or null: x is an RMSNorm's INPUT, this its gain
    float norm_eps, norm_offset; // rmsnorm(x, gain + offset)
    float scale;                 // multiplies the sum after the bias (1 = none)
    int norm_row_scale;          // norm-in in the reference's own arithmetic: the dot runs over bf16(x * (gain + offset)) and the
                                 //   finished row is scaled by 1 / rms(x) (0: the normalised row is rounded first, as the
                                 //   stand-alone RMSNorm stores it)
};
// Several independent linears that read the SAME activations (q, k, v; gate, up), run by ONE launch: the launch's row-block
// space is the matrices' row-blocks one after the other, and a row-block finds its matrix, its packed rows and its output
// through this table (passed by value; count 0 = a single matrix, the plain arguments apply).  What the reference gets by
// fusing the projections at load time (`load_rows_concat`) without re-laying the weights.
#define GEMV_GROUP_MAX 4
struct GemvGroup {
    const uint8_t* packed[GEMV_GROUP_MAX];
    uint16_t* y[GEMV_GROUP_MAX];
    int rb_start[GEMV_GROUP_MAX + 1];    // first row-block of each matrix in the launch's row-block space
    int n[GEMV_GROUP_MAX];               // output channels of each matrix
    int rb_pad[GEMV_GROUP_MAX];          // padded row-blocks of each matrix (where its trailer sits)
    int count;
};
// Matrix of row-block `rb` and everything of it (no dynamic indexing of the by-value table: selects only).
struct GemvGroupPick { const uint8_t* packed; uint16_t* y; int rb_local, n; };
__device__ __forceinline__ GemvGroupPick gemv_group_pick(const GemvGroup& g, int rb) {
    GemvGroupPick p = {g.packed[0], g.y[0], rb, g.n[0]};
#pragma unroll
    for (int i = 1; i < GEMV_GROUP_MAX; ++i)
        if (i < g.count && rb >= g.rb_start[i]) { p.packed = g.packed[i]; p.y = g.y[i]; p.rb_local = rb - g.rb_start[i]; p.n = g.n[i]; }
    return p;
}
__device__ __forceinline__ void gemv_unpack8(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xFFFF0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xFFFF0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xFFFF0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xFFFF0000u);
}
__device__ __forceinline__ uint32_t gemv_pack2(float lo, float hi) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}
constexpr int GEMV_NORM_REG_VECS = 4;     // vectors of 8 a thread keeps in registers: rows up to 8192 wide are read once
// The gain vectors this thread will use (load-time constants: fetched before the dependency wait, hidden under it).
__device__ __forceinline__ void gemv_norm_gain_load(const GemvExtra& ex, int K, uint4 (&gv)[GEMV_NORM_REG_VECS]) {
    const int nv = K >> 3;
#pragma unroll
    for (int i = 0; i < GEMV_NORM_REG_VECS; ++i) {
        const int v = threadIdx.x + i * GEMV_CWARPS * 32;
        gv[i] = v < nv ? *reinterpret_cast<const uint4*>(ex.norm_gain + v * 8) : make_uint4(0, 0, 0, 0);
    }
}
__device__ __forceinline__ uint4 gemv_norm_scale8(const uint4& xv, const uint4& gvec, float inv, float offset) {
    float f[8], w8[8];
    gemv_unpack8(xv, f);
    gemv_unpack8(gvec, w8);
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float g0 = offset != 0.f ? __fadd_rn(w8[2 * j], offset) : w8[2 * j];
        const float g1 = offset != 0.f ? __fadd_rn(w8[2 * j + 1], offset) : w8[2 * j + 1];
        o[j] = gemv_pack2(__fmul_rn(__fmul_rn(f[2 * j], inv), g0), __fmul_rn(__fmul_rn(f[2 * j + 1], inv), g1));
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}
// The norm-in end: the 256 consumer threads normalise the M activation rows into shared memory with the arithmetic AND
// the summation order of the stand-alone RMSNorm kernel (thread t sums the squares of vectors t, t + 256, .. in order,
// a shuffle tree per warp, the eight warp sums in warp order; out = bf16((x * inv_rms) * (gain + offset))), so the
// matvec sees the very bits that kernel would have stored (golden: crates/targets/metal/src/cpu_golden.rs:25-37).
__device__ __forceinline__ void gemv_norm_rows(const uint16_t* __restrict__ x, const GemvExtra& ex, int M, int K, uint8_t* xs,
                                               float* red8, const uint4 (&gv)[GEMV_NORM_REG_VECS]) {
    constexpr int T = GEMV_CWARPS * 32;
    const int tid = threadIdx.x, nv = K >> 3;
    const bool in_regs = nv <= GEMV_NORM_REG_VECS * T;           // block-uniform
    for (int m = 0; m < M; ++m) {
        const uint16_t* xr = x + (size_t)m * K;
        float ss = 0.f;
        uint4 xv[GEMV_NORM_REG_VECS];
        if (in_regs) {
            // one trip to L2 per row: the vectors stay in registers between the sum and the scaling
#pragma unroll
            for (int i = 0; i < GEMV_NORM_REG_VECS; ++i)
                if (tid + i * T < nv) xv[i] = tape_ld_v4(xr + (tid + i * T) * 8);
#pragma unroll
            for (int i = 0; i < GEMV_NORM_REG_VECS; ++i)
                if (tid + i * T < nv) {
                    float f[8];
                    gemv_unpack8(xv[i], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) ss = __fadd_rn(ss, __fmul_rn(f[j], f[j]));
                }
        } else {
            for (int v = tid; v < nv; v += T) {
                float f[8];
                gemv_unpack8(tape_ld_v4(xr + v * 8), f);
#pragma unroll
                for (int j = 0; j < 8; ++j) ss = __fadd_rn(ss, __fmul_rn(f[j], f[j]));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        gemv_consumer_sync();                                    // red8 of the previous row has been read
        if ((tid & 31) == 0) red8[tid >> 5] = ss;
        gemv_consumer_sync();
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < GEMV_CWARPS; ++w) total += red8[w];
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, float(K)), ex.norm_eps)));
        uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)m * K * 2);
        if (in_regs) {
#pragma unroll
            for (int i = 0; i < GEMV_NORM_REG_VECS; ++i)
                if (tid + i * T < nv) dst[tid + i * T] = gemv_norm_scale8(xv[i], gv[i], inv, ex.norm_offset);
        } else {
            for (int v = tid; v < nv; v += T)
                dst[v] = gemv_norm_scale8(tape_ld_v4(xr + v * 8), *reinterpret_cast<const uint4*>(ex.norm_gain + v * 8), inv, ex.norm_offset);
        }
    }
    gemv_consumer_sync();                                        // every row is in shared memory
}

// Norm-in as the reference's matvec does it (crates/targets/metal/tests/affine_qmv_ends_test.rs:6-9: "dots x ⊙ gain and scales
// the row by 1 / rms(x), so it skips the normed row's rounding"): the consumer threads stage bf16(x * (gain + offset)) in shared
// memory and leave each row's sum of squares, per warp, in `sq`; nothing waits for the sum before the first MMA — the thread
// that stores an output multiplies its finished sum by 1 / sqrt(mean(x^2) + eps) (`gemv_row_inv`).  One trip to L2 for up
// to 1024 vectors of 8 (x and gain fetched together), one barrier.
__device__ __forceinline__ void gemv_norm_rows_scaled(const uint16_t* __restrict__ x, const GemvExtra& ex, int M, int K, uint8_t* xs,
                                                      float (*sq)[GEMV_CWARPS]) {
    constexpr int T = GEMV_CWARPS * 32, S = 4;
    const int tid = threadIdx.x, nv = K >> 3, total = M * nv;    // x is [M][K] without padding: vector f is row f / nv
    uint4* dst = reinterpret_cast<uint4*>(xs);
    for (int base = 0; base < total; base += S * T) {
        uint4 xv[S], gv[S];
        int row[S];
#pragma unroll
        for (int i = 0; i < S; ++i) {
            const int f = base + tid + i * T;
            row[i] = f < total ? f / nv : -1;
            if (f < total) {
                xv[i] = tape_ld_v4(x + (size_t)f * 8);
                gv[i] = *reinterpret_cast<const uint4*>(ex.norm_gain + (f - row[i] * nv) * 8);
            }
        }
        float sqv[S];
#pragma unroll
        for (int i = 0; i < S; ++i) {
            sqv[i] = 0.f;
            if (row[i] >= 0) {
                float f8[8], w8[8];
                gemv_unpack8(xv[i], f8);
                gemv_unpack8(gv[i], w8);
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 8; ++j) sqv[i] = __fadd_rn(sqv[i], __fmul_rn(f8[j], f8[j]));
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float g0 = ex.norm_offset != 0.f ? __fadd_rn(w8[2 * j], ex.norm_offset) : w8[2 * j];
                    const float g1 = ex.norm_offset != 0.f ? __fadd_rn(w8[2 * j + 1], ex.norm_offset) : w8[2 * j + 1];
                    o[j] = gemv_pack2(__fmul_rn(f8[2 * j], g0), __fmul_rn(f8[2 * j + 1], g1));
                }
                dst[base + tid + i * T] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
        // a thread's vectors may lie in different rows: per row, its share in slot order, then a fixed shuffle tree
        for (int m = 0; m < M; ++m) {
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < S; ++i) a = __fadd_rn(a, row[i] == m ? sqv[i] : 0.f);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, o));
            if ((tid & 31) == 0) sq[m][tid >> 5] = base == 0 ? a : __fadd_rn(sq[m][tid >> 5], a);
        }
    }
    gemv_consumer_sync();                                        // the staged rows and the sums are in shared memory
}
// 1 / rms of token `tok`'s row from the per-warp sums (warp order), for the thread that stores that token's outputs.
__device__ __forceinline__ float gemv_row_inv(const float (*sq)[GEMV_CWARPS], int tok, int M, int K, float eps) {
    const int m = min(tok, M - 1);
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < GEMV_CWARPS; ++w) t = __fadd_rn(t, sq[m][w]);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, float(K)), eps)));
}

// The plain ends of one finished (row, token) sum: bias, scale, then bf16 / f32 / add into the residual stream.
// GEMV_OUT_RESIDUAL_ADD: y IS the residual stream and receives bf16(y + bf16(sum)) — the bits the separate add produces from the
// matvec's bf16 output (the residual end of `QmvEnds` with the roundings of `fused_add_rmsnorm`, cpu_golden.rs:171-200).
__device__ __forceinline__ void gemv_store_plain(float total, int mode, const GemvExtra& ex, uint16_t* __restrict__ y, size_t at, int n) {
    if (ex.bias) total += __uint_as_float(uint32_t(ex.bias[n]) << 16);
    if (ex.scale != 1.0f) total *= ex.scale;
    if (mode == GEMV_OUT_F32) {
        reinterpret_cast<float*>(y)[at] = total;
        return;
    }
    __nv_bfloat16 v = __float2bfloat16_rn(total);
    if (mode == GEMV_OUT_RESIDUAL_ADD) v = __float2bfloat16_rn(__fadd_rn(__uint_as_float(uint32_t(y[at]) << 16), __bfloat162float(v)));
    y[at] = *reinterpret_cast<const uint16_t*>(&v);
}

// A ring stage holds U blocks per consumer warp (8 * U blocks, one bulk copy): one full/empty handshake, one wait and one
// set of loop bookkeeping per U blocks instead of per block, and U independent dequantise + MMA streams for the
// scheduler to interleave.  Warp w takes blocks w, w + 8, .. of a stage, so a short last stage still spreads over the warps.
template <int U, int GS = 1> struct GemvRing {
    static constexpr int kBlockBytes = aff_block_bytes(GS);
    static constexpr int kStageBlocks = GEMV_CWARPS * U;
    static constexpr int kStageBytes = kStageBlocks * kBlockBytes;
    static constexpr int kStages = (U == 1) ? 4 : 3;
    static constexpr int kBytes = kStages * kStageBytes;
    static constexpr int kCtasPerSm = (U <= 2) ? 3 : 2;
};
// The common case is one try_wait (the stage has landed long ago); the bounded slow path is out of line.
static __device__ __noinline__ void gemv_wait_slow(uint32_t bar, uint32_t parity, int* status) { gemv_wait(bar, parity, status); }
__device__ __forceinline__ void gemv_wait_fast(uint32_t bar, uint32_t parity, int* status) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (!ok) gemv_wait_slow(bar, parity, status);
}

template <int MT, int SPLIT_CLUSTER, bool CHECK, int U, bool NORM, int GS, bool GROUP>
__device__ __forceinline__ void gemv_consumer(const uint16_t* __restrict__ x, uint16_t* __restrict__ y, int M, int N,
                                              int K, int kc_lo, int kc_hi, int nstage, int rb_real, int split, int sp,
                                              int out_f32, const GemvExtra& ex, uint32_t xs_base, int* __restrict__ status, uint32_t ring_base, uint32_t full_base,
                                              uint32_t empty_base, float (*red)[GEMV_CWARPS][32][MT * 4],
                                              float (*cl_part)[16][MT * 8], const GemvEnds& ends, float (*sq_s)[16][16],
                                              const GemvGroup& grp, const float (*norm_sq)[GEMV_CWARPS]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    float cta_sq = 0.f;                        // RESIDUAL_NORM: thread tok's sum of squares over this CTA's row-blocks
    // activation rows this lane feeds into the B operand.  Tokens beyond M read a clamped (valid)
    // row: a column of B only reaches the same column of D, which is discarded for tokens >= M.
    const uint16_t* xrow[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) xrow[mt] = x + (size_t)min(mt * 8 + g, M - 1) * K;

    using R = GemvRing<U, GS>;
    // norm-in, row-scale form: 1 / rms of the token whose outputs this thread stores (the same token for every row-block)
    float row_inv = 1.0f;
    if (NORM && !SPLIT_CLUSTER && ex.norm_row_scale && threadIdx.x < 32 * MT * 4) {
        const int ln0 = threadIdx.x / (MT * 4), idx0 = threadIdx.x % (MT * 4);
        row_inv = gemv_row_inv(norm_sq, (idx0 >> 2) * 8 + (ln0 & 3) * 2 + (idx0 & 1), M, K, ex.norm_eps);
    }
    uint32_t slot = 0, phase = 0;              // ring position and phase of the next stage
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
        for (int j = 0; j < nstage; ++j) {
            const int kc0 = kc_lo + j * R::kStageBlocks + warp;
            // the activations do not depend on the ring: the first block's are fetched while the weights are in flight,
            // the next block's while the current one is computed (L1 hits after the CTA's first row-block)
            uint4 xv[2][MT][4];
            auto load_x = [&](int u, uint4 (&dst)[MT][4]) {
                int k0 = (kc0 + u * GEMV_CWARPS) * 128 + t * 32;
                if (k0 >= K) k0 = 0;                              // padded k (zero weights) or idle warp
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        dst[mt][i] = NORM ? gemv_lds_v4(xs_base + (uint32_t)(min(mt * 8 + g, M - 1) * K + k0 + 8 * i) * 2u)   // the normalised rows
                                          : tape_ld_v4(xrow[mt] + k0 + 8 * i);      // coherent: the preceding kernel wrote x
            };
            load_x(0, xv[0]);
            gemv_wait_fast(full_base + 8u * slot, phase, status);
            const uint32_t stage = ring_base + slot * R::kStageBytes + warp * R::kBlockBytes;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (u + 1 < U) load_x(u + 1, xv[(u + 1) & 1]);
                if (kc0 + u * GEMV_CWARPS < kc_hi)                // warp-uniform
                    gemv_block_compute<MT, CHECK, GS>(stage + u * GEMV_CWARPS * R::kBlockBytes, acc, xv[u & 1], lane);
            }
            __syncwarp();                                         // every lane has consumed the stage
            if (lane == 0) gemv_mbar_arrive(empty_base + 8u * slot);
            if (++slot == R::kStages) { slot = 0; phase ^= 1u; }
        }

        // cross-warp reduction of this row-block, fixed warp order, double-buffered
        const int buf = it & 1;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i)
                red[buf][warp][lane][mt * 4 + i] = (acc[0][mt][i] + acc[1][mt][i]) * (CHECK ? 1.0f : AFF_SCALED_FACTOR);
        gemv_consumer_sync();

        // thread e owns accumulator slot (ln, idx): c0,c1 -> row g, tokens 2t,2t+1 ; c2,c3 -> row g+8
        constexpr int SLOTS = 32 * MT * 4;     // <= 256 consumer threads
        const int e = threadIdx.x;
        const int ln = e / (MT * 4), idx = e % (MT * 4);
        const int row = (ln >> 2) + (((idx & 3) >> 1) ? 8 : 0);
        const int tok = (idx >> 2) * 8 + (ln & 3) * 2 + (idx & 1);
        const int n = rb * 16 + row;
        if (e < SLOTS) {                       // warp-uniform: SLOTS is a multiple of 32
            float total = 0.f;
#pragma unroll
            for (int wdx = 0; wdx < GEMV_CWARPS; ++wdx) total += red[buf][wdx][ln][idx];
            if (NORM && !SPLIT_CLUSTER) total *= row_inv;
            if (SPLIT_CLUSTER) {
                if (tok < M) gemv_st_cluster_rank0_f32(&cl_part[sp][row][tok], total);
            } else if (out_f32 == GEMV_OUT_SILU_PAIRS) {
                gemv_store_silu_pair(total, idx, tok, M, rb * 8 + (ln >> 2), N >> 1, y);
            } else if (out_f32 == GEMV_OUT_RESIDUAL_NORM) {
                sq_s[buf][tok][row] = gemv_residual_update(total, tok, M, n, N, ends);
            } else if (GROUP) {
                const GemvGroupPick gp = gemv_group_pick(grp, rb);
                const int nl = gp.rb_local * 16 + row;
                if (tok < M && nl < gp.n) gemv_store_plain(total, out_f32, ex, gp.y, (size_t)tok * gp.n + nl, nl);
            } else if (tok < M && n < N) {
                gemv_store_plain(total, out_f32, ex, y, (size_t)tok * N + n, n);
            }
        }
        if (!SPLIT_CLUSTER && out_f32 == GEMV_OUT_RESIDUAL_NORM) {
            gemv_consumer_sync();              // sq_s[buf] is complete (red[buf] is not reused before the next sync either)
            if (threadIdx.x < M) {
#pragma unroll
                for (int r = 0; r < 16; ++r) cta_sq = __fadd_rn(cta_sq, sq_s[buf][threadIdx.x][r]);
            }
        }
    }
    if (!SPLIT_CLUSTER && out_f32 == GEMV_OUT_RESIDUAL_NORM)
        gemv_norm_tail(cta_sq, M, N, gridDim.x, blockIdx.x, ends, 1, GEMV_CWARPS * 32);
}

template <int MT, int SPLIT_CLUSTER, int U, bool NORM, int GS, bool GROUP>
__global__ void __launch_bounds__(GEMV_THREADS, (MT == 1 ? GemvRing<U, GS>::kCtasPerSm : 2))
affine_b4_gemv_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                      int M, int N, int K, int RB, int KC, int rb_real, int split, int out_f32,
                      GemvExtra ex, int* __restrict__ status, GemvEnds ends, GemvGroup grp) {
    extern __shared__ __align__(128) uint8_t gemv_ring[];          // [stages][8 * U blocks], then (NORM) the normalised rows [M][K] bf16
    __shared__ float norm_red[GEMV_CWARPS];
    __shared__ float norm_sq[NORM ? 8 : 1][GEMV_CWARPS];          // norm-in, row-scale form: sums of squares [token][warp]
    __shared__ float sq_s[2][16][16];                              // RESIDUAL_NORM: squares of the stored residuals [token][row]
    using R = GemvRing<U, GS>;
    __shared__ __align__(8) uint64_t full_bar[R::kStages];
    __shared__ __align__(8) uint64_t empty_bar[R::kStages];
    __shared__ float red[2][GEMV_CWARPS][32][MT * 4];
    __shared__ float cl_part[SPLIT_CLUSTER ? GEMV_MAX_SPLIT : 1][16][MT * 8];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int d = 0; d < R::kStages; ++d) {
            gemv_mbar_init(gemv_smem_u32(&full_bar[d]), 1);
            gemv_mbar_init(gemv_smem_u32(&empty_bar[d]), GEMV_CWARPS);
        }
    }
    gemv_fence_mbar_init();
    __syncthreads();
    // Programmatic dependent launch: let the next kernel of the stream start its own weight
    // prefetch as this one drains.  Weights are load-time constants, so this kernel's producer
    // starts at once; only the consumers wait for the preceding kernel (which wrote x).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int sp = SPLIT_CLUSTER ? int(gemv_cluster_ctarank()) : 0;
    // k-chunks of this CTA: [kc_lo, kc_hi), consumed 8 at a time
    const int per = (KC + split - 1) / split;
    const int kc_lo = sp * per;
    const int kc_hi = min(KC, kc_lo + per);
    const int nstage = (max(kc_hi - kc_lo, 0) + R::kStageBlocks - 1) / R::kStageBlocks;
    const uint32_t ring_base = gemv_smem_u32(gemv_ring);
    const uint32_t full_base = gemv_smem_u32(&full_bar[0]);
    const uint32_t empty_base = gemv_smem_u32(&empty_bar[0]);

    if (warp == GEMV_CWARPS) {
        // ---- producer warp: one lane streams the row-blocks' k extents into the ring
        if (lane == 0) {
            uint32_t slot = 0, phase = 0;
            for (int rb = blockIdx.x; rb < rb_real; rb += gridDim.x) {
                const uint8_t* src = GROUP ? [&] { const GemvGroupPick gp = gemv_group_pick(grp, rb);
                                                       return gp.packed + ((size_t)gp.rb_local * KC + kc_lo) * R::kBlockBytes; }()
                                               : packed + ((size_t)rb * KC + kc_lo) * R::kBlockBytes;
                for (int j = 0; j < nstage; ++j) {
                    gemv_wait(empty_base + 8u * slot, phase ^ 1u, status);
                    const uint32_t bytes = (uint32_t)min(R::kStageBlocks, kc_hi - kc_lo - j * R::kStageBlocks) * R::kBlockBytes;
                    gemv_arrive_expect_tx(full_base + 8u * slot, bytes);
                    gemv_bulk_g2s(ring_base + slot * R::kStageBytes, src + (size_t)j * R::kStageBytes, bytes, full_base + 8u * slot);
                    if (++slot == R::kStages) { slot = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else {
        // one word per matrix says whether any group needs the exact (two-step rounding) path; it is a
        // load-time constant, so its (cold, HBM) fetch is issued before the wait and hides under it
        unsigned int trailer_flag;
        if (GROUP) {                                               // any matrix of the group that needs the exact path
            trailer_flag = 0;
#pragma unroll
            for (int i = 0; i < GEMV_GROUP_MAX; ++i)
                if (i < grp.count)
                    trailer_flag |= *reinterpret_cast<const volatile unsigned int*>(grp.packed[i] + (size_t)grp.rb_pad[i] * KC * R::kBlockBytes);
        } else {
            trailer_flag = *reinterpret_cast<const volatile unsigned int*>(packed + (size_t)RB * KC * R::kBlockBytes);
        }
        uint4 norm_gv[GEMV_NORM_REG_VECS];
        if (NORM && !ex.norm_row_scale) gemv_norm_gain_load(ex, K, norm_gv);
        asm volatile("griddepcontrol.wait;" ::: "memory");        // x (and y's previous readers) are settled
        const uint32_t xs_base = ring_base + R::kBytes;
        if (NORM) {
            if (ex.norm_row_scale) gemv_norm_rows_scaled(x, ex, M, K, gemv_ring + R::kBytes, norm_sq);
            else gemv_norm_rows(x, ex, M, K, gemv_ring + R::kBytes, norm_red, norm_gv);
        }
        const bool check = trailer_flag != 0;
        if (check)
            gemv_consumer<MT, SPLIT_CLUSTER, true, U, NORM, GS, GROUP>(x, y, M, N, K, kc_lo, kc_hi, nstage, rb_real, split, sp, out_f32, ex, xs_base, status,
                                                            ring_base, full_base, empty_base, red, cl_part, ends, sq_s, grp, norm_sq);
        else
            gemv_consumer<MT, SPLIT_CLUSTER, false, U, NORM, GS, GROUP>(x, y, M, N, K, kc_lo, kc_hi, nstage, rb_real, split, sp, out_f32, ex, xs_base, status,
                                                             ring_base, full_base, empty_base, red, cl_part, ends, sq_s, grp, norm_sq);
    }

    if (SPLIT_CLUSTER) {
        // one row-block per CTA in cluster mode (gridDim.x == rb_real): exchange once, rank order
        gemv_cluster_sync_all();
        constexpr int SLOTS = 32 * MT * 4;
        const int e = threadIdx.x;
        const int ln = e / (MT * 4), idx = e % (MT * 4);
        const int row = (ln >> 2) + (((idx & 3) >> 1) ? 8 : 0);
        const int tok = (idx >> 2) * 8 + (ln & 3) * 2 + (idx & 1);
        const int n = blockIdx.x * 16 + row;
        // norm-in, row-scale form: every CTA of the cluster staged the whole rows, so rank 0 holds the sums of squares
        const float row_inv = (NORM && ex.norm_row_scale && sp == 0 && e < SLOTS) ? gemv_row_inv(norm_sq, tok, M, K, ex.norm_eps) : 1.0f;
        if (out_f32 == GEMV_OUT_RESIDUAL_NORM) {
            if (sp != 0) return;                   // the cluster's CTA 0 owns the row-block's output (block-uniform exit)
            if (e < 256) sq_s[0][e >> 4][e & 15] = 0.f;
            __syncthreads();
            if (e < SLOTS) {
                float s = 0.f;
                for (int r = 0; r < split; ++r) s += cl_part[r][row][tok];
                if (NORM) s *= row_inv;
                sq_s[0][tok][row] = gemv_residual_update(s, tok, M, n, N, ends);
            }
            __syncthreads();
            float cta_sq = 0.f;
            if (e < M) {
#pragma unroll
                for (int r = 0; r < 16; ++r) cta_sq = __fadd_rn(cta_sq, sq_s[0][e][r]);
            }
            gemv_norm_tail(cta_sq, M, N, gridDim.x, blockIdx.x, ends, 2, GEMV_THREADS);
        } else if (sp == 0 && e < SLOTS && out_f32 == GEMV_OUT_SILU_PAIRS) {
            float s = 0.f;
            for (int r = 0; r < split; ++r) s += cl_part[r][row][min(tok, MT * 8 - 1)];
            if (NORM) s *= row_inv;
            gemv_store_silu_pair(s, idx, tok, M, blockIdx.x * 8 + (ln >> 2), N >> 1, y);
        } else if (GROUP && sp == 0 && e < SLOTS) {
            const GemvGroupPick gp = gemv_group_pick(grp, blockIdx.x);
            const int nl = gp.rb_local * 16 + row;
            if (tok < M && nl < gp.n) {
                float s = 0.f;
                for (int r = 0; r < split; ++r) s += cl_part[r][row][tok];
                gemv_store_plain(s, out_f32, ex, gp.y, (size_t)tok * gp.n + nl, nl);
            }
        } else if (sp == 0 && e < SLOTS && tok < M && n < N) {
            float s = 0.f;
            for (int r = 0; r < split; ++r) s += cl_part[r][row][tok];
            if (NORM) s *= row_inv;
            gemv_store_plain(s, out_f32, ex, y, (size_t)tok * N + n, n);
        }
    }
}

// ------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------
static int32_t affine_check_shape(scr_ctx* ctx, int N, int K, int group) {
    if (N <= 0 || K <= 0) return scr_fail(ctx, SCR_E_SHAPE, "N=%d K=%d must be positive", N, K);
    if (group != 32 && group != 64 && group != 128)
        return scr_fail(ctx, SCR_E_DTYPE, "group_size=%d: the affine presets have groups of 32, 64 or 128", group);
    if (K % group != 0) return scr_fail(ctx, SCR_E_SHAPE, "K=%d not divisible by group_size=%d", K, group);
    return SCR_OK;
}

extern "C" int32_t scr_affine_b4_repack_size(int32_t N, int32_t K, int32_t group, size_t* bytes) {
    if (!bytes) return SCR_E_ARG;
    if (N <= 0 || K <= 0) return SCR_E_SHAPE;
    if (group != 32 && group != 64 && group != 128) return SCR_E_DTYPE;
    if (K % group != 0) return SCR_E_SHAPE;
    const AffineGeom g = affine_geom(N, K, group);
    *bytes = affine_packed_bytes(g);
    return SCR_OK;
}

extern "C" int32_t scr_affine_b4_repack(scr_ctx* ctx, const uint32_t* w, const uint16_t* scales, const uint16_t* biases,
                                        int32_t scale_dtype, int32_t N, int32_t K, int32_t group, void* dst, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!w || !scales || !biases || !dst) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    if (scale_dtype != SCR_DTYPE_F16 && scale_dtype != SCR_DTYPE_BF16)
        return scr_fail(ctx, SCR_E_DTYPE, "scales/biases must be F16 or BF16 (dtype %d)", scale_dtype);
    int32_t st = affine_check_shape(ctx, N, K, group);
    if (st) return st;
    if (!scr_aligned16(w) || !scr_aligned16(dst)) return scr_fail(ctx, SCR_E_ALIGN, "w/dst must be 16-byte aligned");
    const AffineGeom g = affine_geom(N, K, group);
    const long long items = (long long)g.RB * g.KC * (64 + (8 << g.gs));
    const int threads = 256;
    const int blocks = (int)std::min<long long>((items + threads - 1) / threads, (long long)ctx->sm_count * 32);
    unsigned int* flag = reinterpret_cast<unsigned int*>((uint8_t*)dst + affine_blocks_bytes(g));
    cudaError_t e = cudaMemsetAsync(flag, 0, AFF_TRAILER_BYTES, (cudaStream_t)stream);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "affine_b4_repack memset: %s", cudaGetErrorString(e));
    affine_b4_repack_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>(w, scales, biases, scale_dtype == SCR_DTYPE_F16, N, K, group, g.gs,
                                                                         g.RB, g.KC, (uint8_t*)dst, flag);
    int32_t st2 = scr_check_launch(ctx, "affine_b4_repack");
    if (st2) return st2;
    affine_b4_repack_fence_kernel<<<1, 32, 0, (cudaStream_t)stream>>>();
    return scr_check_launch(ctx, "affine_b4_repack_fence");
}

extern "C" int32_t scr_affine_b4_dequant_dump(scr_ctx* ctx, const void* packed, int32_t N, int32_t K, int32_t group,
                                              uint16_t* w_bf16, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!packed || !w_bf16) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    int32_t st = affine_check_shape(ctx, N, K, group);
    if (st) return st;
    if (!scr_aligned16(packed) || !scr_aligned16(w_bf16)) return scr_fail(ctx, SCR_E_ALIGN, "pointers must be 16-byte aligned");
    const AffineGeom g = affine_geom(N, K, group);
    const long long items = (long long)g.RB * g.KC * 64;
    const int threads = 256;
    const int blocks = (int)std::min<long long>((items + threads - 1) / threads, (long long)ctx->sm_count * 32);
    affine_b4_dump_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>((const uint8_t*)packed, N, K, g.gs, g.RB, g.KC, w_bf16);
    return scr_check_launch(ctx, "affine_b4_dequant_dump");
}

extern "C" int32_t scr_affine_b4_embed(scr_ctx* ctx, const void* packed, const uint32_t* ids, int32_t n_ids, int32_t vocab,
                                       int32_t hidden, int32_t group, uint16_t* out_bf16, void* stream) {
    SCR_REQUIRE_CTX(ctx);
    if (!packed || !ids || !out_bf16) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    int32_t st = affine_check_shape(ctx, vocab, hidden, group);
    if (st) return st;
    if (n_ids < 0) return scr_fail(ctx, SCR_E_SHAPE, "n_ids=%d", n_ids);
    if (n_ids == 0) return SCR_OK;
    if (!scr_aligned16(packed) || !scr_aligned16(out_bf16)) return scr_fail(ctx, SCR_E_ALIGN, "pointers must be 16-byte aligned");
    const AffineGeom g = affine_geom(vocab, hidden, group);
    const long long items = (long long)n_ids * (hidden / 32);
    const int threads = 128;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)std::min<long long>((items + threads - 1) / threads, (long long)ctx->sm_count * 16));
    cfg.blockDim = dim3(threads);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, affine_b4_embed_kernel, (const uint8_t*)packed, ids, (int)n_ids, (int)vocab, (int)hidden,
                                             g.gs, g.RB, g.KC, out_bf16, ctx->dev_status);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "affine_b4_embed launch: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "affine_b4_embed");
}

// Launch shape.  With enough row-blocks the grid is persistent (two CTAs per SM) and nothing
// is split; with few row-blocks each CTA takes one row-block and a cluster of `split` CTAs
// shares its k-chunks so that about one CTA per SM is busy.
static void affine_gemv_shape(int rb_real, int KC, int sms, int ctas_per_sm, int* grid_x, int* split) {
    // Enough row-blocks: persistent CTAs walk them, nothing is split.
    const int slots = ctas_per_sm * sms;
    if (rb_real >= slots) {
        *grid_x = slots;
        *split = 1;
        return;
    }
    // Fewer: one row-block per CTA and a cluster of `s` CTAs shares its k extent, chosen so that
    // everything is resident at once and the longest CTA runs the fewest ring stages.
    int best = 1, best_stages = (KC + GEMV_CWARPS - 1) / GEMV_CWARPS;
    for (int s = 2; s <= GEMV_MAX_SPLIT && rb_real * s <= slots; ++s) {
        const int per = (KC + s - 1) / s;
        const int stages = (per + GEMV_CWARPS - 1) / GEMV_CWARPS;
        if (stages < best_stages) { best_stages = stages; best = s; }
    }
    *grid_x = rb_real;
    *split = best;
}

// What a forward call asks of the epilogue, passed down as an argument (never parked in the context: a
// context may serve two streams).
struct AffineFwd {
    int out_mode = GEMV_OUT_BF16;            // GEMV_OUT_*
    const uint16_t* bias = nullptr;          // the linear's own bias [N] (bf16), added in f32 before the one rounding
    const uint16_t* norm_gain = nullptr;     // norm-in: x is an RMSNorm's input, this its gain [K]
    float norm_eps = 0.f, norm_offset = 0.f;
    int norm_row_scale = 0;                  // norm-in in the reference's arithmetic (see GemvExtra)
    float scale = 1.0f;                      // multiplies the sum after the bias
    const GemvEnds* ends = nullptr;          // GEMV_OUT_RESIDUAL_NORM only
    int gs = 1;                              // (scale, bias) entries per row and block, log2: set from the group size by affine_forward
    const GemvGroup* grp = nullptr;          // several matrices in one launch (scr_linear_affine_b4_group); N is then unused
    int grp_rb = 0;                          // ... the launch's total row-blocks
};
// Shared memory the norm-in end may take for the normalised rows beside the ring (two CTAs per SM).
#define GEMV_NORM_MAX_BYTES (20 * 1024)

// Blocks per warp and ring stage.  3 costs 173 executed warp instructions per 1152-byte block against 217 with 1, but runs two
// CTAs of 96 registers per SM instead of three of 72.  Measured on Llama-3.2-3B at one token: for launches that follow one
// another in one stream (a decode step; a layer's linears as 4 launches) 3 is faster throughout (the 28 layers' linears one
// after the other 829 against 894 us, as fused projections 641 against 678 us, the batch-1 decode step 1.085-1.100 against
// 1.150 ms, the largest shape alone 5.66 against 5.81 us); only where independent matvecs run on parallel streams and
// overlap their neighbours' tails is 1 ahead (790 against 856 us for the 196 linears on two graph branches); 2 loses in both
// settings.  At 8 tokens, where every lane reads its own activation row, 1 is 2 % faster.  So: 3 up to 4 tokens, 1 above
// (the two-tile kernel for 9..16 tokens has no registers to spare) — except for a matrix whose row-blocks fit the GPU in one
// round at three CTAs per SM but not at two (the fused q|k|v of Llama-3.2-3B: 320 row-blocks for 296 or 444 slots): there
// two dozen CTAs of the two-per-SM form would run a second row-block while the rest idle.
static int affine_gemv_u(int M, int rb_real, int sms) {
    if (M > 4) return 1;
    return (rb_real > 2 * sms && rb_real <= 3 * sms) ? 1 : 3;
}

template <int MT, int U, bool NORM, int GS = 1, bool GROUP = false>
static int32_t affine_gemv_launch_u(scr_ctx* ctx, const uint8_t* packed, const uint16_t* x, uint16_t* y, int M, int N,
                                    int K, const AffineFwd& f, cudaStream_t stream) {
    using R = GemvRing<U, GS>;
    const AffineGeom g = affine_geom(f.grp ? 16 : N, K, GS == 2 ? 32 : 64);   // KC only matters for a group
    const int rb_real = f.grp ? f.grp_rb : scr_ceil_div(N, 16);
    int grid_x = 1, split = 1;
    affine_gemv_shape(rb_real, g.KC, ctx->sm_count, MT == 1 ? R::kCtasPerSm : 2, &grid_x, &split);
    auto kernel = (split == 1) ? affine_b4_gemv_kernel<MT, 0, U, NORM, GS, GROUP> : affine_b4_gemv_kernel<MT, 1, U, NORM, GS, GROUP>;
    const int smem = R::kBytes + (NORM ? M * K * 2 : 0);
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, R::kBytes + (NORM ? GEMV_NORM_MAX_BYTES : 0));
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "affine_b4_gemv smem attribute: %s", cudaGetErrorString(e));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid_x, split, 1);
    cfg.blockDim = dim3(GEMV_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
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
    GemvEnds ends = {};
    if (f.out_mode == GEMV_OUT_RESIDUAL_NORM) {
        if (!f.ends) return scr_fail(ctx, SCR_E_ARG, "residual + norm epilogue requested without its arguments");
        ends = *f.ends;
        if ((size_t)(16 + grid_x * 16) * sizeof(float) > SCR_ENDS_SCRATCH_BYTES)
            return scr_fail(ctx, SCR_E_WORKSPACE, "residual + norm epilogue: %d CTAs exceed the scratch", grid_x);
    }
    const GemvExtra ex = {f.bias, f.norm_gain, f.norm_eps, f.norm_offset, f.scale, f.norm_gain ? f.norm_row_scale : 0};
    const GemvGroup grp = f.grp ? *f.grp : GemvGroup{};
    e = cudaLaunchKernelEx(&cfg, kernel, packed, x, y, M, N, K, g.RB, g.KC, rb_real, split, f.out_mode, ex, ctx->dev_status, ends, grp);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "affine_b4_gemv launch: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "affine_b4_gemv");
}

template <int MT>
static int32_t affine_gemv_launch(scr_ctx* ctx, const uint8_t* packed, const uint16_t* x, uint16_t* y, int M, int N,
                                  int K, const AffineFwd& f, cudaStream_t stream) {
    if (f.gs == 2) {
        // groups of 32: the 1280-byte block, one block per warp and ring stage
        if (f.norm_gain) return scr_fail(ctx, SCR_E_UNSUPPORTED, "norm-in end: not built for groups of 32 (run the norm on its own)");
        return affine_gemv_launch_u<MT, 1, false, 2>(ctx, packed, x, y, M, N, K, f, stream);
    }
    const int u = affine_gemv_u(M, f.grp ? f.grp_rb : scr_ceil_div(N, 16), ctx->sm_count);
    if (f.grp) {
        if (f.gs == 2 || f.norm_gain) return scr_fail(ctx, SCR_E_UNSUPPORTED, "a group launch is built for groups of 64 and 128 without the norm-in end");
        if (u == 3) return affine_gemv_launch_u<1, 3, false, 1, true>(ctx, packed, x, y, M, N, K, f, stream);
        return affine_gemv_launch_u<MT, 1, false, 1, true>(ctx, packed, x, y, M, N, K, f, stream);
    }
    if (f.norm_gain) {
        // the normalised rows sit in shared memory beside the ring: a few tokens only
        if (MT != 1 || (size_t)M * K * 2 > GEMV_NORM_MAX_BYTES)
            return scr_fail(ctx, SCR_E_UNSUPPORTED, "norm-in end: M=%d rows of K=%d exceed %d bytes of shared memory (run the norm on its own)",
                            M, K, GEMV_NORM_MAX_BYTES);
        if (u == 3) return affine_gemv_launch_u<1, 3, true>(ctx, packed, x, y, M, N, K, f, stream);
        return affine_gemv_launch_u<1, 1, true>(ctx, packed, x, y, M, N, K, f, stream);
    }
    if (u == 3) return affine_gemv_launch_u<1, 3, false>(ctx, packed, x, y, M, N, K, f, stream);
    return affine_gemv_launch_u<MT, 1, false>(ctx, packed, x, y, M, N, K, f, stream);
}

// Defined in affine_b4_gemm.cu
int32_t affine_b4_gemm_tc_launch(scr_ctx* ctx, const uint8_t* packed, const uint16_t* x, uint16_t* y, int M, int N,
                                 int K, int gs, int out_f32, const uint16_t* bias, void* workspace, size_t workspace_bytes,
                                 cudaStream_t stream);
size_t affine_b4_gemm_tc_workspace(int M, int N, int K);
bool affine_b4_gemm_tc_enabled();

size_t affine_workspace_bytes(int M, int N, int K) {
    if (M <= 16 || !affine_b4_gemm_tc_enabled()) return 0;
    return affine_b4_gemm_tc_workspace(M, N, K);
}

// The forward dispatch every int4 entry point goes through: the balanced matvec up to 8 tokens, the
// two-tile matvec up to 16, the tensor-core GEMM above.
static int32_t affine_forward(scr_ctx* ctx, const void* packed, const uint16_t* x, int M, int N, int K, int group, void* y_,
                              const AffineFwd& f_in, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (!packed || !x || !y_) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    int32_t st = affine_check_shape(ctx, N, K, group);
    if (st) return st;
    AffineFwd f = f_in;
    f.gs = affine_gs(group);
    if (M <= 0) return scr_fail(ctx, SCR_E_SHAPE, "M=%d must be positive", M);
    if (!scr_aligned16(packed) || !scr_aligned16(x)) return scr_fail(ctx, SCR_E_ALIGN, "packed/x must be 16-byte aligned");
    if ((f.bias || f.scale != 1.0f) && (f.out_mode == GEMV_OUT_SILU_PAIRS || f.out_mode == GEMV_OUT_RESIDUAL_NORM))
        return scr_fail(ctx, SCR_E_UNSUPPORTED, "a bias or a scale cannot be combined with this fused epilogue");
    if (M > 16 && (f.norm_gain || f.scale != 1.0f || f.out_mode == GEMV_OUT_RESIDUAL_ADD))
        return scr_fail(ctx, SCR_E_UNSUPPORTED, "the norm-in, scale and residual ends exist on the matvec path only (M <= 16)");
    if (f.norm_gain && !scr_aligned16(f.norm_gain)) return scr_fail(ctx, SCR_E_ALIGN, "the norm gain must be 16-byte aligned");
    const uint8_t* pk = (const uint8_t*)packed;
    uint16_t* y = static_cast<uint16_t*>(y_);
    if (M <= 8) return affine_gemv_launch<1>(ctx, pk, x, y, M, N, K, f, stream);
    if (M <= 16) return affine_gemv_launch<2>(ctx, pk, x, y, M, N, K, f, stream);
    if (f.out_mode != GEMV_OUT_BF16 && f.out_mode != GEMV_OUT_F32)
        return scr_fail(ctx, SCR_E_UNSUPPORTED, "this fused epilogue exists on the matvec path only (M <= 16)");
    if (affine_b4_gemm_tc_enabled()) {
        const size_t need = affine_b4_gemm_tc_workspace(M, N, K);
        if (need > 0 && (!workspace || workspace_bytes < need))
            return scr_fail(ctx, SCR_E_WORKSPACE, "workspace %zu bytes < required %zu", workspace_bytes, need);
        return affine_b4_gemm_tc_launch(ctx, pk, x, y, M, N, K, f.gs, f.out_mode == GEMV_OUT_F32, f.bias, workspace, workspace_bytes, stream);
    }
    // Token tiles of 16 through the matvec kernel (weights re-streamed per tile).
    const size_t ystride = f.out_mode == GEMV_OUT_F32 ? 2 : 1;
    for (int m0 = 0; m0 < M; m0 += 16) {
        const int mt = std::min(16, M - m0);
        uint16_t* yt = y + (size_t)m0 * N * ystride;
        st = (mt <= 8) ? affine_gemv_launch<1>(ctx, pk, x + (size_t)m0 * K, yt, mt, N, K, f, stream)
                       : affine_gemv_launch<2>(ctx, pk, x + (size_t)m0 * K, yt, mt, N, K, f, stream);
        if (st) return st;
    }
    return SCR_OK;
}

extern "C" int32_t scr_linear_affine_b4(scr_ctx* ctx, const void* packed, const uint16_t* x, int32_t M, int32_t N,
                                        int32_t K, int32_t group, const uint16_t* bias, uint16_t* y, void* workspace,
                                        size_t workspace_bytes, void* stream_) {
    SCR_REQUIRE_CTX(ctx);
    AffineFwd f;
    f.bias = bias;
    return affine_forward(ctx, packed, x, M, N, K, group, y, f, workspace, workspace_bytes, (cudaStream_t)stream_);
}

// A row-parallel linear (o, down) yields a `Partial` in the reference's placement lattice
// (crates/compiler/subtile/src/tensor_parallel.rs:1-63): unrounded f32 sums over the rank's K-slice, to be
// summed over ranks by the all-reduce and rounded to bf16 once afterwards (the bias, if any, is added after
// the sum by whoever rounds).
extern "C" int32_t scr_linear_affine_b4_partial(scr_ctx* ctx, const void* packed, const uint16_t* x, int32_t M, int32_t N,
                                                int32_t K, int32_t group, float* y_f32, void* workspace,
                                                size_t workspace_bytes, void* stream_) {
    SCR_REQUIRE_CTX(ctx);
    AffineFwd f;
    f.out_mode = GEMV_OUT_F32;
    return affine_forward(ctx, packed, x, M, N, K, group, y_f32, f, workspace, workspace_bytes, (cudaStream_t)stream_);
}

// Up to GEMV_GROUP_MAX independent linears over the SAME activations in one launch (q, k, v; gate, up): matrices of one K and
// one group size, each with its own packed buffer and its own output.  Up to 16 tokens it is one matvec launch whose
// row-block space runs over the matrices; above, the linears run one after the other (the GEMM fills the GPU by itself).
extern "C" int32_t scr_linear_affine_b4_group(scr_ctx* ctx, int32_t count, const void* const* packed, const uint16_t* x, int32_t M,
                                              const int32_t* N, int32_t K, int32_t group, uint16_t* const* y, void* workspace,
                                              size_t workspace_bytes, void* stream_) {
    SCR_REQUIRE_CTX(ctx);
    if (!packed || !N || !y || !x) return scr_fail(ctx, SCR_E_ARG, "null pointer");
    if (count < 1 || count > GEMV_GROUP_MAX) return scr_fail(ctx, SCR_E_SHAPE, "a group holds 1 to %d linears (%d)", GEMV_GROUP_MAX, count);
    if (M <= 0) return scr_fail(ctx, SCR_E_SHAPE, "M=%d must be positive", M);
    GemvGroup grp = {};
    grp.count = count;
    int rb = 0;
    for (int i = 0; i < count; ++i) {
        if (!packed[i] || !y[i]) return scr_fail(ctx, SCR_E_ARG, "group member %d: null pointer", i);
        const int32_t st = affine_check_shape(ctx, N[i], K, group);
        if (st) return st;
        if (!scr_aligned16(packed[i])) return scr_fail(ctx, SCR_E_ALIGN, "group member %d: packed must be 16-byte aligned", i);
        grp.packed[i] = static_cast<const uint8_t*>(packed[i]);
        grp.y[i] = y[i];
        grp.n[i] = N[i];
        grp.rb_start[i] = rb;
        grp.rb_pad[i] = affine_geom(N[i], K, group).RB;
        rb += scr_ceil_div(N[i], 16);
    }
    for (int i = count; i <= GEMV_GROUP_MAX; ++i) grp.rb_start[i] = rb;
    if (!scr_aligned16(x)) return scr_fail(ctx, SCR_E_ALIGN, "x must be 16-byte aligned");
    if (M > 16 || count == 1 || group == 32) {            // (groups of 32 have no group launch: member by member)
        for (int i = 0; i < count; ++i) {
            AffineFwd f;
            const int32_t st = affine_forward(ctx, packed[i], x, M, N[i], K, group, y[i], f, workspace, workspace_bytes, (cudaStream_t)stream_);
            if (st) return st;
        }
        return SCR_OK;
    }
    AffineFwd f;
    f.gs = affine_gs(group);
    f.grp = &grp;
    f.grp_rb = rb;
    if (M <= 8) return affine_gemv_launch<1>(ctx, grp.packed[0], x, grp.y[0], M, N[0], K, f, (cudaStream_t)stream_);
    return affine_gemv_launch<2>(ctx, grp.packed[0], x, grp.y[0], M, N[0], K, f, (cudaStream_t)stream_);
}

// The one-row matvec with the reference's ends around it (`QmvEnds`, crates/targets/metal/src/tape/step.rs:472-498).
extern "C" int32_t scr_linear_affine_b4_ends(scr_ctx* ctx, const void* packed, const uint16_t* x, int32_t M, int32_t N, int32_t K,
                                             int32_t group, const scr_qmv_ends* ends, uint16_t* y, void* stream_) {
    SCR_REQUIRE_CTX(ctx);
    if (!ends) return scr_fail(ctx, SCR_E_ARG, "null ends");
    AffineFwd f;
    f.bias = ends->bias;
    f.norm_gain = ends->norm_gain;
    f.norm_eps = ends->norm_eps;
    f.norm_offset = ends->norm_gain_offset;
    f.norm_row_scale = ends->norm_row_scale != 0;
    f.scale = ends->scale == 0.f ? 1.0f : ends->scale;
    if (ends->silu_pairs && ends->residual) return scr_fail(ctx, SCR_E_ARG, "the gate/up pairing and the residual end exclude each other");
    f.out_mode = ends->residual ? GEMV_OUT_RESIDUAL_ADD : (ends->silu_pairs ? GEMV_OUT_SILU_PAIRS : GEMV_OUT_BF16);
    if (ends->silu_pairs && (N <= 0 || N % 16 != 0)) return scr_fail(ctx, SCR_E_SHAPE, "gate/up pairing: %d fused rows (8 gate + 8 up per block)", N);
    if (M > 16) return scr_fail(ctx, SCR_E_UNSUPPORTED, "the matvec ends exist up to 16 tokens (M=%d): run the operators separately", M);
    return affine_forward(ctx, packed, x, M, N, K, group, y, f, nullptr, 0, (cudaStream_t)stream_);
}

extern "C" int32_t scr_linear_affine_b4_residual_rmsnorm(scr_ctx* ctx, const void* packed, const uint16_t* x, int32_t M,
                                                         int32_t N, int32_t K, int32_t group, uint16_t* residual,
                                                         const uint16_t* gain, float eps, uint16_t* normed, void* scratch,
                                                         size_t scratch_bytes, void* stream_) {
    SCR_REQUIRE_CTX(ctx);
    if (M > 16) return scr_fail(ctx, SCR_E_UNSUPPORTED, "fused residual + norm epilogue: M=%d (the matvec path, M <= 16, has it)", M);
    if (!residual || !gain || !normed || !scratch) return scr_fail(ctx, SCR_E_ARG, "fused residual + norm epilogue: null pointer");
    if (N <= 0 || N % 8 != 0) return scr_fail(ctx, SCR_E_SHAPE, "fused residual + norm epilogue: N=%d must be a multiple of 8", N);
    if (scratch_bytes < SCR_ENDS_SCRATCH_BYTES)
        return scr_fail(ctx, SCR_E_WORKSPACE, "fused residual + norm epilogue: scratch %zu bytes < %d", scratch_bytes, SCR_ENDS_SCRATCH_BYTES);
    if (!scr_aligned16(residual) || !scr_aligned16(gain) || !scr_aligned16(normed) || !scr_aligned16(scratch))
        return scr_fail(ctx, SCR_E_ALIGN, "fused residual + norm epilogue: pointers must be 16-byte aligned");
    const GemvEnds ends = {residual, gain, normed, static_cast<float*>(scratch), eps};
    AffineFwd f;
    f.out_mode = GEMV_OUT_RESIDUAL_NORM;
    f.ends = &ends;
    // y is not written in this mode; the residual buffer stands in for the (unused) output pointer
    return affine_forward(ctx, packed, x, M, N, K, group, residual, f, nullptr, 0, (cudaStream_t)stream_);
}

extern "C" int32_t scr_linear_affine_b4_silu_mul(scr_ctx* ctx, const void* packed, const uint16_t* x, int32_t M, int32_t N2,
                                                 int32_t K, int32_t group, uint16_t* out, void* stream_) {
    SCR_REQUIRE_CTX(ctx);
    if (M > 16) return scr_fail(ctx, SCR_E_UNSUPPORTED, "fused silu*up epilogue: M=%d (the matvec path, M <= 16, has it)", M);
    if (N2 <= 0 || N2 % 16 != 0) return scr_fail(ctx, SCR_E_SHAPE, "fused silu*up epilogue: %d fused rows (8 gate + 8 up per block)", N2);
    AffineFwd f;
    f.out_mode = GEMV_OUT_SILU_PAIRS;
    return affine_forward(ctx, packed, x, M, N2, K, group, out, f, nullptr, 0, (cudaStream_t)stream_);
}

// ------------------------------------------------------------------------------------
// Matvec tape: a static list of M <= 16 linears with declared dependencies, one launch.
//
// The reference runs a decode step as a tape of operators fixed at build time
// (crates/targets/metal/src/tape/step.rs); here the linears of such a tape run inside ONE
// persistent cooperative kernel, so that no launch boundary (about 3 us of fixed cost each at these
// sizes) sits between dependent matvecs.  Every CTA walks the jobs in tape order.  Row-blocks are
// dealt round-robin, continuing across jobs, so that small jobs land on different CTAs.  The
// producer lane never waits for anything but ring space: weights are load-time constants, and it
// streams the next jobs' weights while the consumers wait for a dependency.  Consumers wait
// (bounded) until the jobs named in dep[] have stored all their row-blocks — a counter per job,
// bumped with release semantics once per CTA and job — and read activations with ordinary coherent
// loads, never the read-only path (another CTA of this launch may have written them).  The last CTA to leave zeroes the counters,
// so the tape can be replayed from a CUDA graph.  Summation order is fixed: results are
// deterministic and do not depend on which CTA took which row-block.
// ------------------------------------------------------------------------------------
#define TAPE_MAX_DEPS 3
#define TAPE_WAIT_LIMIT (1u << 22)
#define TAPE_ERR_DEP_WAIT 0x0D000001

struct TapeJob {
    const uint8_t* packed;
    const uint16_t* x;
    uint16_t* y;
    int N, K, KC, rb_real;
    int unit_base;                 // row-blocks of all earlier jobs (where the round-robin deal continues)
    int check;                     // the matrix has groups that need the exact (two-step rounding) path
    int dep[TAPE_MAX_DEPS];        // earlier jobs this one waits for (-1 = none)
    int dep_need[TAPE_MAX_DEPS];   // their row-block counts
    int pad[2];
};
static_assert(sizeof(TapeJob) % 16 == 0, "the job table is copied into shared memory 16 bytes at a time");

struct scr_tape {
    scr_ctx* ctx = nullptr;
    int n_jobs = 0;
    int max_rows = 0;              // largest M the x / y buffers were declared for
    TapeJob* jobs = nullptr;       // device
    unsigned int* done = nullptr;  // device: [n_jobs] row-blocks stored per job, [n_jobs] = CTAs that left
    int grid[2] = {0, 0};          // co-resident CTAs: up to 8 rows, up to 16 rows
};

__device__ __forceinline__ void tape_red_release(unsigned int* p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One row-block of one job: the k loop over the ring, the cross-warp sum and the bf16 store.
template <int MT, bool CHECK>
__device__ __forceinline__ void tape_row_block(uint16_t* __restrict__ y, int N, int K, int KC, int rb, int M, int nstage, uint32_t& n_it, int buf,
                                               const uint16_t* const (&xrow)[MT], int* __restrict__ status, uint32_t ring_base,
                                               uint32_t full_base, uint32_t empty_base, float (*red)[GEMV_CWARPS][32][MT * 4]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = lane & 3;
    float acc[2][MT][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[a][mt][i] = 0.f;
#pragma unroll 1
    for (int j = 0; j < nstage; ++j, ++n_it) {
        const int kc = j * GEMV_CWARPS + warp;
        const bool active = kc < KC;
        const uint32_t slot = n_it & (GEMV_STAGES - 1);
        uint4 xv[MT][4];
        int k0 = kc * 128 + t * 32;
        if (k0 >= K) k0 = 0;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[mt][i] = tape_ld_v4(xrow[mt] + k0 + 8 * i);
        gemv_wait(full_base + 8u * slot, (n_it / GEMV_STAGES) & 1u, status);
        if (active) gemv_block_compute<MT, CHECK>(ring_base + slot * GEMV_STAGE_BYTES + warp * AFF_BLOCK_BYTES, acc, xv, lane);
        __syncwarp();
        if (lane == 0) gemv_mbar_arrive(empty_base + 8u * slot);
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i)
            red[buf][warp][lane][mt * 4 + i] = (acc[0][mt][i] + acc[1][mt][i]) * (CHECK ? 1.0f : AFF_SCALED_FACTOR);
    gemv_consumer_sync();
    constexpr int SLOTS = 32 * MT * 4;
    const int e = threadIdx.x;
    if (e < SLOTS) {
        const int ln = e / (MT * 4), idx = e % (MT * 4);
        const int row = (ln >> 2) + (((idx & 3) >> 1) ? 8 : 0);
        const int tok = (idx >> 2) * 8 + (ln & 3) * 2 + (idx & 1);
        const int n = rb * 16 + row;
        float total = 0.f;
#pragma unroll
        for (int wdx = 0; wdx < GEMV_CWARPS; ++wdx) total += red[buf][wdx][ln][idx];
        if (tok < M && n < N) {
            const __nv_bfloat16 v = __float2bfloat16_rn(total);
            y[(size_t)tok * N + n] = *reinterpret_cast<const uint16_t*>(&v);
        }
    }
}

// The job table is copied into shared memory once (a record read from global memory at every job boundary
// stalls the single producer lane for a memory round trip while the ring behind it drains).
template <int MT>
__global__ void __launch_bounds__(GEMV_THREADS, (MT == 1 ? 3 : 2))
affine_b4_tape_kernel(const TapeJob* __restrict__ jobs_g, int n_jobs, int M, unsigned int* done, int* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t gemv_ring[];          // [GEMV_STAGES][8 blocks], then the job table
    __shared__ __align__(8) uint64_t full_bar[GEMV_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[GEMV_STAGES];
    __shared__ float red[2][GEMV_CWARPS][32][MT * 4];
    __shared__ int s_last;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    TapeJob* jobs = reinterpret_cast<TapeJob*>(gemv_ring + GEMV_STAGES * GEMV_STAGE_BYTES);
    {
        const uint4* src = reinterpret_cast<const uint4*>(jobs_g);
        uint4* dst = reinterpret_cast<uint4*>(jobs);
        const int n16 = n_jobs * int(sizeof(TapeJob) / 16);
        for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
    }
    if (threadIdx.x == 0) {
#pragma unroll
        for (int d = 0; d < GEMV_STAGES; ++d) {
            gemv_mbar_init(gemv_smem_u32(&full_bar[d]), 1);
            gemv_mbar_init(gemv_smem_u32(&empty_bar[d]), GEMV_CWARPS);
        }
        s_last = 0;
    }
    gemv_fence_mbar_init();
    __syncthreads();
    const uint32_t ring_base = gemv_smem_u32(gemv_ring);
    const uint32_t full_base = gemv_smem_u32(&full_bar[0]);
    const uint32_t empty_base = gemv_smem_u32(&empty_bar[0]);
    const int G = int(gridDim.x), c = int(blockIdx.x);

    if (warp == GEMV_CWARPS) {
        if (lane == 0) {
            // ---- weights: never waits for anything but ring space
            uint32_t n_it = 0;
            for (int j = 0; j < n_jobs; ++j) {
                const TapeJob& job = jobs[j];
                const int KC = job.KC, rb_real = job.rb_real;
                const int nstage = (KC + GEMV_CWARPS - 1) / GEMV_CWARPS;
                const int first = (c - job.unit_base % G + G) % G;
                for (int rb = first; rb < rb_real; rb += G) {
                    const uint8_t* src = job.packed + (size_t)rb * KC * AFF_BLOCK_BYTES;
                    for (int s = 0; s < nstage; ++s, ++n_it) {
                        const uint32_t slot = n_it & (GEMV_STAGES - 1);
                        gemv_wait(empty_base + 8u * slot, ((n_it / GEMV_STAGES) & 1u) ^ 1u, status);
                        const uint32_t bytes = (uint32_t)min(GEMV_CWARPS, KC - s * GEMV_CWARPS) * AFF_BLOCK_BYTES;
                        gemv_arrive_expect_tx(full_base + 8u * slot, bytes);
                        gemv_bulk_g2s(ring_base + slot * GEMV_STAGE_BYTES, src + (size_t)s * GEMV_STAGE_BYTES, bytes,
                                      full_base + 8u * slot);
                    }
                }
            }
        }
        __syncwarp();
    } else {
        const int g = lane >> 2;
        uint32_t n_it = 0;
        int it = 0;
        for (int j = 0; j < n_jobs; ++j) {
            const TapeJob& job = jobs[j];
            const int rb_real = job.rb_real;
            const int first = (c - job.unit_base % G + G) % G;
            if (first >= rb_real) continue;                    // no row-block of this job here: nothing to wait for or to report
            const int N = job.N, K = job.K, KC = job.KC;
            const bool has_dep = job.dep[0] >= 0 || job.dep[1] >= 0 || job.dep[2] >= 0;
            // one poller per CTA (thousands of pollers on one word starve the writers), with a short back-off
            if (threadIdx.x == 0 && has_dep) {
#pragma unroll 1
                for (int d = 0; d < TAPE_MAX_DEPS; ++d) {
                    const int dep = job.dep[d];
                    if (dep < 0) continue;
                    const unsigned int need = (unsigned int)job.dep_need[d];
                    const volatile unsigned int* ctr = done + dep;
                    bool seen = false;
                    for (unsigned int p = 0; p < TAPE_WAIT_LIMIT; ++p) {
                        if (*ctr >= need) {
                            seen = true;
                            break;
                        }
                        if ((p & 1023u) == 1023u && *reinterpret_cast<volatile int*>(status) != 0) break;
                        __nanosleep(20);
                    }
                    if (!seen) atomicCAS(status, 0, TAPE_ERR_DEP_WAIT);
                }
                __threadfence();                               // acquire: the producers' stores are visible from here on
            }
            if (has_dep) gemv_consumer_sync();
            const bool check = job.check != 0;
            uint16_t* y = job.y;
            const uint16_t* xrow[MT];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) xrow[mt] = job.x + (size_t)min(mt * 8 + g, M - 1) * K;
            const int nstage = (KC + GEMV_CWARPS - 1) / GEMV_CWARPS;
            unsigned int units = 0;
            for (int rb = first; rb < rb_real; rb += G, ++it, ++units) {
                if (check)
                    tape_row_block<MT, true>(y, N, K, KC, rb, M, nstage, n_it, it & 1, xrow, status, ring_base, full_base, empty_base, red);
                else
                    tape_row_block<MT, false>(y, N, K, KC, rb, M, nstage, n_it, it & 1, xrow, status, ring_base, full_base, empty_base, red);
            }
            gemv_consumer_sync();                              // every store of this CTA's row-blocks has been issued ...
            if (threadIdx.x == 0) tape_red_release(done + j, units);      // ... and is released, cumulatively, by this one
        }
    }
    // the last CTA to leave clears the counters for the next replay
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(done + n_jobs, 1u) == (unsigned int)(G - 1)) s_last = 1;
    }
    __syncthreads();
    if (s_last) {
        for (int i = threadIdx.x; i <= n_jobs; i += blockDim.x) done[i] = 0u;
    }
}

#define TAPE_MAX_JOBS 320          // the job table sits in shared memory beside the ring

static size_t tape_smem_bytes(int n_jobs) { return (size_t)GEMV_STAGES * GEMV_STAGE_BYTES + (size_t)n_jobs * sizeof(TapeJob); }

template <int MT>
static int tape_resident_ctas(int sms, int n_jobs) {
    int per_sm = 0;
    const size_t kRingBytes = tape_smem_bytes(n_jobs);
    if (cudaFuncSetAttribute(affine_b4_tape_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tape_smem_bytes(TAPE_MAX_JOBS)) !=
        cudaSuccess)
        return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, affine_b4_tape_kernel<MT>, GEMV_THREADS, kRingBytes) != cudaSuccess)
        return 0;
    return std::min(per_sm, MT == 1 ? 3 : 2) * sms;
}

extern "C" int32_t scr_affine_b4_tape_create(scr_ctx* ctx, const scr_tape_linear* jobs, int32_t n_jobs, int32_t max_rows,
                                             scr_tape** out) {
    SCR_REQUIRE_CTX(ctx);
    if (!jobs || !out) return scr_fail(ctx, SCR_E_ARG, "tape: null pointer");
    *out = nullptr;
    if (n_jobs <= 0) return scr_fail(ctx, SCR_E_SHAPE, "tape: %d jobs", n_jobs);
    if (n_jobs > TAPE_MAX_JOBS) return scr_fail(ctx, SCR_E_UNSUPPORTED, "tape: %d jobs (up to %d per tape; chain several)", n_jobs, TAPE_MAX_JOBS);
    if (max_rows <= 0 || max_rows > 16) return scr_fail(ctx, SCR_E_UNSUPPORTED, "tape: max_rows=%d (the matvec path, 1..16 rows)", max_rows);
    std::vector<TapeJob> host((size_t)n_jobs);
    long long unit_base = 0;
    for (int j = 0; j < n_jobs; ++j) {
        const scr_tape_linear& s = jobs[j];
        if (!s.packed || !s.x || !s.y) return scr_fail(ctx, SCR_E_ARG, "tape job %d: null pointer", j);
        int32_t st = affine_check_shape(ctx, s.N, s.K, s.group);
        if (st) return st;
        if (!scr_aligned16(s.packed) || !scr_aligned16(s.x)) return scr_fail(ctx, SCR_E_ALIGN, "tape job %d: packed/x must be 16-byte aligned", j);
        if (s.group == 32) return scr_fail(ctx, SCR_E_UNSUPPORTED, "tape job %d: the tape kernel is built for groups of 64 and 128", j);
        const AffineGeom g = affine_geom(s.N, s.K, s.group);
        TapeJob& t = host[(size_t)j];
        t.packed = static_cast<const uint8_t*>(s.packed);
        t.x = s.x;
        t.y = s.y;
        t.N = s.N;
        t.K = s.K;
        t.KC = g.KC;
        t.rb_real = scr_ceil_div(s.N, 16);
        t.unit_base = int(unit_base % (1 << 30));
        unit_base += t.rb_real;
        unsigned int flag = 0;
        cudaError_t e = cudaMemcpy(&flag, t.packed + affine_blocks_bytes(g), sizeof(flag), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "tape job %d: reading the matrix trailer: %s", j, cudaGetErrorString(e));
        t.check = flag != 0;
        for (int d = 0; d < TAPE_MAX_DEPS; ++d) {
            const int dep = s.dep[d];
            if (dep >= j) return scr_fail(ctx, SCR_E_ARG, "tape job %d: dependency %d is not an earlier job", j, dep);
            t.dep[d] = dep < 0 ? -1 : dep;
            t.dep_need[d] = dep < 0 ? 0 : host[(size_t)dep].rb_real;
        }
    }
    scr_tape* tp = new (std::nothrow) scr_tape();
    if (!tp) return scr_fail(ctx, SCR_E_CUDA, "tape: out of host memory");
    tp->ctx = ctx;
    tp->n_jobs = n_jobs;
    tp->max_rows = max_rows;
    tp->grid[0] = tape_resident_ctas<1>(ctx->sm_count, n_jobs);
    tp->grid[1] = tape_resident_ctas<2>(ctx->sm_count, n_jobs);
    cudaError_t e = tp->grid[0] > 0 && tp->grid[1] > 0 ? cudaSuccess : cudaErrorLaunchOutOfResources;
    if (e == cudaSuccess) e = cudaMalloc(&tp->jobs, sizeof(TapeJob) * (size_t)n_jobs);
    if (e == cudaSuccess) e = cudaMalloc(&tp->done, sizeof(unsigned int) * ((size_t)n_jobs + 1));
    if (e == cudaSuccess) e = cudaMemcpy(tp->jobs, host.data(), sizeof(TapeJob) * (size_t)n_jobs, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(tp->done, 0, sizeof(unsigned int) * ((size_t)n_jobs + 1));
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        if (tp->jobs) cudaFree(tp->jobs);
        if (tp->done) cudaFree(tp->done);
        delete tp;
        return scr_fail(ctx, SCR_E_CUDA, "tape: %s", cudaGetErrorString(e));
    }
    *out = tp;
    return SCR_OK;
}

extern "C" int32_t scr_tape_destroy(scr_tape* tape) {
    if (!tape) return SCR_OK;
    if (tape->jobs) cudaFree(tape->jobs);
    if (tape->done) cudaFree(tape->done);
    delete tape;
    return SCR_OK;
}

extern "C" int32_t scr_linear_affine_b4_tape(scr_ctx* ctx, scr_tape* tape, int32_t M, void* stream_) {
    SCR_REQUIRE_CTX(ctx);
    if (!tape || tape->ctx != ctx) return scr_fail(ctx, SCR_E_ARG, "tape: null handle or a handle of another context");
    if (M <= 0 || M > tape->max_rows) return scr_fail(ctx, SCR_E_SHAPE, "tape: M=%d outside 1..%d", M, tape->max_rows);
    const size_t kRingBytes = tape_smem_bytes(tape->n_jobs);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tape->grid[M > 8 ? 1 : 0], 1, 1);
    cfg.blockDim = dim3(GEMV_THREADS, 1, 1);
    cfg.dynamicSmemBytes = kRingBytes;
    cfg.stream = (cudaStream_t)stream_;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;       // every CTA resident: a CTA may wait for any other
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const TapeJob* jobs = tape->jobs;
    cudaError_t e = M <= 8 ? cudaLaunchKernelEx(&cfg, affine_b4_tape_kernel<1>, jobs, tape->n_jobs, (int)M, tape->done, ctx->dev_status)
                           : cudaLaunchKernelEx(&cfg, affine_b4_tape_kernel<2>, jobs, tape->n_jobs, (int)M, tape->done, ctx->dev_status);
    if (e != cudaSuccess) return scr_fail(ctx, SCR_E_CUDA, "affine_b4_tape launch: %s", cudaGetErrorString(e));
    return scr_check_launch(ctx, "affine_b4_tape");
}
