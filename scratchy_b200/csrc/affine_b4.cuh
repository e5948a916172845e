// MLX affine int4 (groups of 64; 32 and 128 below): the streaming layout and the one dequantisation routine
// every kernel shares (matvec, tensor-core GEMM, the dump hook), so a weight has the
// same bf16 value wherever it is expanded.
//
// Arithmetic contract (crates/models/quantization/src/affine.rs:120-132 of the reference):
//   w = bf16_rne( f32( f32(scale) * f32(code) + f32(bias) ) )
// The f32 product of a bf16 scale (8 significant bits) and a 4-bit code is exact, so the
// f32 stage rounds once (the add) and the bf16 conversion rounds a second time.
//
// Packed path: one `fma.rn.bf16x2` computes the exact scale*code + bias and rounds ONCE to
// bf16.  That equals the reference's two-step rounding unless the f32 stage is inexact and
// lands on a bf16 half-way point, which needs 0 < |bias| < 2^-13 |scale| (the bias entirely
// below f32's window under the product).  Groups whose (scale, bias) could do that, or that
// hold a value tiny enough for flush-to-zero to matter, take the exact f32 path instead
// (`affine_slow_group`).
//
// Two packed variants exist.  The generic one builds 128 + code with a mask-or, subtracts 128
// and tests every group for the exact path.  The scaled one is used when the repack kernel
// found no group that needs the exact path and every scale below 2 in magnitude (trailer flag
// == 0): a code left in place in bits [0,4) or [4,8) of a 16-bit half IS the bf16 number
// code * 2^-133 (resp. 16 * code * 2^-133, the subnormal/first-binade range is linear in the
// low 8 bits), so fma(scale * 2^126 [or 2^122], bits, bias * 2^-7) = w * 2^-7 with the same
// single rounding; the factor 2^7 is applied, exactly, to the f32 accumulator afterwards.
//
// Streaming layout ("blocks"), produced once at load time by the repack kernel:
//   N is padded to a multiple of 128 rows and K to a multiple of 128; a block covers
//   16 rows x 128 k and is 1152 bytes; block (rb, kc) sits at ((rb * KC) + kc) * 1152
//   with KC = K_pad / 128, i.e. row-block-major: the whole k extent of 16 rows is one
//   contiguous run, which the decode matvec streams with a few large bulk copies.
//   bytes [   0, 512): half 0 = rows 16rb + g,     piece `lane = 4g + t` (16 bytes) holds the
//   bytes [ 512,1024): half 1 = rows 16rb + 8 + g  32 codes k = 128kc + 32t + [0,32) of its row
//   bytes [1024,1152): for (g, h = 0..1): 8 bytes at 1024 + (2g + h) * 8 =
//                      { scale, bias of row g, group 2kc + h ; scale, bias of row g + 8 } (bf16)
//   Inside a piece, word i holds codes e0..e7 = k-offsets 8i..8i+7 with e_{2j} at bits
//   [4j, 4j+4) and e_{2j+1} at bits [16+4j, 16+4j+4): `(word >> 4j) & 0x000F000F` is then
//   the pair (e_{2j}, e_{2j+1}) in the two 16-bit halves, in natural order.
//   Padding rows / k hold code 0, scale 0, bias 0, which dequantise to exactly 0.
//   A 128-byte trailer follows the blocks; its first word is non-zero when some group of the
//   matrix needs the exact path (set by the repack kernel), so the kernels test one word per
//   launch instead of every group.
#pragma once

#include "common.cuh"

#define AFF_BLOCK_BYTES 1152
// Group sizes 32 and 128 (the reference's sibling presets, crates/compiler/subtile/src/lower.rs:112-127) use the same block
// of 16 rows x 128 k.  A lane's 16-byte piece (32 codes) never crosses a group, whichever of the three sizes, so only the
// number of (scale, bias) entries per row and block differs: 2^gs.  Group 128 keeps gs = 1 (its one entry per row is
// stored twice, so every kernel written for group 64 runs it unchanged); group 32 has gs = 2: 4 entries per row, a
// 1280-byte block, entry of (row g, piece t) at 1024 + (g * 4 + t) * 8.
__host__ __device__ constexpr int aff_block_bytes(int gs) { return 1024 + (64 << gs); }
static inline int affine_gs(int group) { return group == 32 ? 2 : 1; }
#define AFF_BLOCK_ROWS 16
#define AFF_BLOCK_K 128
#define AFF_ROW_PAD 128
#define AFF_TRAILER_BYTES 128

struct AffineGeom {
    int N, K;        // logical
    int RB;          // row blocks (N_pad / 16)
    int KC;          // k chunks (ceil(K / 128))
    int gs;          // log2 of the (scale, bias) entries per row and block: 1 (groups of 64 and 128) or 2 (groups of 32)
};

static inline AffineGeom affine_geom(int N, int K, int group) {
    AffineGeom g;
    g.N = N; g.K = K;
    g.gs = affine_gs(group);
    g.RB = scr_ceil_div(N, AFF_ROW_PAD) * (AFF_ROW_PAD / AFF_BLOCK_ROWS);
    g.KC = scr_ceil_div(K, AFF_BLOCK_K);
    return g;
}
static inline size_t affine_blocks_bytes(const AffineGeom& g) { return (size_t)g.RB * g.KC * aff_block_bytes(g.gs); }
static inline size_t affine_packed_bytes(const AffineGeom& g) { return affine_blocks_bytes(g) + AFF_TRAILER_BYTES; }

// True when the packed-bf16 fast path could differ from the reference's two-step rounding
// (see the header comment) or would involve bf16/f32 subnormals.
__host__ __device__ __forceinline__ bool affine_slow_group(uint32_t sb /* scale | bias << 16 */) {
    const uint32_t s = sb & 0x7FFFu, b = (sb >> 16) & 0x7FFFu;      // magnitudes, sign stripped
    const int es = int(s >> 7), eb = int(b >> 7);                    // biased exponents
    const bool tiny = (s != 0 && es < 20) || (b != 0 && eb < 20);
    const bool far_apart = (b != 0 && s != 0 && eb + 12 < es);       // |b| < 2^-12 |s| (conservative)
    const bool special = (es == 255) || (eb == 255);                 // inf / nan: take the exact path
    return tiny || far_apart || special;
}

// Exact reference arithmetic for one word (8 codes) -> 4 bf16x2 registers in natural order.
// Out of line and returning by value, so the common path keeps everything in registers.
static __device__ __noinline__ uint4 affine_dequant_word_exact(uint32_t word, uint32_t sb) {
    const float s = __uint_as_float((sb & 0xFFFFu) << 16);
    const float b = __uint_as_float(sb & 0xFFFF0000u);
    uint32_t out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float q0 = float((word >> (4 * j)) & 0xF);
        const float q1 = float((word >> (16 + 4 * j)) & 0xF);
        const float w0 = __fadd_rn(__fmul_rn(s, q0), b);
        const float w1 = __fadd_rn(__fmul_rn(s, q1), b);
        const __nv_bfloat162 p = __floats2bfloat162_rn(w0, w1);     // .x = low half = w0
        out[j] = *reinterpret_cast<const uint32_t*>(&p);
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

// One word (8 codes) -> 4 bf16x2 registers, natural order.  `s2`/`b2` hold the group's scale
// and bias duplicated in both halves.
__device__ __forceinline__ void affine_dequant_word_fast(uint32_t word, uint32_t s2, uint32_t b2, uint32_t out[4]) {
    const __nv_bfloat162 s = *reinterpret_cast<const __nv_bfloat162*>(&s2);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&b2);
    const uint32_t magic = 0x43004300u;                              // bf16 128.0 in both halves
    const __nv_bfloat162 m128 = *reinterpret_cast<const __nv_bfloat162*>(&magic);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t q = ((word >> (4 * j)) & 0x000F000Fu) | magic;      // (128 + code) in each half, exact
        __nv_bfloat162 qf = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&q), m128);   // exact: code
        __nv_bfloat162 w = __hfma2(s, qf, b);                        // fused, one rounding to bf16
        out[j] = *reinterpret_cast<const uint32_t*>(&w);
    }
}

// True when the scaled variant must not be used for this group.
__host__ __device__ __forceinline__ bool affine_group_needs_generic(uint32_t sb) {
    const uint32_t s = sb & 0x7FFFu;
    return affine_slow_group(sb) || (s != 0 && int(s >> 7) > 127);
}

// Scaled variant: the group's constants, made once per 16-byte piece.
struct AffineScaled {
    uint32_t s_lo;    // scale * 2^126 in both halves (codes in bits [0,4) of a half)
    uint32_t s_hi;    // scale * 2^122 in both halves (codes in bits [4,8) of a half)
    uint32_t b7;      // bias * 2^-7 in both halves
};
__device__ __forceinline__ AffineScaled affine_scaled_consts(uint32_t sb) {
    const uint32_t s2 = __byte_perm(sb, sb, 0x1010), b2 = __byte_perm(sb, sb, 0x3232);
    const uint32_t k126 = 0x7E807E80u, k122 = 0x7C807C80u, km7 = 0x3C003C00u;   // 2^126, 2^122, 2^-7 as bf16x2
    const __nv_bfloat162 s = *reinterpret_cast<const __nv_bfloat162*>(&s2);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&b2);
    const __nv_bfloat162 a = __hmul2(s, *reinterpret_cast<const __nv_bfloat162*>(&k126));
    const __nv_bfloat162 c = __hmul2(s, *reinterpret_cast<const __nv_bfloat162*>(&k122));
    const __nv_bfloat162 d = __hmul2(b, *reinterpret_cast<const __nv_bfloat162*>(&km7));
    AffineScaled r;
    r.s_lo = *reinterpret_cast<const uint32_t*>(&a);
    r.s_hi = *reinterpret_cast<const uint32_t*>(&c);
    r.b7 = *reinterpret_cast<const uint32_t*>(&d);
    return r;
}
// One word (8 codes) -> 4 bf16x2 registers holding w * 2^-7, natural k order.
__device__ __forceinline__ void affine_dequant_word_scaled(uint32_t word, const AffineScaled& c, uint32_t out[4]) {
    const __nv_bfloat162 s_lo = *reinterpret_cast<const __nv_bfloat162*>(&c.s_lo);
    const __nv_bfloat162 s_hi = *reinterpret_cast<const __nv_bfloat162*>(&c.s_hi);
    const __nv_bfloat162 b7 = *reinterpret_cast<const __nv_bfloat162*>(&c.b7);
    const uint32_t w8 = word >> 8;
    const uint32_t q0 = word & 0x000F000Fu, q1 = word & 0x00F000F0u;
    const uint32_t q2 = w8 & 0x000F000Fu, q3 = w8 & 0x00F000F0u;
    const __nv_bfloat162 r0 = __hfma2(s_lo, *reinterpret_cast<const __nv_bfloat162*>(&q0), b7);
    const __nv_bfloat162 r1 = __hfma2(s_hi, *reinterpret_cast<const __nv_bfloat162*>(&q1), b7);
    const __nv_bfloat162 r2 = __hfma2(s_lo, *reinterpret_cast<const __nv_bfloat162*>(&q2), b7);
    const __nv_bfloat162 r3 = __hfma2(s_hi, *reinterpret_cast<const __nv_bfloat162*>(&q3), b7);
    out[0] = *reinterpret_cast<const uint32_t*>(&r0);
    out[1] = *reinterpret_cast<const uint32_t*>(&r1);
    out[2] = *reinterpret_cast<const uint32_t*>(&r2);
    out[3] = *reinterpret_cast<const uint32_t*>(&r3);
}
#define AFF_SCALED_FACTOR 128.0f      // multiply accumulators of scaled weights by this (exact)

// One word with the group's pre-duplicated scale / bias; `slow` (evaluated once per group by the
// caller, only when the matrix's trailer flag is set) selects the exact path.
template <bool CHECK>
__device__ __forceinline__ void affine_dequant_word(uint32_t word, uint32_t sb, uint32_t s2, uint32_t b2, bool slow,
                                                    uint32_t out[4]) {
    if (CHECK && slow) {
        const uint4 r = affine_dequant_word_exact(word, sb);
        out[0] = r.x; out[1] = r.y; out[2] = r.z; out[3] = r.w;
    } else {
        affine_dequant_word_fast(word, s2, b2, out);
    }
}

// A 16-byte piece (32 codes of one row, one group) -> 16 bf16x2 registers in k order.
// CHECK = false is for matrices whose trailer flag says no group needs the exact path.
template <bool CHECK>
__device__ __forceinline__ void affine_dequant_piece(const uint4& piece, uint32_t sb, uint32_t out[16]) {
    if (CHECK && affine_slow_group(sb)) {
        const uint4 r0 = affine_dequant_word_exact(piece.x, sb);
        const uint4 r1 = affine_dequant_word_exact(piece.y, sb);
        const uint4 r2 = affine_dequant_word_exact(piece.z, sb);
        const uint4 r3 = affine_dequant_word_exact(piece.w, sb);
        out[0] = r0.x; out[1] = r0.y; out[2] = r0.z; out[3] = r0.w;
        out[4] = r1.x; out[5] = r1.y; out[6] = r1.z; out[7] = r1.w;
        out[8] = r2.x; out[9] = r2.y; out[10] = r2.z; out[11] = r2.w;
        out[12] = r3.x; out[13] = r3.y; out[14] = r3.z; out[15] = r3.w;
    } else {
        const uint32_t s2 = __byte_perm(sb, sb, 0x1010);             // scale in both halves
        const uint32_t b2 = __byte_perm(sb, sb, 0x3232);             // bias in both halves
        affine_dequant_word_fast(piece.x, s2, b2, out + 0);
        affine_dequant_word_fast(piece.y, s2, b2, out + 4);
        affine_dequant_word_fast(piece.z, s2, b2, out + 8);
        affine_dequant_word_fast(piece.w, s2, b2, out + 12);
    }
}
