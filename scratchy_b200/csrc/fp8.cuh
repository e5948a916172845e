// fp8-dynamic-per-channel: layouts and the device e4m3 encoder shared by the kernels.
//
// Weight pack (written once at load time): N padded to 128 rows, K padded to 128; tile
// (nt, kt) of 128 rows x 128 k bytes is 16384 bytes at ((nt * KT) + kt) * 16384 and is the
// exact shared-memory image a K-major, 128-byte-swizzled tcgen05 operand wants, so a tile
// needs one bulk copy and no tensor map:
//     byte(r, c) = (r / 8) * 1024 + (r % 8) * 128 + (((c / 16) ^ (r % 8)) * 16) + (c % 16)
// The per-channel f32 scales [N_pad] follow the tiles.  Padding is e4m3 zero / scale 0.
//
// Activation pack: [0, align128(4*M)) holds a_scale[M] (f32), then x_q:
//   plain  (M <= 16, matvec path)  : [M][K16] bytes, K16 = K rounded up to 16, row-major
//   tiled  (M  > 16, GEMM path)    : for each k-tile kt: [M_pad128 rows x 128 bytes] in the
//                                    same swizzled image as the weights (row = token)
#pragma once

#include "common.cuh"

#define FP8_TILE 128
#define FP8_TILE_BYTES 16384

struct Fp8Geom {
    int N, K, NT, KT;
};
static inline Fp8Geom fp8_geom(int N, int K) {
    Fp8Geom g;
    g.N = N; g.K = K;
    g.NT = scr_ceil_div(N, FP8_TILE);
    g.KT = scr_ceil_div(K, FP8_TILE);
    return g;
}
static inline size_t fp8_weight_bytes(int N, int K) {
    const Fp8Geom g = fp8_geom(N, K);
    return (size_t)g.NT * g.KT * FP8_TILE_BYTES + (size_t)g.NT * FP8_TILE * sizeof(float);
}

bool fp8_gemm_tc_enabled();
static inline bool fp8_act_tiled(int M) { return M > 16 && fp8_gemm_tc_enabled(); }
static inline size_t fp8_act_scale_bytes(int M) { return ((size_t)M * 4 + 127) / 128 * 128; }
static inline size_t fp8_act_bytes(int M, int K) {
    if (fp8_act_tiled(M))
        return fp8_act_scale_bytes(M) + (size_t)scr_ceil_div(K, FP8_TILE) * scr_ceil_div(M, FP8_TILE) * FP8_TILE_BYTES;
    return fp8_act_scale_bytes(M) + (size_t)M * (size_t)(scr_ceil_div(K, 16) * 16);
}

__host__ __device__ __forceinline__ uint32_t fp8_swizzled_offset(int r, int c) {
    return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((((c >> 4) ^ (r & 7)) << 4) | (c & 15)));
}

// f32 -> float8_e4m3fn with the reference encoder's rule
// (backends/spyre/crates/ktir/ktir-core/src/codec.rs:1023-1070 of the reference):
// nearest, half-way cases AWAY from zero, [448,464) -> 448, >= 464 -> the NaN encoding,
// below 2^-6 the grid is 2^-9.  Integer arithmetic on the f32 bits, no rounding-mode
// dependence.
__device__ __forceinline__ uint32_t e4m3_encode_ref(float v) {
    const uint32_t u = __float_as_uint(v);
    const uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return 0x7Fu;                       // NaN (the reference drops the sign)
    const uint32_t sign = (u >> 24) & 0x80u;
    if (a >= 0x43E80000u) return sign | 0x7Fu;               // >= 464
    if (a >= 0x43E00000u) return sign | 0x7Eu;               // [448, 464)
    if (a < 0x3C800000u) {                                   // < 2^-6: subnormal grid
        const float t = __uint_as_float(a) * 512.0f;         // exact (power-of-two scaling)
        int q = (int)t;                                      // truncation, t in [0, 8)
        if (t - (float)q >= 0.5f) ++q;                       // half away from zero; q <= 8
        return sign | (uint32_t)q;
    }
    uint32_t e = ((a + 0x00080000u) >> 20) - (120u << 3);    // round mantissa to 3 bits, carry into exponent
    if (e > 0x7Eu) e = 0x7Eu;
    return sign | e;
}
