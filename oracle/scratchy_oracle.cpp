// CPU oracle for the quantized-linear hot path. TEST INFRASTRUCTURE ONLY.
//
// This file restates, in plain C++ (OpenMP over output elements only), the
// reference project's own host/test-oracle arithmetic for the two presets the
// CUDA library implements.  Nothing in the product path may call it: only the
// test-suite, the smoke check and the benchmark's CPU-baseline leg load the
// shared object built from this file.
//
// Parity status: PINNED for the int4 affine path and the e4m3 codec (checked
// against the reference's known-answer tests, restated as data in
// tests/test_oracle_kat.py); the end-to-end fp8 W8A8 numerics and the e4m3
// encoder's exact-tie rule are unpinned in the reference itself (it has no
// known-answer test for them), so for those the oracle follows the source line
// by line and the seeded vectors under tests/golden/ become the pin.
//
// Every function cites the reference file:line it follows (paths are relative
// to the reference project's root).
//
// Third-party arithmetic the reference relies on and that is not in its tree:
// the `half` crate 2.7.1 (Cargo.lock) for f32<->bf16/f16 conversion.  Its
// published behaviour is IEEE round-to-nearest-even with NaN quieting; the
// conversions below implement exactly that.

#include <cstdint>
#include <cstring>
#include <cmath>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline float bits_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }
inline uint32_t f32_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }

// half::bf16::to_f32 — exact widening.
inline float bf16_to_f32(uint16_t h) { return bits_f32(uint32_t(h) << 16); }

// half::bf16::from_f32 — round to nearest even, NaN quieted (sets the quiet bit,
// keeps the sign and the upper payload bits).
inline uint16_t f32_to_bf16(float f) {
    uint32_t x = f32_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return uint16_t((x >> 16) | 0x0040u);
    uint32_t round_bit = 0x00008000u;
    if ((x & round_bit) != 0 && (x & (3u * round_bit - 1u)) != 0) return uint16_t((x >> 16) + 1u);
    return uint16_t(x >> 16);
}

// half::f16 conversions — IEEE binary16, RNE.  gcc's _Float16 conversions are
// IEEE-correct (single rounding) on x86-64.
inline float f16_to_f32(uint16_t h) { _Float16 v; std::memcpy(&v, &h, 2); return float(v); }
inline uint16_t f32_to_f16(float f) { _Float16 v = (_Float16)f; uint16_t h; std::memcpy(&h, &v, 2); return h; }

enum { DT_F16 = 0, DT_BF16 = 1 };   // same discriminants as the reference's DType (tensors/src/dtype.rs:7-16)

inline float half_to_f32(uint16_t h, int dt) { return dt == DT_BF16 ? bf16_to_f32(h) : f16_to_f32(h); }
inline uint16_t f32_to_half(float f, int dt) { return dt == DT_BF16 ? f32_to_bf16(f) : f32_to_f16(f); }

}  // namespace

extern "C" {

// The bench's CPU arm runs under launchers that export OMP_NUM_THREADS=1 (torchrun does): it sets the
// thread count explicitly so that the baseline uses the host's cores whatever the environment says.
void orc_set_num_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
}

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
float orc_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

// ---------------------------------------------------------------------------
// int4 affine dequantisation.
//
// Follows crates/models/quantization/src/affine.rs:120-132 (the bits == 4 arm of
// `affine_dequant_b4_to_dtype`), which is also
// crates/targets/metal/src/cpu_reference.rs:69-98 (`affine_dequantize_b4`):
//   byte `offset` holds elements 2*offset (low nibble) and 2*offset+1 (high);
//   group index = element / group_size over the flattened [N, K] tensor;
//   out = round_to_out( f32(scale) * f32(code) + f32(bias) )   (f32 mul, f32 add).
//
// `cast_scale_to_act` != 0 reproduces cpu_reference.rs:90-91, which first narrows
// the scale and bias to the activation dtype; with bf16 scales and a bf16 output
// that is a no-op, and affine.rs never does it.
// ---------------------------------------------------------------------------
void orc_affine_dequant_b4(const uint8_t* packed, const uint16_t* scales, const uint16_t* biases,
                           int64_t n, int64_t k, int64_t group_size, int scale_dt, int out_dt,
                           int cast_scale_to_act, uint16_t* out) {
    const int64_t total = n * k;
#pragma omp parallel for schedule(static)
    for (int64_t offset = 0; offset < total / 2; ++offset) {
        const int64_t oindex = offset * 2;
        const int64_t gindex = oindex / group_size;
        float scale = half_to_f32(scales[gindex], scale_dt);
        float bias = half_to_f32(biases[gindex], scale_dt);
        if (cast_scale_to_act) {
            scale = half_to_f32(f32_to_half(scale, out_dt), out_dt);
            bias = half_to_f32(f32_to_half(bias, out_dt), out_dt);
        }
        const uint8_t byte = packed[offset];
        const float lo = float(byte & 0x0f);
        const float hi = float((byte >> 4) & 0x0f);
        // Two separate roundings (product, then sum) exactly as the Rust source
        // writes it; the build uses -ffp-contract=off so they are never fused.
        out[oindex] = f32_to_half(scale * lo + bias, out_dt);
        out[oindex + 1] = f32_to_half(scale * hi + bias, out_dt);
    }
}

// ---------------------------------------------------------------------------
// int4 affine linear, y = x @ dequant(W)^T.
//
// Follows crates/targets/metal/src/cpu_reference.rs:107-137 (`affine_qmm_t_b4`,
// entry points :478-489 for bf16 activations with bf16 scales, alias :524 for
// the matvec): dequantise W to the activation dtype, then for every output
// element accumulate `acc += f32(x[i,k]) * f32(w[j,k])` for k = 0..K-1 in order
// in f32 and round once.  Parallelism here is over (i, j) only, so each
// element's summation order is the reference's.
//
// `y_f32` (optional) receives the unrounded accumulators — the tensor-parallel
// oracle sums those over ranks before rounding.
// ---------------------------------------------------------------------------
void orc_affine_qmm_t_b4(const uint8_t* packed, const uint16_t* scales, const uint16_t* biases,
                         const uint16_t* x, int64_t m, int64_t n, int64_t k, int64_t group_size,
                         int scale_dt, int act_dt, uint16_t* y, float* y_f32) {
    std::vector<uint16_t> w(size_t(n) * size_t(k));
    orc_affine_dequant_b4(packed, scales, biases, n, k, group_size, scale_dt, act_dt, 1, w.data());
    std::vector<float> wf(size_t(n) * size_t(k));
    std::vector<float> xf(size_t(m) * size_t(k));
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n * k; ++i) wf[i] = half_to_f32(w[i], act_dt);
    for (int64_t i = 0; i < m * k; ++i) xf[i] = half_to_f32(x[i], act_dt);
    // Eight output columns advance together so the eight independent f32 chains
    // overlap; each chain still adds its K products in k order (compiled with
    // -ffp-contract=off and without -ffast-math, so no fusing or re-association).
    const int64_t JB = 8;
#pragma omp parallel for schedule(static)
    for (int64_t j0 = 0; j0 < n; j0 += JB) {
        const int64_t jb = std::min<int64_t>(JB, n - j0);
        for (int64_t i = 0; i < m; ++i) {
            const float* xr = xf.data() + i * k;
            float acc[JB] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (jb == JB) {
                const float* w0 = wf.data() + j0 * k;
                for (int64_t kk = 0; kk < k; ++kk) {
                    const float xv = xr[kk];
                    for (int64_t jj = 0; jj < JB; ++jj) acc[jj] += xv * w0[jj * k + kk];
                }
            } else {
                for (int64_t jj = 0; jj < jb; ++jj) {
                    const float* wr = wf.data() + (j0 + jj) * k;
                    for (int64_t kk = 0; kk < k; ++kk) acc[jj] += xr[kk] * wr[kk];
                }
            }
            for (int64_t jj = 0; jj < jb; ++jj) {
                if (y) y[i * n + j0 + jj] = f32_to_half(acc[jj], act_dt);
                if (y_f32) y_f32[i * n + j0 + jj] = acc[jj];
            }
        }
    }
}

// ---------------------------------------------------------------------------
// float8_e4m3fn codec.
//
// Decode follows backends/spyre/crates/ktir/ktir-core/src/codec.rs:991-1008
// (`e4m3_to_f32_compute`): 1 sign / 4 exponent (bias 7) / 3 mantissa, subnormal
// m * 2^-9, the only NaN is S.1111.111.
// ---------------------------------------------------------------------------
float orc_e4m3_to_f32(uint8_t byte) {
    const float sign = (byte & 0x80) ? -1.0f : 1.0f;
    const int exp = (byte >> 3) & 0x0F;
    const int mant = byte & 0x07;
    if (exp == 0x0F && mant == 0x07) return std::nanf("");
    float mag;
    if (exp == 0) mag = float(mant) * std::ldexp(1.0f, -9);
    else mag = (1.0f + float(mant) / 8.0f) * std::ldexp(1.0f, exp - 7);
    return sign * mag;
}

// Encode follows codec.rs:1023-1070 (`f32_to_e4m3`) statement by statement:
// NaN -> 0x7F; zero keeps its sign; [464, inf] -> NaN encoding; [448, 464) ->
// 0x7E; below 2^-6 the grid is 2^-9 and `(a*512).round()` is clamped to [0, 8];
// otherwise mantissa = `(frac*8).round()` with a carry into the exponent.
// Rust's f32::round rounds half-way cases AWAY from zero, which std::round does too.
uint8_t orc_f32_to_e4m3(float v) {
    if (std::isnan(v)) return 0x7F;
    const uint8_t sign = std::signbit(v) ? 0x80 : 0;
    const float a = std::fabs(v);
    if (a == 0.0f) return sign;
    if (a >= 464.0f) return sign | 0x7F;
    if (a >= 448.0f) return sign | 0x7E;
    if (a < 0.015625f) {
        int q = int(std::round(a * 512.0f));
        q = std::min(std::max(q, 0), 8);
        return sign | uint8_t(q);
    }
    int exp = int((f32_bits(a) >> 23) & 0xFF) - 127;
    const float frac = a / bits_f32(uint32_t(exp + 127) << 23) - 1.0f;
    int mant = int(std::round(frac * 8.0f));
    if (mant == 8) { mant = 0; exp += 1; }
    if (exp + 7 >= 0x0F && mant >= 7) return sign | 0x7E;
    return sign | uint8_t((exp + 7) << 3) | uint8_t(mant & 0x07);
}

// The same encoder with round-half-to-even at exact ties (what `cvt.rn` on NVIDIA
// hardware and torch do).  Not a reference function: reported beside the
// reference rule so the size of the tie-rule difference is visible.
uint8_t orc_f32_to_e4m3_rne(float v) {
    if (std::isnan(v)) return 0x7F;
    const uint8_t sign = std::signbit(v) ? 0x80 : 0;
    const float a = std::fabs(v);
    if (a == 0.0f) return sign;
    if (a >= 464.0f) return sign | 0x7F;
    if (a >= 448.0f) return sign | 0x7E;
    if (a < 0.015625f) {
        int q = int(std::nearbyint(a * 512.0f));   // default rounding mode: to nearest even
        q = std::min(std::max(q, 0), 8);
        return sign | uint8_t(q);
    }
    int exp = int((f32_bits(a) >> 23) & 0xFF) - 127;
    const float frac = a / bits_f32(uint32_t(exp + 127) << 23) - 1.0f;
    int mant = int(std::nearbyint(frac * 8.0f));
    if (mant == 8) { mant = 0; exp += 1; }
    if (exp + 7 >= 0x0F && mant >= 7) return sign | 0x7E;
    return sign | uint8_t((exp + 7) << 3) | uint8_t(mant & 0x07);
}

void orc_e4m3_decode(const uint8_t* bytes, int64_t count, float* out) {
    for (int64_t i = 0; i < count; ++i) out[i] = orc_e4m3_to_f32(bytes[i]);
}
void orc_e4m3_encode(const float* v, int64_t count, int rne, uint8_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) out[i] = rne ? orc_f32_to_e4m3_rne(v[i]) : orc_f32_to_e4m3(v[i]);
}

// ---------------------------------------------------------------------------
// Per-token dynamic activation quantisation (the first half of the W8A8 chain).
//
// Follows backends/spyre/crates/ktir/ktir-superdsc/src/emit/ktir_matmul_fp8.rs
// :300-322 (quantscalepertokenfp8), :430-480 (reciprocal, mul, clip), :517-531
// (qfp8ch) with the constants of superdsc_opspec.rs:1998-2009:
//   a_scale = min(max(absmax * (1/448), 1/448/448), 448)
//   inv     = 1 / a_scale
//   x_q     = e4m3( min(max(x * inv, -448), 448) )
// restated in f32 (the card computes these in fp16).  The constants are the
// reference's f32 expressions `1.0 / 448.0` and `1.0 / 448.0 / 448.0`.
// ---------------------------------------------------------------------------
void orc_fp8_quant_per_token(const uint16_t* x_bf16, int64_t m, int64_t k, int rne,
                             uint8_t* xq, float* a_scale) {
    const float mul_const = 1.0f / 448.0f;
    const float clip_min = 1.0f / 448.0f / 448.0f;
    const float clip_max = 448.0f;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i) {
        const uint16_t* xr = x_bf16 + i * k;
        float amax = 0.0f;
        for (int64_t kk = 0; kk < k; ++kk) amax = std::fmax(amax, std::fabs(bf16_to_f32(xr[kk])));
        const float s = std::fmin(std::fmax(amax * mul_const, clip_min), clip_max);
        a_scale[i] = s;
        const float inv = 1.0f / s;
        for (int64_t kk = 0; kk < k; ++kk) {
            const float c = std::fmin(std::fmax(bf16_to_f32(xr[kk]) * inv, -448.0f), 448.0f);
            xq[i * k + kk] = rne ? orc_f32_to_e4m3_rne(c) : orc_f32_to_e4m3(c);
        }
    }
}

// ---------------------------------------------------------------------------
// fp8 x fp8 contraction with the dequantising tail.
//
// Follows ktir_matmul_fp8.rs:633-720: raw = x_q @ W_q^T, then
// out = (raw * a_scale[m]) * w_scale[n], in that multiply order, restated with an
// f32 accumulator summed in k order (the card accumulates in fp16).
// ---------------------------------------------------------------------------
void orc_fp8_linear(const uint8_t* xq, const float* a_scale, const uint8_t* wq, const float* w_scale,
                    int64_t m, int64_t n, int64_t k, uint16_t* y_bf16, float* y_f32) {
    float table[256];
    for (int b = 0; b < 256; ++b) table[b] = orc_e4m3_to_f32(uint8_t(b));
    std::vector<float> xf(size_t(m) * size_t(k));
    for (int64_t i = 0; i < m * k; ++i) xf[i] = table[xq[i]];
    const int64_t JB = 8;
#pragma omp parallel
    {
        std::vector<float> wr(size_t(k) * JB);
#pragma omp for schedule(static)
        for (int64_t j0 = 0; j0 < n; j0 += JB) {
            const int64_t jb = std::min<int64_t>(JB, n - j0);
            // decoded weights for this column block, k-major so the inner loop is contiguous
            for (int64_t jj = 0; jj < JB; ++jj)
                for (int64_t kk = 0; kk < k; ++kk)
                    wr[kk * JB + jj] = jj < jb ? table[wq[(j0 + jj) * k + kk]] : 0.0f;
            for (int64_t i = 0; i < m; ++i) {
                const float* xr = xf.data() + i * k;
                float acc[JB] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (int64_t kk = 0; kk < k; ++kk) {
                    const float xv = xr[kk];
                    for (int64_t jj = 0; jj < JB; ++jj) acc[jj] += xv * wr[kk * JB + jj];
                }
                for (int64_t jj = 0; jj < jb; ++jj) {
                    const float t = acc[jj] * a_scale[i];
                    const float o = t * w_scale[j0 + jj];
                    if (y_bf16) y_bf16[i * n + j0 + jj] = f32_to_bf16(o);
                    if (y_f32) y_f32[i * n + j0 + jj] = o;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// fp8 weight-only host reference.
//
// Follows backends/spyre/crates/spyre/tests/triton_splice_golden.rs:1690-1713:
// want[m,n] = (sum_k a[m,k] * e4m3_to_f32(w[n,k])) * ws[n], f32, k in order.
// ---------------------------------------------------------------------------
void orc_fp8_weight_only_linear(const float* a, const uint8_t* wq, const float* ws,
                                int64_t m, int64_t n, int64_t k, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < n; ++j) {
        for (int64_t i = 0; i < m; ++i) {
            float acc = 0.0f;
            for (int64_t kk = 0; kk < k; ++kk) {
                acc += a[i * k + kk] * orc_e4m3_to_f32(wq[j * k + kk]);
            }
            out[i * n + j] = acc * ws[j];
        }
    }
}

// ---------------------------------------------------------------------------
// Harness-defined (NOT a reference function; checkpoints arrive quantised):
// per-output-channel weight quantisation of synthetic f32 weights,
// w_scale[n] = absmax(W[n,:]) / 448, W_q = e4m3(W / w_scale) with the reference
// encoder.  The bytes are produced once and shared by the oracle and the GPU,
// so weight rounding cannot diverge between them.
// ---------------------------------------------------------------------------
void orc_fp8_quantize_weight_per_channel(const float* w, int64_t n, int64_t k, uint8_t* wq, float* w_scale) {
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < n; ++j) {
        float amax = 0.0f;
        for (int64_t kk = 0; kk < k; ++kk) amax = std::fmax(amax, std::fabs(w[j * k + kk]));
        float s = amax / 448.0f;
        if (!(s > 0.0f)) s = 1.0f;
        w_scale[j] = s;
        for (int64_t kk = 0; kk < k; ++kk) {
            const float c = std::fmin(std::fmax(w[j * k + kk] / s, -448.0f), 448.0f);
            wq[j * k + kk] = orc_f32_to_e4m3(c);
        }
    }
}

// ---------------------------------------------------------------------------
// All-reduce meaning.
//
// Follows crates/compiler/subtile/src/tensor_parallel.rs:1350-1362
// (`eval_collective`, AllReduce arm): sum the ranks' f32 operands in absolute
// rank order 0..W-1.  `parts` is [world][count].
// ---------------------------------------------------------------------------
void orc_allreduce_rank_order(const float* parts, int world, int64_t count, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        float s = parts[i];
        for (int r = 1; r < world; ++r) s += parts[int64_t(r) * count + i];
        out[i] = s;
    }
}

void orc_f32_to_bf16_array(const float* in, int64_t count, uint16_t* out) {
    for (int64_t i = 0; i < count; ++i) out[i] = f32_to_bf16(in[i]);
}

}  // extern "C"
