"""Independent numpy restatement of the reference lines the C++ oracle follows.

TEST INFRASTRUCTURE ONLY.  Slow and simple on purpose: it exists so the C++ oracle
can be cross-checked on small cases by code that shares nothing with it.
"""
from __future__ import annotations

import numpy as np


def bf16_bits_to_f32(b):
    return (np.asarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(f):
    """Round to nearest even; NaN is quieted (the `half` crate's bf16::from_f32)."""
    x = np.asarray(f, np.float32).view(np.uint32)
    nan = (x & 0x7FFFFFFF) > 0x7F800000
    lsb = (x >> 16) & 1
    rounded = (x + 0x7FFF + lsb) >> 16
    return np.where(nan, (x >> 16) | 0x40, rounded).astype(np.uint16)


def f16_bits_to_f32(b):
    return np.asarray(b, np.uint16).view(np.float16).astype(np.float32)


def f32_to_f16_bits(f):
    return np.asarray(f, np.float32).astype(np.float16).view(np.uint16)


def _dec(b, dt):
    return bf16_bits_to_f32(b) if dt == 1 else f16_bits_to_f32(b)


def _enc(f, dt):
    return f32_to_bf16_bits(f) if dt == 1 else f32_to_f16_bits(f)


def affine_dequant_b4(packed_bytes, scales, biases, n, k, gs, scale_dt=1, out_dt=1, cast_scale_to_act=False):
    """crates/models/quantization/src/affine.rs:120-132 — low nibble is the even element."""
    p = np.asarray(packed_bytes, np.uint8).reshape(-1)
    codes = np.empty(p.size * 2, np.float32)
    codes[0::2] = (p & 0x0F).astype(np.float32)
    codes[1::2] = (p >> 4).astype(np.float32)
    s = _dec(np.asarray(scales, np.uint16).reshape(-1), scale_dt)
    b = _dec(np.asarray(biases, np.uint16).reshape(-1), scale_dt)
    if cast_scale_to_act:                       # cpu_reference.rs:90-91
        s = _dec(_enc(s, out_dt), out_dt)
        b = _dec(_enc(b, out_dt), out_dt)
    g = np.arange(n * k) // gs
    prod = (s[g] * codes).astype(np.float32)    # f32 multiply, rounded
    w = (prod + b[g]).astype(np.float32)        # f32 add, rounded
    return _enc(w, out_dt).reshape(n, k)


def affine_qmm_t_b4(packed_bytes, scales, biases, x, m, n, k, gs, scale_dt=1, act_dt=1):
    """crates/targets/metal/src/cpu_reference.rs:107-137 — sequential f32 accumulation over k."""
    w = _dec(affine_dequant_b4(packed_bytes, scales, biases, n, k, gs, scale_dt, act_dt, True), act_dt)
    xf = _dec(np.asarray(x, np.uint16).reshape(m, k), act_dt)
    acc = np.zeros((m, n), np.float32)
    for kk in range(k):                         # k in order; every (i, j) advances together
        acc = (acc + (xf[:, kk:kk + 1] * w[None, :, kk]).astype(np.float32)).astype(np.float32)
    return _enc(acc, act_dt), acc


def e4m3_to_f32(byte: int) -> float:
    """backends/spyre/crates/ktir/ktir-core/src/codec.rs:991-1008."""
    sign = -1.0 if byte & 0x80 else 1.0
    exp = (byte >> 3) & 0x0F
    mant = byte & 0x07
    if exp == 0x0F and mant == 0x07:
        return float("nan")
    mag = mant * 2.0 ** -9 if exp == 0 else (1.0 + mant / 8.0) * 2.0 ** (exp - 7)
    return sign * mag


def _round_half_away(v: float) -> int:
    import math
    return int(math.floor(abs(v) + 0.5)) * (1 if v >= 0 else -1)


def f32_to_e4m3_log2_spelling(v: float) -> int:
    """The `log2().floor()` spelling the reference pins its fast encoder against
    (codec.rs:841-878 names it `reference`): same branches, exponent from log2."""
    import math
    v = float(np.float32(v))
    if math.isnan(v):
        return 0x7F
    sign = 0x80 if math.copysign(1.0, v) < 0 else 0
    a = abs(v)
    if a == 0.0:
        return sign
    if a >= 464.0:
        return sign | 0x7F
    if a >= 448.0:
        return sign | 0x7E
    if a < 0.015625:
        q = _round_half_away(a * 512.0)
        return sign | max(0, min(8, q))
    exp = int(math.floor(math.log2(a)))
    frac = a / 2.0 ** exp - 1.0
    mant = _round_half_away(frac * 8.0)
    if mant == 8:
        mant, exp = 0, exp + 1
    if exp + 7 >= 0x0F and mant >= 7:
        return sign | 0x7E
    return sign | ((exp + 7) << 3) | (mant & 7)


def fp8_quant_per_token(x_bf16, m, k):
    """ktir_matmul_fp8.rs:300-322,430-480,517-531 with superdsc_opspec.rs:1998-2009, in f32."""
    x = bf16_bits_to_f32(np.asarray(x_bf16, np.uint16).reshape(m, k))
    mul_const = np.float32(1.0) / np.float32(448.0)
    clip_min = np.float32(1.0) / np.float32(448.0) / np.float32(448.0)
    amax = np.abs(x).max(axis=1).astype(np.float32)
    a_scale = np.minimum(np.maximum((amax * mul_const).astype(np.float32), clip_min), np.float32(448.0))
    inv = (np.float32(1.0) / a_scale).astype(np.float32)
    t = np.clip((x * inv[:, None]).astype(np.float32), np.float32(-448.0), np.float32(448.0))
    xq = np.array([f32_to_e4m3_log2_spelling(v) for v in t.reshape(-1)], np.uint8).reshape(m, k)
    return xq, a_scale


def fp8_linear(xq, a_scale, wq, w_scale, m, n, k):
    """ktir_matmul_fp8.rs:633-720 in f32, (raw * a_scale) * w_scale."""
    table = np.array([e4m3_to_f32(b) for b in range(256)], np.float32)
    xf = table[np.asarray(xq, np.uint8).reshape(m, k)]
    wf = table[np.asarray(wq, np.uint8).reshape(n, k)]
    acc = np.zeros((m, n), np.float32)
    for kk in range(k):
        acc = (acc + (xf[:, kk:kk + 1] * wf[None, :, kk]).astype(np.float32)).astype(np.float32)
    t = (acc * np.asarray(a_scale, np.float32)[:, None]).astype(np.float32)
    o = (t * np.asarray(w_scale, np.float32)[None, :]).astype(np.float32)
    return f32_to_bf16_bits(o), o


class SplitMix64:
    """crates/targets/metal/tests/quantized_qmv_test.rs:129-145."""

    def __init__(self, seed: int):
        self.s = seed & 0xFFFFFFFFFFFFFFFF

    def next(self) -> int:
        M = 0xFFFFFFFFFFFFFFFF
        self.s = (self.s + 0x9E3779B97F4A7C15) & M
        z = self.s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        return z ^ (z >> 31)

    def next_byte(self) -> int:
        return self.next() & 0xFF

    def next_unit_f32(self) -> np.float32:
        return np.float32(np.float32(self.next() >> 40) / np.float32(1 << 24))


def make_inputs_bf16(seed, n, k, m, gs):
    """quantized_qmv_test.rs:147-180: random nibble bytes, f16 scales 0.01+0.04u, f16 biases u-0.5, bf16 x 2u-1."""
    rng = SplitMix64(seed)
    packed = np.array([rng.next_byte() for _ in range(n * k // 2)], np.uint8)
    ng = n * k // gs
    scales = f32_to_f16_bits(np.array(
        [np.float32(0.01) + np.float32(0.04) * rng.next_unit_f32() for _ in range(ng)], np.float32))
    biases = f32_to_f16_bits(np.array([rng.next_unit_f32() - np.float32(0.5) for _ in range(ng)], np.float32))
    x = f32_to_bf16_bits(np.array([np.float32(2.0) * rng.next_unit_f32() - np.float32(1.0)
                                   for _ in range(m * k)], np.float32))
    return packed, scales, biases, x
