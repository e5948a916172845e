"""The oracle reproduces the committed golden fixtures (tests/golden/, made by make_golden.py)."""
import glob
import os

import numpy as np
import pytest

import oracle

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "affine_b4_*.npz"))))
def test_affine_golden(path):
    g = np.load(path)
    N, K = g["w"].shape[0], g["w"].shape[1] * 8
    M = g["x"].shape[0]
    packed = g["w"].view(np.uint8).reshape(-1)
    assert np.array_equal(oracle.affine_dequant_b4(packed, g["scales"], g["biases"], N, K, 64), g["w_dequant"])
    assert np.array_equal(oracle.affine_qmm_t_b4(packed, g["scales"], g["biases"], g["x"], M, N, K, 64), g["y"])


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "fp8_*.npz"))))
def test_fp8_golden(path):
    g = np.load(path)
    N, K = g["wq"].shape
    M = g["x"].shape[0]
    xq, a = oracle.fp8_quant_per_token(g["x"], M, K)
    assert np.array_equal(xq, g["xq"]) and np.array_equal(a, g["a_scale"])
    assert np.array_equal(oracle.fp8_linear(xq, a, g["wq"], g["w_scale"], M, N, K), g["y"])


def test_decode_ops_golden():
    """The decode-step oracle reproduces its committed fixture bit for bit (f32 outputs included)."""
    from scratchy_b200 import synth
    g = np.load(os.path.join(GOLD, "decode_ops_small.npz"))
    f, r = synth.bf16_bits_to_f32, synth.f32_to_bf16_bits
    assert np.array_equal(oracle.rmsnorm(f(g["norm_x"]), f(g["norm_gain"]), 1e-5), g["rmsnorm_f32"])
    res, nrm = oracle.fused_add_rmsnorm(f(g["norm_x"]), f(g["norm_delta"]), f(g["norm_gain"]), 1e-5, round_residual_bf16=True)
    assert np.array_equal(r(res), g["addnorm_residual"]) and np.array_equal(nrm, g["addnorm_f32"])
    gu = g["silu_gate_up"]
    assert np.array_equal(oracle.silu_mul(f(gu[:, :128]), f(gu[:, 128:])), g["silu_f32"])
    hq, hkv, hd, bs, _ = (int(v) for v in g["rope_geom"])
    fq = f(g["rope_qkv"])
    ok, ov = f(g["rope_cache_k_in"]).copy(), f(g["rope_cache_v_in"]).copy()
    q_rot = oracle.rope_append(fq[:, :hq * hd], fq[:, hq * hd:(hq + hkv) * hd], fq[:, (hq + hkv) * hd:], g["rope_pos"],
                               g["rope_slots"], g["rope_cos"], g["rope_sin"], ok, ov, hq, hkv, hd, bs)
    assert np.array_equal(r(q_rot), g["rope_q_out"])
    assert np.array_equal(r(ok), g["rope_cache_k_out"]) and np.array_equal(r(ov), g["rope_cache_v_out"])
    att = oracle.attention_via_cache(f(g["attn_q"]), f(g["rope_cache_k_out"]), f(g["rope_cache_v_out"]), g["attn_table"],
                                     g["attn_lens"], hq, hkv, hd, bs, np.float32(hd ** -0.5))
    assert np.array_equal(att, g["attn_f32"])
    assert np.array_equal(oracle.argmax(f(g["argmax_logits"])), g["argmax_ids"]) and g["argmax_ids"][1] == 10
