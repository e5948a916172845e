"""Generates the committed golden fixtures from the CPU oracle on seeded synthetic inputs.

Run from the repository root:  python tests/golden/make_golden.py
The reference project is Rust and cannot be built in this environment, so these vectors come
from the oracle restatement (itself pinned on the reference's known-answer tests); they fix
the oracle's outputs so that a later change to it cannot go unnoticed, and give the GPU
tests inputs with known answers.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from scratchy_b200 import synth  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def affine_case(name, N, K, M, seed):
    w, s, b = synth.affine_int4_weights(N, K, 64, seed)
    x = synth.activations_bf16(M, K, seed + 1)
    packed = w.view(np.uint8).reshape(-1)
    wd = oracle.affine_dequant_b4(packed, s, b, N, K, 64)
    y = oracle.affine_qmm_t_b4(packed, s, b, x, M, N, K, 64)
    np.savez_compressed(os.path.join(OUT, name), w=w, scales=s, biases=b, x=x, w_dequant=wd, y=y)


def fp8_case(name, N, K, M, seed):
    wf = synth.fp8_weights_f32(N, K, seed)
    wq, ws = oracle.fp8_quantize_weight_per_channel(wf)
    x = synth.activations_bf16(M, K, seed + 1)
    xq, a = oracle.fp8_quant_per_token(x, M, K)
    y = oracle.fp8_linear(xq, a, wq, ws, M, N, K)
    np.savez_compressed(os.path.join(OUT, name), wq=wq, w_scale=ws, x=x, xq=xq, a_scale=a, y=y)


def decode_ops_case(name, seed):
    """One small seeded case per decode-step operator; bf16 inputs as bit patterns, outputs as the
    oracle's f32 results rounded to bf16 (f32 kept beside them for the floating-point operators)."""
    rng = np.random.default_rng(seed)
    r, f = synth.f32_to_bf16_bits, synth.bf16_bits_to_f32
    out = {}
    # rmsnorm / fused_add_rmsnorm
    x = r(rng.standard_normal((3, 256)).astype(np.float32) * 2.0)
    d = r(rng.standard_normal((3, 256)).astype(np.float32) * 0.5)
    g = r((1.0 + 0.1 * rng.standard_normal(256)).astype(np.float32))
    out.update(norm_x=x, norm_delta=d, norm_gain=g, rmsnorm_f32=oracle.rmsnorm(f(x), f(g), 1e-5))
    res, nrm = oracle.fused_add_rmsnorm(f(x), f(d), f(g), 1e-5, round_residual_bf16=True)
    out.update(addnorm_residual=r(res), addnorm_f32=nrm)
    # silu(gate) * up on the halves of a fused output
    gu = r(rng.standard_normal((2, 256)).astype(np.float32) * 2.0)
    out.update(silu_gate_up=gu, silu_f32=oracle.silu_mul(f(gu[:, :128]), f(gu[:, 128:])))
    # rope + paged append: 3 tokens, 4 q heads, 2 kv heads, head_dim 64, block 16, 5 blocks
    hq, hkv, hd, bs, nblk = 4, 2, 64, 16, 5
    qkv = r(rng.standard_normal((3, (hq + 2 * hkv) * hd)).astype(np.float32))
    cos = rng.uniform(-1, 1, size=(32, hd)).astype(np.float32)
    sin = rng.uniform(-1, 1, size=(32, hd)).astype(np.float32)
    pos = np.array([5, 0, 31], np.uint32)
    slots = np.array([17, 3, 79], np.uint32)
    ck = r(rng.standard_normal((nblk, hkv, bs, hd)).astype(np.float32))
    cv = r(rng.standard_normal((nblk, hkv, bs, hd)).astype(np.float32))
    ok, ov = f(ck).copy(), f(cv).copy()
    fq = f(qkv)
    q_rot = oracle.rope_append(fq[:, :hq * hd], fq[:, hq * hd:(hq + hkv) * hd], fq[:, (hq + hkv) * hd:], pos, slots, cos, sin,
                               ok, ov, hq, hkv, hd, bs)
    out.update(rope_qkv=qkv, rope_cos=cos, rope_sin=sin, rope_pos=pos, rope_slots=slots, rope_cache_k_in=ck,
               rope_cache_v_in=cv, rope_q_out=r(q_rot), rope_cache_k_out=r(ok), rope_cache_v_out=r(ov),
               rope_geom=np.array([hq, hkv, hd, bs, nblk], np.int32))
    # paged decode attention over the appended caches: two sequences, 37 and 5 tokens
    table = np.array([[4, 1, 0], [2, 3, 0]], np.uint32)
    lens = np.array([37, 5], np.uint32)
    q2 = r(rng.standard_normal((2, hq * hd)).astype(np.float32))
    att = oracle.attention_via_cache(f(q2), f(r(ok)), f(r(ov)), table, lens, hq, hkv, hd, bs, np.float32(hd ** -0.5))
    out.update(attn_q=q2, attn_table=table, attn_lens=lens, attn_f32=att)
    # argmax
    lg = r(rng.standard_normal((3, 1000)).astype(np.float32))
    lg[1, 10] = lg[1, 900] = r(np.array([9.0], np.float32))[0]
    out.update(argmax_logits=lg, argmax_ids=oracle.argmax(f(lg)))
    np.savez_compressed(os.path.join(OUT, name), **out)


CASES = [
    (affine_case, ("affine_b4_n48_k256_m3.npz", 48, 256, 3, 11)),
    (affine_case, ("affine_b4_n128_k192_m16.npz", 128, 192, 16, 12)),
    (affine_case, ("affine_b4_n256_k512_m40.npz", 256, 512, 40, 13)),
    (fp8_case, ("fp8_n48_k256_m3.npz", 48, 256, 3, 21)),
    (fp8_case, ("fp8_n256_k384_m16.npz", 256, 384, 16, 22)),
    (fp8_case, ("fp8_n256_k512_m40.npz", 256, 512, 40, 23)),
    (decode_ops_case, ("decode_ops_small.npz", 31)),
]

if __name__ == "__main__":
    force = "--force" in sys.argv          # without it only missing fixtures are written
    for fn, args in CASES:
        if force or not os.path.exists(os.path.join(OUT, args[0])):
            fn(*args)
            print("wrote", args[0])
