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


if __name__ == "__main__":
    affine_case("affine_b4_n48_k256_m3.npz", 48, 256, 3, 11)
    affine_case("affine_b4_n128_k192_m16.npz", 128, 192, 16, 12)
    affine_case("affine_b4_n256_k512_m40.npz", 256, 512, 40, 13)
    fp8_case("fp8_n48_k256_m3.npz", 48, 256, 3, 21)
    fp8_case("fp8_n256_k384_m16.npz", 256, 384, 16, 22)
    fp8_case("fp8_n256_k512_m40.npz", 256, 512, 40, 23)
    print("wrote fixtures to", OUT)
