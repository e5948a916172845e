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
