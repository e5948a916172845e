"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

No public dataset or checkpoint is involved: weights and activations are random draws with
the distributions the baseline configuration states.  numpy only (runs without a GPU).
"""
from __future__ import annotations

import zlib

import numpy as np

LLAMA_3_2_3B = {"q": (3072, 3072), "k": (3072, 1024), "v": (3072, 1024), "o": (3072, 3072),
                "gate": (3072, 8192), "up": (3072, 8192), "down": (8192, 3072)}          # name -> (K, N)
QWEN_2_5_7B = {"q": (3584, 3584), "k": (3584, 512), "v": (3584, 512), "gate": (3584, 18944),
               "up": (3584, 18944), "down": (18944, 3584)}
LLAMA_3_70B = {"qkv": (8192, 10240), "o": (8192, 8192), "gate_up": (8192, 57344), "down": (28672, 8192)}


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((x + 0x7FFF + ((x >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def seed_for(tag: str, *dims: int) -> int:
    return zlib.crc32((tag + ":" + ",".join(map(str, dims))).encode()) & 0x7FFFFFFF


def affine_int4_weights(N: int, K: int, group: int = 64, seed: int = 0):
    """Codes uniform on [0,15] packed 8 per little-endian uint32 (element k%8 of word k//8 at bit 4*(k%8));
    scales bf16 of |N(0,0.02)|+1e-3; biases bf16 of -8*scale + N(0,1e-3), per (row, group)."""
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 16, size=(N, K), dtype=np.uint32)
    shifts = (np.arange(8, dtype=np.uint32) * 4)[None, None, :]
    w = (codes.reshape(N, K // 8, 8) << shifts).sum(axis=2, dtype=np.uint32)
    s = (np.abs(rng.normal(0.0, 0.02, size=(N, K // group))) + 1e-3).astype(np.float32)
    sb = f32_to_bf16_bits(s)
    b = (-8.0 * bf16_bits_to_f32(sb) + rng.normal(0.0, 1e-3, size=(N, K // group))).astype(np.float32)
    return w, sb, f32_to_bf16_bits(b)


def activations_bf16(M: int, K: int, seed: int = 1) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return f32_to_bf16_bits(rng.standard_normal((M, K)).astype(np.float32))


def fp8_weights_f32(N: int, K: int, seed: int = 0) -> np.ndarray:
    """W ~ N(0, 0.02) in f32; quantise per output channel with the harness rule (scale = absmax/448)."""
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
