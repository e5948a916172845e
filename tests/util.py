"""Shared helpers for the parity tests (numpy <-> torch device buffers, error metrics)."""
import numpy as np


def to_dev(a: np.ndarray, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.view(dtype)
    return t.cuda()


def bf16_dev(bits: np.ndarray):
    import torch
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).cuda()


def u32_dev(words: np.ndarray):
    import torch
    return torch.from_numpy(np.ascontiguousarray(words).view(np.int32)).cuda()


def bits_of(t) -> np.ndarray:
    import torch
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def rel_l2(got_bits: np.ndarray, want_bits: np.ndarray) -> float:
    g = bf16_to_f32(got_bits).astype(np.float64)
    w = bf16_to_f32(want_bits).astype(np.float64)
    return float(np.linalg.norm(g - w) / max(np.linalg.norm(w), 1e-30))


def max_abs(got_bits: np.ndarray, want_bits: np.ndarray) -> float:
    return float(np.max(np.abs(bf16_to_f32(got_bits).astype(np.float64) - bf16_to_f32(want_bits).astype(np.float64))))


def pack_nibbles_bytes(words_u32: np.ndarray) -> np.ndarray:
    """Checkpoint U32 words -> the byte stream the reference's CPU functions take (little endian)."""
    return np.ascontiguousarray(words_u32, np.uint32).view(np.uint8).reshape(-1)
