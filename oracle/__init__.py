"""CPU oracle for the quantized-linear hot path — TEST INFRASTRUCTURE ONLY.

Loads ``liboracle.so`` (built from ``scratchy_oracle.cpp`` by ``make -C oracle``) and
exposes numpy-facing wrappers.  Only the test-suite, the smoke check and the
benchmark's CPU-baseline leg import this package; the product package
``scratchy_b200`` never does.

``numpy_twin`` holds an independent pure-numpy restatement of the same reference
lines, used to cross-check the C++ on small cases.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

F16, BF16 = 0, 1  # discriminants of the reference's DType (crates/tensors/src/dtype.rs:7-16)


def build(force: bool = False) -> str:
    """Compile liboracle.so if it is missing or older than its source."""
    srcs = [os.path.join(_HERE, f) for f in ("scratchy_oracle.cpp", "decode_oracle.cpp")]
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < max(os.path.getmtime(s) for s in srcs):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        L.orc_e4m3_to_f32.restype = ctypes.c_float
        L.orc_e4m3_to_f32.argtypes = [ctypes.c_uint8]
        L.orc_f32_to_e4m3.restype = ctypes.c_uint8
        L.orc_f32_to_e4m3.argtypes = [ctypes.c_float]
        L.orc_f32_to_e4m3_rne.restype = ctypes.c_uint8
        L.orc_f32_to_e4m3_rne.argtypes = [ctypes.c_float]
        L.orc_f32_to_bf16.restype = ctypes.c_uint16
        L.orc_f32_to_bf16.argtypes = [ctypes.c_float]
        L.orc_num_threads.restype = ctypes.c_int
        L.orc_embed.restype = ctypes.c_int
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def set_num_threads(n: int) -> None:
    """OpenMP threads of the following oracle calls (the bench's CPU arm: every host core, whatever OMP_NUM_THREADS
    the launcher exported)."""
    lib().orc_set_num_threads(ctypes.c_int(int(n)))


def num_threads() -> int:
    return int(lib().orc_num_threads())


# --------------------------------------------------------------------------- bf16 helpers
def f32_to_bf16_bits(a) -> np.ndarray:
    a = _c(a, np.float32)
    out = np.empty(a.shape, np.uint16)
    lib().orc_f32_to_bf16_array(_p(a), ctypes.c_int64(a.size), _p(out))
    return out


def bf16_bits_to_f32(a) -> np.ndarray:
    a = _c(a, np.uint16)
    return (a.astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------- int4 affine
def affine_dequant_b4(packed_bytes, scales, biases, n, k, group_size, scale_dt=BF16, out_dt=BF16,
                      cast_scale_to_act=False) -> np.ndarray:
    """crates/models/quantization/src/affine.rs:120-132 / cpu_reference.rs:69-98. Returns [n,k] 16-bit patterns."""
    packed_bytes = _c(packed_bytes, np.uint8).reshape(-1)
    scales = _c(scales, np.uint16).reshape(-1)
    biases = _c(biases, np.uint16).reshape(-1)
    assert k % group_size == 0 and packed_bytes.size == n * k // 2
    assert scales.size == n * k // group_size == biases.size
    out = np.empty((n, k), np.uint16)
    lib().orc_affine_dequant_b4(_p(packed_bytes), _p(scales), _p(biases), ctypes.c_int64(n), ctypes.c_int64(k),
                                ctypes.c_int64(group_size), scale_dt, out_dt, int(cast_scale_to_act), _p(out))
    return out


def affine_qmm_t_b4(packed_bytes, scales, biases, x, m, n, k, group_size, scale_dt=BF16, act_dt=BF16,
                    want_f32=False):
    """crates/targets/metal/src/cpu_reference.rs:107-137. x, y are 16-bit patterns ([m,k] / [m,n])."""
    packed_bytes = _c(packed_bytes, np.uint8).reshape(-1)
    scales = _c(scales, np.uint16).reshape(-1)
    biases = _c(biases, np.uint16).reshape(-1)
    x = _c(x, np.uint16).reshape(-1)
    assert x.size == m * k and packed_bytes.size == n * k // 2
    y = np.empty((m, n), np.uint16)
    yf = np.empty((m, n), np.float32) if want_f32 else None
    lib().orc_affine_qmm_t_b4(_p(packed_bytes), _p(scales), _p(biases), _p(x), ctypes.c_int64(m),
                              ctypes.c_int64(n), ctypes.c_int64(k), ctypes.c_int64(group_size), scale_dt, act_dt,
                              _p(y), _p(yf) if want_f32 else None)
    return (y, yf) if want_f32 else y


def affine_qmm_t_b4_bias(packed_bytes, scales, biases, x, linear_bias, m, n, k, group_size, scale_dt=BF16):
    """The linear with its own bias [n] (bf16 patterns): the reference's matvec adds `float(bias[n])` to the f32
    dot and rounds once (crates/targets/metal/shaders/quantized_qmv.metal:104-112, `qmv_store`)."""
    _, acc = affine_qmm_t_b4(packed_bytes, scales, biases, x, m, n, k, group_size, scale_dt=scale_dt, want_f32=True)
    bias = bf16_bits_to_f32(_c(linear_bias, np.uint16).reshape(1, n))
    return f32_to_bf16_bits(acc.astype(np.float32) + bias.astype(np.float32))


# --------------------------------------------------------------------------- e4m3 / fp8
def e4m3_to_f32(b) -> np.ndarray:
    b = _c(b, np.uint8)
    out = np.empty(b.shape, np.float32)
    lib().orc_e4m3_decode(_p(b), ctypes.c_int64(b.size), _p(out))
    return out


def f32_to_e4m3(v, rne=False) -> np.ndarray:
    v = _c(v, np.float32)
    out = np.empty(v.shape, np.uint8)
    lib().orc_e4m3_encode(_p(v), ctypes.c_int64(v.size), int(rne), _p(out))
    return out


def fp8_quant_per_token(x_bf16, m, k, rne=False):
    """ktir_matmul_fp8.rs:300-322,430-480,517-531 in f32. Returns (xq [m,k] u8, a_scale [m] f32)."""
    x_bf16 = _c(x_bf16, np.uint16).reshape(-1)
    assert x_bf16.size == m * k
    xq = np.empty((m, k), np.uint8)
    a = np.empty((m,), np.float32)
    lib().orc_fp8_quant_per_token(_p(x_bf16), ctypes.c_int64(m), ctypes.c_int64(k), int(rne), _p(xq), _p(a))
    return xq, a


def fp8_linear(xq, a_scale, wq, w_scale, m, n, k, want_f32=False):
    """ktir_matmul_fp8.rs:633-720 in f32: y = bf16((sum_k xq*wq) * a_scale[m] * w_scale[n])."""
    xq = _c(xq, np.uint8).reshape(-1)
    wq = _c(wq, np.uint8).reshape(-1)
    a_scale = _c(a_scale, np.float32).reshape(-1)
    w_scale = _c(w_scale, np.float32).reshape(-1)
    assert xq.size == m * k and wq.size == n * k and a_scale.size == m and w_scale.size == n
    y = np.empty((m, n), np.uint16)
    yf = np.empty((m, n), np.float32) if want_f32 else None
    lib().orc_fp8_linear(_p(xq), _p(a_scale), _p(wq), _p(w_scale), ctypes.c_int64(m), ctypes.c_int64(n),
                         ctypes.c_int64(k), _p(y), _p(yf) if want_f32 else None)
    return (y, yf) if want_f32 else y


def fp8_dynamic_linear(x_bf16, wq, w_scale, m, n, k, rne=False, want_f32=False):
    """The whole generated Linear for fp8-dynamic-per-channel: quantise per token, contract, dequantise."""
    xq, a = fp8_quant_per_token(x_bf16, m, k, rne=rne)
    return fp8_linear(xq, a, wq, w_scale, m, n, k, want_f32=want_f32)


def fp8_dynamic_linear_bias(x_bf16, wq, w_scale, linear_bias, m, n, k) -> np.ndarray:
    """The fp8 dynamic linear with the linear's own bias [n] (bf16 patterns): the bias is added in f32 to the
    dequantised sum and the result rounded once, the order of the reference's matvec epilogue
    (crates/targets/metal/shaders/quantized_qmv.metal:104-112, `qmv_store`)."""
    _, acc = fp8_dynamic_linear(x_bf16, wq, w_scale, m, n, k, want_f32=True)
    bias = bf16_bits_to_f32(_c(linear_bias, np.uint16).reshape(1, n))
    return f32_to_bf16_bits(acc.astype(np.float32) + bias.astype(np.float32))


def fp8_weight_only_linear(a, wq, ws, m, n, k) -> np.ndarray:
    """backends/spyre/crates/spyre/tests/triton_splice_golden.rs:1690-1713."""
    a = _c(a, np.float32).reshape(-1)
    wq = _c(wq, np.uint8).reshape(-1)
    ws = _c(ws, np.float32).reshape(-1)
    out = np.empty((m, n), np.float32)
    lib().orc_fp8_weight_only_linear(_p(a), _p(wq), _p(ws), ctypes.c_int64(m), ctypes.c_int64(n),
                                     ctypes.c_int64(k), _p(out))
    return out


def fp8_quantize_weight_per_channel(w_f32):
    """Harness-defined synthetic weight quantisation: w_scale = absmax/448, wq = e4m3(w / w_scale)."""
    w = _c(w_f32, np.float32)
    n, k = w.shape
    wq = np.empty((n, k), np.uint8)
    ws = np.empty((n,), np.float32)
    lib().orc_fp8_quantize_weight_per_channel(_p(w), ctypes.c_int64(n), ctypes.c_int64(k), _p(wq), _p(ws))
    return wq, ws


# --------------------------------------------------------------------------- tensor parallel
def slice_rows(full: np.ndarray, world: int, rank: int) -> np.ndarray:
    """SourceShard::Rows of crates/compiler/subtile/src/tensor_parallel.rs:1186-1189 applied to a 2-D array."""
    lr = full.shape[0] // world
    return np.ascontiguousarray(full[rank * lr:(rank + 1) * lr])


def slice_cols(full: np.ndarray, world: int, rank: int) -> np.ndarray:
    """SourceShard::Cols of tensor_parallel.rs:1190-1199 applied to a 2-D array."""
    lc = full.shape[1] // world
    return np.ascontiguousarray(full[:, rank * lc:(rank + 1) * lc])


def allreduce_rank_order(parts) -> np.ndarray:
    """tensor_parallel.rs:1350-1362: f32 sum over ranks in absolute rank order."""
    parts = _c(np.stack(parts), np.float32)
    world = parts.shape[0]
    out = np.empty(parts.shape[1:], np.float32)
    lib().orc_allreduce_rank_order(_p(parts), world, ctypes.c_int64(out.size), _p(out))
    return out


def affine_embed_b4(packed_bytes, scales, biases, ids, vocab, hidden, group_size, scale_dt=BF16) -> np.ndarray:
    """The quantized embedding's host reference (crates/targets/metal/tests/quantized_affine_embed_test.rs:27-90, after MLX
    `nn.QuantizedEmbedding.__call__`): gather the packed row, its scales and its offsets by token id, then dequantise
    the row — scale and offset narrowed to the activation type first, `bf16(f32(scale) * f32(code) + f32(bias))`.
    Returns [len(ids), hidden] bf16 bit patterns."""
    packed = _c(packed_bytes, np.uint8).reshape(vocab, hidden // 2)
    sc = _c(scales, np.uint16).reshape(vocab, hidden // group_size)
    bi = _c(biases, np.uint16).reshape(vocab, hidden // group_size)
    ids = np.asarray(ids).astype(np.int64).reshape(-1)
    if ids.size and (ids.min() < 0 or ids.max() >= vocab):
        raise ValueError("token id beyond the vocabulary")
    return affine_dequant_b4(packed[ids], sc[ids], bi[ids], ids.size, hidden, group_size, scale_dt=scale_dt,
                             cast_scale_to_act=True)


def allgather_cols_rank_order(parts, cols: int) -> np.ndarray:
    """tensor_parallel.rs:1363-1386 (`SubOp::AllGather{cols}`): every rank's [rows, lc] column block side by side in
    absolute rank order, row by row, cropped to `cols` (a padded last block's tail is cut off).  Any dtype; values
    are moved, never changed."""
    parts = [np.asarray(p) for p in parts]
    rows, lc = parts[0].shape
    if lc * len(parts) < cols:
        raise ValueError(f"{len(parts)} blocks of {lc} columns cannot restore {cols}")
    out = np.empty((rows, cols), parts[0].dtype)
    for i in range(rows):
        row = []
        for p in parts:
            row.extend(p[i, :lc].tolist())
        out[i, :] = np.asarray(row[:cols], dtype=parts[0].dtype)
    return out


# --------------------------------------------------------------------------- decode-step operators
# f32 in, f32 out, exactly as the reference's host golden (decode_oracle.cpp cites the lines).
def rmsnorm(x, weight, eps=1e-5) -> np.ndarray:
    x = _c(x, np.float32)
    w = _c(weight, np.float32)
    rows, hidden = x.reshape(-1, w.size).shape
    out = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), _p(out), ctypes.c_int64(rows), ctypes.c_int64(hidden), ctypes.c_float(eps))
    return out


def fused_add_rmsnorm(residual, delta, weight, eps=1e-5, round_residual_bf16=False):
    """Returns (residual_after_add, normed); the inputs are not modified."""
    w = _c(weight, np.float32)
    res = np.array(residual, dtype=np.float32, order="C", copy=True)
    dl = np.array(delta, dtype=np.float32, order="C", copy=True)
    rows, hidden = res.reshape(-1, w.size).shape
    lib().orc_fused_add_rmsnorm(_p(res), _p(dl), _p(w), ctypes.c_float(eps), ctypes.c_int64(rows),
                                ctypes.c_int64(hidden), ctypes.c_int(1 if round_residual_bf16 else 0))
    return res, dl


def silu_mul(gate, up) -> np.ndarray:
    g = _c(gate, np.float32)
    u = _c(up, np.float32)
    out = np.empty_like(g)
    lib().orc_silu_mul(_p(g), _p(u), _p(out), ctypes.c_int64(g.size))
    return out


def embed(ids, table) -> np.ndarray:
    ids = _c(ids, np.uint32)
    table = _c(table, np.float32)
    vocab, hidden = table.shape
    out = np.empty((ids.size, hidden), np.float32)
    rc = lib().orc_embed(_p(ids), ctypes.c_int64(ids.size), _p(table), ctypes.c_int64(vocab),
                         ctypes.c_int64(hidden), _p(out))
    if rc != 0:
        raise IndexError("token id outside the embedding table")
    return out


def rope_append(q, k, v, positions, slot_mapping, cos_table, sin_table, cache_k, cache_v, num_q_heads,
                num_kv_heads, head_dim, block_size):
    """Returns q_out; cache_k / cache_v (f32, C-contiguous) are updated in place."""
    q = _c(q, np.float32)
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    pos = _c(positions, np.uint32)
    slots = _c(slot_mapping, np.uint32)
    cos = _c(cos_table, np.float32)
    sin = _c(sin_table, np.float32)
    assert cache_k.dtype == np.float32 and cache_k.flags.c_contiguous
    assert cache_v.dtype == np.float32 and cache_v.flags.c_contiguous
    assert cache_k.size % (num_kv_heads * block_size * head_dim) == 0 and cache_k.size == cache_v.size
    q_out = np.empty_like(q)
    lib().orc_rope_append(_p(q), _p(k), _p(v), _p(pos), _p(slots), _p(cos), _p(sin), _p(q_out), _p(cache_k),
                          _p(cache_v), ctypes.c_int64(pos.size), ctypes.c_int64(num_q_heads),
                          ctypes.c_int64(num_kv_heads), ctypes.c_int64(head_dim), ctypes.c_int64(block_size))
    return q_out


def attention_via_cache(q, cache_k, cache_v, block_table, seq_used_k, num_q_heads, num_kv_heads, head_dim,
                        block_size, attn_scale) -> np.ndarray:
    q = _c(q, np.float32)
    ck = _c(cache_k, np.float32)
    cv = _c(cache_v, np.float32)
    bt = _c(block_table, np.uint32)
    used = _c(seq_used_k, np.uint32)
    batch = used.size
    max_blocks = bt.size // max(batch, 1)
    out = np.zeros((batch, num_q_heads * head_dim), np.float32)
    lib().orc_attention_via_cache(_p(q), _p(ck), _p(cv), _p(bt), _p(used), _p(out), ctypes.c_int64(batch),
                                  ctypes.c_int64(num_q_heads), ctypes.c_int64(num_kv_heads),
                                  ctypes.c_int64(head_dim), ctypes.c_int64(block_size),
                                  ctypes.c_int64(max_blocks), ctypes.c_float(attn_scale))
    return out


def argmax(logits) -> np.ndarray:
    lg = _c(logits, np.float32)
    rows, width = lg.shape
    out = np.empty(rows, np.uint32)
    lib().orc_argmax(_p(lg), ctypes.c_int64(rows), ctypes.c_int64(width), _p(out))
    return out
