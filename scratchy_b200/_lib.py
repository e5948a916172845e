"""ctypes binding of ``libscratchy_cuda.so`` — the same entry points a Rust `extern "C"` shim binds."""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libscratchy_cuda.so")

OK = 0
STATUS = {0: "SCR_OK", -1: "SCR_E_ARG", -2: "SCR_E_SHAPE", -3: "SCR_E_ALIGN", -4: "SCR_E_DTYPE", -5: "SCR_E_CUDA",
          -6: "SCR_E_WORKSPACE", -7: "SCR_E_UNSUPPORTED", -8: "SCR_E_TIMEOUT", -9: "SCR_E_COMM"}
DTYPE_F16, DTYPE_BF16 = 0, 1     # the reference's DType discriminants (crates/tensors/src/dtype.rs:7-16)
KIND_AFFINE_B4 = 0
KIND_FP8_DYNAMIC = 1


class ScratchyCudaError(RuntimeError):
    def __init__(self, status: int, detail: str = ""):
        self.status = status
        self.name = STATUS.get(status, f"status {status}")
        super().__init__(f"{self.name}: {detail}" if detail else self.name)


def lib_path() -> str:
    return _LIB_PATH


_vp, _i32, _i64, _sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t
_psz = ctypes.POINTER(ctypes.c_size_t)

# name -> (restype, argtypes); one row per declaration in include/scratchy_cuda.h
SIGNATURES = {
    "scr_status_string": (ctypes.c_char_p, [_i32]),
    "scr_last_error": (ctypes.c_char_p, [_vp]),
    "scr_cuda_init": (_i32, [_i32, ctypes.POINTER(_vp)]),
    "scr_cuda_destroy": (_i32, [_vp]),
    "scr_launch_count": (_i64, [_vp]),
    "scr_device_status": (_i32, [_vp, _vp, ctypes.POINTER(_i32)]),
    "scr_affine_b4_repack_size": (_i32, [_i32, _i32, _i32, _psz]),
    "scr_affine_b4_repack": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "scr_affine_b4_dequant_dump": (_i32, [_vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "scr_affine_b4_embed": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "scr_linear_workspace_size": (_i32, [_i32, _i32, _i32, _i32, _psz]),
    "scr_linear_affine_b4": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _sz, _vp]),
    "scr_linear_affine_b4_ends": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "scr_linear_affine_b4_group": (_i32, [_vp, _i32, ctypes.POINTER(_vp), _vp, _i32, ctypes.POINTER(_i32), _i32, _i32, ctypes.POINTER(_vp), _vp, ctypes.c_size_t, _vp]),
    "scr_linear_affine_b4_silu_mul": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp]),
    "scr_linear_affine_b4_residual_rmsnorm": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, ctypes.c_float, _vp,
                                                     _vp, _sz, _vp]),
    "scr_affine_b4_tape_create": (_i32, [_vp, _vp, _i32, _i32, ctypes.POINTER(_vp)]),
    "scr_linear_affine_b4_tape": (_i32, [_vp, _vp, _i32, _vp]),
    "scr_tape_destroy": (_i32, [_vp]),
    "scr_fp8_repack_size": (_i32, [_i32, _i32, _psz]),
    "scr_fp8_repack": (_i32, [_vp, _vp, _vp, _i32, _i32, _vp, _vp]),
    "scr_fp8_act_size": (_i32, [_i32, _i32, _psz]),
    "scr_fp8_quant_per_token": (_i32, [_vp, _vp, _i32, _i32, _vp, _vp]),
    "scr_rmsnorm_fp8_quant": (_i32, [_vp, _vp, _vp, ctypes.c_float, _i32, _i32, _vp, _vp, _vp]),
    "scr_fp8_act_unpack": (_i32, [_vp, _vp, _i32, _i32, _vp, _vp, _vp]),
    "scr_e4m3_encode": (_i32, [_vp, _vp, _i64, _vp, _vp]),
    "scr_linear_fp8": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _sz, _vp]),
    "scr_linear_fp8_dynamic": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _vp, _sz, _vp]),
    "scr_linear_affine_b4_partial": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _sz, _vp]),
    "scr_linear_fp8_partial": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _sz, _vp]),
    "scr_linear_fp8_dynamic_partial": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _sz, _vp]),
    "scr_partial_to_bf16": (_i32, [_vp, _vp, _i64, _vp, _vp]),
    "scr_tp_comm_create": (_i32, [_vp, _i32, _i32, _i64, ctypes.POINTER(_vp), _vp]),
    "scr_tp_comm_connect": (_i32, [_vp, _vp]),
    "scr_tp_comm_base": (_i32, [_vp, ctypes.POINTER(_vp)]),
    "scr_tp_comm_connect_local": (_i32, [_vp, ctypes.POINTER(_vp), ctypes.POINTER(_i32)]),
    "scr_tp_comm_set_wait_limit": (_i32, [_vp, ctypes.c_uint32]),
    "scr_tp_allreduce_partial": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp]),
    "scr_tp_allgather_cols": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "scr_tp_comm_destroy": (_i32, [_vp]),
    "scr_linear_fp8_dynamic_allreduce": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "scr_linear_fp8_dynamic_static": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "scr_embed_bf16": (_i32, [_vp, _vp, _i32, _vp, _i32, _i32, _vp, _vp]),
    "scr_rmsnorm_bf16": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, ctypes.c_float, _vp]),
    "scr_fused_add_rmsnorm_bf16": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, ctypes.c_float, _vp]),
    "scr_silu_mul_bf16": (_i32, [_vp, _vp, _vp, _i64, _vp, _i32, _i32, _vp]),
    "scr_silu_mul_pairs8_bf16": (_i32, [_vp, _vp, _i64, _vp, _i32, _i32, _vp]),
    "scr_rope_append_bf16": (_i32, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _i32, _vp, _i64, _vp, _vp,
                                    _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "scr_attention_via_cache_bf16": (_i32, [_vp, _vp, _i64, _vp, _vp, _i32, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32,
                                            _i32, _i32, ctypes.c_float, _vp]),
    "scr_rope_attention_via_cache_bf16": (_i32, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _i32, _vp, _vp, _i32,
                                                 _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _i32, ctypes.c_float,
                                                 _vp]),
    "scr_argmax_bf16": (_i32, [_vp, _vp, _i64, _i32, _i32, _vp, _vp]),
}



class QmvEnds(ctypes.Structure):
    """`scr_qmv_ends` of include/scratchy_cuda.h."""
    _fields_ = [("norm_gain", _vp), ("norm_eps", ctypes.c_float), ("norm_gain_offset", ctypes.c_float), ("bias", _vp),
                ("scale", ctypes.c_float), ("residual", _i32), ("silu_pairs", _i32), ("norm_row_scale", _i32)]


class TapeLinear(ctypes.Structure):
    """`scr_tape_linear` of include/scratchy_cuda.h."""
    _fields_ = [("packed", _vp), ("x", _vp), ("y", _vp), ("N", _i32), ("K", _i32), ("group", _i32), ("dep", _i32 * 3)]


_lib = None
_lock = threading.Lock()


def lib() -> ctypes.CDLL:
    """Load the C-ABI library; raise (never fall back) if it has not been built."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(_LIB_PATH):
                raise ScratchyCudaError(-5, f"{_LIB_PATH} is missing: run `python -m scratchy_b200.build` "
                                            "(there is no CPU fallback)")
            L = ctypes.CDLL(_LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(L, name)          # AttributeError here = header and library disagree
                fn.restype, fn.argtypes = res, args
            _lib = L
    return _lib


class Context:
    """Owns one ``scr_ctx`` (one per device).  ``check`` turns a status into an exception."""

    def __init__(self, device: int = 0):
        self._h = _vp()
        st = lib().scr_cuda_init(int(device), ctypes.byref(self._h))
        if st != OK:
            raise ScratchyCudaError(st, f"scr_cuda_init(device={device})")
        self.device = int(device)

    @property
    def handle(self):
        return self._h

    def check(self, status: int) -> None:
        if status != OK:
            detail = lib().scr_last_error(self._h)
            raise ScratchyCudaError(status, detail.decode() if detail else "")

    def device_status(self, stream=None) -> None:
        """Synchronise and raise if a bounded device-side wait ran out (`scr_device_status`)."""
        self.check(lib().scr_device_status(self._h, stream, None))

    def launch_count(self) -> int:
        return int(lib().scr_launch_count(self._h))

    def close(self) -> None:
        if self._h:
            lib().scr_cuda_destroy(self._h)
            self._h = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_contexts: dict[int, Context] = {}


def context(device: int) -> Context:
    """Process-wide context of ``device``."""
    with _lock:
        c = _contexts.get(device)
    if c is None:
        c = Context(device)
        with _lock:
            _contexts[device] = c
    return c
