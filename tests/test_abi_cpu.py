"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

from scratchy_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "scratchy_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(scr_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = ctypes.CDLL(_lib.lib_path())
    names = header_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/scratchy_cuda.h but not exported"


def test_binding_table_matches_header():
    assert sorted(_lib.SIGNATURES) == header_symbols()


def test_status_strings():
    L = _lib.lib()
    assert L.scr_status_string(0) == b"SCR_OK"
    assert L.scr_status_string(-2) == b"SCR_E_SHAPE"
    assert L.scr_status_string(-123) == b"SCR_E_UNKNOWN"


def test_affine_repack_size_law():
    L = _lib.lib()
    s = ctypes.c_size_t()
    # 4.5 bits per weight: codes + bf16 scale and bias per group of 64, no padding at 128-multiples,
    # plus a 128-byte trailer
    assert L.scr_affine_b4_repack_size(8192, 3072, 64, ctypes.byref(s)) == 0
    assert s.value == 8192 * 3072 // 2 + 2 * 2 * 8192 * 3072 // 64 + 128
    # rows pad to 128, k to 128
    assert L.scr_affine_b4_repack_size(8, 64, 64, ctypes.byref(s)) == 0
    assert s.value == (128 // 16) * 1 * 1152 + 128
    # the sibling presets: groups of 32 carry four (scale, bias) entries per row and 128 k, groups of 128 store theirs twice
    assert L.scr_affine_b4_repack_size(256, 256, 32, ctypes.byref(s)) == 0
    assert s.value == (256 // 16) * 2 * 1280 + 128
    assert L.scr_affine_b4_repack_size(256, 256, 128, ctypes.byref(s)) == 0
    assert s.value == (256 // 16) * 2 * 1152 + 128
    # the preset's law: K % group == 0, groups of 32, 64 or 128 (crates/compiler/subtile/src/lower.rs:112-127)
    assert L.scr_affine_b4_repack_size(16, 96, 64, ctypes.byref(s)) == -2
    assert L.scr_affine_b4_repack_size(16, 192, 128, ctypes.byref(s)) == -2
    assert L.scr_affine_b4_repack_size(16, 96, 48, ctypes.byref(s)) == -4
    assert L.scr_affine_b4_repack_size(0, 128, 64, ctypes.byref(s)) == -2
    assert L.scr_affine_b4_repack_size(16, 128, 64, None) == -1


def test_fp8_sizes():
    L = _lib.lib()
    s = ctypes.c_size_t()
    assert L.scr_fp8_repack_size(3584, 3584, ctypes.byref(s)) == 0
    assert s.value == 3584 * 3584 + 3584 * 4
    assert L.scr_fp8_repack_size(100, 200, ctypes.byref(s)) == 0
    assert s.value == 128 * 256 + 128 * 4
    assert L.scr_fp8_act_size(1, 3584, ctypes.byref(s)) == 0
    assert s.value == 128 + 3584
    assert L.scr_fp8_act_size(0, 3584, ctypes.byref(s)) == -2
    assert L.scr_linear_workspace_size(0, 1, 8192, 3072, ctypes.byref(s)) == 0 and s.value == 0
    assert L.scr_linear_workspace_size(1, 4, 512, 3584, ctypes.byref(s)) == 0 and s.value >= 128 + 4 * 3584
    assert L.scr_linear_workspace_size(7, 4, 512, 3584, ctypes.byref(s)) == -1


def test_null_context_is_an_argument_error_not_a_crash():
    L = _lib.lib()
    assert L.scr_linear_affine_b4(None, None, None, 1, 16, 64, 64, None, None, None, 0, None) == -1
    assert L.scr_fp8_quant_per_token(None, None, 1, 64, None, None) == -1
    assert L.scr_cuda_destroy(None) == -1
    assert L.scr_launch_count(None) == 0


def test_init_without_a_gpu_reports_cuda_error():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = ctypes.c_void_p()
    assert _lib.lib().scr_cuda_init(0, ctypes.byref(h)) == -5
    assert not h.value
    with pytest.raises(_lib.ScratchyCudaError):
        _lib.Context(0)


def test_struct_mirrors_have_the_layout_the_c_compiler_gives(tmp_path):
    """The ctypes mirrors of the header's structs (`scr_qmv_ends`, `scr_tape_linear`) against the C compiler's own sizes
    and field offsets: a field added to the header and not to the mirror (or in another place) would shift every
    argument after it."""
    import shutil
    import subprocess
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    fields = {"scr_qmv_ends": [f[0] for f in _lib.QmvEnds._fields_], "scr_tape_linear": [f[0] for f in _lib.TapeLinear._fields_]}
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "scratchy_cuda.h"', 'int main(void) {']
    for s, fs in fields.items():
        lines.append(f'  printf("{s} %zu\\n", sizeof({s}));')
        for f in fs:
            lines.append(f'  printf("{s}.{f} %zu\\n", offsetof({s}, {f}));')
    lines += ['  return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.check_call([cc, "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    got = dict(line.split() for line in subprocess.check_output([str(exe)], text=True).splitlines())
    for s, cls in (("scr_qmv_ends", _lib.QmvEnds), ("scr_tape_linear", _lib.TapeLinear)):
        assert int(got[s]) == ctypes.sizeof(cls), s
        for f in fields[s]:
            assert int(got[f"{s}.{f}"]) == getattr(cls, f).offset, f"{s}.{f}"
