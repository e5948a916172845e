"""`scr_linear_fp8_dynamic_static`: the fp8 dynamic linear for callers that cannot allocate.

Some callers of this library have no device allocator on the step path (a runtime whose arena
already owns all device memory, code inside a no-allocation region, a thin FFI shim that owns
only the input and output tensors).  The entry point keeps the activation pack in an 8 MiB array
built into the library instead of a caller workspace.  It must produce exactly what
`scr_linear_fp8_dynamic` produces — bit for bit: up to 4 tokens that entry point takes the one-launch
self-quantising matvec while this one always quantises into the array first, and the two do the same
arithmetic statement for statement — also on a second call that finds the previous call's contents in
the array; it must not change the device's free memory; and it must refuse requests that do not fit.

This file sorts last on purpose, so a run that stops at the first failure has already run
every other test.
"""
import ctypes

import numpy as np
import pytest

from scratchy_b200 import synth

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _both(layer, x, M, N, K):
    import torch
    from scratchy_b200 import _lib
    ctx = _lib.context(0)
    L = _lib.lib()
    y_ref = layer.forward(x)
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ctx.check(L.scr_linear_fp8_dynamic_static(ctx.handle, _ptr(layer.packed), _ptr(x), M, N, K, _ptr(y), stream))
    torch.cuda.synchronize()
    # the first call above resolved the array's address; from here on a call must leave the device's memory alone
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(2):
        ctx.check(L.scr_linear_fp8_dynamic_static(ctx.handle, _ptr(layer.packed), _ptr(x), M, N, K, _ptr(y), stream))
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"the call changed the device's free memory by {free0 - free1} bytes"
    return y, y_ref


@pytest.mark.parametrize("N,K,M1,M2", [(384, 512, 3, 16), (512, 384, 200, 40), (256, 1024, 64, 2)])
def test_static_scratch_matches_workspace_entry_point_twice(N, K, M1, M2):
    import torch
    from scratchy_b200 import Fp8Linear
    rng = np.random.default_rng(3)
    w = torch.from_numpy(rng.integers(0, 0x7E, size=(N, K), dtype=np.uint8)).cuda()
    ws = torch.from_numpy((rng.random(N) * 1e-3 + 1e-4).astype(np.float32)).cuda()
    layer = Fp8Linear.from_tensors(w, ws)
    for M, seed in ((M1, 5), (M2, 6)):      # two calls in a row share the built-in array
        x = torch.from_numpy(synth.activations_bf16(M, K, seed).view(np.int16)).view(torch.bfloat16).cuda().reshape(M, K)
        y, y_ref = _both(layer, x, M, N, K)
        assert torch.equal(y, y_ref)        # the same arithmetic on the same bytes: bit-identical


def test_requests_beyond_the_array_are_refused():
    import torch
    from scratchy_b200 import _lib
    ctx = _lib.context(0)
    L = _lib.lib()
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = _ptr(buf)
    # M=4096 tokens x K=8192 needs a 32 MiB pack: refused before anything is launched
    st = L.scr_linear_fp8_dynamic_static(ctx.handle, p, p, 4096, 128, 8192, p, None)
    assert st == -6
    assert b"built-in array" in L.scr_last_error(ctx.handle)
    assert L.scr_linear_fp8_dynamic_static(ctx.handle, None, p, 1, 128, 128, p, None) == -1
