"""GPU parity of the fp8-dynamic-per-channel path against the CPU oracle (through the C ABI).

Bars: the e4m3 encoder and the per-token quantisation (x_q bytes, a_scale) are bit-exact;
bf16 outputs within relative L2 1e-3 of the oracle's f32-accumulated result.
"""
import ctypes
import glob
import os

import numpy as np
import pytest

import oracle
from scratchy_b200 import synth
from util import bf16_dev, bits_of, max_abs, rel_l2, to_dev

pytestmark = pytest.mark.gpu
REL_L2_TOL = 1e-3
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def make_layer(wq, ws):
    from scratchy_b200 import Fp8Linear
    return Fp8Linear.from_tensors(to_dev(wq), to_dev(ws))


def test_device_e4m3_encoder_matches_reference_rule():
    import torch
    from scratchy_b200 import _lib
    # every e4m3 grid point, every midpoint between neighbours (the exact ties), one ulp either
    # side of each, the subnormal grid, the [448, 464) band, specials, and a random sweep
    grid = oracle.e4m3_to_f32(np.arange(0, 0x7F, dtype=np.uint8))
    mids = ((grid[:-1].astype(np.float64) + grid[1:].astype(np.float64)) / 2).astype(np.float32)
    vals = [grid, mids, np.nextafter(mids, np.float32(0)), np.nextafter(mids, np.float32(1e9)),
            np.array([0.0, 448.0, 463.99, 464.0, 1e9, np.inf, np.nan, 2.0 ** -10, 2.0 ** -11, 3 * 2.0 ** -11,
                      1e-45, 0.015625, 0.0156249], np.float32)]
    rng = np.random.default_rng(0)
    vals.append((rng.standard_normal(200000) * 100).astype(np.float32))
    vals.append(rng.uniform(0, 0.02, 50000).astype(np.float32))
    v = np.concatenate(vals)
    v = np.concatenate([v, -v])
    want = oracle.f32_to_e4m3(v)
    ctx = _lib.context(0)
    dv = to_dev(v)
    out = torch.empty(v.size, dtype=torch.uint8, device="cuda")
    ctx.check(_lib.lib().scr_e4m3_encode(ctx.handle, ctypes.c_void_p(dv.data_ptr()), v.size,
                                         ctypes.c_void_p(out.data_ptr()), None))
    got = out.cpu().numpy()
    bad = np.argwhere(got != want)
    assert bad.size == 0, f"{bad.size} mismatches, first v={v[bad[0, 0]]!r} got={got[bad[0, 0]]:#x} want={want[bad[0, 0]]:#x}"


@pytest.mark.parametrize("M,K", [(1, 3584), (16, 3584), (3, 256), (5, 72), (40, 512), (300, 384), (2, 18944)])
def test_quant_per_token_bit_exact(M, K):
    from scratchy_b200 import Fp8Linear
    x = synth.activations_bf16(M, K, synth.seed_for("q", M, K))
    x.reshape(-1)[:3] = synth.f32_to_bf16_bits(np.array([0.0, -0.0, 37.5], np.float32))
    if M > 1:
        x[1, :] = 0                                     # an all-zero (padded) row keeps the scale floor
    pack = Fp8Linear.quantize_activation(bf16_dev(x).reshape(M, K))
    xq, a = pack.unpack()
    want_q, want_a = oracle.fp8_quant_per_token(x, M, K)
    assert np.array_equal(a.cpu().numpy(), want_a)
    assert np.array_equal(xq.cpu().numpy(), want_q)
    rne_q, _ = oracle.fp8_quant_per_token(x, M, K, rne=True)
    print(f"M={M} K={K}: bytes that differ under a round-half-even encoder: {int((rne_q != want_q).sum())}")


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "fp8_*.npz"))))
def test_golden_fixtures(path):
    import torch
    from scratchy_b200 import Fp8Linear
    g = np.load(path)
    N, K = g["wq"].shape
    M = g["x"].shape[0]
    layer = make_layer(g["wq"], g["w_scale"])
    xdev = bf16_dev(g["x"]).reshape(M, K)
    pack = Fp8Linear.quantize_activation(xdev)
    xq, a = pack.unpack()
    assert np.array_equal(xq.cpu().numpy(), g["xq"]) and np.array_equal(a.cpu().numpy(), g["a_scale"])
    y1 = bits_of(layer.forward_quantized(pack)).reshape(M, N)
    y2 = bits_of(layer.forward(xdev)).reshape(M, N)
    torch.cuda.synchronize()
    assert np.array_equal(y1, y2)
    assert rel_l2(y1, g["y"]) <= REL_L2_TOL


def run_case(N, K, M, seed):
    import torch
    wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(N, K, seed))
    x = synth.activations_bf16(M, K, seed + 1)
    layer = make_layer(wq, ws)
    y = layer.forward(bf16_dev(x).reshape(M, K))
    torch.cuda.synchronize()
    want = oracle.fp8_dynamic_linear(x, wq, ws, M, N, K)
    return bits_of(y).reshape(M, N), want


@pytest.mark.parametrize("name", ["q", "k", "gate", "down"])
@pytest.mark.parametrize("M", [1, 16])
def test_qwen_7b_shapes_decode(name, M):
    K, N = synth.QWEN_2_5_7B[name]
    got, want = run_case(N, K, M, synth.seed_for("fp8", N, K, M))
    r = rel_l2(got, want)
    print(f"{name} M={M} rel_l2={r:.3e} max_abs={max_abs(got, want):.3e}")
    assert r <= REL_L2_TOL


@pytest.mark.parametrize("N,K,M", [(8, 64, 1), (24, 200, 5), (130, 328, 9), (100, 1024, 16), (256, 512, 64), (384, 256, 33)])
def test_ragged_and_small_shapes(N, K, M):
    got, want = run_case(N, K, M, synth.seed_for("f8r", N, K, M))
    assert rel_l2(got, want) <= REL_L2_TOL


def test_weight_only_program_bound():
    """The reference's own fp8 check (triton_splice_golden.rs:1690-1726): weight-only math on its
    formula inputs, max-abs < 0.05 against the host loop.  The W8A8 result obeys the same bound."""
    import torch
    m, k, n = 4, 256, 128
    a = np.array([(i % 13) * np.float32(0.01) - np.float32(0.06) for i in range(m * k)], np.float32).reshape(m, k)
    w_val = np.array([(i % 17) * np.float32(0.02) - np.float32(0.16) for i in range(k * n)], np.float32)
    wq = oracle.f32_to_e4m3(w_val).reshape(n, k)
    ws = np.array([(i % 7) * np.float32(0.05) + np.float32(0.1) for i in range(n)], np.float32)
    want = oracle.fp8_weight_only_linear(a, wq, ws, m, n, k)
    layer = make_layer(wq, ws)
    y = layer.forward(bf16_dev(synth.f32_to_bf16_bits(a)).reshape(m, k))
    torch.cuda.synchronize()
    got = y.float().cpu().numpy()
    assert np.max(np.abs(got - want)) < 0.05


def test_determinism_full_size():
    import torch
    K, N = synth.QWEN_2_5_7B["gate"]
    wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(N, K, 3))
    layer = make_layer(wq, ws)
    x = bf16_dev(synth.activations_bf16(4, K, 4)).reshape(4, K)
    y1, y2 = layer.forward(x), layer.forward(x)
    y3 = layer.forward(x * 2)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    assert torch.equal(y1 * 2, y3)       # the per-token scale doubles, x_q is unchanged


# ---------------------------------------------------------------- prefill (tensor-core GEMM, M > 16)
def _device_ok():
    from scratchy_b200 import _lib
    _lib.context(0).device_status()


@pytest.mark.parametrize("N,K,M", [(128, 128, 32), (128, 256, 128), (256, 512, 130), (384, 200, 200), (130, 328, 77),
                                   (512, 384, 300)])
def test_prefill_gemm_small(N, K, M):
    got, want = run_case(N, K, M, synth.seed_for("g8", N, K, M))
    _device_ok()
    r = rel_l2(got, want)
    print(f"N={N} K={K} M={M} rel_l2={r:.3e} max_abs={max_abs(got, want):.3e}")
    assert r <= REL_L2_TOL


@pytest.mark.parametrize("name,M", [("k", 256), ("q", 256)])
def test_prefill_gemm_qwen_shapes_full_oracle(name, M):
    K, N = synth.QWEN_2_5_7B[name]
    got, want = run_case(N, K, M, synth.seed_for("g8f", N, K, M))
    _device_ok()
    r = rel_l2(got, want)
    print(f"{name} M={M} rel_l2={r:.3e} max_abs={max_abs(got, want):.3e}")
    assert r <= REL_L2_TOL


@pytest.mark.parametrize("M", [256, 2048, 8192])
@pytest.mark.parametrize("name", ["q", "k", "gate", "down"])
def test_prefill_gemm_full_size_sampled_rows(name, M):
    """Every prefill cell of the Qwen2.5-7B sweep (v has k's shape, up has gate's; down at 8192 tokens takes the
    tail-split plan): oracle on a seeded subset of 16 token rows; x_q and a_scale of those rows must be bit-exact
    and the outputs within tolerance; the whole output must be finite."""
    import torch
    from scratchy_b200 import Fp8Linear
    K, N = synth.QWEN_2_5_7B[name]
    wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(N, K, synth.seed_for("g8s", N, K)))
    x = synth.activations_bf16(M, K, synth.seed_for("g8sx", M, K))
    layer = make_layer(wq, ws)
    xdev = bf16_dev(x).reshape(M, K)
    y = layer.forward(xdev)
    torch.cuda.synchronize()
    _device_ok()
    assert bool(torch.isfinite(y.float()).all())
    rows = np.sort(np.random.default_rng(1).choice(M, 16, replace=False))
    xq_want, a_want = oracle.fp8_quant_per_token(x[rows], len(rows), K)
    xq, a = Fp8Linear.quantize_activation(xdev).unpack()
    assert np.array_equal(xq.cpu().numpy()[rows], xq_want) and np.array_equal(a.cpu().numpy()[rows], a_want)
    want = oracle.fp8_linear(xq_want, a_want, wq, ws, len(rows), N, K)
    got = bits_of(y).reshape(M, N)[rows]
    r = rel_l2(got, want)
    print(f"{name} M={M} sampled rel_l2={r:.3e} max_abs={max_abs(got, want):.3e}")
    assert r <= REL_L2_TOL


@pytest.mark.parametrize("N,K,M", [(3584, 3584, 1), (512, 3584, 4), (18944, 3584, 2), (130, 328, 3), (24, 200, 1),
                                  (1280, 8192, 2), (8192, 1024, 1), (64, 16384, 1)])
def test_matvec_quantises_by_itself_with_the_same_bits(N, K, M):
    """For M <= 4 (and up to 14 KiB of codes) the whole linear is one launch: the matvec computes a_scale and x_q in
    shared memory.
    Its output must equal, bit for bit, the two-step path (quantise kernel, then the matvec on the pack),
    and the f32 partial variant must equal the pack's partial variant."""
    import torch
    from scratchy_b200 import Fp8Linear, _lib
    wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(N, K, synth.seed_for("fuse", N, K)))
    layer = make_layer(wq, ws)
    x = bf16_dev(synth.activations_bf16(M, K, 7)).reshape(M, K)
    n0 = _lib.context(0).launch_count()
    fused = layer.forward(x)
    fuses = M <= 4 and M * ((K + 15) // 16 * 16) <= 14 * 1024          # beyond that the quantise kernel runs once
    assert _lib.context(0).launch_count() - n0 == (1 if fuses else 2)
    two_step = layer.forward_quantized(Fp8Linear.quantize_activation(x))
    part = layer.forward_partial(x)
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(fused), bits_of(two_step))
    assert np.array_equal(bits_of(part.to(torch.bfloat16)), bits_of(fused))
    want = oracle.fp8_dynamic_linear(bits_of(x).reshape(M, K), wq, ws, M, N, K)
    assert rel_l2(bits_of(fused).reshape(M, N), want) <= REL_L2_TOL


@pytest.mark.parametrize("M,K", [(1, 3584), (16, 8192), (40, 3584), (300, 256), (3, 72)])
def test_rmsnorm_fused_with_the_quantisation(M, K):
    """The W8A8 activation producer straight from the residual stream (norm-side quantisation,
    crates/targets/metal/src/shaders/norm_w4a8_quant.h:1-12): codes, scales and the bf16 normed rows must equal the
    two-kernel path (rmsnorm, then quantise) bit for bit, and the oracle within its bars."""
    import torch
    from scratchy_b200 import Fp8Linear, decode
    from util import bf16_to_f32
    rng = np.random.default_rng(synth.seed_for("normq", M, K))
    xb = synth.f32_to_bf16_bits((rng.standard_normal((M, K)) * 2.0).astype(np.float32))
    gb = synth.f32_to_bf16_bits((1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32))
    x, g = bf16_dev(xb).reshape(M, K), bf16_dev(gb)
    normed = torch.empty((M, K), dtype=torch.bfloat16, device="cuda")
    fused = Fp8Linear.quantize_rmsnorm(x, g, 1e-5, normed_out=normed)
    two_norm = decode.rmsnorm(x, g, 1e-5)
    two = Fp8Linear.quantize_activation(two_norm)
    xq_a, sc_a = fused.unpack()
    xq_b, sc_b = two.unpack()
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(normed), bits_of(two_norm))
    assert torch.equal(xq_a, xq_b) and torch.equal(sc_a, sc_b)
    want_norm = synth.f32_to_bf16_bits(oracle.rmsnorm(bf16_to_f32(xb), bf16_to_f32(gb), 1e-5))
    assert rel_l2(bits_of(normed).reshape(M, K), want_norm) <= REL_L2_TOL
    want_q, want_s = oracle.fp8_quant_per_token(want_norm, M, K)
    assert np.allclose(sc_a.cpu().numpy(), want_s, rtol=1e-2)
    assert np.mean(xq_a.cpu().numpy().reshape(M, K) == want_q) > 0.97


@pytest.mark.parametrize("N,K,M", [(3584, 3584, 1), (512, 3584, 1), (512, 3584, 16), (512, 3584, 64), (3584, 3584, 2048),
                                   (1000, 1088, 3)])
def test_linear_bias_in_the_epilogue(N, K, M):
    """`{prefix}.bias` on the fp8 path (Qwen2.5's q/k/v carry one): added in f32 to the dequantised sum before the one
    rounding (the order of crates/targets/metal/shaders/quantized_qmv.metal:104-112), on the self-quantising matvec,
    the pack matvec and the tensor-core GEMM."""
    import torch
    from scratchy_b200 import Fp8Linear
    wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(N, K, synth.seed_for("f8bias", N, K, M)))
    x = synth.activations_bf16(M, K, synth.seed_for("f8biasx", N, K, M))
    rng = np.random.default_rng(synth.seed_for("f8biasb", N, K, M))
    bias = synth.f32_to_bf16_bits(rng.normal(0.0, 2.0, N).astype(np.float32))
    layer = Fp8Linear.from_tensors(to_dev(wq), to_dev(ws), linear_bias=bf16_dev(bias))
    y = bits_of(layer.forward(bf16_dev(x).reshape(M, K))).reshape(M, N)
    torch.cuda.synchronize()
    rows = np.arange(M) if M <= 64 else np.sort(np.random.default_rng(1).choice(M, 48, replace=False))
    xs = x.reshape(M, K)[rows]
    want = oracle.fp8_dynamic_linear_bias(xs, wq, ws, bias, len(rows), N, K)
    plain = oracle.fp8_dynamic_linear(xs, wq, ws, len(rows), N, K)
    r = rel_l2(y[rows], want)
    print(f"fp8 bias N={N} K={K} M={M} rel_l2={r:.3e} max_abs={max_abs(y[rows], want):.3e}")
    assert r <= REL_L2_TOL
    assert rel_l2(y[rows], plain) > 0.1, "the bias must have been applied"


@pytest.mark.parametrize("N,K,M", [(18944, 384, 512), (18944, 256, 768), (4864, 3584, 2048)])
def test_two_cta_gemm_against_the_oracle(N, K, M):
    """Shapes the CTA-pair kernel takes (whole 256 x 256 tiles, full rounds of 74 pairs; K = 384 is an odd number of
    k-tiles, so the last ring stage is half full): bf16 with a bias, the unrounded f32 partials of a row-parallel layer,
    and run-to-run identical bits.  Rows are sampled over both CTAs of a pair."""
    import torch
    from scratchy_b200 import Fp8Linear
    wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(N, K, synth.seed_for("pair", N, K, M)))
    x = synth.activations_bf16(M, K, synth.seed_for("pairx", N, K, M))
    bias = synth.f32_to_bf16_bits(np.random.default_rng(7).normal(0.0, 2.0, N).astype(np.float32))
    xd = bf16_dev(x).reshape(M, K)
    layer = Fp8Linear.from_tensors(to_dev(wq), to_dev(ws), linear_bias=bf16_dev(bias))
    y = layer.forward(xd)
    y2 = layer.forward(xd)
    plain = Fp8Linear.from_tensors(to_dev(wq), to_dev(ws))
    part = plain.forward_partial(xd)
    torch.cuda.synchronize()
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))
    rows = np.unique(np.concatenate([np.arange(0, M, 37), [0, 127, 128, 255, 256, M - 129, M - 128, M - 1]]))
    xs = x.reshape(M, K)[rows]
    want = oracle.fp8_dynamic_linear_bias(xs, wq, ws, bias, len(rows), N, K)
    assert rel_l2(bits_of(y).reshape(M, N)[rows], want) <= REL_L2_TOL
    _, acc = oracle.fp8_dynamic_linear(xs, wq, ws, len(rows), N, K, want_f32=True)
    got = part.cpu().numpy().reshape(M, N)[rows].astype(np.float64)
    assert np.linalg.norm(got - acc) / np.linalg.norm(acc) <= 1e-5
    from scratchy_b200 import _lib
    _lib.context(0).device_status(None)


def test_misaligned_pointers_are_refused_on_the_host():
    """Every fp8 forward entry point refuses a pointer that is not 16-byte aligned with SCR_E_ALIGN before anything
    is launched: the matvec's bulk copies would otherwise fault on the device."""
    import torch
    from scratchy_b200 import _lib
    ctx = _lib.context(0)
    L = _lib.lib()
    N, K = 64, 128
    wq, ws = oracle.fp8_quantize_weight_per_channel(synth.fp8_weights_f32(N, K, 3))
    layer = make_layer(wq, ws)
    x = torch.zeros((17, K), dtype=torch.bfloat16, device="cuda")
    y = torch.empty((17, N), dtype=torch.bfloat16, device="cuda")
    wsz = layer.workspace_bytes(17)
    wsb = torch.empty(wsz + 64, dtype=torch.uint8, device="cuda")
    p, xp, yp, wp = layer.packed.data_ptr(), x.data_ptr(), y.data_ptr(), wsb.data_ptr()
    before = ctx.launch_count()
    for M in (1, 17):
        assert L.scr_linear_fp8_dynamic(ctx.handle, p + 2, xp, M, N, K, None, yp, wp, wsb.numel(), None) == -3
        assert L.scr_linear_fp8_dynamic(ctx.handle, p, xp + 2, M, N, K, None, yp, wp, wsb.numel(), None) == -3
        assert L.scr_linear_fp8_dynamic_static(ctx.handle, p + 2, xp, M, N, K, yp, None) == -3
        assert L.scr_linear_fp8_dynamic_static(ctx.handle, p, xp + 2, M, N, K, yp, None) == -3
        assert L.scr_linear_fp8(ctx.handle, p + 2, wp, M, N, K, None, yp, wp, wsb.numel(), None) == -3
        assert L.scr_linear_fp8(ctx.handle, p, wp + 2, M, N, K, None, yp, wp, wsb.numel(), None) == -3
    assert ctx.launch_count() == before, "a refused call must not launch anything"
