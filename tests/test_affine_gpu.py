"""GPU parity of the MLX affine int4 path against the CPU oracle (through the C ABI).

Bars: dequantised weights bit-exact; bf16 outputs within relative L2 1e-3 of the oracle's
f32-accumulated result (the tolerance the baseline configuration states), max-abs printed.
"""
import ctypes
import glob
import os

import numpy as np
import pytest

import oracle
from scratchy_b200 import synth
from util import bf16_dev, bits_of, max_abs, rel_l2, u32_dev

pytestmark = pytest.mark.gpu
REL_L2_TOL = 1e-3
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def make_layer(w, s, b):
    from scratchy_b200 import AffineQuantLinear
    return AffineQuantLinear.from_tensors(u32_dev(w), bf16_dev(s), bf16_dev(b), 64, 4)


def run_case(N, K, M, seed, w=None, s=None, b=None, x=None):
    import torch
    if w is None:
        w, s, b = synth.affine_int4_weights(N, K, 64, seed)
        x = synth.activations_bf16(M, K, seed + 1)
    layer = make_layer(w, s, b)
    y = layer.forward(bf16_dev(x).reshape(M, K))
    torch.cuda.synchronize()
    want = oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), s, b, x, M, N, K, 64)
    got = bits_of(y).reshape(M, N)
    return got, want


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "affine_b4_*.npz"))))
def test_golden_fixtures(path):
    import torch
    g = np.load(path)
    N, K, M = g["w"].shape[0], g["w"].shape[1] * 8, g["x"].shape[0]
    layer = make_layer(g["w"], g["scales"], g["biases"])
    wd = bits_of(layer.dequantize()).reshape(N, K)
    assert np.array_equal(wd, g["w_dequant"]), "dequantised weights must be bit-exact"
    y = bits_of(layer.forward(bf16_dev(g["x"]).reshape(M, K))).reshape(M, N)
    torch.cuda.synchronize()
    assert rel_l2(y, g["y"]) <= REL_L2_TOL


@pytest.mark.parametrize("N,K", [(8192, 3072), (1024, 3072), (3072, 8192), (8, 64), (24, 192), (130, 320)])
def test_dequant_bit_exact(N, K):
    w, s, b = synth.affine_int4_weights(N, K, 64, synth.seed_for("deq", N, K))
    layer = make_layer(w, s, b)
    got = bits_of(layer.dequantize()).reshape(N, K)
    want = oracle.affine_dequant_b4(w.view(np.uint8).reshape(-1), s, b, N, K, 64)
    assert np.array_equal(got, want)


def test_dequant_bit_exact_adversarial_scales():
    """Scales/biases that stress the rounding contract: the reference test distribution
    (scales 0.01+0.04u, biases u-0.5), zero scale/bias, tiny biases far below the product
    (the double-rounding case), large magnitudes, negative scales, subnormal values."""
    N, K = 64, 256
    rng = np.random.default_rng(5)
    w, s, b = synth.affine_int4_weights(N, K, 64, 9)
    G = K // 64
    sf = (0.01 + 0.04 * rng.random((N, G))).astype(np.float32)
    bf = (rng.random((N, G)) - 0.5).astype(np.float32)
    sf[0] = 0.0
    bf[1] = 0.0
    bf[2] = 1e-30
    bf[3] = -1e-20
    sf[4] = 1.5
    bf[4] = 2.0 ** -14
    sf[5] = -0.037
    sf[6] = 3.0e4
    bf[6] = -2.4e5
    sf[7] = 1e-40
    bf[8] = 1e-39
    sf[9] = 1.0078125       # 1 + 2^-7 : products land on bf16 half-way points for odd codes
    bf[9] = 2.0 ** -20
    sf[10] = 1.0078125
    bf[10] = -(2.0 ** -30)
    sf[11] = 257.0
    bf[11] = 1e-6
    s = synth.f32_to_bf16_bits(sf)
    b = synth.f32_to_bf16_bits(bf)
    layer = make_layer(w, s, b)
    got = bits_of(layer.dequantize()).reshape(N, K)
    want = oracle.affine_dequant_b4(w.view(np.uint8).reshape(-1), s, b, N, K, 64)
    bad = np.argwhere(got != want)
    assert bad.size == 0, f"first mismatches (row, k): {bad[:8].tolist()}"


def test_config0_single_linear_m1():
    """Benchmark configuration 0: M=1, K=3072, N=8192, seed 0."""
    w, s, b = synth.affine_int4_weights(8192, 3072, 64, 0)
    x = synth.activations_bf16(1, 3072, 1)
    got, want = run_case(8192, 3072, 1, 0, w, s, b, x)
    r = rel_l2(got, want)
    print(f"config0 rel_l2={r:.3e} max_abs={max_abs(got, want):.3e} exact={np.mean(got == want):.4f}")
    assert r <= REL_L2_TOL


@pytest.mark.parametrize("name", ["q", "k", "gate", "down"])
@pytest.mark.parametrize("M", [1, 4, 16])
def test_llama_3b_shapes_decode(name, M):
    K, N = synth.LLAMA_3_2_3B[name]
    got, want = run_case(N, K, M, synth.seed_for("aff", N, K, M))
    r = rel_l2(got, want)
    print(f"{name} M={M} rel_l2={r:.3e} max_abs={max_abs(got, want):.3e}")
    assert r <= REL_L2_TOL


@pytest.mark.parametrize("N,K,M", [(8, 64, 1), (16, 64, 2), (24, 192, 5), (130, 320, 9), (100, 1024, 16), (48, 128, 7)])
def test_ragged_and_small_shapes(N, K, M):
    got, want = run_case(N, K, M, synth.seed_for("rag", N, K, M))
    assert rel_l2(got, want) <= REL_L2_TOL


@pytest.mark.parametrize("M", [17, 64, 100])
def test_prefill_rows_small_matrix(M):
    got, want = run_case(256, 512, M, synth.seed_for("pre", M))
    assert rel_l2(got, want) <= REL_L2_TOL


def test_linearity_and_determinism_full_size():
    """Size-independent properties at a full layer shape: y(2x) == 2 y(x) exactly (power-of-two
    scaling commutes with every rounding), and two runs are bit-identical (fixed reduction order)."""
    import torch
    K, N = synth.LLAMA_3_2_3B["gate"]
    w, s, b = synth.affine_int4_weights(N, K, 64, 3)
    layer = make_layer(w, s, b)
    x = bf16_dev(synth.activations_bf16(4, K, 4)).reshape(4, K)
    y1 = layer.forward(x)
    y2 = layer.forward(x)
    y3 = layer.forward(x * 2)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    assert torch.equal(y1 * 2, y3)


def test_zero_activation_gives_zero():
    import torch
    w, s, b = synth.affine_int4_weights(64, 128, 64, 3)
    layer = make_layer(w, s, b)
    y = layer.forward(torch.zeros((3, 128), dtype=torch.bfloat16, device="cuda"))
    assert not y.any()


def test_error_codes_through_the_abi():
    import torch
    from scratchy_b200 import _lib
    ctx = _lib.context(0)
    L = _lib.lib()
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = ctypes.c_void_p(buf.data_ptr())
    assert L.scr_linear_affine_b4(ctx.handle, p, p, 1, 16, 96, 64, None, p, None, 0, None) == -2     # K % group
    assert L.scr_linear_affine_b4(ctx.handle, p, p, 1, 16, 96, 48, None, p, None, 0, None) == -4     # groups are 32, 64 or 128
    assert L.scr_linear_affine_b4(ctx.handle, p, p, 0, 16, 128, 64, None, p, None, 0, None) == -2    # M
    assert L.scr_linear_affine_b4(ctx.handle, None, p, 1, 16, 128, 64, None, p, None, 0, None) == -1
    mis = ctypes.c_void_p(buf.data_ptr() + 4)
    assert L.scr_linear_affine_b4(ctx.handle, mis, p, 1, 16, 128, 64, None, p, None, 0, None) == -3
    assert b"aligned" in L.scr_last_error(ctx.handle)


# ---------------------------------------------------------------- prefill (tensor-core GEMM, M > 16)
def _device_ok():
    from scratchy_b200 import _lib
    _lib.context(0).device_status()


@pytest.mark.parametrize("N,K,M", [(128, 128, 32), (128, 256, 128), (256, 512, 130), (384, 192, 200), (130, 320, 77)])
def test_prefill_gemm_small(N, K, M):
    got, want = run_case(N, K, M, synth.seed_for("g4", N, K, M))
    _device_ok()
    r = rel_l2(got, want)
    print(f"N={N} K={K} M={M} rel_l2={r:.3e} max_abs={max_abs(got, want):.3e}")
    assert r <= REL_L2_TOL


@pytest.mark.parametrize("name,M", [("k", 512), ("q", 64)])
def test_prefill_gemm_llama_shapes_full_oracle(name, M):
    K, N = synth.LLAMA_3_2_3B[name]
    got, want = run_case(N, K, M, synth.seed_for("g4f", N, K, M))
    _device_ok()
    r = rel_l2(got, want)
    print(f"{name} M={M} rel_l2={r:.3e} max_abs={max_abs(got, want):.3e}")
    assert r <= REL_L2_TOL


@pytest.mark.parametrize("M", [64, 512, 2048])
@pytest.mark.parametrize("name", ["q", "k", "gate", "down"])
def test_prefill_gemm_full_size_sampled_rows(name, M):
    """Every prefill cell of the Llama-3.2-3B sweep (o has q's shape, v has k's, up has gate's; each (M, N, K) picks
    its own tile and split-K plan): the oracle evaluates a seeded subset of 24 token rows (each output row depends
    only on its own activation row), and the whole output must be finite."""
    import torch
    K, N = synth.LLAMA_3_2_3B[name]
    w, s, b = synth.affine_int4_weights(N, K, 64, synth.seed_for("g4s", N, K))
    x = synth.activations_bf16(M, K, synth.seed_for("g4sx", M, K))
    layer = make_layer(w, s, b)
    y = layer.forward(bf16_dev(x).reshape(M, K))
    torch.cuda.synchronize()
    _device_ok()
    assert bool(torch.isfinite(y.float()).all())
    rows = np.sort(np.random.default_rng(1).choice(M, 24, replace=False))
    want = oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), s, b, x[rows], len(rows), N, K, 64)
    got = bits_of(y).reshape(M, N)[rows]
    r = rel_l2(got, want)
    print(f"{name} M={M} sampled rel_l2={r:.3e} max_abs={max_abs(got, want):.3e}")
    assert r <= REL_L2_TOL


def test_prefill_matches_decode_kernel_rows():
    """The GEMM and the matvec expand identical bf16 weights, so a row computed in a batch of 64
    must match the same row computed alone up to f32 summation order."""
    import torch
    K, N = 1024, 512
    w, s, b = synth.affine_int4_weights(N, K, 64, 77)
    layer = make_layer(w, s, b)
    x = bf16_dev(synth.activations_bf16(64, K, 78)).reshape(64, K)
    yb = layer.forward(x)
    y1 = layer.forward(x[5:6])
    torch.cuda.synchronize()
    _device_ok()
    assert rel_l2(bits_of(yb[5:6]), bits_of(y1)) <= 2e-4


@pytest.mark.parametrize("M", [1, 7, 40])
def test_rows_concat_equals_its_parts(M):
    """crates/targets/metal/src/layers_quant.rs:363-450: the fused projection's rows are its parts' rows in
    order: its dequantised rows are the parts' rows bit for bit, and its output columns are the parts'
    outputs side by side (up to the f32 summation order, which the launch shape picks from N)."""
    import torch
    from scratchy_b200 import AffineQuantLinear, GpuWeights
    K, rows = 512, {"q": 384, "k": 128, "v": 128}
    ck, parts = {}, {}
    for i, (name, n) in enumerate(rows.items()):
        w, s, b = synth.affine_int4_weights(n, K, 64, 40 + i)
        ck[f"a.{name}.weight"], ck[f"a.{name}.scales"], ck[f"a.{name}.biases"] = u32_dev(w), bf16_dev(s), bf16_dev(b)
        parts[name] = make_layer(w, s, b)
    fused = AffineQuantLinear.load_rows_concat(GpuWeights(ck), ["a.q", "a.k", "a.v"], 64, 4, K)
    assert fused.out_features == 640 and fused.in_features == K
    x = bf16_dev(synth.activations_bf16(M, K, 50)).reshape(M, K)
    got = bits_of(fused.forward(x)).reshape(M, 640)
    want = np.concatenate([bits_of(parts[n].forward(x)).reshape(M, -1) for n in rows], axis=1)
    torch.cuda.synchronize()
    wd = np.concatenate([bits_of(parts[n].dequantize()) for n in rows], axis=0)
    assert np.array_equal(bits_of(fused.dequantize()), wd)
    assert rel_l2(got, want) <= 1e-4 and np.mean(got == want) > 0.99


@pytest.mark.parametrize("M", [1, 5, 16, 40])
@pytest.mark.parametrize("inter,K", [(1024, 512), (200, 256), (8192, 3072)])
def test_gate_up_with_fused_silu_mul(M, inter, K):
    """`FusedGateUpSiluMul` (crates/targets/metal/src/cpu_golden.rs:211-219) as the matvec's epilogue: against the
    oracle (two linears rounded to bf16, then silu*up in f32), and — up to 16 tokens — bit for bit against the
    unfused path on the same interleaved matrix (linear, then the pairing silu*up kernel)."""
    import torch
    from scratchy_b200 import AffineQuantLinear, GpuWeights, _lib
    from util import bf16_to_f32
    ck, host = {}, {}
    for i, name in enumerate(("gate", "up")):
        w, s, b = synth.affine_int4_weights(inter, K, 64, synth.seed_for("gu", inter, K) + i)
        host[name] = (w, s, b)
        ck[f"m.{name}.weight"], ck[f"m.{name}.scales"], ck[f"m.{name}.biases"] = u32_dev(w), bf16_dev(s), bf16_dev(b)
    lin = AffineQuantLinear.load_rows_interleave8(GpuWeights(ck), "m.gate", "m.up", 64, 4, K)
    xb = synth.activations_bf16(M, K, 77)
    x = bf16_dev(xb).reshape(M, K)
    n0 = _lib.context(0).launch_count()
    got = bits_of(lin.forward_silu_mul(x)).reshape(M, inter)
    launches = _lib.context(0).launch_count() - n0
    torch.cuda.synchronize()
    g, u = (oracle.affine_qmm_t_b4(host[n][0].view(np.uint8).reshape(-1), host[n][1], host[n][2], xb, M, inter, K, 64)
            for n in ("gate", "up"))
    want = synth.f32_to_bf16_bits(oracle.silu_mul(bf16_to_f32(g), bf16_to_f32(u)))
    assert rel_l2(got, want) <= REL_L2_TOL
    if M <= 16:
        assert launches == 1
        fused_cols = lin.forward(x)                                   # [M, 2*inter], 8 gate / 8 up columns alternating
        ctx = _lib.context(0)
        two_step = torch.empty((M, inter), dtype=torch.bfloat16, device="cuda")
        ctx.check(_lib.lib().scr_silu_mul_pairs8_bf16(ctx.handle, fused_cols.data_ptr(), 2 * inter, two_step.data_ptr(), M, inter,
                                                      None))
        torch.cuda.synchronize()
        assert np.array_equal(got, bits_of(two_step).reshape(M, inter))


@pytest.mark.parametrize("M", [1, 5, 16, 40])
@pytest.mark.parametrize("N,K", [(3072, 3072), (3072, 8192), (8192, 3072), (24, 192), (136, 320)])
def test_residual_add_and_rmsnorm_in_the_epilogue(N, K, M):
    """`fused_add_rmsnorm` (crates/targets/metal/src/cpu_golden.rs:171-200) folded into the o / down matvec: the stored
    residual must equal the two-kernel path bit for bit (same matvec sums, same roundings), the norm must meet the
    oracle bar; repeated calls and graph replays must keep working (the ticket counter resets itself)."""
    import torch
    from scratchy_b200 import AffineQuantLinear, decode
    from util import bf16_to_f32
    w, s, b = synth.affine_int4_weights(N, K, 64, synth.seed_for("ends", N, K))
    lin = make_layer(w, s, b)
    rng = np.random.default_rng(M)
    xb = synth.activations_bf16(M, K, 91)
    res0 = synth.f32_to_bf16_bits(rng.standard_normal((M, N)).astype(np.float32))
    gain = synth.f32_to_bf16_bits((1.0 + 0.1 * rng.standard_normal(N)).astype(np.float32))
    x, g = bf16_dev(xb).reshape(M, K), bf16_dev(gain)
    # two kernels: linear, then add + norm
    res_a = bf16_dev(res0)
    normed_a = decode.fused_add_rmsnorm(res_a, lin.forward(x), g, 1e-5)
    # one launch (up to 16 tokens)
    scratch = torch.zeros(AffineQuantLinear.ENDS_SCRATCH_BYTES, dtype=torch.uint8, device="cuda")
    res_b = bf16_dev(res0)
    normed_b = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    lin.forward_residual_rmsnorm(x, res_b, g, 1e-5, normed_b, scratch)
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(res_b), bits_of(res_a)), "residual after the add"
    assert rel_l2(bits_of(normed_b), bits_of(normed_a)) <= 1e-4 and np.mean(bits_of(normed_b) == bits_of(normed_a)) > 0.98
    y = oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), s, b, xb, M, N, K, 64)
    want_res, want = oracle.fused_add_rmsnorm(bf16_to_f32(res0), bf16_to_f32(y), bf16_to_f32(gain), 1e-5, round_residual_bf16=True)
    assert rel_l2(bits_of(normed_b), synth.f32_to_bf16_bits(want)) <= REL_L2_TOL
    assert rel_l2(bits_of(res_b), synth.f32_to_bf16_bits(want_res)) <= REL_L2_TOL
    assert int(scratch.view(torch.int32)[0]) == 0, "the ticket counter is left at zero"
    if M <= 16:
        # again, eagerly and from a graph: same inputs, same outputs
        side = torch.cuda.Stream()
        res_c = bf16_dev(res0)
        normed_c = torch.empty_like(normed_b)
        lin.forward_residual_rmsnorm(x, res_c, g, 1e-5, normed_c, scratch)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            lin.forward_residual_rmsnorm(x, res_c, g, 1e-5, normed_c, scratch)
        for _ in range(3):
            res_c.copy_(bf16_dev(res0))
            graph.replay()
            torch.cuda.synchronize()
            assert np.array_equal(bits_of(res_c), bits_of(res_b)) and np.array_equal(bits_of(normed_c), bits_of(normed_b))


@pytest.mark.parametrize("N,K,M", [(3584, 3584, 1), (512, 3584, 1), (512, 3584, 16), (1000, 1088, 3), (3584, 3584, 64),
                                   (512, 3584, 2048)])
def test_linear_bias_in_the_epilogue(N, K, M):
    """`{prefix}.bias` (the q/k/v projections of Qwen2.5 carry one): added in f32 to the sum before the one rounding,
    as the reference's matvec epilogue does (crates/targets/metal/shaders/quantized_qmv.metal:104-112), on the
    matvec (M <= 16) and on the tensor-core GEMM, split-K tiles included."""
    import torch
    from scratchy_b200 import AffineQuantLinear
    w, s, b = synth.affine_int4_weights(N, K, 64, synth.seed_for("bias", N, K, M))
    x = synth.activations_bf16(M, K, synth.seed_for("biasx", N, K, M))
    rng = np.random.default_rng(synth.seed_for("biasb", N, K, M))
    bias = synth.f32_to_bf16_bits(rng.normal(0.0, 2.0, N).astype(np.float32))
    layer = AffineQuantLinear.from_tensors(u32_dev(w), bf16_dev(s), bf16_dev(b), 64, 4, linear_bias=bf16_dev(bias))
    y = bits_of(layer.forward(bf16_dev(x).reshape(M, K))).reshape(M, N)
    torch.cuda.synchronize()
    rows = np.arange(M) if M <= 64 else np.sort(np.random.default_rng(1).choice(M, 48, replace=False))
    xs = x.reshape(M, K)[rows]
    want = oracle.affine_qmm_t_b4_bias(w.view(np.uint8).reshape(-1), s, b, xs, bias, len(rows), N, K, 64)
    plain = oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), s, b, xs, len(rows), N, K, 64)
    r = rel_l2(y[rows], want)
    print(f"bias N={N} K={K} M={M} rel_l2={r:.3e} max_abs={max_abs(y[rows], want):.3e}")
    assert r <= REL_L2_TOL
    assert rel_l2(y[rows], plain) > 0.1, "the bias must have been applied"


def test_bias_is_refused_where_no_epilogue_has_it():
    """A fused gate/up pairing has no bias end: the call is refused, never silently dropped."""
    import torch
    from scratchy_b200 import AffineQuantLinear, ScratchyCudaError
    w, s, b = synth.affine_int4_weights(64, 128, 64, 5)
    bias = synth.f32_to_bf16_bits(np.ones(64, np.float32))
    layer = AffineQuantLinear.from_tensors(u32_dev(w), bf16_dev(s), bf16_dev(b), 64, 4, linear_bias=bf16_dev(bias))
    layer.pairs8 = True
    with pytest.raises((ScratchyCudaError, ValueError)):
        layer.forward_silu_mul(torch.zeros((1, 128), dtype=torch.bfloat16, device="cuda"))


def _f16_bits(a):
    return np.asarray(a, np.float32).astype(np.float16).view(np.uint16)


def test_f16_scales_kat_values_through_the_dump_hook():
    """F16 scale/bias storage with bf16 activations — what every mlx-community 4-bit checkpoint ships
    (crates/targets/metal/src/cpu_reference.rs:63-68).  The scale/bias/code triples of the reference's known-answer
    test `dequant_b4_bf16_scale_bias_apply_per_group` (crates/targets/metal/tests/cpu_reference_test.rs:33-54: scale 2,
    bias 1, codes 3,4,5,6 -> 7,9,11,13; scale 0.5, bias -1, codes 1,2,3,4 -> -0.5,0,0.5,1), laid out at this preset's
    group size, must come back from the repacked buffer bit for bit."""
    import torch
    from scratchy_b200 import AffineQuantLinear
    N, K = 16, 128
    codes = np.zeros((N, K), np.uint32)
    codes[0, 0:4] = [3, 4, 5, 6]
    codes[0, 64:68] = [1, 2, 3, 4]
    shifts = (np.arange(8, dtype=np.uint32) * 4)[None, None, :]
    w = (codes.reshape(N, K // 8, 8) << shifts).sum(axis=2, dtype=np.uint32)
    sc = np.ones((N, 2), np.float32)
    bi = np.zeros((N, 2), np.float32)
    sc[0] = [2.0, 0.5]
    bi[0] = [1.0, -1.0]
    layer = AffineQuantLinear.from_tensors(u32_dev(w), torch.from_numpy(_f16_bits(sc).view(np.float16)).cuda(),
                                           torch.from_numpy(_f16_bits(bi).view(np.float16)).cuda(), 64, 4)
    got = bits_of(layer.dequantize()).reshape(N, K)
    from util import bf16_to_f32
    assert bf16_to_f32(got[0, 0:4]).tolist() == [7.0, 9.0, 11.0, 13.0]
    assert bf16_to_f32(got[0, 64:68]).tolist() == [-0.5, 0.0, 0.5, 1.0]
    want = oracle.affine_dequant_b4(w.view(np.uint8).reshape(-1), _f16_bits(sc), _f16_bits(bi), N, K, 64, oracle.F16, oracle.BF16,
                                    True)      # scale narrowed to the activation type first: cpu_reference.rs:90-92
    assert np.array_equal(got, want)


@pytest.mark.parametrize("N,K,M", [(3072, 3072, 1), (1024, 3072, 16), (256, 512, 100)])
def test_f16_scales_match_the_oracle(N, K, M):
    """F16 scales that are NOT bf16-representable (11 significant bits): the narrowing to the activation type at load
    time must be the reference's (`TAct::from_f32(scale.to_f32())`, cpu_reference.rs:90-92) — dequantised weights bit
    for bit, outputs within the bar."""
    import torch
    from scratchy_b200 import AffineQuantLinear
    rng = np.random.default_rng(synth.seed_for("f16s", N, K, M))
    w, _, _ = synth.affine_int4_weights(N, K, 64, synth.seed_for("f16w", N, K))
    sc = (np.abs(rng.normal(0.0, 0.02, (N, K // 64))) + 1e-3).astype(np.float16)
    bi = (-8.0 * sc.astype(np.float32) + rng.normal(0.0, 1e-3, (N, K // 64))).astype(np.float16)
    x = synth.activations_bf16(M, K, synth.seed_for("f16x", N, K, M))
    layer = AffineQuantLinear.from_tensors(u32_dev(w), torch.from_numpy(sc).cuda(), torch.from_numpy(bi).cuda(), 64, 4)
    wd = bits_of(layer.dequantize()).reshape(N, K)
    want_w = oracle.affine_dequant_b4(w.view(np.uint8).reshape(-1), sc.view(np.uint16), bi.view(np.uint16), N, K, 64, oracle.F16,
                                      oracle.BF16, True)
    assert np.array_equal(wd, want_w)
    y = bits_of(layer.forward(bf16_dev(x).reshape(M, K))).reshape(M, N)
    torch.cuda.synchronize()
    want = oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), sc.view(np.uint16), bi.view(np.uint16), x, M, N, K, 64,
                                  scale_dt=oracle.F16)
    assert rel_l2(y, want) <= REL_L2_TOL


# ---- the sibling presets: groups of 32 and 128 (crates/compiler/subtile/src/lower.rs:112-127) ------------------------
def _group_layer(N, K, group, seed, f16=False):
    from scratchy_b200 import AffineQuantLinear
    w, s, b = synth.affine_int4_weights(N, K, group, seed)
    return w, s, b, AffineQuantLinear.from_tensors(u32_dev(w), bf16_dev(s), bf16_dev(b), group, 4)


@pytest.mark.parametrize("group", [32, 128])
@pytest.mark.parametrize("N,K", [(8192, 3072), (1024, 3072), (3072, 8192), (8, 128), (24, 384), (130, 640)])
def test_group_sizes_dequant_bit_exact(N, K, group):
    w, s, b, layer = _group_layer(N, K, group, synth.seed_for("deqg", N, K, group))
    got = bits_of(layer.dequantize()).reshape(N, K)
    want = oracle.affine_dequant_b4(w.view(np.uint8).reshape(-1), s, b, N, K, group)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("group", [32, 128])
@pytest.mark.parametrize("N,K,M", [(8192, 3072, 1), (3072, 8192, 1), (1024, 3072, 4), (3072, 3072, 8), (3072, 3072, 16), (24, 384, 5),
                                   (130, 640, 9), (256, 512, 130), (1024, 3072, 64), (3072, 8192, 512)])
def test_group_sizes_match_the_oracle(N, K, M, group):
    """Matvec (one and two token tiles, persistent and cluster-split grids) and the tensor-core GEMM at groups of 32 and 128."""
    import torch
    w, s, b, layer = _group_layer(N, K, group, synth.seed_for("lg", N, K, group))
    x = synth.activations_bf16(M, K, synth.seed_for("lgx", N, K, M))
    y = layer.forward(bf16_dev(x).reshape(M, K))
    torch.cuda.synchronize()
    rows = np.arange(M) if M * N * K <= 2 ** 31 else np.unique(np.random.default_rng(1).integers(0, M, 24))
    want = oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), s, b, x[rows], len(rows), N, K, group)
    assert rel_l2(bits_of(y).reshape(M, N)[rows], want) <= REL_L2_TOL


@pytest.mark.parametrize("group", [32, 128])
def test_group_sizes_fused_ends_and_refusals(group):
    """The ends that ride on the matvec keep their bits at the other group sizes; what is not built is refused by name."""
    import torch
    from scratchy_b200 import _lib, decode
    N, K, M = 3072, 1024, 2
    w, s, b, lin = _group_layer(N, K, group, 77)
    x = bf16_dev(synth.activations_bf16(M, K, 78)).reshape(M, K)
    res0 = synth.activations_bf16(M, N, 79)
    y = lin.forward_ends(x, torch.empty((M, N), dtype=torch.bfloat16, device="cuda"))
    want_res = (bf16_dev(res0).reshape(M, N).float() + y.float()).to(torch.bfloat16)
    got_res = lin.forward_ends(x, bf16_dev(res0).reshape(M, N), residual=True)
    assert torch.equal(got_res.view(torch.int16), want_res.view(torch.int16))
    want = oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), s, b, bits_of(x), M, N, K, group)
    assert rel_l2(bits_of(y), want) <= REL_L2_TOL
    gain = bf16_dev(synth.f32_to_bf16_bits(np.ones(K, np.float32)))
    if group == 32:
        with pytest.raises(_lib.ScratchyCudaError) as e:
            lin.forward_ends(x, torch.empty((M, N), dtype=torch.bfloat16, device="cuda"), norm_gain=gain, norm_eps=1e-5)
        assert e.value.name == "SCR_E_UNSUPPORTED"
    else:
        got = lin.forward_ends(x, torch.empty((M, N), dtype=torch.bfloat16, device="cuda"), norm_gain=gain, norm_eps=1e-5)
        assert torch.equal(got.view(torch.int16), lin.forward_ends(decode.rmsnorm(x, gain, 1e-5), torch.empty_like(got)).view(torch.int16))


def test_two_cta_gemm_gives_the_bits_of_the_one_cta_kernel(tmp_path):
    """The CTA-pair int4 GEMM (`tcgen05.mma.cta_group::2`, each CTA dequantising half of the pair's channels) is opt-in
    through the environment, read once per process: a child process runs it on a shape it takes (whole 256 x 256 tiles,
    two full rounds of 74 pairs), this process runs the one-CTA kernel; same bits, and the oracle's bound on sampled rows."""
    import subprocess
    import sys
    import torch
    N, K, M, group = 18944, 256, 512, 64
    w, s, b = synth.affine_int4_weights(N, K, group, 3)
    x = synth.activations_bf16(M, K, 4)
    bias = synth.f32_to_bf16_bits(np.random.default_rng(5).normal(0.0, 1.0, N).astype(np.float32))
    np.savez(tmp_path / "in.npz", w=w, s=s, b=b, x=x, bias=bias)
    child = (
        "import sys, numpy as np, torch\n"
        f"sys.path.insert(0, {os.path.dirname(os.path.dirname(os.path.abspath(__file__)))!r})\n"
        f"sys.path.insert(0, {os.path.dirname(os.path.abspath(__file__))!r})\n"
        "from scratchy_b200 import AffineQuantLinear, _lib\n"
        "from util import bf16_dev, bits_of, u32_dev\n"
        f"g = np.load({str(tmp_path / 'in.npz')!r})\n"
        f"lin = AffineQuantLinear.from_tensors(u32_dev(g['w']), bf16_dev(g['s']), bf16_dev(g['b']), {group}, 4, linear_bias=bf16_dev(g['bias']))\n"
        f"y = lin.forward(bf16_dev(g['x']).reshape({M}, {K}))\n"
        "torch.cuda.synchronize(); _lib.context(0).device_status(None)\n"
        f"np.save({str(tmp_path / 'y.npy')!r}, bits_of(y))\n")
    env = dict(os.environ, SCR_AFFINE_GEMM_PAIR="1")
    subprocess.run([sys.executable, "-c", child], check=True, env=env, timeout=300)
    from scratchy_b200 import AffineQuantLinear
    lin = AffineQuantLinear.from_tensors(u32_dev(w), bf16_dev(s), bf16_dev(b), group, 4, linear_bias=bf16_dev(bias))
    here = bits_of(lin.forward(bf16_dev(x).reshape(M, K)))
    torch.cuda.synchronize()
    pair = np.load(tmp_path / "y.npy")
    assert np.array_equal(pair, here)
    rows = np.array([0, 127, 128, 255, 256, 383, 384, 511])
    want = oracle.affine_qmm_t_b4_bias(w.view(np.uint8).reshape(-1), s, b, x[rows], bias, len(rows), N, K, group)
    assert rel_l2(pair.reshape(M, N)[rows], want) <= REL_L2_TOL


@pytest.mark.parametrize("M", [1, 3, 8, 16, 40])
@pytest.mark.parametrize("ns,K", [((3072, 1024, 1024), 3072), ((8192, 8192), 3072), ((24, 136, 8, 40), 320), ((3072,), 8192)])
def test_group_launch_gives_each_member_the_bits_of_its_own_launch(ns, K, M):
    """`scr_linear_affine_b4_group`: q, k, v (or gate, up) over the same activations in one launch.  A member's summation
    order is that of its own row-block, so its bits are those of `forward` wherever the two launches split k alike, and
    within rounding otherwise; both are held to the oracle's bound.  Outputs are prefilled with NaN to catch an unwritten row."""
    import torch
    from scratchy_b200 import AffineQuantLinear
    trip = [synth.affine_int4_weights(n, K, 64, synth.seed_for("grp", n, K, i)) for i, n in enumerate(ns)]
    lins = [make_layer(w, s, b) for w, s, b in trip]
    x = synth.activations_bf16(M, K, synth.seed_for("grpx", K, M))
    xd = bf16_dev(x).reshape(M, K)
    outs = [torch.full((M, n), float("nan"), dtype=torch.bfloat16, device="cuda") for n in ns]
    AffineQuantLinear.forward_group(lins, xd, outs)
    torch.cuda.synchronize()
    for (w, s, b), lin, out, n in zip(trip, lins, outs, ns):
        want = oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), s, b, x, M, n, K, 64)
        got = bits_of(out).reshape(M, n)
        assert rel_l2(got, want) <= REL_L2_TOL
        alone = bits_of(lin.forward(xd)).reshape(M, n)
        assert rel_l2(got, alone) <= 1e-4 and np.mean(got == alone) > 0.98
    from scratchy_b200 import _lib
    _lib.context(0).device_status(None)


def test_group_launch_refusals():
    import torch
    from scratchy_b200 import AffineQuantLinear
    a = make_layer(*synth.affine_int4_weights(32, 128, 64, 1))
    b = make_layer(*synth.affine_int4_weights(32, 256, 64, 2))
    x = bf16_dev(synth.activations_bf16(1, 128, 3)).reshape(1, 128)
    with pytest.raises(ValueError):
        AffineQuantLinear.forward_group([a, b], x)                      # different in_features
    with pytest.raises(ValueError):
        AffineQuantLinear.forward_group([a] * 5, x)                     # more than four
