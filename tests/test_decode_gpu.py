"""GPU parity of the decode-step operators and of one whole decode step against the CPU oracle.

Bars: index / byte work (embed, RoPE'd values, cache appends, argmax) bit-exact; floating-point
operators within relative L2 1e-3 of the oracle's f32 result rounded to bf16; the chained step
(dozens of bf16 roundings in sequence) within 1e-2 on the logits, with the tolerance stated here.
"""
import math

import numpy as np
import pytest

import oracle
from scratchy_b200 import synth
from util import bf16_dev, bf16_to_f32, bits_of, rel_l2, to_dev, u32_dev

pytestmark = pytest.mark.gpu
REL_L2_TOL = 1e-3
STEP_REL_L2_TOL = 1e-2


@pytest.fixture(autouse=True)
def _status_word_is_clean_between_tests():
    """A test that trips a device-side check must not leak the recorded code into the next test."""
    yield
    from scratchy_b200 import _lib
    try:
        _lib.context(0).device_status(None)
    except _lib.ScratchyCudaError:
        pass


def rbits(a):
    return synth.f32_to_bf16_bits(np.asarray(a, np.float32))


def i32_dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, np.uint32).view(np.int32)).cuda()


def test_embed_bit_exact_and_checked():
    import torch
    from scratchy_b200 import _lib, decode
    rng = np.random.default_rng(1)
    table = rbits(rng.standard_normal((1000, 256)))
    ids = rng.integers(0, 1000, size=37).astype(np.uint32)
    out = decode.embed(i32_dev(ids), bf16_dev(table))
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(out), table[ids])
    # an id outside the table: the row is zero-filled and the context reports the check
    bad = ids.copy()
    bad[5] = 1000
    out = decode.embed(i32_dev(bad), bf16_dev(table))
    with pytest.raises(_lib.ScratchyCudaError) as e:
        _lib.context(0).device_status(None)
    assert e.value.status == -1
    got = bits_of(out)
    assert np.all(got[5] == 0) and np.array_equal(got[6], table[bad[6]])
    _lib.context(0).device_status(None)          # cleared


@pytest.mark.parametrize("rows,hidden", [(1, 3072), (8, 3072), (32, 8192), (3, 256), (2, 16384)])
def test_rmsnorm(rows, hidden):
    import torch
    from scratchy_b200 import decode
    rng = np.random.default_rng(synth.seed_for("rmsnorm", rows, hidden))
    x = rbits(rng.standard_normal((rows, hidden)) * 3.0)
    w = rbits(1.0 + 0.1 * rng.standard_normal(hidden))
    out = decode.rmsnorm(bf16_dev(x), bf16_dev(w), 1e-5)
    torch.cuda.synchronize()
    want = rbits(oracle.rmsnorm(bf16_to_f32(x), bf16_to_f32(w), 1e-5))
    assert rel_l2(bits_of(out), want) <= REL_L2_TOL
    assert np.mean(bits_of(out) == want) > 0.98          # the sum order differs: a few 1-ulp flips at most


@pytest.mark.parametrize("rows,hidden", [(1, 3072), (32, 3072), (5, 8192)])
def test_fused_add_rmsnorm(rows, hidden):
    import torch
    from scratchy_b200 import decode
    rng = np.random.default_rng(synth.seed_for("addnorm", rows, hidden))
    r = rbits(rng.standard_normal((rows, hidden)))
    d = rbits(rng.standard_normal((rows, hidden)) * 0.5)
    w = rbits(1.0 + 0.1 * rng.standard_normal(hidden))
    res = bf16_dev(r)
    out = decode.fused_add_rmsnorm(res, bf16_dev(d), bf16_dev(w), 1e-5)
    torch.cuda.synchronize()
    want_res, want = oracle.fused_add_rmsnorm(bf16_to_f32(r), bf16_to_f32(d), bf16_to_f32(w), 1e-5,
                                              round_residual_bf16=True)
    assert np.array_equal(bits_of(res), rbits(want_res)), "the stored residual is bf16(r + d) exactly"
    assert rel_l2(bits_of(out), rbits(want)) <= REL_L2_TOL
    # the norm may be written over delta, as the reference does
    dl = bf16_dev(d)
    res2 = bf16_dev(r)
    decode.fused_add_rmsnorm(res2, dl, bf16_dev(w), 1e-5, out=dl)
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(dl), bits_of(out))


@pytest.mark.parametrize("rows,inter", [(1, 8192), (32, 8192), (3, 64)])
def test_silu_mul_on_fused_halves(rows, inter):
    import torch
    from scratchy_b200 import decode
    rng = np.random.default_rng(synth.seed_for("silu", rows, inter))
    gu = rbits(rng.standard_normal((rows, 2 * inter)) * 2.0)
    t = bf16_dev(gu)
    out = decode.silu_mul(t[:, :inter], t[:, inter:])
    torch.cuda.synchronize()
    want = rbits(oracle.silu_mul(bf16_to_f32(gu[:, :inter]), bf16_to_f32(gu[:, inter:])))
    assert rel_l2(bits_of(out), want) <= REL_L2_TOL
    assert np.mean(bits_of(out) == want) > 0.99


def test_silu_mul_reference_signs():
    """crates/targets/metal/src/cpu_golden.rs:1198-1209, on the device (8 columns: the vector width)."""
    import torch
    from scratchy_b200 import decode
    g = rbits(np.array([[0.0, 1.0, -1.0, 0, 0, 0, 0, 0]]))
    u = rbits(np.array([[5.0, 2.0, -1.0, 0, 0, 0, 0, 0]]))
    out = bf16_to_f32(bits_of(decode.silu_mul(bf16_dev(g), bf16_dev(u))))
    torch.cuda.synchronize()
    assert abs(out[0, 0]) < 1e-5 and abs(out[0, 1] - 1.4621172) < 1e-2 and abs(out[0, 2] - 0.26894143) < 2e-3


def _rope_case(tokens, hq, hkv, d, bs, nblk, seed):
    rng = np.random.default_rng(seed)
    qkv = rbits(rng.standard_normal((tokens, (hq + 2 * hkv) * d)))
    cos, sin = (rng.uniform(-1, 1, size=(64, d)).astype(np.float32) for _ in range(2))
    pos = rng.integers(0, 64, size=tokens).astype(np.uint32)
    slots = rng.permutation(nblk * bs)[:tokens].astype(np.uint32)
    ck = rbits(rng.standard_normal((nblk, hkv, bs, d)))
    cv = rbits(rng.standard_normal((nblk, hkv, bs, d)))
    return qkv, cos, sin, pos, slots, ck, cv


@pytest.mark.parametrize("tokens,hq,hkv,d,bs,nblk", [(1, 24, 8, 128, 16, 9), (32, 24, 8, 128, 16, 40), (5, 4, 2, 64, 4, 7),
                                                    (3, 2, 1, 8, 2, 5)])
def test_rope_append_bit_exact(tokens, hq, hkv, d, bs, nblk):
    import torch
    from scratchy_b200 import decode
    qkv, cos, sin, pos, slots, ck, cv = _rope_case(tokens, hq, hkv, d, bs, nblk, synth.seed_for("rope", tokens, hq, d))
    qd, kd = hq * d, hkv * d
    t = bf16_dev(qkv)
    dk, dv = bf16_dev(ck), bf16_dev(cv)
    decode.rope_append(t[:, :qd], t[:, qd:qd + kd], t[:, qd + kd:], i32_dev(pos), i32_dev(slots), to_dev(cos), to_dev(sin),
                       dk, dv, hq, hkv, d, bs)
    torch.cuda.synchronize()
    f = bf16_to_f32(qkv)
    ok, ov = bf16_to_f32(ck).copy(), bf16_to_f32(cv).copy()
    q_want = oracle.rope_append(f[:, :qd], f[:, qd:qd + kd], f[:, qd + kd:], pos, slots, cos, sin, ok, ov, hq, hkv, d, bs)
    got = bits_of(t)
    assert np.array_equal(got[:, :qd], rbits(q_want)), "rotated q must equal the rounded reference value"
    assert np.array_equal(got[:, qd:], qkv[:, qd:]), "k and v inputs are not modified"
    assert np.array_equal(bits_of(dk), rbits(ok)) and np.array_equal(bits_of(dv), rbits(ov))


def _attention_case(lens, hq, hkv, d, bs, seed, scale=None):
    import torch
    from scratchy_b200 import decode
    rng = np.random.default_rng(seed)
    batch = len(lens)
    max_blocks = max(1, max((n + bs - 1) // bs for n in lens)) + 1
    nblk = batch * max_blocks + 3
    table = rng.permutation(nblk)[:batch * max_blocks].reshape(batch, max_blocks).astype(np.uint32)
    ck = rbits(rng.standard_normal((nblk, hkv, bs, d)))
    cv = rbits(rng.standard_normal((nblk, hkv, bs, d)))
    q = rbits(rng.standard_normal((batch, hq * d)))
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    out = decode.attention_via_cache(bf16_dev(q), bf16_dev(ck), bf16_dev(cv), i32_dev(table), i32_dev(np.array(lens)),
                                     hq, hkv, d, bs, scale)
    torch.cuda.synchronize()
    from scratchy_b200 import _lib
    _lib.context(0).device_status(None)          # no bounded wait ran out, no block id was refused
    want = oracle.attention_via_cache(bf16_to_f32(q), bf16_to_f32(ck), bf16_to_f32(cv), table, np.array(lens, np.uint32),
                                      hq, hkv, d, bs, np.float32(scale))
    return bits_of(out), rbits(want)


@pytest.mark.parametrize("lens,hq,hkv,d,bs", [
    ([2049], 24, 8, 128, 16),                 # Llama-3.2-3B geometry at context 2048 + the new token
    ([2049, 77, 1, 300, 16, 17, 128, 640], 24, 8, 128, 16),
    ([1, 7, 8, 9], 8, 8, 64, 4),              # one query head per kv head, fewer tokens than splits
    ([513, 31], 8, 1, 128, 16),               # 8 query heads on one kv head
    ([200, 95], 28, 4, 128, 32),              # 7 query heads per kv head
    ([100], 4, 2, 64, 1),                     # block_size 1
    ([700 - 13 * i for i in range(10)], 24, 8, 128, 16),      # 80 (sequence, kv head) pairs: clusters of 4
    ([300 + 7 * i for i in range(20)], 24, 8, 128, 16),       # 160 pairs: clusters of 2
    ([1 + 11 * i for i in range(40)], 24, 8, 128, 16),        # 320 pairs: one CTA per pair, no cluster
    ([5000, 33], 8, 2, 128, 32),              # more blocks per CTA than ring stages: the ring wraps
    ([200, 33, 16], 8, 8, 64, 16),            # head_dim 64 on the tensor-core path, one query head per kv head
    ([1000], 16, 2, 64, 64),                  # head_dim 64, 8 query heads per kv head, 64-token blocks
])
def test_attention_via_cache(lens, hq, hkv, d, bs):
    got, want = _attention_case(lens, hq, hkv, d, bs, synth.seed_for("attn", len(lens), hq, hkv, d, bs))
    assert rel_l2(got, want) <= REL_L2_TOL


def test_attention_zero_kv_len_is_zero():
    """crates/targets/metal/src/cpu_golden.rs:1410-1435: seq_used_k = 0 leaves zeros."""
    got, want = _attention_case([0, 5], 4, 2, 64, 4, 3)
    assert np.all(bf16_to_f32(got[0]) == 0.0)
    assert rel_l2(got[1], want[1]) <= REL_L2_TOL


def test_attention_sharp_softmax():
    """A large scale makes the softmax nearly one-hot: the running-maximum merge must not lose it."""
    got, want = _attention_case([777, 1500], 24, 8, 128, 16, 5, scale=4.0)
    assert rel_l2(got, want) <= REL_L2_TOL


@pytest.mark.parametrize("lens,hq,hkv,d,bs", [
    ([2049], 24, 8, 128, 16),                 # the newest token opens a block of its own (slot 0), clusters of 8
    ([2048, 77, 1, 300, 16, 17, 128, 640], 24, 8, 128, 16),   # last slot of a block, a one-token sequence, ...
    ([700 - 13 * i for i in range(10)], 24, 8, 128, 16),      # clusters of 4
    ([1 + 11 * i for i in range(40)], 24, 8, 128, 16),        # one CTA per pair
    ([200, 33, 16], 8, 8, 64, 16),            # head_dim 64
    ([1000, 65], 16, 2, 64, 64),              # 8 query heads per kv head, 64-token blocks
    ([5000, 33], 8, 2, 128, 32),              # the ring wraps before the newest block arrives
])
def test_rope_attention_one_launch_equals_the_two_operators(lens, hq, hkv, d, bs):
    """RoPE + append folded into the attention launch: the cache and the output are the bits that
    `rope_append` followed by `attention_via_cache` produce, and both match the oracle."""
    import torch
    from scratchy_b200 import _lib, decode
    rng = np.random.default_rng(synth.seed_for("ropeattn", len(lens), hq, hkv, d, bs))
    batch = len(lens)
    max_blocks = max((n + bs - 1) // bs for n in lens) + 1
    nblk = batch * max_blocks + 3
    table = rng.permutation(nblk)[:batch * max_blocks].reshape(batch, max_blocks).astype(np.uint32)
    ck = rbits(rng.standard_normal((nblk, hkv, bs, d)))
    cv = rbits(rng.standard_normal((nblk, hkv, bs, d)))
    qkv = rbits(rng.standard_normal((batch, (hq + 2 * hkv) * d)))
    cos, sin = (rng.uniform(-1, 1, size=(64, d)).astype(np.float32) for _ in range(2))
    pos = rng.integers(0, 64, size=batch).astype(np.uint32)
    used = np.array(lens, np.uint32)
    slots = np.array([table[b, (lens[b] - 1) // bs] * bs + (lens[b] - 1) % bs for b in range(batch)], np.uint32)
    qd, kd = hq * d, hkv * d
    scale = 1.0 / math.sqrt(d)
    # the two operators
    t = bf16_dev(qkv)
    k2, v2 = bf16_dev(ck), bf16_dev(cv)
    decode.rope_append(t[:, :qd], t[:, qd:qd + kd], t[:, qd + kd:], i32_dev(pos), i32_dev(slots), to_dev(cos), to_dev(sin),
                       k2, v2, hq, hkv, d, bs)
    two = decode.attention_via_cache(t[:, :qd], k2, v2, i32_dev(table), i32_dev(used), hq, hkv, d, bs, scale)
    # one launch
    u = bf16_dev(qkv)
    k1, v1 = bf16_dev(ck), bf16_dev(cv)
    one = decode.rope_attention_via_cache(u[:, :qd], u[:, qd:qd + kd], u[:, qd + kd:], i32_dev(pos), to_dev(cos), to_dev(sin),
                                          k1, v1, i32_dev(table), i32_dev(used), hq, hkv, d, bs, scale)
    torch.cuda.synchronize()
    _lib.context(0).device_status(None)
    assert np.array_equal(bits_of(u), qkv), "the fused call leaves q, k, v as the projection wrote them"
    assert np.array_equal(bits_of(k1), bits_of(k2)) and np.array_equal(bits_of(v1), bits_of(v2)), "cache contents"
    assert np.array_equal(bits_of(one), bits_of(two)), "attention output"
    f = bf16_to_f32(qkv)
    ok, ov = bf16_to_f32(ck).copy(), bf16_to_f32(cv).copy()
    q_rot = oracle.rope_append(f[:, :qd], f[:, qd:qd + kd], f[:, qd + kd:], pos, slots, cos, sin, ok, ov, hq, hkv, d, bs)
    assert np.array_equal(bits_of(k1), rbits(ok)) and np.array_equal(bits_of(v1), rbits(ov))
    want = oracle.attention_via_cache(bf16_to_f32(rbits(q_rot)), bf16_to_f32(rbits(ok)), ov, table, used, hq, hkv, d, bs,
                                      np.float32(scale))
    assert rel_l2(bits_of(one), rbits(want)) <= REL_L2_TOL


def test_rope_attention_refuses_what_it_cannot_stream():
    """Blocks that are not a multiple of 16 tokens have no one-launch form: the call says so and touches nothing."""
    import torch
    from scratchy_b200 import _lib, decode
    rng = np.random.default_rng(4)
    hq, hkv, d, bs = 4, 2, 64, 4
    ck = rbits(rng.standard_normal((6, hkv, bs, d)))
    k1, v1 = bf16_dev(ck), bf16_dev(ck)
    u = bf16_dev(rbits(rng.standard_normal((1, (hq + 2 * hkv) * d))))
    tab = to_dev(np.zeros((64, d), np.float32))
    with pytest.raises(_lib.ScratchyCudaError) as e:
        decode.rope_attention_via_cache(u[:, :hq * d], u[:, hq * d:(hq + hkv) * d], u[:, (hq + hkv) * d:], i32_dev(np.array([3])),
                                        tab, tab, k1, v1, i32_dev(np.array([[1, 2]])), i32_dev(np.array([4])), hq, hkv, d, bs, 0.125)
    assert e.value.status == -7
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(k1), ck) and not decode.rope_attention_supported(bs)


def test_argmax_bit_exact():
    import torch
    from scratchy_b200 import decode
    rng = np.random.default_rng(9)
    width = 128256
    lg = rbits(rng.standard_normal((6, width)))
    f = bf16_to_f32(lg).copy()
    f[1, 777] = f[1, 90000] = 50.0            # equal maxima: the smaller id wins
    f[2, :] = np.nan                          # NaN never wins: id 0
    f[3, 5] = np.nan
    f[3, 128255] = 60.0                       # the last element
    f[4, :] = -np.inf
    lg = rbits(f)
    out = decode.argmax(bf16_dev(lg))
    torch.cuda.synchronize()
    want = oracle.argmax(bf16_to_f32(lg))
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want)
    assert want[1] == 777 and want[2] == 0 and want[3] == 128255 and want[4] == 0
    # a ragged width (not a multiple of the vector width) behind a padded row stride
    pad = bf16_dev(rbits(rng.standard_normal((3, 1008))))
    got = decode.argmax(pad[:, :1003]).cpu().numpy().view(np.uint32)
    assert np.array_equal(got, oracle.argmax(bf16_to_f32(bits_of(pad))[:, :1003]))


# ------------------------------------------------------------------------------------ whole step
def _oracle_linear(ck, prefixes, x_bits, k):
    w = np.concatenate([ck[f"{p}.weight"] for p in prefixes], 0)
    s = np.concatenate([ck[f"{p}.scales"] for p in prefixes], 0)
    b = np.concatenate([ck[f"{p}.biases"] for p in prefixes], 0)
    return oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), s, b, x_bits, x_bits.shape[0], w.shape[0], k, 64)


def _oracle_step(cfg, ck, ids, pos, slots, table, used, cache_k, cache_v, cos, sin, bs):
    """The step as a chain of oracle operators, rounding to bf16 wherever the device stores bf16."""
    f, r = bf16_to_f32, rbits
    qd, kd = cfg.q_dim, cfg.kv_dim
    if "model.embed_tokens.scales" in ck:                                  # an AffineQuantEmbedding: gather + dequantise
        e = "model.embed_tokens"
        residual = oracle.affine_embed_b4(ck[f"{e}.weight"].view(np.uint8).reshape(-1), ck[f"{e}.scales"], ck[f"{e}.biases"], ids,
                                          cfg.vocab, cfg.hidden, 64)
    else:
        residual = ck["model.embed_tokens.weight"][ids]                   # bf16 bits
    normed = r(oracle.rmsnorm(f(residual), f(ck["model.layers.0.input_layernorm.weight"]), cfg.rms_eps))
    for i in range(cfg.n_layers):
        root = f"model.layers.{i}"
        qkv = _oracle_linear(ck, [f"{root}.self_attn.{p}_proj" for p in "qkv"], normed, cfg.hidden)
        fq = f(qkv)
        q_rot = oracle.rope_append(fq[:, :qd], fq[:, qd:qd + kd], fq[:, qd + kd:], pos, slots, cos, sin, cache_k[i],
                                   cache_v[i], cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, bs)
        cache_k[i][...] = f(r(cache_k[i]))                                 # the device cache holds bf16
        attn = r(oracle.attention_via_cache(f(r(q_rot)), cache_k[i], cache_v[i], table, used, cfg.n_q_heads,
                                            cfg.n_kv_heads, cfg.head_dim, bs, np.float32(1.0 / math.sqrt(cfg.head_dim))))
        delta = _oracle_linear(ck, [f"{root}.self_attn.o_proj"], attn, qd)
        res, nrm = oracle.fused_add_rmsnorm(f(residual), f(delta), f(ck[f"{root}.post_attention_layernorm.weight"]),
                                            cfg.rms_eps, round_residual_bf16=True)
        residual, normed = r(res), r(nrm)
        gu = f(_oracle_linear(ck, [f"{root}.mlp.gate_proj", f"{root}.mlp.up_proj"], normed, cfg.hidden))
        act = r(oracle.silu_mul(gu[:, :cfg.intermediate], gu[:, cfg.intermediate:]))
        delta = _oracle_linear(ck, [f"{root}.mlp.down_proj"], act, cfg.intermediate)
        nxt = ck[f"model.layers.{i + 1}.input_layernorm.weight"] if i + 1 < cfg.n_layers else ck["model.norm.weight"]
        res, nrm = oracle.fused_add_rmsnorm(f(residual), f(delta), f(nxt), cfg.rms_eps, round_residual_bf16=True)
        residual, normed = r(res), r(nrm)
    return _oracle_linear(ck, ["lm_head" if "lm_head.weight" in ck else "model.embed_tokens"], normed, cfg.hidden)


@pytest.mark.parametrize("group,f16", [(64, False), (32, False), (128, True)])
@pytest.mark.parametrize("vocab,hidden,n", [(1000, 256, 7), (128256, 3072, 5), (40, 128, 40)])
def test_quantized_embedding_gathers_and_dequantises_bit_exact(vocab, hidden, n, group, f16):
    """`AffineQuantEmbedding` (quantized_dequantize.metal:82-157; host reference quantized_affine_embed_test.rs:27-90):
    every gathered row has the bits of the oracle's dequantisation; the tied head multiplies with the same buffer; an
    id beyond the vocabulary is reported and yields zeros."""
    import torch
    from scratchy_b200 import AffineQuantEmbedding, _lib
    w, s, b = synth.affine_int4_weights(vocab, hidden, group, synth.seed_for("qembed", vocab, hidden, group))
    sdt = oracle.BF16
    st, bt = bf16_dev(s), bf16_dev(b)
    if f16:
        s = bf16_to_f32(s).astype(np.float16).view(np.uint16)
        b = bf16_to_f32(b).astype(np.float16).view(np.uint16)
        st, bt = (torch.from_numpy(v.view(np.float16)).cuda() for v in (s, b))
        sdt = oracle.F16
    emb = AffineQuantEmbedding.from_tensors(u32_dev(w), st, bt, group, 4)
    rng = np.random.default_rng(n)
    ids = rng.integers(0, vocab, size=n).astype(np.uint32)
    ids[0], ids[-1] = 0, vocab - 1
    got = emb.forward(i32_dev(ids))
    torch.cuda.synchronize()
    want = oracle.affine_embed_b4(w.view(np.uint8).reshape(-1), s, b, ids, vocab, hidden, group, scale_dt=sdt)
    assert np.array_equal(bits_of(got), want)
    assert emb.as_linear().packed.data_ptr() == emb.table.packed.data_ptr() and emb.as_linear().out_features == vocab
    ctx = _lib.context(0)
    ctx.device_status(None)
    bad = ids.copy()
    bad[1 % n] = vocab
    got = emb.forward(i32_dev(bad))
    with pytest.raises(_lib.ScratchyCudaError) as e:
        ctx.device_status(None)
    assert e.value.name == "SCR_E_ARG"
    assert not bits_of(got)[1 % n].any()
    ctx.device_status(None)


def test_decoder_health_check_reports_a_bad_token_id_and_clears():
    """`LlamaDecoder.check_health` is the step-level reader of the device status word: a token id beyond the vocabulary
    is skipped on the device, reported once as SCR_E_ARG, and the next check is clean."""
    import torch
    from scratchy_b200 import _lib, decode
    cfg = decode.LlamaConfig(hidden=256, n_layers=1, n_q_heads=4, n_kv_heads=2, head_dim=64, intermediate=512,
                             vocab=1024, rope_theta=10000.0)
    dec = decode.LlamaDecoder(cfg, decode.synthetic_checkpoint(cfg, seed=2), "cuda:0", max_pos=64)
    cache = decode.PagedKvCache(cfg, 8, 4, "cuda:0")
    buf = dec.buffers(1, 8)
    buf.block_table.copy_(i32_dev(np.arange(8, dtype=np.uint32).reshape(1, 8)))
    for tok, bad in ((5, False), (cfg.vocab + 3, True), (7, False)):
        buf.ids.copy_(i32_dev(np.array([tok], np.uint32)))
        buf.positions.copy_(i32_dev(np.array([2], np.uint32)))
        buf.slot_mapping.copy_(i32_dev(np.array([2], np.uint32)))
        buf.seq_used_k.copy_(i32_dev(np.array([3], np.uint32)))
        dec.step(buf, cache)
        if bad:
            with pytest.raises(_lib.ScratchyCudaError) as e:
                dec.check_health()
            assert e.value.name == "SCR_E_ARG"
        dec.check_health()


def test_decode_step_with_a_tied_quantized_embedding():
    """A checkpoint whose `model.embed_tokens` is quantized and that has no `lm_head`: the embedding gathers from, and the
    vocabulary head multiplies with, one buffer."""
    import torch
    from scratchy_b200 import decode
    cfg = decode.LlamaConfig(hidden=256, n_layers=2, n_q_heads=4, n_kv_heads=2, head_dim=64, intermediate=512,
                             vocab=1024, rope_theta=10000.0)
    ck = decode.synthetic_checkpoint(cfg, seed=5)
    for suffix in ("weight", "scales", "biases"):
        ck[f"model.embed_tokens.{suffix}"] = ck.pop(f"lm_head.{suffix}")
    dec = decode.LlamaDecoder(cfg, dict(ck), "cuda:0", max_pos=128)
    assert dec.embed_table is None and dec.lm_head is dec.quant_embed.as_linear()
    batch, bs, max_blocks = 3, 4, 8
    nblk = batch * max_blocks
    cache = decode.PagedKvCache(cfg, nblk, bs, "cuda:0")
    rng = np.random.default_rng(3)
    ctx_len = rng.integers(3, 20, size=batch)
    table = rng.permutation(nblk).reshape(batch, max_blocks).astype(np.uint32)
    hist = [rbits(rng.standard_normal((nblk, cfg.n_kv_heads, bs, cfg.head_dim))) for _ in range(2 * cfg.n_layers)]
    for i in range(cfg.n_layers):
        cache.k[i].copy_(bf16_dev(hist[2 * i]))
        cache.v[i].copy_(bf16_dev(hist[2 * i + 1]))
    ok = [bf16_to_f32(hist[2 * i]).copy() for i in range(cfg.n_layers)]
    ov = [bf16_to_f32(hist[2 * i + 1]).copy() for i in range(cfg.n_layers)]
    cos, sin = decode.rope_tables(128, cfg.head_dim, cfg.rope_theta)
    buf = dec.buffers(batch, max_blocks)
    buf.block_table.copy_(i32_dev(table))
    ids = rng.integers(0, cfg.vocab, size=batch).astype(np.uint32)
    pos = ctx_len.astype(np.uint32)
    slots = np.array([table[q, pos[q] // bs] * bs + pos[q] % bs for q in range(batch)], np.uint32)
    used = (pos + 1).astype(np.uint32)
    buf.ids.copy_(i32_dev(ids))
    buf.positions.copy_(i32_dev(pos))
    buf.slot_mapping.copy_(i32_dev(slots))
    buf.seq_used_k.copy_(i32_dev(used))
    dec.step(buf, cache)
    torch.cuda.synchronize()
    want = _oracle_step(cfg, ck, ids, pos, slots, table, used, ok, ov, cos, sin, bs)
    assert rel_l2(bits_of(buf.logits), want) <= STEP_REL_L2_TOL


@pytest.mark.parametrize("batch,fuse_residual_norm,head_dim,bs,max_ctx,fuse_rope", [
    (1, False, 64, 4, 20, True), (3, False, 64, 4, 20, True), (20, False, 64, 4, 20, True), (3, True, 64, 4, 20, True),
    # 16-token blocks and head_dim 128: the TMA + tensor-core attention.  With RoPE + append as a kernel of their
    # own it streams the old cache blocks while that kernel is still running and waits only for the newest block;
    # with them folded in (the default) it patches the newest token into its shared-memory tile itself.
    (2, False, 128, 16, 100, False), (9, False, 128, 16, 100, False),
    (2, False, 128, 16, 100, True), (9, False, 128, 16, 100, True), (20, False, 64, 16, 100, True)])
def test_decode_step_matches_oracle_chain(batch, fuse_residual_norm, head_dim, bs, max_ctx, fuse_rope):
    """Two consecutive steps of a small random-init decoder (eager, then the same step replayed from a
    CUDA graph) against the oracle chain; batch 20 takes the tensor-core linear path."""
    import torch
    from scratchy_b200 import decode
    cfg = decode.LlamaConfig(hidden=256, n_layers=2, n_q_heads=4, n_kv_heads=2, head_dim=head_dim, intermediate=512,
                             vocab=1024, rope_theta=10000.0)
    ck = decode.synthetic_checkpoint(cfg, seed=batch)
    dec = decode.LlamaDecoder(cfg, ck, "cuda:0", max_pos=128, fuse_residual_norm=fuse_residual_norm, fuse_rope=fuse_rope)
    max_blocks = 8
    nblk = batch * max_blocks
    cache = decode.PagedKvCache(cfg, nblk, bs, "cuda:0")
    rng = np.random.default_rng(batch)
    ctx_len = rng.integers(3, max_ctx, size=batch)
    if bs == 16:
        ctx_len[0] = 2 * bs - 1                      # the second step's token opens a new block
    table = rng.permutation(nblk).reshape(batch, max_blocks).astype(np.uint32)
    # pre-fill the caches with random history
    hist_k = [rbits(rng.standard_normal((nblk, cfg.n_kv_heads, bs, cfg.head_dim))) for _ in range(cfg.n_layers)]
    hist_v = [rbits(rng.standard_normal((nblk, cfg.n_kv_heads, bs, cfg.head_dim))) for _ in range(cfg.n_layers)]
    for i in range(cfg.n_layers):
        cache.k[i].copy_(bf16_dev(hist_k[i]))
        cache.v[i].copy_(bf16_dev(hist_v[i]))
    ok = [bf16_to_f32(a).copy() for a in hist_k]
    ov = [bf16_to_f32(a).copy() for a in hist_v]
    cos, sin = decode.rope_tables(128, cfg.head_dim, cfg.rope_theta)
    buf = dec.buffers(batch, max_blocks)
    buf.block_table.copy_(i32_dev(table))
    ids = rng.integers(0, cfg.vocab, size=batch).astype(np.uint32)
    graph = None
    for step in range(2):
        pos = (ctx_len + step).astype(np.uint32)
        slots = np.array([table[b, pos[b] // bs] * bs + pos[b] % bs for b in range(batch)], np.uint32)
        used = (pos + 1).astype(np.uint32)
        buf.ids.copy_(i32_dev(ids))
        buf.positions.copy_(i32_dev(pos))
        buf.slot_mapping.copy_(i32_dev(slots))
        buf.seq_used_k.copy_(i32_dev(used))
        if step == 0:
            dec.step(buf, cache)
        else:
            # capture warms the step once more on the same inputs: appends are idempotent for fixed slots
            graph = dec.capture(buf, cache)
            graph.replay()
        torch.cuda.synchronize()
        want = _oracle_step(cfg, ck, ids, pos, slots, table, used, ok, ov, cos, sin, bs)
        got = bits_of(buf.logits)
        err = rel_l2(got, want)
        assert err <= STEP_REL_L2_TOL, f"step {step}: logits rel-L2 {err:.3e}"
        for i in range(cfg.n_layers):
            assert rel_l2(bits_of(cache.v[i]), rbits(ov[i])) <= STEP_REL_L2_TOL
        want_ids = oracle.argmax(bf16_to_f32(got))
        assert np.array_equal(buf.next_ids.cpu().numpy().view(np.uint32), want_ids), "argmax of the device logits"
        ids = want_ids.astype(np.uint32)
    from scratchy_b200 import _lib
    _lib.context(0).device_status(None)


@pytest.mark.parametrize("batch", [1, 8])
def test_llama_3b_layer_at_real_geometry_operator_by_operator(batch):
    """One decoder layer at the Llama-3.2-3B geometry of the decode benchmark (hidden 3072, 24 query / 8 kv heads of
    128, intermediate 8192, RoPE theta 500000, context 2048 in 16-token blocks): every operator of the step is given
    the ORACLE's input for it (as the bf16 bits the device would hold) and must meet the per-operator bar — index and
    byte work bit for bit, floating point within 1e-3 — so no operator hides behind the chain's accumulated error; then
    the whole step through `LlamaDecoder.step` against the oracle chain."""
    import torch
    from scratchy_b200 import _lib, decode
    f, r = bf16_to_f32, rbits
    cfg = decode.LlamaConfig(hidden=3072, n_layers=1, n_q_heads=24, n_kv_heads=8, head_dim=128, intermediate=8192,
                             vocab=4096, rope_theta=500000.0)
    ck = decode.synthetic_checkpoint(cfg, seed=40 + batch)
    dec = decode.LlamaDecoder(cfg, ck, "cuda:0", max_pos=2048)
    layer = dec.layers[0]
    bs, ctx = 16, 2048
    max_blocks = ctx // bs
    nblk = batch * max_blocks
    rng = np.random.default_rng(batch)
    table = rng.permutation(nblk).reshape(batch, max_blocks).astype(np.uint32)
    hist_k = rbits(rng.standard_normal((nblk, cfg.n_kv_heads, bs, cfg.head_dim)))
    hist_v = rbits(rng.standard_normal((nblk, cfg.n_kv_heads, bs, cfg.head_dim)))
    cos, sin = decode.rope_tables(2048, cfg.head_dim, cfg.rope_theta)
    ids = rng.integers(0, cfg.vocab, size=batch).astype(np.uint32)
    pos = np.full(batch, ctx - 1, np.uint32)
    if batch > 1:
        pos[1:] = rng.integers(1, ctx - 1, size=batch - 1)                 # ragged histories, one of them full
    used = (pos + 1).astype(np.uint32)
    slots = np.array([table[b, pos[b] // bs] * bs + pos[b] % bs for b in range(batch)], np.uint32)
    qd, kd = cfg.q_dim, cfg.kv_dim
    root = "model.layers.0"

    def check(name, got_bits, want_bits, exact=False):
        if exact:
            assert np.array_equal(got_bits, want_bits), f"{name}: must be bit-exact"
        else:
            e = rel_l2(got_bits, want_bits)
            assert e <= REL_L2_TOL, f"{name}: rel-L2 {e:.3e}"

    # embed, norm
    residual = ck["model.embed_tokens.weight"][ids]
    check("embed", bits_of(decode.embed(i32_dev(ids), dec.embed_table)), residual, exact=True)
    normed = r(oracle.rmsnorm(f(residual), f(ck[f"{root}.input_layernorm.weight"]), cfg.rms_eps))
    check("rmsnorm", bits_of(decode.rmsnorm(bf16_dev(residual), layer.input_norm, cfg.rms_eps)), normed)
    # fused q|k|v projection
    qkv = _oracle_linear(ck, [f"{root}.self_attn.{p}_proj" for p in "qkv"], normed, cfg.hidden)
    check("qkv", bits_of(layer.qkv.forward(bf16_dev(normed))), qkv)
    # RoPE + append + attention in one launch
    ok, ov = f(hist_k).copy(), f(hist_v).copy()
    fq = f(qkv)
    q_rot = oracle.rope_append(fq[:, :qd], fq[:, qd:qd + kd], fq[:, qd + kd:], pos, slots, cos, sin, ok, ov, cfg.n_q_heads,
                               cfg.n_kv_heads, cfg.head_dim, bs)
    attn = r(oracle.attention_via_cache(f(r(q_rot)), f(r(ok)), ov, table, used, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, bs,
                                        np.float32(1.0 / math.sqrt(cfg.head_dim))))
    t = bf16_dev(qkv)
    ckd, cvd = bf16_dev(hist_k), bf16_dev(hist_v)
    got_attn = decode.rope_attention_via_cache(t[:, :qd], t[:, qd:qd + kd], t[:, qd + kd:], i32_dev(pos), dec.cos, dec.sin, ckd, cvd,
                                               i32_dev(table), i32_dev(used), cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, bs,
                                               dec.attn_scale)
    check("cache k", bits_of(ckd), r(ok), exact=True)
    check("cache v", bits_of(cvd), r(ov), exact=True)
    check("attention", bits_of(got_attn), attn)
    # o projection, residual add + norm
    delta = _oracle_linear(ck, [f"{root}.self_attn.o_proj"], attn, qd)
    check("o", bits_of(layer.o.forward(bf16_dev(attn))), delta)
    res, nrm = oracle.fused_add_rmsnorm(f(residual), f(delta), f(ck[f"{root}.post_attention_layernorm.weight"]), cfg.rms_eps,
                                        round_residual_bf16=True)
    res_d = bf16_dev(residual)
    got_n = decode.fused_add_rmsnorm(res_d, bf16_dev(delta), layer.post_norm, cfg.rms_eps)
    check("residual after o", bits_of(res_d), r(res), exact=True)
    check("post-attention norm", bits_of(got_n), r(nrm))
    # gate|up with silu*up in the epilogue, down projection
    gu = f(_oracle_linear(ck, [f"{root}.mlp.gate_proj", f"{root}.mlp.up_proj"], r(nrm), cfg.hidden))
    act = r(oracle.silu_mul(gu[:, :cfg.intermediate], gu[:, cfg.intermediate:]))
    check("silu(gate)*up", bits_of(layer.gate_up.forward_silu_mul(bf16_dev(r(nrm)))), act)
    delta2 = _oracle_linear(ck, [f"{root}.mlp.down_proj"], act, cfg.intermediate)
    check("down", bits_of(layer.down.forward(bf16_dev(act))), delta2)
    torch.cuda.synchronize()
    _lib.context(0).device_status(None)

    # the whole step through the decoder, from the same history
    cache = decode.PagedKvCache(cfg, nblk, bs, "cuda:0")
    cache.k[0].copy_(bf16_dev(hist_k))
    cache.v[0].copy_(bf16_dev(hist_v))
    buf = dec.buffers(batch, max_blocks)
    buf.block_table.copy_(i32_dev(table))
    buf.ids.copy_(i32_dev(ids))
    buf.positions.copy_(i32_dev(pos))
    buf.slot_mapping.copy_(i32_dev(slots))
    buf.seq_used_k.copy_(i32_dev(used))
    dec.step(buf, cache)
    torch.cuda.synchronize()
    want = _oracle_step(cfg, ck, ids, pos, slots, table, used, [f(hist_k).copy()], [f(hist_v).copy()], cos, sin, bs)
    e = rel_l2(bits_of(buf.logits), want)
    print(f"3B layer batch={batch}: logits rel-L2 {e:.3e}")
    assert e <= STEP_REL_L2_TOL
    _lib.context(0).device_status(None)


@pytest.mark.parametrize("batch", [1, 2, 3])
def test_matvec_ends_give_the_bits_of_the_separate_operators(batch):
    """The reference's `QmvEnds` on the decode path: RMSNorm inside the matvec that consumes it, the residual add inside the
    matvec that produces its summand.  A decoder that uses them (five launches per layer) with the norm-in end in its
    rounded-row form and one that runs the norms and adds as kernels of their own (seven) must produce the same logits,
    residual stream and next token, bit for bit, over two steps at the Llama-3.2-3B hidden size, and so must the default
    decoder (the residual end alone, the norms as plain RMSNorm launches); with the norm-in end in the
    reference matvec's own arithmetic (the row scaled by 1 / rms(x) after the dot: no rounded normalised row) the step agrees
    within the step tolerance.  The ends are also checked one by one against the operators they replace."""
    import torch
    from scratchy_b200 import _lib, decode
    cfg = decode.LlamaConfig(hidden=3072, n_layers=2, n_q_heads=24, n_kv_heads=8, head_dim=128, intermediate=8192,
                             vocab=2048, rope_theta=500000.0)
    ck = decode.synthetic_checkpoint(cfg, seed=70 + batch)
    a = decode.LlamaDecoder(cfg, ck, "cuda:0", max_pos=256, fuse_ends=True, exact_norm_in=True)
    b = decode.LlamaDecoder(cfg, ck, "cuda:0", max_pos=256, fuse_ends=False, fuse_residual=False)
    c = decode.LlamaDecoder(cfg, ck, "cuda:0", max_pos=256, fuse_ends=True)
    d = decode.LlamaDecoder(cfg, ck, "cuda:0", max_pos=256)         # the default: the residual end alone, plain norms
    bs, max_blocks = 16, 8
    nblk = batch * max_blocks
    rng = np.random.default_rng(batch)
    table = rng.permutation(nblk).reshape(batch, max_blocks).astype(np.uint32)
    hist = [rbits(rng.standard_normal((nblk, cfg.n_kv_heads, bs, cfg.head_dim))) for _ in range(2 * cfg.n_layers)]
    ids = rng.integers(0, cfg.vocab, size=batch).astype(np.uint32)
    ctx_len = rng.integers(20, 100, size=batch)
    outs = []
    for dec in (a, b, c, d):
        cache = decode.PagedKvCache(cfg, nblk, bs, "cuda:0")
        for i in range(cfg.n_layers):
            cache.k[i].copy_(bf16_dev(hist[2 * i]))
            cache.v[i].copy_(bf16_dev(hist[2 * i + 1]))
        buf = dec.buffers(batch, max_blocks)
        buf.block_table.copy_(i32_dev(table))
        cur, res = ids.copy(), []
        n0 = _lib.context(0).launch_count()
        for step in range(2):
            pos = (ctx_len + step).astype(np.uint32)
            buf.ids.copy_(i32_dev(cur))
            buf.positions.copy_(i32_dev(pos))
            buf.slot_mapping.copy_(i32_dev(np.array([table[q, pos[q] // bs] * bs + pos[q] % bs for q in range(batch)], np.uint32)))
            buf.seq_used_k.copy_(i32_dev(pos + 1))
            dec.step(buf, cache)
            torch.cuda.synchronize()
            res.append((bits_of(buf.logits).copy(), bits_of(buf.residual).copy(), buf.next_ids.cpu().numpy().copy()))
            # every decoder is fed the separate operators' tokens, so that the steps stay comparable
            cur = (res[-1][2] if dec is not c else outs[1][0][step][2]).view(np.uint32).copy()
        outs.append((res, _lib.context(0).launch_count() - n0))
    (ra, la), (rb, lb), (rc, lc), (rd, ld) = outs
    assert la < lb and lc == la and ld == lb, f"the ends must save launches ({la}, {lc} against {lb}, {ld})"
    for step in range(2):
        assert np.array_equal(ra[step][1], rb[step][1]), f"step {step}: residual stream"
        assert np.array_equal(ra[step][0], rb[step][0]), f"step {step}: logits"
        assert np.array_equal(ra[step][2], rb[step][2]), f"step {step}: next token"
        assert all(np.array_equal(rd[step][j], rb[step][j]) for j in range(3)), f"step {step}: the residual end alone"
        assert rel_l2(rc[step][1], rb[step][1]) <= STEP_REL_L2_TOL, f"step {step}: residual stream, row-scale norm-in"
        assert rel_l2(rc[step][0], rb[step][0]) <= STEP_REL_L2_TOL, f"step {step}: logits, row-scale norm-in"
    _lib.context(0).device_status(None)


@pytest.mark.parametrize("N,K,M", [(1024, 3072, 1), (3072, 3072, 3), (8192, 3072, 2), (3072, 8192, 1), (5120, 2048, 4), (136, 320, 5)])
def test_each_matvec_end_against_the_operator_it_replaces(N, K, M):
    import torch
    from scratchy_b200 import AffineQuantLinear, decode
    from util import u32_dev
    rng = np.random.default_rng(synth.seed_for("ends1", N, K, M))
    w, s, b = synth.affine_int4_weights(N, K, 64, synth.seed_for("endsw", N, K))
    bias = rbits(rng.normal(0, 1, N))
    lin = AffineQuantLinear.from_tensors(u32_dev(w), bf16_dev(s), bf16_dev(b), 64, 4)
    linb = AffineQuantLinear.from_tensors(u32_dev(w), bf16_dev(s), bf16_dev(b), 64, 4, linear_bias=bf16_dev(bias))
    x = bf16_dev(rbits(rng.standard_normal((M, K)) * 3.0))
    gain = bf16_dev(rbits(1.0 + 0.1 * rng.standard_normal(K)))
    res0 = rbits(rng.standard_normal((M, N)))
    # the operator an end replaces is the same matvec (the ends entry point with no end set) followed by the separate operator
    def plain(v):
        return lin.forward_ends(v, torch.empty((M, N), dtype=torch.bfloat16, device="cuda"))
    # norm-in == rmsnorm, then the plain linear
    want = plain(decode.rmsnorm(x, gain, 1e-5))
    got = lin.forward_ends(x, torch.empty((M, N), dtype=torch.bfloat16, device="cuda"), norm_gain=gain, norm_eps=1e-5)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)), "norm-in"
    # residual end == the linear, then residual <- bf16(residual + y)
    y = plain(x)
    want_res = (bf16_dev(res0).float() + y.float()).to(torch.bfloat16)
    got_res = lin.forward_ends(x, bf16_dev(res0), residual=True)
    assert torch.equal(got_res.view(torch.int16), want_res.view(torch.int16)), "residual"
    # bias and scale against the oracle's f32 sums
    _, acc = oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), s, b, bits_of(x), M, N, K, 64, want_f32=True)
    want_bs = rbits((acc + bf16_to_f32(bias)[None, :]) * np.float32(0.125))
    got_bs = linb.forward_ends(x, torch.empty((M, N), dtype=torch.bfloat16, device="cuda"), scale=0.125)
    torch.cuda.synchronize()
    assert rel_l2(bits_of(got_bs), want_bs) <= REL_L2_TOL, "bias + scale"
    # everything at once: norm-in, bias, scale, residual
    yn = linb.forward_ends(x, torch.empty((M, N), dtype=torch.bfloat16, device="cuda"), norm_gain=gain, norm_eps=1e-5, scale=0.5)
    want_all = (bf16_dev(res0).float() + yn.float()).to(torch.bfloat16)
    got_all = linb.forward_ends(x, bf16_dev(res0), norm_gain=gain, norm_eps=1e-5, scale=0.5, residual=True)
    torch.cuda.synchronize()
    assert torch.equal(got_all.view(torch.int16), want_all.view(torch.int16)), "all ends"


def _unit(rng, shape):
    return rng.uniform(-1.0, 1.0, size=shape)


@pytest.mark.parametrize("K,N,offset,f16_scales", [(3072, 1024, 0.0, False), (3072, 1024, 1.0, False), (3072, 1024, 0.0, True),
                                                   (896, 136, 0.0, False), (128, 256, 0.0, False), (2048, 7, 0.0, False)])
@pytest.mark.parametrize("M", [1, 2, 3, 5])
def test_norm_in_is_as_close_to_the_exact_normed_product_as_the_norm_then_the_matvec(K, N, offset, f16_scales, M):
    """The reference's own test of its normalising matvec, at its shapes, value distributions and bound
    (crates/targets/metal/tests/affine_qmv_ends_test.rs:86-93 cases, :152-186 weights, :278-296 inputs and the exact
    product, :361-377 the bound, :421-447 the three arms; the wide variant :449-470 for 2 to 5 rows): against the exact
    `W . rmsnorm(x, gain + offset)` in f64 over the un-rounded decoded weights, every output must lie within one rounding of
    the output plus 2 ulp of the row's sum of |terms| — for the RMSNorm followed by the plain matvec, for the norm-in end
    in the reference's arithmetic (row scaled by 1 / rms after the dot) and in the rounded-row form; the plain matvec of
    the raw x must fall outside, or the bound could not see a missing norm.  Inputs are seeded draws from the reference
    test's distributions."""
    import torch
    from scratchy_b200 import AffineQuantLinear, decode
    from util import u32_dev
    if not AffineQuantLinear.norm_in_supported(M, K):
        pytest.skip("the normalised rows of this case exceed the end's shared memory")
    rng = np.random.default_rng(K * 7 + N + 1000 * M + (1 if f16_scales else 0) + int(offset * 10))
    words = rng.integers(0, 2 ** 32, size=(N, K // 8), dtype=np.uint64).astype(np.uint32)
    sc = (0.5 + np.abs(_unit(rng, (N, K // 64)))) * 0.02 / 15.0
    bi = -sc * 7.5 * (1.0 + 0.1 * _unit(rng, (N, K // 64)))
    if f16_scales:
        s_st, b_st = sc.astype(np.float16), bi.astype(np.float16)
        s_val, b_val = s_st.astype(np.float64), b_st.astype(np.float64)
        s_dev, b_dev = torch.from_numpy(s_st).cuda(), torch.from_numpy(b_st).cuda()
    else:
        s_st, b_st = rbits(sc), rbits(bi)
        s_val, b_val = bf16_to_f32(s_st).astype(np.float64), bf16_to_f32(b_st).astype(np.float64)
        s_dev, b_dev = bf16_dev(s_st), bf16_dev(b_st)
    codes = ((words[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))[None, None, :]) & 0xF).reshape(N, K).astype(np.float64)
    decoded = np.repeat(s_val, 64, axis=1) * codes + np.repeat(b_val, 64, axis=1)
    x_bits = rbits(4.0 * _unit(rng, (M, K)))
    g_bits = rbits(1.0 - offset + 0.25 * _unit(rng, K))
    x, gain = bf16_to_f32(x_bits).astype(np.float64), bf16_to_f32(g_bits).astype(np.float64)
    eps = 1e-5
    inv = 1.0 / np.sqrt((x * x).sum(axis=1, keepdims=True) / K + np.float64(np.float32(eps)))
    xn = x * inv * (gain + offset)[None, :]
    exact = xn @ decoded.T                                           # [M, N]
    scale = np.abs(xn) @ np.abs(decoded).T                           # the sum of the terms' magnitudes
    ulp = 2.0 ** -8
    bound = ulp * np.abs(exact) + 2.0 * ulp * scale

    lin = AffineQuantLinear.from_tensors(u32_dev(words), s_dev, b_dev, 64, 4)
    xd, gd = bf16_dev(x_bits), bf16_dev(g_bits)
    def out():
        return torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    def within(t):
        torch.cuda.synchronize()
        return bool(np.all(np.abs(bf16_to_f32(bits_of(t)).astype(np.float64) - exact) <= bound))
    # the separate operator takes its gain as stored: fold the offset into a gain of its own (exact for these values or not,
    # the bound has room for one rounding of the gain)
    gain_plus = bf16_dev(rbits(gain + offset)) if offset else gd
    assert within(lin.forward_ends(decode.rmsnorm(xd, gain_plus, eps), out())), "the norm, then the matvec"
    assert within(lin.forward_ends(xd, out(), norm_gain=gd, norm_eps=eps, norm_gain_offset=offset, norm_row_scale=True)), \
        "the normalising matvec, the reference's arithmetic"
    assert within(lin.forward_ends(xd, out(), norm_gain=gd, norm_eps=eps, norm_gain_offset=offset)), \
        "the normalising matvec, rounded-row form"
    assert not within(lin.forward_ends(xd, out())), "the bound accepts the raw matvec: it cannot see a missing norm"


def test_row_scale_norm_in_with_every_other_end():
    """Norm-in in the reference's arithmetic together with the bias, a scale and the residual add, and with the gate/up
    pairing: each equals the same call without the later ends followed by the separate operator (the order of the ends is
    norm, dot, bias, scale, residual), bit for bit."""
    import torch
    from scratchy_b200 import AffineQuantLinear, decode
    from util import u32_dev
    N, K, M = 3072, 3072, 2
    rng = np.random.default_rng(synth.seed_for("ends-rs", N, K, M))
    w, s, b = synth.affine_int4_weights(N, K, 64, synth.seed_for("endsw-rs", N, K))
    bias = rbits(rng.normal(0, 1, N))
    linb = AffineQuantLinear.from_tensors(u32_dev(w), bf16_dev(s), bf16_dev(b), 64, 4, linear_bias=bf16_dev(bias))
    x = bf16_dev(rbits(rng.standard_normal((M, K)) * 3.0))
    gain = bf16_dev(rbits(1.0 + 0.1 * rng.standard_normal(K)))
    res0 = rbits(rng.standard_normal((M, N)))
    kw = dict(norm_gain=gain, norm_eps=1e-5, norm_row_scale=True, scale=0.5)
    yn = linb.forward_ends(x, torch.empty((M, N), dtype=torch.bfloat16, device="cuda"), **kw)
    want = (bf16_dev(res0).float() + yn.float()).to(torch.bfloat16)
    got = linb.forward_ends(x, bf16_dev(res0), residual=True, **kw)
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16)), "norm-in, bias, scale, residual"
    # against the oracle's f32 sums over the staged row bf16(x * gain): (acc * inv_rms + bias) * scale
    xf, gf = bf16_to_f32(bits_of(x)), bf16_to_f32(bits_of(gain))
    staged = rbits(xf * gf[None, :])
    _, acc = oracle.affine_qmm_t_b4(w.view(np.uint8).reshape(-1), s, b, staged, M, N, K, 64, want_f32=True)
    inv = 1.0 / np.sqrt((xf.astype(np.float64) ** 2).sum(axis=1, keepdims=True) / K + 1e-5)
    want_y = rbits((acc * inv + bf16_to_f32(bias)[None, :]) * 0.5)
    assert rel_l2(bits_of(yn), want_y) <= REL_L2_TOL
    assert np.mean(bits_of(yn) == want_y) > 0.97, "the same roundings as the restatement up to the sums' order"
    # the gate/up pairing
    pair = AffineQuantLinear.from_tensors(u32_dev(w), bf16_dev(s), bf16_dev(b), 64, 4)
    pair.pairs8 = True                                              # rows read as runs of 8 gate, 8 up
    act = pair.forward_ends(x, torch.empty((M, N // 2), dtype=torch.bfloat16, device="cuda"), norm_gain=gain, norm_eps=1e-5,
                            norm_row_scale=True, silu_pairs=True)
    full = pair.forward_ends(x, torch.empty((M, N), dtype=torch.bfloat16, device="cuda"), norm_gain=gain, norm_eps=1e-5,
                             norm_row_scale=True)
    fr = full.view(M, N // 16, 2, 8)
    want_act = decode.silu_mul(fr[:, :, 0, :].reshape(M, N // 2).contiguous(), fr[:, :, 1, :].reshape(M, N // 2).contiguous())
    torch.cuda.synchronize()
    assert rel_l2(bits_of(act), bits_of(want_act)) <= REL_L2_TOL
    assert np.mean(bits_of(act) == bits_of(want_act)) > 0.99


def test_decode_ops_against_the_committed_fixture():
    """tests/golden/decode_ops_small.npz (written by tests/golden/make_golden.py from the oracle)."""
    import os
    import torch
    from scratchy_b200 import decode
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decode_ops_small.npz"))
    gain = bf16_dev(g["norm_gain"])
    assert rel_l2(bits_of(decode.rmsnorm(bf16_dev(g["norm_x"]), gain, 1e-5)), rbits(g["rmsnorm_f32"])) <= REL_L2_TOL
    res = bf16_dev(g["norm_x"])
    nrm = decode.fused_add_rmsnorm(res, bf16_dev(g["norm_delta"]), gain, 1e-5)
    assert np.array_equal(bits_of(res), g["addnorm_residual"])
    assert rel_l2(bits_of(nrm), rbits(g["addnorm_f32"])) <= REL_L2_TOL
    gu = bf16_dev(g["silu_gate_up"])
    assert rel_l2(bits_of(decode.silu_mul(gu[:, :128], gu[:, 128:])), rbits(g["silu_f32"])) <= REL_L2_TOL
    hq, hkv, hd, bs, _ = (int(v) for v in g["rope_geom"])
    qkv = bf16_dev(g["rope_qkv"])
    ck, cv = bf16_dev(g["rope_cache_k_in"]), bf16_dev(g["rope_cache_v_in"])
    decode.rope_append(qkv[:, :hq * hd], qkv[:, hq * hd:(hq + hkv) * hd], qkv[:, (hq + hkv) * hd:], i32_dev(g["rope_pos"]),
                       i32_dev(g["rope_slots"]), to_dev(g["rope_cos"]), to_dev(g["rope_sin"]), ck, cv, hq, hkv, hd, bs)
    assert np.array_equal(bits_of(qkv)[:, :hq * hd], g["rope_q_out"])
    assert np.array_equal(bits_of(ck), g["rope_cache_k_out"]) and np.array_equal(bits_of(cv), g["rope_cache_v_out"])
    att = decode.attention_via_cache(bf16_dev(g["attn_q"]), ck, cv, i32_dev(g["attn_table"]), i32_dev(g["attn_lens"]), hq, hkv,
                                     hd, bs, hd ** -0.5)
    assert rel_l2(bits_of(att), rbits(g["attn_f32"])) <= REL_L2_TOL
    ids = decode.argmax(bf16_dev(g["argmax_logits"]))
    torch.cuda.synchronize()
    assert np.array_equal(ids.cpu().numpy().view(np.uint32), g["argmax_ids"])


def test_decoder_from_a_safetensors_directory(tmp_path):
    """Checkpoint files -> mmap -> pinned staging -> device -> repack: the decoder loaded from disk produces
    the same logits, bit for bit, as the one built from the in-memory tensors."""
    import torch
    from scratchy_b200 import decode
    from scratchy_b200.weights import CheckpointWeights, write_safetensors
    cfg = decode.LlamaConfig(hidden=256, n_layers=2, n_q_heads=4, n_kv_heads=2, head_dim=64, intermediate=512,
                             vocab=1024, rope_theta=10000.0)
    ck = decode.synthetic_checkpoint(cfg, seed=5)
    on_disk = {k: ((v, "BF16") if v.dtype == np.uint16 else v) for k, v in ck.items()}
    names = sorted(on_disk)
    write_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), {k: on_disk[k] for k in names[::2]})
    write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), {k: on_disk[k] for k in names[1::2]})
    gw = CheckpointWeights.from_dir(str(tmp_path), "cuda:0")
    from_disk = decode.LlamaDecoder(cfg, gw, "cuda:0", max_pos=64)
    assert not gw.contains("model.layers.0.self_attn.q_proj.weight") and not gw.contains("lm_head.scales")
    in_memory = decode.LlamaDecoder(cfg, ck, "cuda:0", max_pos=64)
    logits = []
    for dec in (from_disk, in_memory):
        cache = decode.PagedKvCache(cfg, 8, 4, "cuda:0")
        buf = dec.buffers(2, 4)
        buf.ids.copy_(i32_dev([3, 900]))
        buf.positions.copy_(i32_dev([0, 5]))
        buf.block_table.copy_(i32_dev([[0, 1, 2, 3], [4, 5, 6, 7]]))
        buf.slot_mapping.copy_(i32_dev([0, 21]))
        buf.seq_used_k.copy_(i32_dev([1, 6]))
        dec.step(buf, cache)
        torch.cuda.synchronize()
        logits.append(bits_of(buf.logits))
    assert np.array_equal(logits[0], logits[1])
    gw.close()
