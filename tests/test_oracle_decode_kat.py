"""Pins the decode-step oracle against the reference's own known-answer tests.

Each case restates, as data, a test of the reference's host golden
(crates/targets/metal/src/cpu_golden.rs, the `tests` module at :1091-1436) or of its
argmax contract (crates/targets/metal/tests/argmax_split_test.rs:24-33, :60-160).
"""
import numpy as np

import oracle


def test_rmsnorm_identity():                       # cpu_golden.rs:1091-1102
    out = oracle.rmsnorm(np.ones((1, 128), np.float32), np.ones(128, np.float32), 1e-5)
    assert np.all(np.abs(out - 1.0) < 1e-3)


def test_rmsnorm_scaling():                        # cpu_golden.rs:1104-1114
    out = oracle.rmsnorm(np.full((1, 64), 2.0, np.float32), np.full(64, 0.5, np.float32), 1e-5)
    assert np.all(np.abs(out - 0.5) < 1e-3)


def test_fused_add_rmsnorm_two_rows():             # cpu_golden.rs:1172-1196
    weight = np.array([1.0, 0.5, 0.5, 1.0], np.float32)
    res, normed = oracle.fused_add_rmsnorm(np.zeros((2, 4), np.float32), np.full((2, 4), 2.0, np.float32),
                                           weight, 1e-5)
    assert np.all(np.abs(res - 2.0) < 1e-5)
    assert np.all(np.abs(normed - weight[None, :]) < 1e-3)


def test_fused_add_rmsnorm_is_add_then_rmsnorm():
    rng = np.random.default_rng(3)
    r = rng.standard_normal((5, 96)).astype(np.float32)
    d = rng.standard_normal((5, 96)).astype(np.float32)
    w = rng.standard_normal(96).astype(np.float32)
    res, normed = oracle.fused_add_rmsnorm(r, d, w, 1e-5)
    assert np.array_equal(res, r + d)
    assert np.array_equal(normed, oracle.rmsnorm(r + d, w, 1e-5))


def test_fused_gate_up_silu_mul_signs():           # cpu_golden.rs:1198-1209
    out = oracle.silu_mul(np.array([0.0, 1.0, -1.0], np.float32), np.array([5.0, 2.0, -1.0], np.float32))
    assert abs(out[0]) < 1e-5
    assert abs(out[1] - 1.4621172) < 1e-4
    assert abs(out[2] - 0.26894143) < 1e-4


def test_embed_gather():                           # cpu_golden.rs:1137-1153
    table = np.array([[0.1, 0.2, 0.3], [1.1, 1.2, 1.3], [2.1, 2.2, 2.3], [3.1, 3.2, 3.3]], np.float32)
    out = oracle.embed([2, 0, 3], table)
    assert np.array_equal(out, np.array([[2.1, 2.2, 2.3], [0.1, 0.2, 0.3], [3.1, 3.2, 3.3]], np.float32))
    try:
        oracle.embed([4], table)
    except IndexError:
        pass
    else:
        raise AssertionError("an id outside the table must be refused")


def test_rope_append_writes_paged_cache():         # cpu_golden.rs:1211-1277
    head_dim, block_size, num_blocks = 4, 2, 3
    q_in = np.array([[1.0, 2.0, 3.0, 4.0]], np.float32)
    k_in = np.array([[5.0, 6.0, 7.0, 8.0]], np.float32)
    v_in = np.array([[9.0, 10.0, 11.0, 12.0]], np.float32)
    cos = np.zeros((1, head_dim), np.float32)
    cos[0, :head_dim // 2] = 1.0
    sin = np.zeros((1, head_dim), np.float32)
    ck = np.zeros(num_blocks * 1 * block_size * head_dim, np.float32)
    cv = np.zeros_like(ck)
    q_out = oracle.rope_append(q_in, k_in, v_in, [0], [3], cos, sin, ck, cv, 1, 1, head_dim, block_size)
    assert np.array_equal(q_out, q_in)
    assert np.array_equal(ck[12:16], k_in[0]) and np.array_equal(cv[12:16], v_in[0])
    untouched = np.ones(ck.size, bool)
    untouched[12:16] = False
    assert np.all(ck[untouched] == 0.0) and np.all(cv[untouched] == 0.0)


def test_rope_append_actually_rotates():           # cpu_golden.rs:1279-1319
    ck = np.zeros(2, np.float32)
    cv = np.zeros(2, np.float32)
    q_out = oracle.rope_append([[3.0, 4.0]], [[5.0, 6.0]], [[7.0, 8.0]], [0], [0],
                               np.array([[0.0, 0.0]], np.float32), np.array([[1.0, 0.0]], np.float32),
                               ck, cv, 1, 1, 2, 1)
    assert q_out.tolist() == [[-4.0, 3.0]]
    assert ck.tolist() == [-6.0, 5.0]
    assert cv.tolist() == [7.0, 8.0]


def _contiguous_decode(q, k, v, scale):
    """cpu_golden.rs:469-520 (`attention_decode`): exact 1/sum_exp, contiguous K/V."""
    s = (k @ q) * scale
    p = np.exp(s - s.max())
    return (p / p.sum()) @ v


def test_attention_via_cache_matches_decode_ref():  # cpu_golden.rs:1321-1408
    head_dim, block_size, kv_len = 4, 2, 3
    q = np.array([[1.0, 0.0, 0.0, 0.0]], np.float32)
    k = np.array([[1, 0, 0, 0], [0, 1, 0, 0], [1, 1, 0, 0]], np.float32)
    v = np.arange(1, 13, dtype=np.float32).reshape(3, 4)
    ck = np.zeros((2, 1, block_size, head_dim), np.float32)
    cv = np.zeros_like(ck)
    for t in range(kv_len):
        ck[t // block_size, 0, t % block_size] = k[t]
        cv[t // block_size, 0, t % block_size] = v[t]
    scale = np.float32(1.0 / np.sqrt(head_dim))
    out = oracle.attention_via_cache(q, ck, cv, [[0, 1]], [kv_len], 1, 1, head_dim, block_size, scale)
    want = _contiguous_decode(q[0], k, v, scale)
    assert np.all(np.abs(out[0] - want) < 1e-4)


def test_attention_via_cache_zero_kv_len():        # cpu_golden.rs:1410-1435
    out = oracle.attention_via_cache(np.ones((1, 4), np.float32), np.zeros(8, np.float32),
                                     np.zeros(8, np.float32), [[0, 0]], [0], 1, 1, 4, 2, 0.5)
    assert np.all(out == 0.0)


def test_attention_via_cache_follows_block_table_and_gqa():
    rng = np.random.default_rng(11)
    hq, hkv, d, bs, nblk = 4, 2, 8, 4, 6
    ck = rng.standard_normal((nblk, hkv, bs, d)).astype(np.float32)
    cv = rng.standard_normal((nblk, hkv, bs, d)).astype(np.float32)
    q = rng.standard_normal((2, hq * d)).astype(np.float32)
    table = np.array([[5, 2, 0], [1, 3, 4]], np.uint32)
    used = np.array([9, 6], np.uint32)
    out = oracle.attention_via_cache(q, ck, cv, table, used, hq, hkv, d, bs, 0.3)
    for b in range(2):
        for h in range(hq):
            kv = h // (hq // hkv)
            ks = np.stack([ck[table[b, t // bs], kv, t % bs] for t in range(used[b])])
            vs = np.stack([cv[table[b, t // bs], kv, t % bs] for t in range(used[b])])
            want = _contiguous_decode(q[b, h * d:(h + 1) * d], ks, vs, np.float32(0.3))
            assert np.allclose(out[b, h * d:(h + 1) * d], want, atol=1e-5)


def test_argmax_contract():                        # argmax_split_test.rs:24-33
    row = np.array([[1.0, 7.0, 3.0, 7.0, np.nan, -np.inf]], np.float32)
    assert oracle.argmax(row).tolist() == [1]       # largest value, smallest id among equal ones
    assert oracle.argmax(np.full((1, 5), np.nan, np.float32)).tolist() == [0]   # NaN never wins
    assert oracle.argmax(np.full((1, 5), -np.inf, np.float32)).tolist() == [0]
    # the reference's planted-maximum pattern (argmax_split_test.rs:36-52): value (i*7919 + r*104729) % 4093
    width = 1000
    rows = np.array([[((i * 7919 + r * 104729) % 4093) * 1e-3 for i in range(width)] for r in range(3)],
                    np.float32)
    rows[0, 17] = 9.0
    rows[1, 999] = 9.0
    rows[2, 0] = 9.0
    rows[2, 500] = 9.0
    assert oracle.argmax(rows).tolist() == [17, 999, 0]
