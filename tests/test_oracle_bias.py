"""Pins of the additive-bias oracle: tests/m13_attention_bias_oracle.rs and
tests/m13_bias_public_api.rs restated against the C++ restatement of src/attention_bias.rs."""
import numpy as np
import pytest

from oracle import binding as ob

ERR_LENGTH_MISMATCH = 7
ERR_NON_FINITE = 9
ERR_POSITION_OVERFLOW = 6


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def fixture(n, phase):
    # tests/m13_attention_bias_oracle.rs:11-15
    return ob.fixture(n, 0.071, phase, 0.625)


def small_shape():
    return ob.Shape(1, 4, 2, 3, 5, 8, 2)


ROPE = (10000.0, 17, 13)


# tests/m13_attention_bias_oracle.rs:37-63
@pytest.mark.parametrize("causal", [False, True])
def test_no_bias_is_bitwise_identical_to_unbiased_oracle(causal):
    s = small_shape()
    q, k, v = fixture(96, 0.2), fixture(80, 0.8), fixture(80, 1.4)
    e = ob.forward_reference_projection_grouped_rope_asymmetric(q, k, v, s, *ROPE, causal=causal)
    a = ob.forward_reference_projection_grouped_rope_asymmetric_biased(q, k, v, s, *ROPE, causal=causal)
    assert np.array_equal(bits(a[0]), bits(e[0])) and np.array_equal(bits(a[1]), bits(e[1]))


# tests/m13_attention_bias_oracle.rs:65-101
def test_dense_bias_changes_softmax():
    s = ob.Shape(1, 1, 1, 1, 2, 2, 0)
    out, lse = ob.forward_reference_projection_grouped_rope_asymmetric_biased(
        [0, 0], [0, 0, 0, 0], [1, 2, 3, 4], s, 10000.0, 0, 0, dense=[0.0, np.log(np.float32(3.0))])
    assert abs(out[0] - 2.5) <= 1e-6 and abs(out[1] - 3.5) <= 1e-6
    assert abs(lse[0] - np.log(np.float32(4.0))) <= 1e-6


# tests/m13_attention_bias_oracle.rs:103-156
def test_alibi_matches_equivalent_dense_bias():
    s = small_shape()
    q, k, v = fixture(96, 0.3), fixture(80, 0.9), fixture(80, 1.5)
    slopes = np.array([0.25, 0.5, 0.75, 1.0], np.float32)
    q0, k0 = 31, 29
    dense = np.empty((1, 4, 3, 5), np.float32)
    for h in range(4):
        for i in range(3):
            for j in range(5):
                dense[0, h, i, j] = slopes[h] * (np.float32(k0 + j) - np.float32(q0 + i))
    d = ob.forward_reference_projection_grouped_rope_asymmetric_biased(q, k, v, s, *ROPE, dense=dense)
    a = ob.forward_reference_projection_grouped_rope_asymmetric_biased(q, k, v, s, *ROPE, alibi=(slopes, q0, k0))
    assert np.array_equal(bits(a[0]), bits(d[0])) and np.array_equal(bits(a[1]), bits(d[1]))


# tests/m13_attention_bias_oracle.rs:158-203
def test_malformed_biases_fail_explicitly():
    s = small_shape()
    q, k, v = fixture(96, 0.2), fixture(80, 0.8), fixture(80, 1.4)
    with pytest.raises(ob.OracleError) as e:
        ob.forward_reference_projection_grouped_rope_asymmetric_biased(q, k, v, s, *ROPE, dense=[0.0])
    assert e.value.status == ERR_LENGTH_MISMATCH and "attention bias" in e.value.detail
    with pytest.raises(ob.OracleError) as e:
        ob.forward_reference_projection_grouped_rope_asymmetric_biased(
            q, k, v, s, *ROPE, alibi=([0.0, np.nan, 0.0, 0.0], 0, 0))
    assert e.value.status == ERR_NON_FINITE and "ALiBi slopes" in e.value.detail and "1" in e.value.detail
    with pytest.raises(ob.OracleError) as e:
        ob.forward_reference_projection_grouped_rope_asymmetric_biased(
            q, k, v, s, *ROPE, alibi=([0.0] * 4, 2 ** 64 - 2, 0))
    assert e.value.status == ERR_POSITION_OVERFLOW


# tests/m13_bias_public_api.rs:6-33
def test_single_key_returns_value_row():
    s = ob.Shape(1, 1, 1, 1, 1, 2, 0)
    out, _ = ob.forward_reference_projection_grouped_rope_asymmetric_biased(
        [1.0, 0.0], [1.0, 0.0], [2.0, 3.0], s, 10000.0, 0, 0)
    assert out.tolist() == [2.0, 3.0]


def test_alibi_against_two_pass_softmax():
    """Independent check: materialised scores + bias, two-pass softmax in f64."""
    rng = np.random.default_rng(5)
    B, Hq, Hkv, Nq, Nkv, D = 2, 4, 2, 6, 11, 16
    s = ob.Shape(B, Hq, Hkv, Nq, Nkv, D, 5)
    q = rng.standard_normal((B, Nq, Hq, D)).astype(np.float32)
    k = rng.standard_normal((B, Nkv, Hkv, D)).astype(np.float32)
    v = rng.standard_normal((B, Nkv, Hkv, D)).astype(np.float32)
    slopes = np.array([0.5, 0.25, 0.125, 0.0625], np.float32)
    out, lse = ob.forward_reference_projection_grouped_rope_asymmetric_biased(
        q, k, v, s, 10000.0, 3, 1, causal=True, alibi=(slopes, 40, 38))
    qpos = np.arange(3, 3 + Nq, dtype=np.uint64)
    kpos = np.arange(1, 1 + Nkv, dtype=np.uint64)
    qr = ob.rotate_rows(q.transpose(0, 2, 1, 3).reshape(-1, D), D, np.tile(qpos, B * Hq), 10000.0).reshape(B, Hq, Nq, D)
    kr = ob.rotate_rows(k.transpose(0, 2, 1, 3).reshape(-1, D), D, np.tile(kpos, B * Hkv), 10000.0).reshape(B, Hkv, Nkv, D)
    vv = v.transpose(0, 2, 1, 3)
    out = out.reshape(B, Nq, Hq, D)
    lse = lse.reshape(B, Hq, Nq)
    for b in range(B):
        for h in range(Hq):
            for i in range(Nq):
                keys = min(Nkv, 5 + i + 1)
                sc = kr[b, h // 2, :keys].astype(np.float64) @ qr[b, h, i].astype(np.float64) / 4.0
                sc += slopes[h] * ((38 + np.arange(keys)) - (40.0 + i))
                m = sc.max()
                p = np.exp(sc - m)
                assert np.abs(out[b, i, h] - (p / p.sum()) @ vv[b, h // 2, :keys]).max() <= 2e-5
                assert abs(lse[b, h, i] - (m + np.log(p.sum()))) <= 2e-5


def test_alibi_row_sampling_is_bitwise_identical_to_the_full_biased_oracle():
    """forward_rows_alibi (the sampled-row route the large-shape parity gates use) against the full biased oracle:
    with the rotation materialised first the sampled rows carry the same bits."""
    s = ob.Shape(2, 4, 2, 6, 9, 8, 3)
    q, k, v = fixture(2 * 6 * 4 * 8, 0.3), fixture(2 * 9 * 2 * 8, 0.9), fixture(2 * 9 * 2 * 8, 1.7)
    slopes = np.array([0.5, -0.25, 0.125, 0.0625], np.float32)
    theta, q_off, kv_off = 10000.0, 11, 4
    for causal in (False, True):
        fo, fl = ob.forward_reference_projection_grouped_rope_asymmetric_biased(q, k, v, s, theta, q_off, kv_off, causal=causal,
                                                                               alibi=(slopes, 7, 2))
        qpos = np.repeat(np.tile(np.arange(6, dtype=np.uint64) + q_off, 2), 4)
        kpos = np.repeat(np.tile(np.arange(9, dtype=np.uint64) + kv_off, 2), 2)
        rq, rk = ob.rotate_rows(q, 8, qpos, theta), ob.rotate_rows(k, 8, kpos, theta)
        rows = [(b, h, r) for b in range(2) for h in range(4) for r in range(6)]
        ro, rl = ob.forward_rows_alibi(rq, rk, v, s, ob.PROJECTION, rows, slopes, 7, 2, causal=causal, threads=2)
        full_o = fo.reshape(2, 6, 4, 8)
        full_l = fl.reshape(2, 4, 6)
        for i, (b, h, r) in enumerate(rows):
            assert np.array_equal(bits(ro[i]), bits(full_o[b, r, h])), (causal, b, h, r)
            assert bits(rl[i:i + 1])[0] == bits(full_l[b, h, r:r + 1])[0]
