"""Pins of the CPU oracle: the reference's own oracle-only tests restated against the C++
restatement (cross-oracle bit-exact equalities, invariants, validation behaviour)."""
import numpy as np
import pytest

from oracle import binding as ob

INF = np.float32(np.inf)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bit_equal(a, b, what=""):
    assert np.array_equal(bits(a), bits(b)), what


# ---- tests/parity.rs:3-109: online softmax vs naive two-pass softmax, tol 2e-6 -------------
def naive_forward(q, k, v, B, H, N, D, causal, scale):
    q = q.reshape(B, H, N, D).astype(np.float32)
    k = k.reshape(B, H, N, D).astype(np.float32)
    v = v.reshape(B, H, N, D).astype(np.float32)
    out = np.zeros_like(q)
    lse = np.zeros((B, H, N), np.float32)
    for b in range(B):
        for h in range(H):
            for qi in range(N):
                keys = qi + 1 if causal else N
                s = (k[b, h, :keys] @ q[b, h, qi]).astype(np.float32) * np.float32(scale)
                m = s.max()
                p = np.exp(s - m, dtype=np.float32)
                den = p.sum(dtype=np.float32)
                out[b, h, qi] = (p / den) @ v[b, h, :keys]
                lse[b, h, qi] = m + np.log(den, dtype=np.float32)
    return out.reshape(-1), lse.reshape(-1)


@pytest.mark.parametrize("B,H,N,D,causal,scale", [(2, 3, 7, 5, False, None), (1, 2, 9, 8, True, 0.25)])
def test_online_softmax_matches_naive(B, H, N, D, causal, scale):
    n = B * H * N * D
    q = ob.fixture(n, 0.173, -0.7, 1.0)
    k = np.cos(np.arange(n, dtype=np.float32) * np.float32(0.119) + np.float32(0.2), dtype=np.float32)
    v = ob.fixture(n, 0.071, -0.4, 1.7)
    out, lse = ob.forward_reference(q, k, v, B, H, N, D, causal, scale)
    s = scale if scale is not None else 1.0 / np.sqrt(np.float32(D))
    eo, el = naive_forward(q, k, v, B, H, N, D, causal, s)
    assert np.abs(out - eo).max() <= 2.0e-6
    assert np.abs(lse - el).max() <= 2.0e-6


# ---- src/lib.rs:524-551 --------------------------------------------------------------------
def test_default_scale_and_bad_lengths():
    # default scale 1/sqrt(64) == 0.125 exactly: explicit 0.125 must give identical bits
    n = 1 * 1 * 3 * 64
    q, k, v = ob.fixture(n, 0.1, 0.0, 1.0), ob.fixture(n, 0.2, 0.3, 1.0), ob.fixture(n, 0.3, 0.5, 1.0)
    a = ob.forward_reference(q, k, v, 1, 1, 3, 64, False, None)
    b = ob.forward_reference(q, k, v, 1, 1, 3, 64, False, 0.125)
    assert_bit_equal(a[0], b[0]) and assert_bit_equal(a[1], b[1])
    with pytest.raises(ob.OracleError) as e:
        ob.forward_reference(np.zeros(4), np.zeros(3), np.zeros(4), 1, 1, 2, 2)
    assert e.value.status == 7 and "K" in e.value.detail


def test_validation_errors():
    z = np.zeros(4, np.float32)
    with pytest.raises(ob.OracleError) as e:
        ob.forward_reference(z, z, z, 0, 1, 2, 2)
    assert e.value.status == 1  # ZeroDimension
    bad = z.copy()
    bad[2] = np.nan
    with pytest.raises(ob.OracleError) as e:
        ob.forward_reference(z, z, bad, 1, 1, 2, 2)
    assert e.value.status == 9 and "V" in e.value.detail and "index 2" in e.value.detail
    for s in (0.0, -1.0, np.inf, np.nan):
        with pytest.raises(ob.OracleError) as e:
            ob.forward_reference(z, z, z, 1, 1, 2, 2, False, s)
        assert e.value.status == 8
    with pytest.raises(ob.OracleError) as e:  # src/asymmetric_grouped.rs:611-641
        ob.forward_reference_grouped_asymmetric(z, z, z, ob._shape(1, 6, 4, 1, 8, 32, 7))
    assert e.value.status == 3
    with pytest.raises(ob.OracleError) as e:
        ob.forward_reference_grouped_rope(np.zeros(3), np.zeros(3), np.zeros(3), 1, 1, 1, 1, 3, 1e4, 0)
    assert e.value.status == 4  # odd head_dim
    for theta in (0.0, -1.0, np.inf):
        with pytest.raises(ob.OracleError) as e:
            ob.forward_reference_grouped_rope(z, z, z, 1, 1, 1, 2, 2, theta, 0)
        assert e.value.status == 5
    with pytest.raises(ob.OracleError) as e:  # src/projection_asymmetric.rs:349-360
        ob.forward_reference_projection_grouped_rope_asymmetric(
            np.zeros(2 * 64), np.zeros(8 * 64), np.zeros(8 * 64), ob._shape(1, 1, 1, 2, 8, 64), 1e4,
            2**64 - 1, 0)
    assert e.value.status == 6


# ---- tests/grouped.rs:32-92: GQA oracle == MHA oracle on expanded K/V, bit-exact -----------
def gfix(n, phase):
    return ob.fixture(n, 0.037, phase, 1.75, 0.41, 0.25)


@pytest.mark.parametrize("q_heads,kv_heads", [(8, 8), (8, 2), (8, 1)])
def test_grouped_matches_expanded_mha_bit_exact(q_heads, kv_heads):
    B, N, D = 2, 7, 16
    q = gfix(B * q_heads * N * D, 0.1)
    k = gfix(B * kv_heads * N * D, 0.7)
    v = gfix(B * kv_heads * N * D, 1.3)
    g = q_heads // kv_heads
    ek = np.repeat(k.reshape(B, kv_heads, N * D), g, axis=1).reshape(-1)
    ev = np.repeat(v.reshape(B, kv_heads, N * D), g, axis=1).reshape(-1)
    for causal in (False, True):
        for scale in (None, 0.19):
            go, gl = ob.forward_reference_grouped(q, k, v, B, q_heads, kv_heads, N, D, causal, scale)
            mo, ml = ob.forward_reference(q, ek, ev, B, q_heads, N, D, causal, scale)
            assert_bit_equal(go, mo)
            assert_bit_equal(gl, ml)


# ---- tests/rotary_grouped.rs:48-143: fused RoPE == materialised RoPE then grouped ----------
def rfix(n, phase):
    return ob.fixture(n, 0.029, phase, 1.5, 0.37, 0.375)


def materialize_head_major(x, B, H, N, D, theta, off):
    pos = np.tile(np.arange(N, dtype=np.uint64) + np.uint64(off), B * H)
    return ob.rotate_rows(x, D, pos, theta)


@pytest.mark.parametrize("B,Hq,Hkv,N,D", [(1, 4, 4, 7, 16), (2, 8, 2, 9, 64), (1, 8, 1, 5, 32)])
def test_fused_rope_matches_materialised(B, Hq, Hkv, N, D):
    q, k, v = rfix(B * Hq * N * D, 0.2), rfix(B * Hkv * N * D, 0.8), rfix(B * Hkv * N * D, 1.4)
    for theta, off in ((10_000.0, 0), (500_000.0, 37)):
        rq = materialize_head_major(q, B, Hq, N, D, theta, off)
        rk = materialize_head_major(k, B, Hkv, N, D, theta, off)
        for causal in (False, True):
            fo, fl = ob.forward_reference_grouped_rope(q, k, v, B, Hq, Hkv, N, D, theta, off, causal)
            mo, ml = ob.forward_reference_grouped(rq, rk, v, B, Hq, Hkv, N, D, causal)
            assert_bit_equal(fo, mo)
            assert_bit_equal(fl, ml)


def test_rope_frequency_table_matches_rotated_pair():
    for theta, D in ((1e4, 64), (5e5, 128)):
        f = ob.rope_frequencies(theta, D)
        pos = np.array([12345], dtype=np.uint64)
        x = np.zeros(D, np.float32)
        x[0::2] = 1.0
        r = ob.rotate_rows(x, D, pos, theta)
        ang = np.float32(12345) * f
        # even' = cos(angle), odd' = sin(angle) for (1, 0) pairs
        assert np.abs(r[0::2] - np.cos(ang.astype(np.float64))).max() < 1e-6
        assert np.abs(r[1::2] - np.sin(ang.astype(np.float64))).max() < 1e-6


# ---- tests/projection_grouped.rs:64-181: projection layout == head-major after transpose ---
def pfix(n, phase):
    return ob.fixture(n, 0.023, phase, 1.875, 0.61, 0.3125)


def proj_to_head_major(x, B, H, N, D):
    return np.ascontiguousarray(x.reshape(B, N, H, D).transpose(0, 2, 1, 3)).reshape(-1)


def head_major_to_proj(x, B, H, N, D):
    return np.ascontiguousarray(x.reshape(B, H, N, D).transpose(0, 2, 1, 3)).reshape(-1)


@pytest.mark.parametrize("B,Hq,Hkv,N,D", [(1, 4, 4, 7, 16), (2, 8, 2, 9, 64), (2, 8, 1, 5, 32)])
def test_projection_layout_bit_exact_with_head_major(B, Hq, Hkv, N, D):
    q, k, v = pfix(B * N * Hq * D, 0.3), pfix(B * N * Hkv * D, 0.9), pfix(B * N * Hkv * D, 1.5)
    for theta, off in ((10_000.0, 0), (500_000.0, 19)):
        for causal in (False, True):
            po, pl = ob.forward_reference_projection_grouped_rope(q, k, v, B, Hq, Hkv, N, D, theta, off, causal)
            ho, hl = ob.forward_reference_grouped_rope(
                proj_to_head_major(q, B, Hq, N, D), proj_to_head_major(k, B, Hkv, N, D),
                proj_to_head_major(v, B, Hkv, N, D), B, Hq, Hkv, N, D, theta, off, causal)
            assert_bit_equal(po, head_major_to_proj(ho, B, Hq, N, D))
            assert_bit_equal(pl, hl)  # LSE stays head-major in both


# ---- src/projection_asymmetric.rs:253-347 --------------------------------------------------
def afix(n, phase):
    return ob.fixture(n, 0.071, phase, 0.625)


def test_asymmetric_equal_length_is_r2_oracle_and_decode_is_last_row():
    B, Hq, Hkv, N, D = 1, 4, 2, 7, 8
    q, k, v = afix(B * N * Hq * D, 0.3), afix(B * N * Hkv * D, 0.9), afix(B * N * Hkv * D, 1.5)
    full_o, full_l = ob.forward_reference_projection_grouped_rope(q, k, v, B, Hq, Hkv, N, D, 1e4, 11, True)
    width = Hq * D
    dq = q[(N - 1) * width:N * width]
    o, l = ob.forward_reference_projection_grouped_rope_asymmetric(
        dq, k, v, ob._shape(1, Hq, Hkv, 1, N, D, N - 1), 1e4, 11 + N - 1, 11, True)
    assert_bit_equal(o, full_o[(N - 1) * width:N * width])
    assert_bit_equal(l, full_l.reshape(Hq, N)[:, N - 1])


# ---- src/asymmetric_grouped.rs:351-546 -----------------------------------------------------
def dfix(n, phase):
    return ob.fixture(n, 0.173, phase, 0.7)


def test_asymmetric_grouped_matches_grouped_and_decode_last_row():
    B, Hq, Hkv, N, D = 2, 8, 2, 6, 16
    q, k, v = dfix(B * Hq * N * D, 0.1), dfix(B * Hkv * N * D, 0.7), dfix(B * Hkv * N * D, 1.3)
    for causal in (False, True):
        a = ob.forward_reference_grouped_asymmetric(q, k, v, ob._shape(B, Hq, Hkv, N, N, D, 0), causal)
        g = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, causal)
        assert_bit_equal(a[0], g[0]) and assert_bit_equal(a[1], g[1])
    B, Hq, Hkv, N, D = 1, 4, 2, 9, 8
    q, k, v = dfix(Hq * N * D, 0.2), dfix(Hkv * N * D, 0.8), dfix(Hkv * N * D, 1.4)
    fo, fl = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, True)
    dq = q.reshape(Hq, N, D)[:, N - 1].reshape(-1)
    o, l = ob.forward_reference_grouped_asymmetric(dq, k, v, ob._shape(1, Hq, Hkv, 1, N, D, N - 1), True)
    assert_bit_equal(o, fo.reshape(Hq, N, D)[:, N - 1].reshape(-1))
    assert_bit_equal(l, fl.reshape(Hq, N)[:, N - 1])


def test_variable_lengths_match_independent_calls_and_padding_is_inert():
    B, Hq, Hkv, Nq, Nkv, D = 2, 4, 2, 5, 7, 8
    shape = ob._shape(B, Hq, Hkv, Nq, Nkv, D)
    q, k, v = dfix(B * Hq * Nq * D, 0.15), dfix(B * Hkv * Nkv * D, 0.75), dfix(B * Hkv * Nkv * D, 1.35)
    active = [(3, 5, 2), (5, 7, 0)]
    for causal in (False, True):
        bo, bl = ob.forward_reference_variable_lengths(q, k, v, shape, active, causal)
        bo, bl = bo.reshape(B, Hq, Nq, D), bl.reshape(B, Hq, Nq)
        for b, (aq, akv, off) in enumerate(active):
            q1 = q.reshape(B, Hq, Nq, D)[b, :, :aq].reshape(-1)
            k1 = k.reshape(B, Hkv, Nkv, D)[b, :, :akv].reshape(-1)
            v1 = v.reshape(B, Hkv, Nkv, D)[b, :, :akv].reshape(-1)
            eo, el = ob.forward_reference_grouped_asymmetric(q1, k1, v1, ob._shape(1, Hq, Hkv, aq, akv, D, off), causal)
            assert_bit_equal(bo[b, :, :aq], eo.reshape(Hq, aq, D))
            assert_bit_equal(bl[b, :, :aq], el.reshape(Hq, aq))
            assert np.all(bo[b, :, aq:] == 0.0)
            assert np.all(bl[b, :, aq:] == -INF)
    # poisoned padding (src/asymmetric_grouped.rs:497-546)
    shape = ob._shape(1, 4, 2, 4, 6, 8)
    q, k, v = dfix(4 * 4 * 8, 0.25), dfix(2 * 6 * 8, 0.85), dfix(2 * 6 * 8, 1.45)
    pq, pk, pv = q.reshape(4, 4, 8).copy(), k.reshape(2, 6, 8).copy(), v.reshape(2, 6, 8).copy()
    pq[:, 2:] = 1.0e20
    pk[:, 3:] = -1.0e20
    pv[:, 3:] = 1.0e20
    clean = ob.forward_reference_variable_lengths(q, k, v, shape, [(2, 3, 1)], True)
    poisoned = ob.forward_reference_variable_lengths(pq, pk, pv, shape, [(2, 3, 1)], True)
    assert_bit_equal(clean[0], poisoned[0]) and assert_bit_equal(clean[1], poisoned[1])


def test_variable_length_metadata_is_validated():
    shape = ob._shape(2, 4, 2, 4, 6, 8)
    q, k, v = np.zeros(2 * 4 * 4 * 8), np.zeros(2 * 2 * 6 * 8), np.zeros(2 * 2 * 6 * 8)
    for active, status, word in (([(1, 1, 0)], 7, "metadata"), ([(5, 1, 0), (1, 1, 0)], 7, "query"),
                                 ([(1, 7, 0), (1, 1, 0)], 7, "KV"), ([(0, 1, 0), (1, 1, 0)], 1, "")):
        with pytest.raises(ob.OracleError) as e:
            ob.forward_reference_variable_lengths(q, k, v, shape, active)
        assert e.value.status == status and word in e.value.detail


# ---- src/chunked_projection_prefill.rs:215-285 ---------------------------------------------
def cfix(n, phase):
    return ob.fixture(n, 0.021, phase, 1.125, 0.43, 0.3125)


@pytest.mark.parametrize("shape,causal,chunk", [((2, 4, 2, 9, 8), c, s) for c in (False, True) for s in (1, 2, 3, 4, 8, 16)]
                         + [((2, 4, 1, 7, 8), c, s) for c in (False, True) for s in (1, 2, 3, 4, 8, 16)]
                         + [((1, 6, 2, 5, 16), True, 64)])
def test_chunked_prefill_bit_exact(shape, causal, chunk):
    B, Hq, Hkv, N, D = shape
    q, k, v = cfix(B * N * Hq * D, 0.2), cfix(B * N * Hkv * D, 0.8), cfix(B * N * Hkv * D, 1.4)
    co, cl = ob.forward_reference_projection_grouped_rope(q, k, v, B, Hq, Hkv, N, D, 1e4, 7, causal)
    ho, hl = ob.forward_reference_projection_grouped_rope_chunked_prefill(q, k, v, B, Hq, Hkv, N, D, 1e4, 7, chunk, causal)
    assert_bit_equal(co, ho)
    assert_bit_equal(cl, hl)


def test_zero_query_chunk_size_rejected():
    with pytest.raises(ob.OracleError) as e:
        ob.forward_reference_projection_grouped_rope_chunked_prefill([1, 2], [3, 4], [5, 6], 1, 1, 1, 1, 2, 1e4, 0, 0)
    assert e.value.status == 50


# ---- tests/m38_property_stress.rs:44-143 ---------------------------------------------------
class Lcg:
    def __init__(self, seed):
        self.s = seed

    def next_u32(self):
        self.s = (self.s * 6364136223846793005 + 1442695040888963407) % (1 << 64)
        return self.s >> 32

    def pick(self, upper):
        return self.next_u32() % upper

    def finite(self):
        return np.float32((self.next_u32() / 4294967295.0 * 2.0 - 1.0) * 3.0)


def test_randomized_grouped_invariants():
    rng = Lcg(0x4D385EEDCAFEBABE)
    for case in range(64):
        B = 1 + rng.pick(2)
        Hq = [1, 2, 4, 8][rng.pick(4)]
        divs = [d for d in range(1, Hq + 1) if Hq % d == 0]
        Hkv = divs[rng.pick(len(divs))]
        N = 1 + rng.pick(33)
        D = [1, 2, 4, 8, 16, 32, 64, 128][rng.pick(8)]
        q = np.array([rng.finite() for _ in range(B * Hq * N * D)], np.float32)
        k = np.array([rng.finite() for _ in range(B * Hkv * N * D)], np.float32)
        v = np.array([rng.finite() for _ in range(B * Hkv * N * D)], np.float32)
        causal = case % 2 == 0
        o, l = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, causal)
        assert np.isfinite(o).all() and np.isfinite(l).all()
        on, _ = ob.forward_reference_grouped(q, k, np.ones_like(v), B, Hq, Hkv, N, D, causal)
        assert np.abs(on - 1.0).max() <= 3.0e-5
        if causal:
            g = Hq // Hkv
            o4, v4 = o.reshape(B, Hq, N, D), v.reshape(B, Hkv, N, D)
            for h in range(Hq):
                e = v4[:, h // g, 0]
                assert np.all(np.abs(o4[:, h, 0] - e) <= 2.0e-4 + 1.0e-3 * np.abs(e))


def test_extreme_scores_stay_finite_and_normalised():
    B, Hq, Hkv, N, D = 1, 8, 1, 33, 128
    q = np.where(np.arange(Hq * N * D) % 2 == 0, 1000.0, -1000.0).astype(np.float32)
    k = np.where(np.arange(Hkv * N * D) % 3 == 0, -1000.0, 1000.0).astype(np.float32)
    v = np.ones(Hkv * N * D, np.float32)
    for causal in (False, True):
        o, l = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, causal)
        assert np.isfinite(o).all() and np.isfinite(l).all()
        assert np.abs(o - 1.0).max() <= 3.0e-5


# ---- tests/numerical_policy.rs:12-107: adversarial fixtures, finite and bit-repeatable ------
def test_adversarial_corpus_is_finite_and_repeatable():
    B, H, N, D = 1, 2, 17, 32
    n = B * H * N * D
    i = np.arange(n)
    f32 = np.float32
    corpus = [
        (np.zeros(n, f32), np.ones(n, f32), ((i % 17) * 0.125 - 1.0).astype(f32)),
        (np.sin(i.astype(f32) * f32(1e-5)).astype(f32) * f32(1e-2), np.cos(i.astype(f32) * f32(1e-5)).astype(f32) * f32(1e-2),
         np.sin(i.astype(f32) * f32(0.031)).astype(f32)),
        (np.where(i % 2 == 0, 7.75, -7.75).astype(f32), np.where((i // 3) % 2 == 0, -6.5, 6.5).astype(f32),
         np.where((i // 5) % 2 == 0, 3.0, -3.0).astype(f32)),
        (np.where(i % 2 == 0, 24.0, -24.0).astype(f32), np.where((i // 2) % 2 == 0, 22.0, -22.0).astype(f32),
         (np.cos(i.astype(f32) * f32(0.017)) * 4.0).astype(f32)),
    ]
    for q, k, v in corpus:
        for causal in (False, True):
            for scale in (None, 1.0e-3, 0.25, 2.0):
                a = ob.forward_reference(q, k, v, B, H, N, D, causal, scale)
                b = ob.forward_reference(q, k, v, B, H, N, D, causal, scale)
                assert np.isfinite(a[0]).all() and np.isfinite(a[1]).all()
                assert_bit_equal(a[0], b[0]) and assert_bit_equal(a[1], b[1])


# ---- tests/wgpu_matrix.rs:161-195 (oracle side): zero Q/K, causal row 0 == V[0] bit-exact ---
def test_causal_row_zero_is_v0():
    B, H, N, D = 1, 1, 9, 8
    v = ob.fixture(N * D, 0.3, 0.1, 2.0)
    z = np.zeros(N * D, np.float32)
    o, l = ob.forward_reference(z, z, v, B, H, N, D, True)
    assert_bit_equal(o[:D], v[:D])
    assert l[0] == 0.0


# ---- sampled-row API equals the full oracle bit for bit --------------------------------------
def test_forward_rows_equals_full_oracle():
    B, Hq, Hkv, Nq, Nkv, D = 2, 4, 2, 5, 11, 16
    shape = ob._shape(B, Hq, Hkv, Nq, Nkv, D, 6)
    q, k, v = dfix(B * Hq * Nq * D, 0.1), dfix(B * Hkv * Nkv * D, 0.5), dfix(B * Hkv * Nkv * D, 0.9)
    fo, fl = ob.forward_reference_grouped_asymmetric(q, k, v, shape, True)
    rows = [(b, h, r) for b in range(B) for h in range(Hq) for r in range(Nq)]
    ro, rl = ob.forward_rows(q, k, v, shape, ob.HEAD_MAJOR, rows, True, threads=3)
    assert_bit_equal(ro.reshape(-1), fo)
    assert_bit_equal(rl, fl)
