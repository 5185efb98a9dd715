"""Pins of the CPU oracle (backward and paged-KV metadata): the reference's unit tests restated."""
import numpy as np
import pytest

from oracle import binding as ob


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def bfix(n, phase, step=0.31, a=0.65, c=0.43, b=0.23):
    return ob.fixture(n, step, phase, a, c, b)


def objective(q, k, v, d_out, B, Hq, Hkv, N, D, causal, scale):
    o, _ = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, causal, scale)
    acc = np.float32(0.0)
    for x, g in zip(o, d_out):  # serial f32 sum like the Rust iterator
        acc = np.float32(acc + np.float32(x * g))
    return acc


def finite_difference(t, idx, eps, fn):
    orig = t[idx]
    t[idx] = orig + np.float32(eps)
    plus = fn(t)
    t[idx] = orig - np.float32(eps)
    minus = fn(t)
    t[idx] = orig
    return np.float32((plus - minus) / np.float32(2.0 * eps))


# src/backward.rs:158-211 (MHA, tol 3e-3 + 1.5e-2|x|) and src/backward_grouped.rs:153-206
# (GQA/MQA, tol 4e-3 + 2e-2|x|)
@pytest.mark.parametrize("Hq,Hkv,causal,scale,fx,atol,rtol", [
    (1, 1, False, 0.73, dict(step=0.37, a=0.7, c=0.41, b=0.2), 3.0e-3, 1.5e-2),
    (1, 1, True, 0.73, dict(step=0.37, a=0.7, c=0.41, b=0.2), 3.0e-3, 1.5e-2),
    (4, 2, True, 0.67, {}, 4.0e-3, 2.0e-2),
    (4, 1, False, 0.67, {}, 4.0e-3, 2.0e-2),
])
def test_backward_matches_finite_differences(Hq, Hkv, causal, scale, fx, atol, rtol):
    B, N, D = 1, 3, 2
    q, k, v = bfix(B * Hq * N * D, 0.1, **fx), bfix(B * Hkv * N * D, 0.8, **fx), bfix(B * Hkv * N * D, 1.4, **fx)
    d_out = bfix(B * Hq * N * D, 2.2 if Hq == 1 else 2.1, **fx)
    fo, fl = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, causal, scale)
    dq, dk, dv = ob.backward_reference_grouped(q, k, v, d_out, fo, fl, B, Hq, Hkv, N, D, causal, scale)
    eps = 1.0e-3
    nq = [finite_difference(q, i, eps, lambda c: objective(c, k, v, d_out, B, Hq, Hkv, N, D, causal, scale)) for i in range(q.size)]
    nk = [finite_difference(k, i, eps, lambda c: objective(q, c, v, d_out, B, Hq, Hkv, N, D, causal, scale)) for i in range(k.size)]
    nv = [finite_difference(v, i, eps, lambda c: objective(q, k, c, d_out, B, Hq, Hkv, N, D, causal, scale)) for i in range(v.size)]
    for an, nu in ((dq, nq), (dk, nk), (dv, nv)):
        nu = np.array(nu, np.float32)
        assert np.all(np.abs(an - nu) <= atol + rtol * np.abs(nu))


def test_backward_rejects_malformed_forward():
    z = np.zeros(4, np.float32)
    with pytest.raises(ob.OracleError) as e:
        ob.backward_reference(z, z, z, z, np.zeros(3), np.zeros(2), 1, 1, 2, 2)
    assert e.value.status == 7 and "O" in e.value.detail


def test_backward_cardinality_and_units_equal_full():
    B, Hq, Hkv, N, D = 2, 8, 2, 5, 4
    q, k, v = bfix(B * Hq * N * D, 0.2), bfix(B * Hkv * N * D, 0.8), bfix(B * Hkv * N * D, 1.3)
    d_out = bfix(B * Hq * N * D, 1.9)
    for causal in (False, True):
        fo, fl = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, causal)
        dq, dk, dv = ob.backward_reference_grouped(q, k, v, d_out, fo, fl, B, Hq, Hkv, N, D, causal)
        assert dq.size == q.size and dk.size == k.size and dv.size == v.size
        units = [(b, h) for b in range(B) for h in range(Hkv)]
        uq, uk, uv = ob.backward_units(q, k, v, d_out, fo, fl, B, Hq, Hkv, N, D, units, causal, threads=2)
        assert np.array_equal(bits(uq.reshape(-1)), bits(dq))
        assert np.array_equal(bits(uk.reshape(-1)), bits(dk))
        assert np.array_equal(bits(uv.reshape(-1)), bits(dv))


def test_backward_rows_equal_full_oracle():
    B, Hq, Hkv, N, D = 2, 4, 2, 7, 8
    q, k, v = bfix(B * Hq * N * D, 0.2), bfix(B * Hkv * N * D, 0.8), bfix(B * Hkv * N * D, 1.3)
    d_out = bfix(B * Hq * N * D, 1.9)
    for causal in (False, True):
        fo, fl = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, causal)
        dq, dk, dv = ob.backward_reference_grouped(q, k, v, d_out, fo, fl, B, Hq, Hkv, N, D, causal)
        qr = [(b, h, r) for b in range(B) for h in range(Hq) for r in range(N)]
        kr = [(b, h, r) for b in range(B) for h in range(Hkv) for r in range(N)]
        rq, rk, rv = ob.backward_rows(q, k, v, d_out, fo, fl, B, Hq, Hkv, N, D, qr, kr, causal, threads=3)
        assert np.array_equal(bits(rq.reshape(-1)), bits(dq))
        assert np.array_equal(bits(rk.reshape(-1)), bits(dk))
        assert np.array_equal(bits(rv.reshape(-1)), bits(dv))


# ---- src/paged_kv.rs:200-270 ------------------------------------------------------------------
def test_mapping_is_stable_across_page_boundaries():
    t = ob.PagedKvTable(4, 3)
    t.append(9)
    assert t.address(0)[0] == 0
    assert t.address(3)[1] == 3
    assert t.address(4)[0] == 1
    assert t.address(8)[0] == 2
    assert t.address(9) is None


def test_telemetry_reports_exact_internal_fragmentation():
    t = ob.PagedKvTable(8, 4)
    t.append(9)
    assert t.telemetry() == dict(live_tokens=9, capacity_tokens=32, mapped_pages=2, free_pages=2,
                                 internal_fragmentation_tokens=7, generation=0)


def test_reset_invalidates_old_generation_before_page_reuse():
    t = ob.PagedKvTable(2, 2)
    t.append(1)
    old = t.address(0)
    t.reset()
    assert t.address(0) is None
    t.append(1)
    new = t.address(0)
    assert old[0] == new[0] and old[2] != new[2]


def test_capacity_overflow_is_explicit_and_non_mutating():
    t = ob.PagedKvTable(4, 2)
    t.append(7)
    before = t.telemetry()
    with pytest.raises(ob.OracleError) as e:
        t.append(2)
    assert e.value.status == 41 and "9" in e.value.detail and "8" in e.value.detail
    assert t.telemetry() == before
    with pytest.raises(ob.OracleError) as e:
        ob.PagedKvTable(0, 2)
    assert e.value.status == 1
