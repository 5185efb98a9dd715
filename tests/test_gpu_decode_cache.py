"""Resident / paged KV caches and q_len = 1 decode against the CPU oracle (f32 and bf16):
tests/m14_resident_kv_cache.rs, m15_growing_cache.rs, m15_external_resident.rs, m16_paged_decode.rs,
m16_paged_kv_cache.rs, plus the batched paged decode of benchmark configuration 3 (reduced and full size)."""
import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.gpu_util import assert_close, bf16_round, ctx, dev, fa, ramp

pytestmark = pytest.mark.gpu
TOL = (2.0e-4, 1.0e-3)  # tests/m16_paged_decode.rs:12-13


def oracle_decode(q, k_rows, v_rows, Hq, Hkv, D, theta, q_pos, kv_off, pre_rotated, scale=None):
    """q [Hq*D]; k_rows/v_rows [n, Hkv*D] in logical order.  With pre-rotated K the rotation of Q is
    materialised with the oracle formula and the no-RoPE rectangular oracle is used (bit-identical
    route, tests/rotary_grouped.rs:48-143)."""
    n = k_rows.shape[0]
    if pre_rotated:
        rq = ob.rotate_rows(q, D, np.full(Hq, q_pos, np.uint64), theta)
        kh = k_rows.reshape(n, Hkv, D).transpose(1, 0, 2)
        vh = v_rows.reshape(n, Hkv, D).transpose(1, 0, 2)
        return ob.forward_reference_grouped_asymmetric(rq, kh, vh, ob._shape(1, Hq, Hkv, 1, n, D, n - 1), True, scale)
    return ob.forward_reference_projection_grouped_rope_asymmetric(q, k_rows, v_rows, ob._shape(1, Hq, Hkv, 1, n, D, n - 1),
                                                                   theta, q_pos, kv_off, True, scale)


def unpack(out, dtype, rows, D):
    raw = out.cpu()
    es = 2 if dtype == fa.BF16 else 4
    o = raw[:rows * D * es].view(fa.torch_dtype(dtype)).float().numpy().reshape(rows, D)
    l = raw[rows * D * es:rows * D * es + rows * 4].view(torch.float32).numpy()
    return o, l


# ---- resident cache ---------------------------------------------------------------------------
def test_resident_cache_append_prefix_stride_reset():
    c = ctx()
    B, Hkv, cap, D = 2, 2, 7, 16
    cache = fa.CudaResidentKvCache(c, fa.F32, B, Hkv, cap, D)
    W = Hkv * D
    k1, v1 = ramp(B * 3 * W, 0.1).reshape(B, 3, W), ramp(B * 3 * W, 0.6).reshape(B, 3, W)
    assert cache.record_append(dev(k1), dev(v1), 3) == 3
    k2, v2 = ramp(B * 2 * W, 1.1).reshape(B, 2, W), ramp(B * 2 * W, 1.6).reshape(B, 2, W)
    assert cache.record_append(dev(k2), dev(v2), 2) == 5
    c.synchronize()
    K, V = cache.download()
    assert np.array_equal(K[:, :3].numpy(), k1) and np.array_equal(K[:, 3:5].numpy(), k2)
    assert np.array_equal(V[:, :3].numpy(), v1) and np.array_equal(V[:, 3:5].numpy(), v2)
    assert cache.remaining_capacity() == 2
    with pytest.raises(fa.FlatAttentionError) as e:
        cache.record_append(dev(k1), dev(v1), 3)
    assert e.value.kind == "CapacityExceeded" and len(cache) == 5
    with pytest.raises(fa.FlatAttentionError) as e:
        cache.record_append(dev(k1), dev(v1), 0)
    assert e.value.kind == "ZeroDimension"
    with pytest.raises(fa.FlatAttentionError) as e:
        cache.record_append(dev(k2.reshape(-1)[:-1]), dev(v2), 2)
    assert e.value.kind == "BufferTooSmall"
    cache.reset()
    assert len(cache) == 0
    with pytest.raises(fa.FlatAttentionError) as e:
        fa.CudaResidentKvCache(c, fa.F32, 0, 1, 1, 1)
    assert e.value.kind == "ZeroDimension"


@pytest.mark.parametrize("dtype", [fa.F32, fa.BF16])
def test_token_by_token_growth_resident_decode(dtype):
    # tests/m15_growing_cache.rs:146-270: grow 1..6 tokens, decode after each append
    c = ctx()
    Hq, Hkv, D, cap, theta, off = 4, 1, 32, 8, 1e4, 5
    td = fa.torch_dtype(dtype)
    cache = fa.CudaResidentKvCache(c, dtype, 1, Hkv, cap, D)
    W = Hkv * D
    k_raw = ramp(6 * W, 0.3).reshape(6, W)
    v_all = ramp(6 * W, 0.8).reshape(6, W)
    k_rot = ob.rotate_rows(k_raw, D, np.repeat(np.arange(6, dtype=np.uint64) + off, Hkv), theta).reshape(6, W)
    if dtype == fa.BF16:
        k_rot, v_all = bf16_round(k_rot), bf16_round(v_all)
    for step in range(6):
        cache.record_append(dev(k_rot[step:step + 1], td), dev(v_all[step:step + 1], td), 1)
        n = step + 1
        q = ramp(Hq * D, 0.05 * step)
        if dtype == fa.BF16:
            q = bf16_round(q)
        out = c.empty_bytes(Hq * D * 4 + Hq * 4)
        c.decode_resident(dtype, 1, Hq, Hkv, D, n, cap, fa.config(True), theta, off + n - 1, dev(q, td),
                          cache.k_buffer(), cache.v_buffer(), out)
        o, l = unpack(out, dtype, Hq, D)
        eo, el = oracle_decode(q, k_rot[:n], v_all[:n], Hq, Hkv, D, theta, off + n - 1, off, True)
        tol = TOL if dtype == fa.F32 else (2e-2, 0.0)
        assert_close("O", o, eo, *tol)
        assert_close("LSE", l, el, *(TOL if dtype == fa.F32 else (2e-3, 0.0)))


def test_external_capacity_strided_decode_with_poison():
    # tests/m15_external_resident.rs: B=2, Hq=4, Hkv=2, kv 3, capacity 7, D=32; inactive rows poisoned
    c = ctx()
    B, Hq, Hkv, n, cap, D, theta, qpos = 2, 4, 2, 3, 7, 32, 1e4, 9
    W = Hkv * D
    K = np.full((B, cap, W), 17.0, np.float32)
    V = np.full((B, cap, W), -19.0, np.float32)
    k_live, v_live = ramp(B * n * W, 0.2).reshape(B, n, W), ramp(B * n * W, 0.7).reshape(B, n, W)
    K[:, :n], V[:, :n] = k_live, v_live
    q = ramp(B * Hq * D, 0.4).reshape(B, Hq * D)
    out = c.empty_bytes(B * Hq * D * 4 + B * Hq * 4)
    c.decode_resident(fa.F32, B, Hq, Hkv, D, n, cap, fa.config(True), theta, qpos, dev(q), dev(K), dev(V), out)
    o, l = unpack(out, fa.F32, B * Hq, D)
    for b in range(B):
        eo, el = oracle_decode(q[b], k_live[b], v_live[b], Hq, Hkv, D, theta, qpos, 0, True)
        assert_close("O", o[b * Hq:(b + 1) * Hq], eo, *TOL)
        assert_close("LSE", l[b * Hq:(b + 1) * Hq], el, *TOL)
    # validation (src/wgpu_decode.rs:419-435,470-478)
    for args, kind in (((0, cap, qpos), "EmptyCache"), ((8, cap, qpos), "InvalidCacheLength"), ((3, cap, 1), "CausalVisibilityMismatch")):
        with pytest.raises(fa.FlatAttentionError) as e:
            c.decode_resident(fa.F32, B, Hq, Hkv, D, args[0], args[1], fa.config(True), theta, args[2], dev(q), dev(K), dev(V), out)
        assert e.value.kind == kind
    with pytest.raises(fa.FlatAttentionError) as e:
        c.decode_resident(fa.F32, B, Hq, Hkv, D, n, cap, fa.config(True), float("nan"), qpos, dev(q), dev(K), dev(V), out)
    assert e.value.kind == "InvalidTheta"


# ---- paged cache + single-sequence decode -----------------------------------------------------
def test_paged_decode_with_poisoned_unmapped_rows():
    # tests/m16_paged_decode.rs:171-284: Hq4 Hkv2 kv 7 page 3 pages 4 D64, K=17 / V=-19 outside live rows
    c = ctx()
    Hq, Hkv, n, ps, pages, D, theta, qpos = 4, 2, 7, 3, 4, 64, 1e4, 6
    W = Hkv * D
    table = fa.PagedKvTable(ps, pages)
    table.append(n)
    K = np.full((pages * ps, W), 17.0, np.float32)
    V = np.full((pages * ps, W), -19.0, np.float32)
    k_live, v_live = ramp(n * W, 0.2).reshape(n, W), ramp(n * W, 0.7).reshape(n, W)
    for t in range(n):
        page, offset, _ = table.address(t)
        K[page * ps + offset], V[page * ps + offset] = k_live[t], v_live[t]
    q = ramp(Hq * D, 0.4)
    out = c.empty_bytes(Hq * D * 4 + Hq * 4)
    c.decode_paged(fa.F32, table, Hq, Hkv, D, fa.config(True), theta, qpos, dev(q), dev(K), dev(V), out)
    o, l = unpack(out, fa.F32, Hq, D)
    eo, el = oracle_decode(q, k_live, v_live, Hq, Hkv, D, theta, qpos, 0, True)
    assert_close("O", o, eo, *TOL)
    assert_close("LSE", l, el, *TOL)
    with pytest.raises(fa.FlatAttentionError) as e:
        c.decode_paged(fa.F32, table, Hq, Hkv, D, fa.config(True), theta, 3, dev(q), dev(K), dev(V), out)
    assert e.value.kind == "CausalVisibilityMismatch"
    with pytest.raises(fa.FlatAttentionError) as e:
        c.decode_paged(fa.F32, fa.PagedKvTable(ps, pages), Hq, Hkv, D, fa.config(True), theta, qpos, dev(q), dev(K), dev(V), out)
    assert e.value.kind == "EmptyTable"
    with pytest.raises(fa.FlatAttentionError) as e:
        c.decode_paged(fa.F32, table, Hq, Hkv, D, fa.config(True), theta, qpos, dev(q), dev(K[:-1]), dev(V), out)
    assert e.value.kind == "BufferTooSmall"


def test_paged_cache_append_reset_reuse_then_decode():
    # tests/m16_paged_kv_cache.rs:159-396: page 3 x 4, append 2 then 4, reset, reuse; cache -> decode
    c = ctx()
    ps, pages, Hkv, D = 3, 4, 1, 8
    cache = fa.CudaPagedKvCache(c, fa.F32, ps, pages, Hkv, D)
    W = Hkv * D
    k_all, v_all = ramp(6 * W, 0.1).reshape(6, W), ramp(6 * W, 0.6).reshape(6, W)
    assert cache.record_append(dev(k_all[:2]), dev(v_all[:2]), 2) == 2
    assert cache.record_append(dev(k_all[2:]), dev(v_all[2:]), 4) == 6
    c.synchronize()
    K, V = cache.download()
    tab = cache.table()
    for t in range(6):
        page, offset, gen = tab.address(t)
        assert gen == 0
        assert np.array_equal(K[page * ps + offset].numpy(), k_all[t]) and np.array_equal(V[page * ps + offset].numpy(), v_all[t])
    with pytest.raises(fa.FlatAttentionError) as e:
        cache.record_append(dev(ramp(7 * W, 0.3)), dev(ramp(7 * W, 0.4)), 7)
    assert e.value.kind == "CapacityExceeded" and len(cache) == 6
    cache.reset()
    assert len(cache) == 0 and cache.generation() == 1 and cache.table().address(0) is None
    cache.record_append(dev(v_all[:4]), dev(k_all[:4]), 4)
    c.synchronize()
    K, V = cache.download()
    assert np.array_equal(K[:4].numpy(), v_all[:4])  # lowest physical pages are reused first

    Hq, Hkv, n, ps, D, theta = 4, 1, 5, 2, 32, 1e4
    cache = fa.CudaPagedKvCache(c, fa.F32, ps, 4, Hkv, D)
    k_raw, v_live = ramp(n * D, 0.3).reshape(n, D), ramp(n * D, 0.9).reshape(n, D)
    cache.record_append_rotating(dev(k_raw[:3]), dev(v_live[:3]), 3, theta, 2)
    cache.record_append_rotating(dev(k_raw[3:]), dev(v_live[3:]), 2, theta, 2)
    q = ramp(Hq * D, 0.4)
    out = c.empty_bytes(Hq * D * 4 + Hq * 4)
    c.decode_paged(fa.F32, cache.table(), Hq, Hkv, D, fa.config(True), theta, 2 + n - 1, dev(q), cache.k_buffer(),
                   cache.v_buffer(), out)
    o, l = unpack(out, fa.F32, Hq, D)
    eo, el = oracle_decode(q, k_raw, v_live, Hq, Hkv, D, theta, 2 + n - 1, 2, False)
    assert_close("O", o, eo, *TOL)
    assert_close("LSE", l, el, *TOL)


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 1, 80), (12, 4, 64), (6, 2, 30)])
def test_paged_decode_shapes_outside_the_streaming_kernel(Hq, Hkv, D):
    """head_dim / group sizes the 16-byte-lane kernel does not take go through the generic kernel."""
    c = ctx()
    n, ps, pages, theta = 21, 4, 8, 5e5
    W = Hkv * D
    table = fa.PagedKvTable(ps, pages)
    table.append(n)
    K, V = np.zeros((pages * ps, W), np.float32), np.zeros((pages * ps, W), np.float32)
    k_live, v_live = ramp(n * W, 0.2).reshape(n, W), ramp(n * W, 0.7).reshape(n, W)
    K[:n], V[:n] = k_live, v_live
    q = ramp(Hq * D, 0.4)
    out = c.empty_bytes(Hq * D * 4 + Hq * 4)
    c.decode_paged(fa.F32, table, Hq, Hkv, D, fa.config(True), theta, n - 1, dev(q), dev(K), dev(V), out)
    o, l = unpack(out, fa.F32, Hq, D)
    eo, el = oracle_decode(q, k_live, v_live, Hq, Hkv, D, theta, n - 1, 0, True)
    assert_close("O", o, eo, *TOL)
    assert_close("LSE", l, el, *TOL)


# ---- batched paged decode (benchmark configuration 3) -------------------------------------------------
def make_paged_batch(num_seqs, Hq, Hkv, D, ps, lo, hi, dtype, seed=5):
    rng = np.random.default_rng(seed)
    lens = (lo + rng.integers(0, hi - lo + 1, num_seqs)).astype(np.int32)
    pages_per = (lens + ps - 1) // ps
    pool = int(pages_per.sum()) + 7
    perm = np.random.default_rng(seed + 1).permutation(pool).astype(np.int32)
    maxp = int(pages_per.max())
    tables = np.full((num_seqs, maxp), -1, np.int32)
    at = 0
    for s in range(num_seqs):
        tables[s, :pages_per[s]] = perm[at:at + pages_per[s]]
        at += pages_per[s]
    g = torch.Generator().manual_seed(seed + 2)
    td = fa.torch_dtype(dtype)
    K = torch.randn(pool * ps, Hkv * D, generator=g).to(td)
    V = torch.randn(pool * ps, Hkv * D, generator=g).to(td)
    Q = torch.randn(num_seqs, Hq * D, generator=g).to(td)
    return lens, tables, pool, maxp, Q, K, V


def run_batched(c, dtype, lens, tables, pool, maxp, Q, K, V, Hq, Hkv, D, ps, theta, splits=0, Kd=None, Vd=None):
    n = len(lens)
    qpos = (lens - 1).astype(np.int32)
    safe = np.where(tables < 0, 0, tables).astype(np.int32)
    es = 2 if dtype == fa.BF16 else 4
    out = c.empty_bytes(n * Hq * D * es + n * Hq * 4)
    out.fill_(0x7f)
    c.decode_paged_batched(dtype, n, Hq, Hkv, D, ps, pool, maxp, torch.from_numpy(safe).cuda(), torch.from_numpy(lens).cuda(),
                           torch.from_numpy(qpos).cuda(), safe, lens, qpos, fa.config(True), theta, Q.cuda(),
                           K.cuda() if Kd is None else Kd, V.cuda() if Vd is None else Vd, out, kv_splits=splits)
    return unpack(out, dtype, n * Hq, D)


def check_batched(o, l, lens, tables, Q, K, V, Hq, Hkv, D, ps, theta, otol, ltol, seqs=None):
    Kf, Vf, Qf = K.float().numpy(), V.float().numpy(), Q.float().numpy()
    for s in (range(len(lens)) if seqs is None else seqs):
        rows = np.array([tables[s, t // ps] * ps + t % ps for t in range(lens[s])])
        eo, el = oracle_decode(Qf[s], Kf[rows], Vf[rows], Hq, Hkv, D, theta, int(lens[s]) - 1, 0, True)
        assert_close("O seq %d" % s, o[s * Hq:(s + 1) * Hq], eo, *otol)
        assert_close("LSE seq %d" % s, l[s * Hq:(s + 1) * Hq], el, *ltol)


@pytest.mark.parametrize("dtype,Hq,Hkv,D,splits", [(fa.F32, 8, 2, 64, 0), (fa.F32, 8, 2, 64, 3), (fa.BF16, 32, 8, 128, 0),
                                                     (fa.BF16, 32, 8, 128, 1), (fa.BF16, 32, 8, 128, 5), (fa.BF16, 16, 16, 64, 2),
                                                     (fa.F32, 8, 1, 128, 4)])
def test_batched_paged_decode_permuted_pages(dtype, Hq, Hkv, D, splits):
    c = ctx()
    ps, theta = 16, 5e5
    lens, tables, pool, maxp, Q, K, V = make_paged_batch(6, Hq, Hkv, D, ps, 17, 700, dtype)
    o, l = run_batched(c, dtype, lens, tables, pool, maxp, Q, K, V, Hq, Hkv, D, ps, theta, splits)
    if dtype == fa.F32:
        check_batched(o, l, lens, tables, Q, K, V, Hq, Hkv, D, ps, theta, TOL, TOL)
    else:
        check_batched(o, l, lens, tables, Q, K, V, Hq, Hkv, D, ps, theta, (2e-2, 0.0), (2e-3, 0.0))
    assert c.device_status() == 0


def test_batched_paged_decode_validation():
    c = ctx()
    Hq, Hkv, D, ps, theta = 8, 2, 64, 16, 1e4
    lens, tables, pool, maxp, Q, K, V = make_paged_batch(3, Hq, Hkv, D, ps, 17, 100, fa.F32)
    qpos = (lens - 1).astype(np.int32)
    safe = np.where(tables < 0, 0, tables).astype(np.int32)
    out = c.empty_bytes(3 * Hq * D * 4 + 3 * Hq * 4)
    dt, dl, dq = torch.from_numpy(safe).cuda(), torch.from_numpy(lens).cuda(), torch.from_numpy(qpos).cuda()

    def call(tab=safe, ln=lens, qp=qpos, pool_=pool):
        c.decode_paged_batched(fa.F32, 3, Hq, Hkv, D, ps, pool_, maxp, dt, dl, dq, tab, ln, qp, fa.config(True), theta,
                               Q.cuda(), K.cuda(), V.cuda(), out)
    bad = safe.copy(); bad[1, 0] = pool
    with pytest.raises(fa.FlatAttentionError) as e:
        call(tab=bad)
    assert e.value.kind == "PageOutOfRange"
    bad = safe.copy(); bad[2, 0] = safe[0, 0]
    with pytest.raises(fa.FlatAttentionError) as e:
        call(tab=bad)
    assert e.value.kind == "PageShared"
    with pytest.raises(fa.FlatAttentionError) as e:
        call(qp=(lens - 2).astype(np.int32))
    assert e.value.kind == "CausalVisibilityMismatch"
    bad = lens.copy(); bad[0] = 0
    with pytest.raises(fa.FlatAttentionError) as e:
        call(ln=bad)
    assert e.value.kind == "EmptyTable"
    call()


def test_config3_full_size_properties_and_sampled_oracle():
    """64 sequences, Hq=32 Hkv=8 D=128 bf16, page 16, ctx U[512,8192], permuted pool.  Oracle on four
    sequences (shortest, longest, two others); for all of them: V = 1 gives O = 1, and the result
    is invariant to the split along KV within tolerance."""
    c = ctx()
    Hq, Hkv, D, ps, theta = 32, 8, 128, 16, 5e5
    lens, tables, pool, maxp, Q, K, V = make_paged_batch(64, Hq, Hkv, D, ps, 512, 8192, fa.BF16)
    Kd, Vd = K.cuda(), V.cuda()
    o, l = run_batched(c, fa.BF16, lens, tables, pool, maxp, Q, K, V, Hq, Hkv, D, ps, theta, 0, Kd, Vd)
    picks = sorted({int(np.argmin(lens)), int(np.argmax(lens)), 7, 40})
    check_batched(o, l, lens, tables, Q, K, V, Hq, Hkv, D, ps, theta, (2e-2, 0.0), (2e-3, 0.0), seqs=picks)
    o1, l1 = run_batched(c, fa.BF16, lens, tables, pool, maxp, Q, K, V, Hq, Hkv, D, ps, theta, 1, Kd, Vd)
    assert np.abs(o - o1).max() <= 2e-2 and np.abs(l - l1).max() <= 2e-4
    ones = torch.ones_like(V).cuda()
    oo, lo = run_batched(c, fa.BF16, lens, tables, pool, maxp, Q, K, V, Hq, Hkv, D, ps, theta, 0, Kd, ones)
    assert np.abs(oo - 1.0).max() <= 8e-3  # bf16 rounding of an output that is 1 up to f32 error
    assert np.abs(lo - l).max() == 0.0     # LSE does not depend on V
    assert c.device_status() == 0


def test_splitkv_merge_matches_unsplit():
    c = ctx()
    parts, rows, D = 5, 24, 128
    g = torch.Generator().manual_seed(3)
    po = torch.randn(parts, rows, D, generator=g)
    pl = torch.randn(parts, rows, generator=g) * 3
    out = c.empty_bytes(rows * D * 4 + rows * 4)
    c.splitkv_merge(fa.F32, parts, rows, D, po.cuda(), pl.cuda(), out)
    o, l = unpack(out, fa.F32, rows, D)
    tot = torch.logsumexp(pl.double(), 0)
    w = torch.exp(pl.double() - tot)
    eo = (w[:, :, None] * po.double()).sum(0)
    assert_close("O", o, eo.float().numpy(), 1e-5, 1e-5)
    assert_close("LSE", l, tot.float().numpy(), 1e-5, 1e-5)


@pytest.mark.parametrize("parts", [2, 8])
def test_kv_split_across_ranks_emulated_on_one_gpu(parts):
    """Single-sequence long-context decode split along KV: every 'rank' holds a contiguous page range
    in its own cache slice, computes the f32 partial (O_i, LSE_i); the packed partials (the all-gather
    output) are merged.  Result = unsplit decode = oracle."""
    import importlib.util, os
    spec = importlib.util.spec_from_file_location("fd", os.path.join(os.path.dirname(fa.__file__), "distributed.py"))
    fd = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(fd)
    c = ctx()
    Hq, Hkv, D, ps, theta, n = 32, 8, 128, 16, 5e5, 16 * 515 + 7
    g = torch.Generator().manual_seed(9)
    K = torch.randn(n, Hkv * D, generator=g).bfloat16()
    V = torch.randn(n, Hkv * D, generator=g).bfloat16()
    Q = torch.randn(1, Hq * D, generator=g).bfloat16()
    qpos = np.array([n - 1], np.int32)
    blocks = []
    for r in range(parts):
        first, count = fd.shard_pages(n, ps, parts, r)
        pages = (count + ps - 1) // ps
        pool = pages + 3
        perm = np.random.default_rng(r).permutation(pool).astype(np.int32)[:pages]
        Kc, Vc = torch.zeros(pool * ps, Hkv * D, dtype=torch.bfloat16), torch.zeros(pool * ps, Hkv * D, dtype=torch.bfloat16)
        for i in range(pages):
            lo, hi = first + i * ps, min(first + count, first + (i + 1) * ps)
            Kc[perm[i] * ps:perm[i] * ps + hi - lo] = K[lo:hi]
            Vc[perm[i] * ps:perm[i] * ps + hi - lo] = V[lo:hi]
        lens = np.array([count], np.int32)
        tab = perm.reshape(1, pages)
        out = torch.empty(Hq * (D + 1), dtype=torch.float32, device="cuda")
        c.decode_paged_batched_partial(fa.BF16, 1, Hq, Hkv, D, ps, pool, pages, torch.from_numpy(tab).cuda(),
                                       torch.from_numpy(lens).cuda(), torch.from_numpy(qpos).cuda(), tab, lens,
                                       fa.config(True), theta, Q.cuda(), Kc.cuda(), Vc.cuda(), out)
        blocks.append(out)
    gathered = torch.stack(blocks)
    final = c.empty_bytes(Hq * D * 2 + Hq * 4)
    c.splitkv_merge_packed(fa.BF16, parts, Hq, D, gathered, final)
    o, l = unpack(final, fa.BF16, Hq, D)
    eo, el = oracle_decode(Q[0].float().numpy(), K.float().numpy(), V.float().numpy(), Hq, Hkv, D, theta, n - 1, 0, True)
    assert_close("O", o, eo, 2e-2, 0.0)
    assert_close("LSE", l, el, 2e-3, 0.0)
    # the reference merge formula on the same partials
    po = gathered[:, :Hq * D].reshape(parts, Hq, D).cpu()
    pl = gathered[:, Hq * D:].cpu()
    mo, ml = fd.merge_partials_reference(po, pl)
    assert_close("merge O", o, mo.numpy(), 8e-3, 0.0)
    assert_close("merge LSE", l, ml.numpy(), 1e-5, 0.0)


def _one_sequence_slice(n, Hq=32, Hkv=8, D=128, ps=16, seed=21):
    g = torch.Generator().manual_seed(seed)
    K = torch.randn(n, Hkv * D, generator=g).bfloat16()
    V = torch.randn(n, Hkv * D, generator=g).bfloat16()
    Q = torch.randn(1, Hq * D, generator=g).bfloat16()
    pages = (n + ps - 1) // ps
    pool = pages + 2
    perm = np.random.default_rng(seed).permutation(pool).astype(np.int32)[:pages]
    Kc, Vc = torch.zeros(pool * ps, Hkv * D, dtype=torch.bfloat16), torch.zeros(pool * ps, Hkv * D, dtype=torch.bfloat16)
    for i in range(pages):
        lo, hi = i * ps, min(n, (i + 1) * ps)
        Kc[perm[i] * ps:perm[i] * ps + hi - lo] = K[lo:hi]
        Vc[perm[i] * ps:perm[i] * ps + hi - lo] = V[lo:hi]
    tab, lens, qpos = perm.reshape(1, pages), np.array([n], np.int32), np.array([n - 1], np.int32)
    args = (1, Hq, Hkv, D, ps, pool, pages, torch.from_numpy(tab).cuda(), torch.from_numpy(lens).cuda(),
            torch.from_numpy(qpos).cuda(), tab, lens, fa.config(True), 5e5, Q.cuda(), Kc.cuda(), Vc.cuda())
    return args, Hq, D


def test_peer_exchange_with_one_rank_equals_partial_plus_merge():
    """flat_splitkv_decode_peer on a one-rank exchange (no peer to map): the exchange kernel stores the partial into
    the rank's own buffer, sees its own flag and merges one part.  Same bits as the partial followed by
    flat_splitkv_merge_packed, step after step (both receive buffers and the device-side step counter)."""
    c = ctx()
    args, Hq, D = _one_sequence_slice(16 * 133 + 3)
    part = torch.empty(Hq * (D + 1), dtype=torch.float32, device="cuda")
    c.decode_paged_batched_partial(fa.BF16, *args, part)
    want = c.create_decode_output_buffer(fa.BF16, 1, Hq, D)
    c.splitkv_merge_packed(fa.BF16, 1, Hq, D, part, want)
    x = fa.SplitKvPeerExchange(c, 0, 1, Hq, D)
    try:
        for step in range(4):
            got = c.create_decode_output_buffer(fa.BF16, 1, Hq, D)
            got.zero_()
            c.splitkv_decode_peer(x, fa.BF16, *args, got)
            c.synchronize()
            assert torch.equal(got, want), f"step {step}"
        assert c.device_status() == 0
    finally:
        x.close()


def test_peer_exchange_wait_gives_up_when_a_rank_never_arrives():
    """The exchange kernel's wait for the other ranks' flags is bounded: a two-rank exchange whose second rank does
    not exist (its handle slot names this process's own buffer, so the stores have a place to go) runs into the limit
    after about a second, the status word reports FLAT_ERR_DEVICE_WAIT_TIMEOUT with the absent rank, and the context
    goes on working."""
    c = ctx()
    args, Hq, D = _one_sequence_slice(16 * 40)
    x = fa.SplitKvPeerExchange(c, 0, 2, Hq, D)
    try:
        x.connect(x.handle() * 2)
        out = c.create_decode_output_buffer(fa.BF16, 1, Hq, D)
        c.splitkv_decode_peer(x, fa.BF16, *args, out)
        c.synchronize()
        assert c.device_status() == 60  # FLAT_ERR_DEVICE_WAIT_TIMEOUT, cleared by the read
    finally:
        x.close()
    # the context still decodes
    part = torch.empty(Hq * (D + 1), dtype=torch.float32, device="cuda")
    c.decode_paged_batched_partial(fa.BF16, *args, part)
    c.synchronize()
    assert c.device_status() == 0 and bool(torch.isfinite(part).all())
