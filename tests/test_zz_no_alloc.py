"""The allocation-free split-KV paged decode (flat_decode_paged_batched_static_scratch).

Some callers cannot allocate device memory at the moment they decode: latency-critical serving
loops (an allocation would synchronise the device), plug-ins under a
framework allocator that forbids side allocations, processes with a memory budget fixed at start-up.
For them the library keeps the split-KV partials in a fixed 8 MiB device array instead of the
growable context workspace.  This test calls that entry point through the C ABI twice in a row and
checks both results against the regular entry point and against the CPU oracle within the decode
tolerances (tensor-core route with pages of 16, streaming route with pages of 8), checks that the
context workspace never grew, that short contexts (one chunk, no scratch needed) run, that shapes
beyond the fixed array are refused, and that a page-table entry outside the pool is masked and
reported instead of being read.

Collected last on purpose, so a run that stops at the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

from tests.gpu_util import fa
from tests.test_gpu_decode_cache import check_batched, make_paged_batch, unpack

pytestmark = pytest.mark.gpu


def run_pair(c, dtype, Hq, Hkv, D, ps, seed, splits, lo=40, hi=900, oracle_seqs=None):
    theta = 5e5
    lens, tables, pool, maxp, Q, K, V = make_paged_batch(5, Hq, Hkv, D, ps, lo, hi, dtype, seed=seed)
    n = len(lens)
    qpos = (lens - 1).astype(np.int32)
    safe = np.where(tables < 0, 0, tables).astype(np.int32)
    es = 2 if dtype == fa.BF16 else 4
    d_tab, d_len, d_pos = torch.from_numpy(safe).cuda(), torch.from_numpy(lens).cuda(), torch.from_numpy(qpos).cuda()
    dQ, dK, dV = Q.cuda(), K.cuda(), V.cuda()
    ref_ctx = fa.Context(0)
    ref = ref_ctx.empty_bytes(n * Hq * D * es + n * Hq * 4)
    ref_ctx.decode_paged_batched(dtype, n, Hq, Hkv, D, ps, pool, maxp, d_tab, d_len, d_pos, safe, lens, qpos,
                                 fa.config(True), theta, dQ, dK, dV, ref, kv_splits=splits)
    out = c.empty_bytes(n * Hq * D * es + n * Hq * 4)
    out.fill_(0x7f)
    c.decode_paged_batched_static_scratch(dtype, n, Hq, Hkv, D, ps, pool, maxp, d_tab, d_len, d_pos, lens, qpos,
                                          fa.config(True), theta, dQ, dK, dV, out, kv_splits=splits)
    o, l = unpack(out, dtype, n * Hq, D)
    ro, rl = unpack(ref, dtype, n * Hq, D)
    otol, ltol = (2e-2, 2e-3) if dtype == fa.BF16 else (2e-4, 2e-4)
    assert np.isfinite(o).all() and np.isfinite(l).all()
    assert np.abs(o - ro).max() <= otol, float(np.abs(o - ro).max())
    assert np.abs(l - rl).max() <= ltol, float(np.abs(l - rl).max())
    if oracle_seqs is not None:
        tol = ((2e-2, 0.0), (2e-3, 0.0)) if dtype == fa.BF16 else ((2e-4, 1e-3), (2e-4, 1e-3))
        check_batched(o, l, lens, tables, Q, K, V, Hq, Hkv, D, ps, theta, tol[0], tol[1], seqs=oracle_seqs)


def test_static_scratch_decode_matches_regular_entry_point_twice_and_never_allocates():
    c = fa.Context(0)  # fresh context: its workspace starts empty and must stay empty
    assert c.workspace_bytes() == 0
    run_pair(c, fa.BF16, 32, 8, 128, 16, seed=21, splits=0, oracle_seqs=[0, 3])
    run_pair(c, fa.F32, 8, 2, 64, 16, seed=22, splits=3)   # second call reuses the array with other contents
    run_pair(c, fa.BF16, 32, 8, 128, 16, seed=23, splits=4)
    run_pair(c, fa.BF16, 16, 4, 64, 8, seed=25, splits=3, oracle_seqs=[1, 4])  # pages of 8: the streaming kernel
    c.synchronize()
    assert c.workspace_bytes() == 0
    assert c.device_status() == 0


def test_static_scratch_decode_of_short_contexts_needs_no_scratch():
    """The first tokens of a sequence: every context fits one 64-token chunk, the plan has a single chunk and the
    kernel writes O and LSE directly.  An explicit kv_splits = 1 and a split that the chunk rounding collapses
    behave the same."""
    c = fa.Context(0)
    for splits in (0, 1, 2):
        run_pair(c, fa.BF16, 32, 8, 128, 16, seed=26, splits=splits, lo=1, hi=64, oracle_seqs=[0, 2])
    run_pair(c, fa.F32, 8, 2, 64, 4, seed=27, splits=0, lo=1, hi=40, oracle_seqs=[1])
    c.synchronize()
    assert c.workspace_bytes() == 0
    assert c.device_status() == 0


def test_out_of_range_page_entry_is_masked_and_reported_not_read():
    """No host copy of the page tables reaches this entry point, so entries are checked on the device: an entry
    outside the pool is skipped (never dereferenced) and the context reports PageOutOfRange."""
    for ps, Hq, Hkv, D in ((16, 32, 8, 128), (8, 16, 4, 64)):
        c = fa.Context(0)
        lens, tables, pool, maxp, Q, K, V = make_paged_batch(3, Hq, Hkv, D, ps, 100, 300, fa.BF16, seed=28)
        qpos = (lens - 1).astype(np.int32)
        safe = np.where(tables < 0, 0, tables).astype(np.int32)
        bad = safe.copy()
        bad[1, 0] = pool + 5       # beyond the pool
        bad[2, 1] = -7             # negative
        d_len, d_pos = torch.from_numpy(lens).cuda(), torch.from_numpy(qpos).cuda()
        out = c.empty_bytes(3 * Hq * D * 2 + 3 * Hq * 4)
        c.decode_paged_batched_static_scratch(fa.BF16, 3, Hq, Hkv, D, ps, pool, maxp, torch.from_numpy(bad).cuda(), d_len,
                                              d_pos, lens, qpos, fa.config(True), 5e5, Q.cuda(), K.cuda(), V.cuda(), out,
                                              kv_splits=2)
        assert c.device_status() == 35  # PageOutOfRange, and the word is cleared by the read
        assert c.device_status() == 0
        o, l = unpack(out, fa.BF16, 3 * Hq, D)
        assert np.isfinite(o).all()
        # the untouched sequence is exact against the clean call
        ref = c.empty_bytes(3 * Hq * D * 2 + 3 * Hq * 4)
        c.decode_paged_batched_static_scratch(fa.BF16, 3, Hq, Hkv, D, ps, pool, maxp, torch.from_numpy(safe).cuda(), d_len,
                                              d_pos, lens, qpos, fa.config(True), 5e5, Q.cuda(), K.cuda(), V.cuda(), ref,
                                              kv_splits=2)
        ro, rl = unpack(ref, fa.BF16, 3 * Hq, D)
        assert np.array_equal(o[:Hq], ro[:Hq]) and np.array_equal(l[:Hq], rl[:Hq])
        assert c.device_status() == 0


def test_static_scratch_decode_refuses_what_does_not_fit():
    c = fa.Context(0)
    Hq, Hkv, D, ps = 32, 8, 128, 16
    lens, tables, pool, maxp, Q, K, V = make_paged_batch(4, Hq, Hkv, D, ps, 40, 200, fa.BF16, seed=24)
    qpos = (lens - 1).astype(np.int32)
    safe = np.where(tables < 0, 0, tables).astype(np.int32)
    d_tab, d_len, d_pos = torch.from_numpy(safe).cuda(), torch.from_numpy(lens).cuda(), torch.from_numpy(qpos).cuda()
    out = c.empty_bytes(4 * Hq * D * 2 + 4 * Hq * 4)

    def call(splits, heads=Hq):
        c.decode_paged_batched_static_scratch(fa.BF16, 4, heads, Hkv, D, ps, pool, maxp, d_tab, d_len, d_pos, lens, qpos,
                                              fa.config(True), 5e5, Q.cuda(), K.cuda(), V.cuda(), out, kv_splits=splits)
    with pytest.raises(fa.FlatAttentionError) as e:
        call(200)  # 200 * 4*32 * 129 * 4 bytes = 13.2 MB > 8 MiB
    assert e.value.kind == "UnsupportedShape" and str(8 << 20) in e.value.detail
    call(1)  # a single chunk needs no scratch: it runs
    with pytest.raises(fa.FlatAttentionError) as e:
        call(2, heads=24)  # group of 3 is outside the streaming kernel
    assert e.value.kind == "UnsupportedShape"
    call(2)
    assert c.workspace_bytes() == 0


def test_static_scratch_decode_survives_hostile_geometry():
    """The entry point shares the regular one's validation: sizes that would wrap 64-bit products or divide by a
    wrapped zero come back as typed errors (tests/m39_host_api_fuzz.rs:54-105: no panics on hostile input)."""
    import ctypes as C
    c = fa.Context(0)
    lib = fa.lib()
    t = torch.zeros(64, dtype=torch.int32, device="cuda")
    big = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    lens = np.array([5], np.int32)
    b = fa.buf(big)

    def call(num_seqs=1, hq=8, hkv=2, d=64, ps=16, pages=4, maxp=4, theta=1e4, cfg=fa.config(True), q=b, splits=0):
        return lib.flat_decode_paged_batched_static_scratch(
            c.h, C.c_int32(fa.BF16), C.c_uint64(num_seqs), C.c_uint64(hq), C.c_uint64(hkv), C.c_uint64(d), C.c_uint64(ps),
            C.c_uint64(pages), C.c_uint64(maxp), C.c_void_p(t.data_ptr()), C.c_void_p(t.data_ptr()), C.c_void_p(t.data_ptr()),
            lens.ctypes.data_as(C.POINTER(C.c_int32)), None, C.byref(cfg), C.c_float(theta), C.c_uint32(splits), q, b, b, b)

    assert fa.STATUS[call(hq=1 << 62, hkv=1 << 62)] == "DispatchLimit"      # wrapped sizes used to divide by zero
    assert fa.STATUS[call(hq=(1 << 62) + 3, hkv=1 << 62)] == "InvalidHeadGrouping"
    assert fa.STATUS[call(d=(1 << 63) + 2)] == "UnsupportedHeadDim"
    assert fa.STATUS[call(d=63)] == "InvalidRotaryHeadDim"
    assert fa.STATUS[call(pages=1 << 40, ps=1 << 40)] == "IndexSpaceExceeded"
    assert fa.STATUS[call(num_seqs=0)] == "ZeroDimension"
    assert fa.STATUS[call(theta=float("nan"))] == "InvalidTheta"
    assert fa.STATUS[call(cfg=fa.config(True, -1.0))] == "InvalidScale"
    assert fa.STATUS[call(q=fa.Buffer(big.data_ptr(), 8))] == "BufferTooSmall"
    assert fa.STATUS[call(q=fa.Buffer(big.data_ptr() + 2, 1 << 15))] == "MisalignedBuffer"
    assert fa.STATUS[call(splits=1 << 31)] == "UnsupportedShape"
    assert call() == 0
    c.synchronize()
    assert c.workspace_bytes() == 0
