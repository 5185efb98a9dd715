"""The allocation-free split-KV paged decode (flat_decode_paged_batched_static_scratch).

Some callers cannot allocate device memory at the moment they decode: latency-critical serving
loops (an allocation would synchronise the device), plug-ins under a
framework allocator that forbids side allocations, processes with a memory budget fixed at start-up.
For them the library keeps the split-KV partials in a fixed 8 MiB device array instead of the
growable context workspace.  This test calls that entry point through the C ABI twice in a row and
checks both results against the regular entry point within the decode tolerances, checks that the
context workspace never grew, and that shapes beyond the fixed array are refused.

Collected last on purpose, so a run that stops at the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

from tests.gpu_util import fa
from tests.test_gpu_decode_cache import make_paged_batch, unpack

pytestmark = pytest.mark.gpu


def run_pair(c, dtype, Hq, Hkv, D, ps, seed, splits):
    theta = 5e5
    lens, tables, pool, maxp, Q, K, V = make_paged_batch(5, Hq, Hkv, D, ps, 40, 900, dtype, seed=seed)
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


def test_static_scratch_decode_matches_regular_entry_point_twice_and_never_allocates():
    c = fa.Context(0)  # fresh context: its workspace starts empty and must stay empty
    assert c.workspace_bytes() == 0
    run_pair(c, fa.BF16, 32, 8, 128, 16, seed=21, splits=0)
    run_pair(c, fa.F32, 8, 2, 64, 16, seed=22, splits=3)   # second call reuses the array with other contents
    run_pair(c, fa.BF16, 32, 8, 128, 16, seed=23, splits=4)
    c.synchronize()
    assert c.workspace_bytes() == 0
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
    with pytest.raises(fa.FlatAttentionError) as e:
        call(1)
    assert e.value.kind == "UnsupportedShape"
    with pytest.raises(fa.FlatAttentionError) as e:
        call(2, heads=24)  # group of 3 is outside the streaming kernel
    assert e.value.kind == "UnsupportedShape"
    call(2)
    assert c.workspace_bytes() == 0
