"""Chunked prefill (contiguous and against the growing paged cache) and backward against the CPU
oracle: tests/m16_chunked_prefill_wgpu.rs, m18_wgpu_backward.rs, m19_*, m20_*, m21_*, m23/m26 chain."""
import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.gpu_util import assert_close, bf16_round, ctx, dev, fa, ramp

pytestmark = pytest.mark.gpu
TOL = (2.0e-4, 1.0e-3)


@pytest.mark.parametrize("B,Hq,Hkv,N,D,causal,chunk", [(2, 4, 2, 7, 32, True, 3), (2, 4, 1, 5, 32, False, 2),
                                                        (1, 8, 2, 70, 64, True, 32), (1, 4, 4, 9, 16, True, 64)])
def test_chunked_prefill_equals_contiguous(B, Hq, Hkv, N, D, causal, chunk):
    c = ctx()
    theta, off = 1e4, 5
    q, k, v = ramp(B * N * Hq * D, 0.2), ramp(B * N * Hkv * D, 0.8), ramp(B * N * Hkv * D, 1.4)
    shp = fa.shape(B, Hq, Hkv, N, N, D)
    out = c.create_output_buffer(fa.F32, shp)
    c.chunked_prefill(fa.F32, shp, fa.config(causal), fa.rotary(theta, off), chunk, dev(q), dev(k), dev(v), out)
    o, l = c.split_output(out, fa.F32, shp, fa.PROJECTION)
    eo, el = ob.forward_reference_projection_grouped_rope(q, k, v, B, Hq, Hkv, N, D, theta, off, causal)
    assert_close("O", o.cpu().numpy(), eo, *TOL)
    assert_close("LSE", l.cpu().numpy(), el, *TOL)
    # chunking never changes the result: identical bits to the one-chunk call
    out1 = c.create_output_buffer(fa.F32, shp)
    c.chunked_prefill(fa.F32, shp, fa.config(causal), fa.rotary(theta, off), N, dev(q), dev(k), dev(v), out1)
    assert torch.equal(out, out1)
    with pytest.raises(fa.FlatAttentionError) as e:
        c.chunked_prefill(fa.F32, shp, fa.config(causal), fa.rotary(theta, off), 0, dev(q), dev(k), dev(v), out)
    assert e.value.kind == "ZeroQueryChunkSize"


@pytest.mark.parametrize("dtype,Hq,Hkv,D,N,chunk,ps", [(fa.F32, 4, 2, 32, 23, 5, 4), (fa.F32, 8, 1, 64, 40, 16, 16),
                                                        (fa.BF16, 8, 2, 128, 300, 128, 16), (fa.BF16, 4, 4, 64, 90, 32, 16),
                                                        # more (query block, head) items than SMs, ragged last block
                                                        (fa.BF16, 64, 8, 64, 700, 640, 16)])
@pytest.mark.parametrize("shadow", [False, True])
def test_chunked_prefill_into_growing_paged_cache(dtype, Hq, Hkv, D, N, chunk, ps, shadow):
    """Each chunk appends rotated K and V to the paged cache, then attends causally to the whole
    cache.  Oracle: the cache contents as stored (pre-rotated K), Q rotation materialised.  With the binary16
    K shadow (bf16 caches) the attention kernel reads K tiles without converting them; results agree bit for bit
    with the converting kernel's tolerance class (the shadow holds the same bf16 values)."""
    c = ctx()
    theta, off = 5e5, 3
    td = fa.torch_dtype(dtype)
    pages = (N + ps - 1) // ps + 2
    cache = fa.CudaPagedKvCache(c, dtype, ps, pages, Hkv, D)
    if shadow:
        if dtype != fa.BF16:
            with pytest.raises(fa.FlatAttentionError) as e:
                cache.enable_prefill_shadow()
            assert e.value.kind == "UnsupportedDtype"
            return
        # switched on after the first chunk is in: the existing rows are converted, later appends write both copies
        first = min(chunk, N)
        warm = c.empty_bytes(first * Hq * D * 2 + Hq * first * 4)
        q0 = bf16_round(ramp(N * Hq * D, 0.2).reshape(N, Hq * D))
        k0 = bf16_round(ramp(N * Hkv * D, 0.8).reshape(N, Hkv * D))
        v0 = bf16_round(ramp(N * Hkv * D, 1.4).reshape(N, Hkv * D))
        c.chunked_prefill_paged(cache, Hq, first, fa.config(True), theta, off, dev(q0[:first], td), dev(k0[:first], td),
                                dev(v0[:first], td), warm)
        cache.enable_prefill_shadow()
        cache.enable_prefill_shadow()  # idempotent
        cache.reset()
    q, k, v = ramp(N * Hq * D, 0.2).reshape(N, Hq * D), ramp(N * Hkv * D, 0.8).reshape(N, Hkv * D), \
        ramp(N * Hkv * D, 1.4).reshape(N, Hkv * D)
    if dtype == fa.BF16:
        q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
    es = 2 if dtype == fa.BF16 else 4
    outs = []
    for start in range(0, N, chunk):
        n = min(chunk, N - start)
        out = c.empty_bytes(n * Hq * D * es + Hq * n * 4)
        c.chunked_prefill_paged(cache, Hq, n, fa.config(True), theta, off, dev(q[start:start + n], td),
                                dev(k[start:start + n], td), dev(v[start:start + n], td), out)
        outs.append((start, n, out))
    c.synchronize()
    assert len(cache) == N
    K, V = cache.download()
    tab = cache.table()
    rows = np.array([tab.address(t)[0] * ps + tab.address(t)[1] for t in range(N)])
    k_cache, v_cache = K.float().numpy()[rows], V.float().numpy()[rows]
    # cache holds rotated K (rounded to the storage type) and raw V
    k_rot = ob.rotate_rows(k, D, np.repeat(np.arange(N, dtype=np.uint64) + off, Hkv), theta).reshape(N, Hkv * D)
    assert np.array_equal(v_cache, v)
    assert_close("cached K", k_cache, k_rot, 1e-5 if dtype == fa.F32 else 0.0, 0.0 if dtype == fa.F32 else 2.0 ** -7)
    kh, vh = k_cache.reshape(N, Hkv, D).transpose(1, 0, 2), v_cache.reshape(N, Hkv, D).transpose(1, 0, 2)
    for start, n, out in outs:
        raw = out.cpu()
        o = raw[:n * Hq * D * es].view(td).float().numpy().reshape(n, Hq, D)
        l = raw[n * Hq * D * es:].view(torch.float32).numpy().reshape(Hq, n)
        rq = ob.rotate_rows(q[start:start + n], D, np.repeat(np.arange(n, dtype=np.uint64) + off + start, Hq), theta)
        rq = rq.reshape(n, Hq, D).transpose(1, 0, 2)  # head-major
        kv_len = start + n
        eo, el = ob.forward_reference_grouped_asymmetric(rq, kh[:, :kv_len], vh[:, :kv_len],
                                                         ob._shape(1, Hq, Hkv, n, kv_len, D, start), True)
        eo = eo.reshape(Hq, n, D).transpose(1, 0, 2)
        if dtype == fa.F32:
            assert_close("O", o, eo, *TOL)
            assert_close("LSE", l, el, *TOL)
        else:
            assert_close("O", o, eo, 2e-2, 0.0)
            assert_close("LSE", l, el, 2e-3, 0.0)


def test_config4_chunked_prefill_full_size_sampled_rows():
    """One sequence of 32768 tokens fed in 2048-token chunks into the growing paged cache (page 16), Hq=64,
    Hkv=8, D=128, causal, bf16, theta 5e5: 16 launches with up to 256 KV tiles and 2048 pages per work item.
    Per chunk the oracle (no-RoPE rectangular rows on the cache contents as stored, Q rotation materialised)
    checks the first and last row, the rows either side of a tile border (127/128) and of a page border (15/16)
    and random rows, each on sampled query heads."""
    c = ctx()
    Hq, Hkv, D, N, chunk, ps, theta = 64, 8, 128, 32768, 2048, 16, 5e5
    q = torch.randn(N, Hq * D, generator=torch.Generator().manual_seed(31)).bfloat16()
    k = torch.randn(N, Hkv * D, generator=torch.Generator().manual_seed(32)).bfloat16()
    v = torch.randn(N, Hkv * D, generator=torch.Generator().manual_seed(33)).bfloat16()
    cache = fa.CudaPagedKvCache(c, fa.BF16, ps, N // ps + 8, Hkv, D)
    cache.enable_prefill_shadow()  # as the benchmark runs it: K tiles reach the tensor core without conversion
    out = c.empty_bytes(chunk * Hq * D * 2 + Hq * chunk * 4)
    rng = np.random.default_rng(4)
    picked = []  # (chunk start, [(head, row)], O rows, LSE values)
    for start in range(0, N, chunk):
        c.chunked_prefill_paged(cache, Hq, chunk, fa.config(True), theta, 0, q[start:start + chunk].cuda(),
                                k[start:start + chunk].cuda(), v[start:start + chunk].cuda(), out)
        rows = [0, 15, 16, 127, 128, chunk - 1] + [int(r) for r in rng.integers(0, chunk, 3)]
        # (no pair twice: the oracle's Q rotation below is applied once per listed pair)
        pairs = list(dict.fromkeys([(int(rng.integers(Hq)), r) for r in rows] + [(Hq - 1, chunk - 1), (0, 0)]))
        o = out[:chunk * Hq * D * 2].view(torch.bfloat16).view(chunk, Hq, D)
        l = out[chunk * Hq * D * 2:].view(torch.float32).view(Hq, chunk)
        picked.append((start, pairs, torch.stack([o[r, h] for (h, r) in pairs]).float().cpu().numpy(),
                       np.array([float(l[h, r]) for (h, r) in pairs], np.float32)))
    c.synchronize()
    assert c.device_status() == 0
    assert len(cache) == N
    K, V = cache.download()
    tab = cache.table()
    entries = np.array(tab.export(), np.int64)
    rows = (entries[:, None] * ps + np.arange(ps)[None, :]).reshape(-1)[:N]
    k_cache, v_cache = K.float().numpy()[rows], V.float().numpy()[rows]
    assert np.array_equal(v_cache, v.float().numpy())
    some = np.array([0, 1, 15, 16, 2047, 2048, N - 1] + [int(r) for r in rng.integers(0, N, 32)])
    k_rot = ob.rotate_rows(k.float().numpy()[some], D, np.repeat(some.astype(np.uint64), Hkv), theta).reshape(len(some), Hkv * D)
    assert_close("cached K", k_cache[some], k_rot, 0.0, 2.0 ** -7)
    qf = q.float().numpy()
    worst_o = worst_l = 0.0
    for start, pairs, ao, al in picked:
        kv_len = start + chunk
        rq = qf[start:start + chunk].reshape(chunk, Hq, D).copy()
        for (h, r) in pairs:
            rq[r, h] = ob.rotate_rows(rq[r, h], D, [start + r], theta)
        eo, el = ob.forward_rows(rq, k_cache[:kv_len], v_cache[:kv_len], ob._shape(1, Hq, Hkv, chunk, kv_len, D, start),
                                 ob.PROJECTION, [(0, h, r) for (h, r) in pairs], True, threads=8)
        worst_o = max(worst_o, float(np.abs(ao - eo).max()))
        worst_l = max(worst_l, float(np.abs(al - el).max()))
    assert worst_o <= 2e-2 and worst_l <= 2e-3, (worst_o, worst_l)


# ---- backward -----------------------------------------------------------------------------------
def run_backward(dtype, B, Hq, Hkv, N, D, causal, scale, q, k, v, do, fo, fl, mha=False):
    c = ctx()
    shp = fa.shape(B, Hq, Hkv, N, N, D)
    L = fa.backward_layout(dtype, shp)
    td = fa.torch_dtype(dtype)
    packed = torch.zeros(L.input_bytes, dtype=torch.uint8)
    for off, arr in ((L.q_offset, q), (L.k_offset, k), (L.v_offset, v), (L.d_out_offset, do), (L.out_offset, fo)):
        t = torch.as_tensor(np.ascontiguousarray(arr, dtype=np.float32)).reshape(-1).to(td)
        packed[off:off + t.numel() * t.element_size()] = t.view(torch.uint8)
    t = torch.as_tensor(np.ascontiguousarray(fl, dtype=np.float32)).reshape(-1)
    packed[L.lse_offset:L.lse_offset + 4 * t.numel()] = t.view(torch.uint8)
    grads = c.empty_bytes(L.output_bytes)
    grads.fill_(0x7f)
    (c.backward_mha if mha else c.backward_grouped)(dtype, shp, fa.config(causal, scale), packed.cuda(), grads)
    raw = grads.cpu()
    dq = raw[L.dq_offset:L.dq_offset + L.q_elements * 4].view(torch.float32).numpy()   # gradients are f32 in both modes
    dk = raw[L.dk_offset:L.dk_offset + L.kv_elements * 4].view(torch.float32).numpy()
    dv = raw[L.dv_offset:L.dv_offset + L.kv_elements * 4].view(torch.float32).numpy()
    return dq, dk, dv


def bfix(n, phase):
    return ob.fixture(n, 0.31, phase, 0.65, 0.43, 0.23)


BWD = [(2, 2, 2, 3, 4, None), (2, 4, 2, 5, 8, 0.41), (2, 4, 1, 5, 8, 0.41), (2, 8, 2, 5, 16, None), (1, 4, 1, 5, 8, None),
       (1, 1, 1, 1, 2, None), (1, 4, 4, 3, 8, None), (1, 8, 1, 9, 32, None), (2, 12, 3, 7, 6, None), (1, 4, 4, 7, 8, None),
       (1, 8, 2, 9, 16, None), (2, 4, 1, 5, 12, None), (1, 8, 2, 17, 64, None), (1, 8, 1, 33, 32, None), (1, 4, 2, 70, 128, None)]


@pytest.mark.parametrize("B,Hq,Hkv,N,D,scale", BWD)
@pytest.mark.parametrize("causal", [False, True])
def test_backward_f32(B, Hq, Hkv, N, D, scale, causal):
    q, k, v, do = bfix(B * Hq * N * D, 0.1), bfix(B * Hkv * N * D, 0.8), bfix(B * Hkv * N * D, 1.4), bfix(B * Hq * N * D, 2.1)
    fo, fl = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, causal, scale)
    edq, edk, edv = ob.backward_reference_grouped(q, k, v, do, fo, fl, B, Hq, Hkv, N, D, causal, scale)
    dq, dk, dv = run_backward(fa.F32, B, Hq, Hkv, N, D, causal, scale, q, k, v, do, fo, fl, mha=(Hq == Hkv))
    for name, a, e in (("dQ", dq, edq), ("dK", dk, edk), ("dV", dv, edv)):
        assert_close(name, a, e, 4.0e-4, 2.0e-3)  # tests/m19_grouped_backward_wgpu.rs:12-13
    again = run_backward(fa.F32, B, Hq, Hkv, N, D, causal, scale, q, k, v, do, fo, fl)
    assert all(np.array_equal(x.view(np.uint32), y.view(np.uint32)) for x, y in zip((dq, dk, dv), again))


def test_backward_validation():
    c = ctx()
    shp = fa.shape(1, 4, 2, 5, 5, 8)
    L = fa.backward_layout(fa.F32, shp)
    inp, out = c.empty_bytes(L.input_bytes), c.empty_bytes(L.output_bytes)
    with pytest.raises(fa.FlatAttentionError) as e:
        c.backward_grouped(fa.F32, shp, fa.config(), inp[:-4], out)
    assert e.value.kind == "BufferTooSmall" and str(L.input_bytes) in e.value.detail
    with pytest.raises(fa.FlatAttentionError) as e:
        c.backward_grouped(fa.F32, shp, fa.config(), inp, out[:-4])
    assert e.value.kind == "BufferTooSmall"
    with pytest.raises(fa.FlatAttentionError) as e:
        c.backward_mha(fa.F32, shp, fa.config(), inp, out)
    assert e.value.kind == "InvalidHeadGrouping"
    big_in, big_out = c.empty_bytes(L.input_bytes + 128), c.empty_bytes(L.output_bytes + 128)
    big_in.zero_()
    c.backward_grouped(fa.F32, shp, fa.config(), big_in, big_out)  # over-provisioned buffers are accepted


@pytest.mark.parametrize("B,Hq,Hkv,N,D,causal,scale", [(1, 4, 2, 7, 16, True, None), (2, 4, 1, 5, 8, False, 0.31)])
def test_training_chain_forward_then_backward_on_device(B, Hq, Hkv, N, D, causal, scale):
    # tests/m26_wgpu_public_training_chain.rs:148-349: forward -> pack -> backward, one stream, no host sync between
    c = ctx()
    q, k, v, do = bfix(B * Hq * N * D, 0.1), bfix(B * Hkv * N * D, 0.8), bfix(B * Hkv * N * D, 1.4), bfix(B * Hq * N * D, 2.1)
    shp = fa.shape(B, Hq, Hkv, N, N, D)
    FL, L = fa.forward_layout(fa.F32, shp), fa.backward_layout(fa.F32, shp)
    dq_, dk_, dv_, ddo = dev(q), dev(k), dev(v), dev(do)
    fwd = c.create_output_buffer(fa.F32, shp)
    c.forward_grouped(fa.F32, shp, fa.config(causal, scale), dq_, dk_, dv_, fwd)
    packed = c.empty_bytes(L.input_bytes)
    for off, t in ((L.q_offset, dq_), (L.k_offset, dk_), (L.v_offset, dv_), (L.d_out_offset, ddo)):
        packed[off:off + t.numel() * 4] = t.view(torch.uint8).reshape(-1)
    packed[L.out_offset:L.out_offset + FL.q_bytes] = fwd[:FL.q_bytes]
    packed[L.lse_offset:L.lse_offset + 4 * FL.lse_elements] = fwd[FL.lse_byte_offset:FL.lse_byte_offset + 4 * FL.lse_elements]
    grads = c.empty_bytes(L.output_bytes)
    c.backward_grouped(fa.F32, shp, fa.config(causal, scale), packed, grads)
    g = grads.cpu().view(torch.float32).numpy()
    fo, fl = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, causal, scale)
    e = np.concatenate(ob.backward_reference_grouped(q, k, v, do, fo, fl, B, Hq, Hkv, N, D, causal, scale))
    assert_close("dQ|dK|dV", g, e, 6.0e-4, 2.5e-3)
