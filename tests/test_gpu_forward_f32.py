"""f32 parity of the CUDA forward path against the CPU oracle, on the reference's GPU-test shape
inventory (tests/wgpu_device.rs, wgpu_matrix.rs, wgpu_grouped.rs, wgpu_rotary_grouped.rs,
wgpu_external*.rs) and on benchmark configuration 1.  The required tolerance for the f32 mode: 1e-4."""
import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.gpu_util import assert_close, ctx, fa, ramp, run_forward

pytestmark = pytest.mark.gpu

O_TOL = (2.0e-5, 2.0e-4)     # tests/wgpu_device.rs:8-11
LSE_TOL = (3.0e-5, 3.0e-4)
ROPE_TOL = (1.5e-4, 1.0e-3)  # tests/wgpu_rotary_grouped.rs


def test_config1_mha_causal_f32_max_abs_1e4():
    B, H, N, D = 1, 2, 128, 64
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(B * H * N * D, generator=torch.Generator().manual_seed(s)).numpy() for s in (1, 2, 3))
    o, l = run_forward("mha", fa.F32, fa.shape(B, H, H, N, N, D), fa.config(True), q, k, v)
    eo, el = ob.forward_reference(q, k, v, B, H, N, D, True)
    assert np.abs(o - eo).max() <= 1e-4
    assert np.abs(l - el).max() <= 1e-4


MATRIX = [(1, 1, 17, d) for d in (1, 8, 16, 32, 64, 80, 96, 128)] + [(1, 2, 9, d) for d in (1, 8, 80, 128)] + \
         [(1, 1, n, 16) for n in (1, 7, 8, 9, 15, 16, 17, 31, 32, 63, 64, 65, 127, 128, 129)] + \
         [(1, 1, n, 32) for n in (1, 33, 65, 129)] + [(2, 3, 31, 16), (3, 4, 17, 32)]


@pytest.mark.parametrize("B,H,N,D", MATRIX)
@pytest.mark.parametrize("causal", [False, True])
def test_mha_shape_matrix(B, H, N, D, causal):
    n = B * H * N * D
    q, k, v = ramp(n, 0.1, 0.173, 1.0, 0.3, 0.2), ramp(n, 0.6, 0.119, 1.0, 0.5, 0.1), ramp(n, 1.1, 0.071, 1.7, 0.2, 0.3)
    o, l = run_forward("mha", fa.F32, fa.shape(B, H, H, N, N, D), fa.config(causal), q, k, v)
    eo, el = ob.forward_reference(q, k, v, B, H, N, D, causal)
    assert_close("O", o, eo, *O_TOL)
    assert_close("LSE", l, el, *LSE_TOL)


def test_adversarial_magnitudes():
    B, H, N, D = 1, 2, 17, 32
    n = B * H * N * D
    i = np.arange(n)
    q = np.where(i % 2 == 0, 7.0, -7.0).astype(np.float32)
    k = np.where((i // 3) % 2 == 0, -7.0, 7.0).astype(np.float32)
    v = ramp(n, 0.2)
    for causal in (False, True):
        o, l = run_forward("mha", fa.F32, fa.shape(B, H, H, N, N, D), fa.config(causal, 0.125), q, k, v)
        eo, el = ob.forward_reference(q, k, v, B, H, N, D, causal, 0.125)
        assert_close("O", o, eo, 8.0e-5, 8.0e-4)
        assert_close("LSE", l, el, 2.0e-4, 8.0e-4)


def test_causal_future_token_isolation():
    # tests/wgpu_device.rs:191-243, tests/wgpu_matrix.rs:161-195
    B, H, N, D = 1, 1, 9, 8
    q, k, v = ramp(N * D, 0.1), ramp(N * D, 0.5), ramp(N * D, 0.9)
    base_o, _ = run_forward("mha", fa.F32, fa.shape(B, H, H, N, N, D), fa.config(True), q, k, v)
    k2, v2 = k.copy().reshape(N, D), v.copy().reshape(N, D)
    k2[1:] = np.where(np.arange((N - 1) * D).reshape(N - 1, D) % 2 == 0, 1000.0, -1000.0)
    v2[1:] = 500.0 + np.arange((N - 1) * D).reshape(N - 1, D)
    o, _ = run_forward("mha", fa.F32, fa.shape(B, H, H, N, N, D), fa.config(True), q, k2, v2)
    assert np.array_equal(o[:D], base_o[:D])
    assert np.abs(o[:D] - v[:D]).max() <= 1e-6
    z = np.zeros(N * D, np.float32)
    o, l = run_forward("mha", fa.F32, fa.shape(B, H, H, N, N, D), fa.config(True), z, z, v)
    assert np.array_equal(o[:D].view(np.uint32), v[:D].view(np.uint32))
    assert l[0] == 0.0


GQA = [(1, 4, 4, 17, 32), (1, 8, 2, 17, 64), (2, 8, 1, 9, 80), (1, 16, 4, 5, 128), (2, 12, 3, 17, 64)]


@pytest.mark.parametrize("B,Hq,Hkv,N,D", GQA)
@pytest.mark.parametrize("causal", [False, True])
def test_grouped(B, Hq, Hkv, N, D, causal):
    q, k, v = ramp(B * Hq * N * D, 0.1, 0.037, 1.75, 0.41, 0.25), ramp(B * Hkv * N * D, 0.7, 0.037, 1.75, 0.41, 0.25), \
        ramp(B * Hkv * N * D, 1.3, 0.037, 1.75, 0.41, 0.25)
    o, l = run_forward("grouped", fa.F32, fa.shape(B, Hq, Hkv, N, N, D), fa.config(causal), q, k, v)
    eo, el = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, causal)
    assert_close("O", o, eo, 6.0e-5, 6.0e-4)
    assert_close("LSE", l, el, 6.0e-5, 6.0e-4)


def test_invalid_grouping_rejected():
    z = np.zeros(6 * 2 * 4, np.float32)
    with pytest.raises(fa.FlatAttentionError) as e:
        run_forward("grouped", fa.F32, fa.shape(1, 6, 4, 2, 2, 4), fa.config(), z, z, z)
    assert e.value.kind == "InvalidHeadGrouping"


@pytest.mark.parametrize("B,Hq,Hkv,N,D", [g for g in GQA if g[4] % 2 == 0])
@pytest.mark.parametrize("theta,off", [(1e4, 0), (5e5, 11), (1e4, 23)])
def test_grouped_rope_head_major(B, Hq, Hkv, N, D, theta, off):
    q, k, v = ramp(B * Hq * N * D, 0.2, 0.029, 1.5, 0.37, 0.375), ramp(B * Hkv * N * D, 0.8, 0.029, 1.5, 0.37, 0.375), \
        ramp(B * Hkv * N * D, 1.4, 0.029, 1.5, 0.37, 0.375)
    for causal in (False, True):
        o, l = run_forward("grouped_rope", fa.F32, fa.shape(B, Hq, Hkv, N, N, D), fa.config(causal), q, k, v,
                           rot=fa.rotary(theta, off))
        eo, el = ob.forward_reference_grouped_rope(q, k, v, B, Hq, Hkv, N, D, theta, off, causal)
        assert_close("O", o, eo, *ROPE_TOL)
        assert_close("LSE", l, el, *ROPE_TOL)


@pytest.mark.parametrize("B,Hq,Hkv,N,D,theta,off", [(1, 8, 2, 17, 64, 1e4, 13), (2, 8, 1, 9, 80, 5e5, 21)])
def test_projection_rope(B, Hq, Hkv, N, D, theta, off):
    q, k, v = ramp(B * N * Hq * D, 0.3, 0.023, 1.875, 0.61, 0.3125), ramp(B * N * Hkv * D, 0.9, 0.023, 1.875, 0.61, 0.3125), \
        ramp(B * N * Hkv * D, 1.5, 0.023, 1.875, 0.61, 0.3125)
    for causal in (False, True):
        o, l = run_forward("projection_rope", fa.F32, fa.shape(B, Hq, Hkv, N, N, D), fa.config(causal), q, k, v,
                           rot=fa.rotary(theta, off))
        eo, el = ob.forward_reference_projection_grouped_rope(q, k, v, B, Hq, Hkv, N, D, theta, off, causal)
        assert_close("O", o, eo, *ROPE_TOL)
        assert_close("LSE", l, el, *ROPE_TOL)


RECT = [  # (B,Hq,Hkv,Nq,Nkv,D, causal, causal_off, theta, q_rope, kv_rope)  tests/wgpu_external_asymmetric.rs:200-321
    (1, 8, 2, 1, 17, 64, True, 16, 1e4, 29, 13),
    (2, 8, 1, 5, 9, 80, False, 0, 5e5, 7, 3),
    (1, 8, 2, 17, 17, 64, True, 0, 1e4, 5, 5),
    (1, 8, 2, 17, 17, 128, True, 0, 1e4, 5, 5),
    (1, 4, 2, 3, 7, 80, True, 4, 1e4, 11, 7),
    (1, 4, 2, 40, 70, 32, True, 30, 5e5, 30, 0),
]


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nkv,D,causal,coff,theta,qr,kr", RECT)
def test_rectangular_projection(B, Hq, Hkv, Nq, Nkv, D, causal, coff, theta, qr, kr):
    q, k, v = ramp(B * Nq * Hq * D, 0.3, 0.071, 0.625, 0.3, 0.2), ramp(B * Nkv * Hkv * D, 0.9, 0.071, 0.625, 0.3, 0.2), \
        ramp(B * Nkv * Hkv * D, 1.5, 0.071, 0.625, 0.3, 0.2)
    shp = fa.shape(B, Hq, Hkv, Nq, Nkv, D, coff)
    o, l = run_forward("projection_rope_asymmetric", fa.F32, shp, fa.config(causal), q, k, v, rot=fa.rotary(theta, qr, kr))
    eo, el = ob.forward_reference_projection_grouped_rope_asymmetric(q, k, v, ob._shape(B, Hq, Hkv, Nq, Nkv, D, coff),
                                                                     theta, qr, kr, causal)
    assert_close("O", o, eo, *ROPE_TOL)
    assert_close("LSE", l, el, *ROPE_TOL)


@pytest.mark.parametrize("Hq,Hkv,Nkv,D,theta", [(8, 2, 17, 64, 1e4), (8, 1, 65, 80, 5e5)])
def test_pre_rotated_k_decode(Hq, Hkv, Nkv, D, theta):
    # tests/wgpu_prerotated_k_decode.rs:227-234: K rotated once on the host, rotate_k = 0
    q, k, v = ramp(Hq * D, 0.3), ramp(Nkv * Hkv * D, 0.9), ramp(Nkv * Hkv * D, 1.5)
    pos = np.repeat(np.arange(Nkv, dtype=np.uint64) + 3, Hkv)
    k_rot = ob.rotate_rows(k, D, pos, theta)
    shp = fa.shape(1, Hq, Hkv, 1, Nkv, D, Nkv - 1)
    o, l = run_forward("projection_rope_asymmetric", fa.F32, shp, fa.config(True), q, k_rot, v,
                       rot=fa.rotary(theta, 3 + Nkv - 1, 3, rotate_k=False))
    eo, el = ob.forward_reference_projection_grouped_rope_asymmetric(q, k, v, ob._shape(1, Hq, Hkv, 1, Nkv, D, Nkv - 1),
                                                                     theta, 3 + Nkv - 1, 3, True)
    assert_close("O", o, eo, *ROPE_TOL)
    assert_close("LSE", l, el, *ROPE_TOL)


VARLEN = [  # tests/wgpu_external_variable.rs:160-387
    (2, 8, 2, 5, 9, 64, True, None, 1e4, 11, [(3, 6, 3, 17), (5, 9, 4, 29)]),
    (3, 8, 1, 6, 10, 80, False, 0.125, 5e5, 0, [(6, 10, 0, 0), (1, 1, 0, 5), (4, 7, 2, 9)]),
]


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nkv,D,causal,scale,theta,kvoff,meta", VARLEN)
def test_variable_length_projection(B, Hq, Hkv, Nq, Nkv, D, causal, scale, theta, kvoff, meta):
    q = ramp(B * Nq * Hq * D, 0.15).reshape(B, Nq, Hq * D)
    k = ramp(B * Nkv * Hkv * D, 0.75).reshape(B, Nkv, Hkv * D)
    v = ramp(B * Nkv * Hkv * D, 1.35).reshape(B, Nkv, Hkv * D)
    for b, (aq, akv, _, _) in enumerate(meta):  # poison the padding
        q[b, aq:] = 1.0e20
        k[b, akv:] = -1.0e20
        v[b, akv:] = 1.0e20
    seqs = [fa.VarlenSequence(*m) for m in meta]
    o, l = run_forward("projection_rope_varlen", fa.F32, fa.shape(B, Hq, Hkv, Nq, Nkv, D), fa.config(causal, scale),
                       q, k, v, rot=fa.rotary(theta, 0, kvoff), sequences=seqs)
    o, l = o.reshape(B, Nq, Hq, D), l.reshape(B, Hq, Nq)
    for b, (aq, akv, coff, qr) in enumerate(meta):
        eo, el = ob.forward_reference_projection_grouped_rope_asymmetric(
            q[b, :aq], k[b, :akv], v[b, :akv], ob._shape(1, Hq, Hkv, aq, akv, D, coff), theta, qr, kvoff, causal, scale)
        assert_close("O", o[b, :aq], eo, *ROPE_TOL)
        assert_close("LSE", l[b, :, :aq], el, *ROPE_TOL)
        assert np.all(o[b, aq:] == 0.0)
        assert np.all(l[b, :, aq:].view(np.uint32) == 0xFF800000)


def test_varlen_metadata_and_buffers_are_validated():
    B, Hq, Hkv, Nq, Nkv, D = 2, 4, 2, 4, 6, 8
    shp = fa.shape(B, Hq, Hkv, Nq, Nkv, D)
    q, k = np.zeros(B * Nq * Hq * D, np.float32), np.zeros(B * Nkv * Hkv * D, np.float32)
    rot = fa.rotary(1e4, 0, 0)
    for meta, kind in (([(1, 1, 0, 0)], "LengthMismatch"), ([(5, 1, 0, 0), (1, 1, 0, 0)], "LengthMismatch"),
                       ([(1, 7, 0, 0), (1, 1, 0, 0)], "LengthMismatch"), ([(0, 1, 0, 0), (1, 1, 0, 0)], "ZeroDimension"),
                       ([(2, 1, 2**32 - 1, 0), (1, 1, 0, 0)], "PositionOverflow")):
        with pytest.raises(fa.FlatAttentionError) as e:
            run_forward("projection_rope_varlen", fa.F32, shp, fa.config(), q, k, k, rot=rot,
                        sequences=[fa.VarlenSequence(*m) for m in meta])
        assert e.value.kind == kind
    # undersized buffers are rejected with exact byte counts; oversized ones are accepted
    c = ctx()
    dq, dk = torch.zeros(q.size, device="cuda"), torch.zeros(k.size, device="cuda")
    out = c.create_output_buffer(fa.F32, shp)
    with pytest.raises(fa.FlatAttentionError) as e:
        c.forward_projection_rope_asymmetric(fa.F32, shp, fa.config(), rot, dq, dk[:-1], dk, out)
    assert e.value.kind == "BufferTooSmall" and "K" in e.value.detail and str(k.size * 4) in e.value.detail
    with pytest.raises(fa.FlatAttentionError) as e:
        c.forward_projection_rope_asymmetric(fa.F32, shp, fa.config(), rot, dq, dk, dk, out[:-4])
    assert e.value.kind == "BufferTooSmall"
    big = torch.zeros(out.numel() + 64, dtype=torch.uint8, device="cuda")
    c.forward_projection_rope_asymmetric(fa.F32, shp, fa.config(), rot, dq, dk, dk, big)
    for scale in (0.0, -1.0, float("inf"), float("nan")):
        with pytest.raises(fa.FlatAttentionError) as e:
            c.forward_projection_rope_asymmetric(fa.F32, shp, fa.config(False, scale), rot, dq, dk, dk, out)
        assert e.value.kind == "InvalidScale"
    with pytest.raises(fa.FlatAttentionError) as e:
        c.forward_projection_rope_asymmetric(fa.F32, shp, fa.config(), fa.rotary(-1.0), dq, dk, dk, out)
    assert e.value.kind == "InvalidRotaryTheta"


def test_repeat_no_drift():
    # tests/m38_property_stress.rs:161-201: 32 resident dispatches, bitwise repeatable
    B, Hq, Hkv, N, D = 1, 8, 2, 17, 32
    q, k, v = ramp(B * Hq * N * D, 0.1), ramp(B * Hkv * N * D, 0.7), ramp(B * Hkv * N * D, 1.3)
    eo, el = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, True)
    first = None
    for _ in range(32):
        o, l = run_forward("grouped", fa.F32, fa.shape(B, Hq, Hkv, N, N, D), fa.config(True), q, k, v)
        if first is None:
            first = (o.copy(), l.copy())
            assert_close("O", o, eo, 2.0e-4, 1.0e-3)
            assert_close("LSE", l, el, 2.0e-4, 1.0e-3)
        assert np.array_equal(o.view(np.uint32), first[0].view(np.uint32))
        assert np.array_equal(l.view(np.uint32), first[1].view(np.uint32))


def test_owning_executor_forward_host_to_host():
    ex = fa.CudaFlatAttention(0, fa.F32)
    B, H, N, D = 1, 2, 33, 16
    q, k, v = ramp(B * H * N * D, 0.1), ramp(B * H * N * D, 0.7), ramp(B * H * N * D, 1.3)
    r = ex.forward(q, k, v, fa.shape(B, H, H, N, N, D), fa.config(True))
    eo, el = ob.forward_reference(q, k, v, B, H, N, D, True)
    assert_close("O", r.output.numpy(), eo, *O_TOL)
    assert_close("LSE", r.lse.numpy(), el, *LSE_TOL)


def test_host_slice_forward_validates_like_validate_input():
    # src/lib.rs:428-447 through the host-slice entry point: exact lengths, first non-finite index by tensor name
    c = ctx()
    B, H, N, D = 1, 2, 9, 8
    shp = fa.shape(B, H, H, N, N, D)
    q, k, v = (torch.as_tensor(ramp(B * H * N * D, ph)) for ph in (0.1, 0.7, 1.3))
    out = torch.empty(fa.forward_layout(fa.F32, shp).combined_bytes, dtype=torch.uint8)
    c.forward_host(fa.F32, fa.HEAD_MAJOR, shp, fa.config(True), None, q, k, v, out, check_finite=True)
    eo, el = ob.forward_reference(q.numpy(), k.numpy(), v.numpy(), B, H, N, D, True)
    assert_close("O", out[:4 * q.numel()].view(torch.float32).numpy(), eo, *O_TOL)
    assert_close("LSE", out[4 * q.numel():].view(torch.float32).numpy(), el, *LSE_TOL)
    with pytest.raises(fa.FlatAttentionError) as e:
        c.forward_host(fa.F32, fa.HEAD_MAJOR, shp, fa.config(True), None, q, k[:-1], v, out, check_finite=True)
    assert e.value.kind == "LengthMismatch" and "K" in e.value.detail and str(k.numel() - 1) in e.value.detail
    bad = v.clone()
    bad[5] = float("inf")
    with pytest.raises(fa.FlatAttentionError) as e:
        c.forward_host(fa.F32, fa.HEAD_MAJOR, shp, fa.config(True), None, q, k, bad, out, check_finite=True)
    assert e.value.kind == "NonFiniteInput" and "V" in e.value.detail and "index 5" in e.value.detail
    badb = q.bfloat16()
    badb[3] = float("nan")
    with pytest.raises(fa.FlatAttentionError) as e:
        c.forward_host(fa.BF16, fa.HEAD_MAJOR, shp, fa.config(True), None, badb, k.bfloat16(), v.bfloat16(), out, check_finite=True)
    assert e.value.kind == "NonFiniteInput" and "Q" in e.value.detail and "index 3" in e.value.detail
    with pytest.raises(fa.FlatAttentionError) as e:
        c.forward_host(fa.F32, fa.HEAD_MAJOR, shp, fa.config(True), None, q, k, v, out[:-1], check_finite=True)
    assert e.value.kind == "BufferTooSmall"
