"""IEEE binary16 storage on the forward entry points against the CPU oracle evaluated on the
de-quantised inputs, as tests/wgpu_f16.rs does: O is compared with the oracle's output rounded to
binary16 (ATOL 2e-3, RTOL 5e-3), LSE with the oracle's f32 LSE (ATOL 8e-4, RTOL 2e-3)."""
import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.gpu_util import assert_close, ctx, fa

pytestmark = pytest.mark.gpu

O_ATOL, O_RTOL, LSE_ATOL, LSE_RTOL = 2.0e-3, 5.0e-3, 8.0e-4, 2.0e-3  # tests/wgpu_f16.rs:8-11


def fixture(n):
    # tests/wgpu_f16.rs:13-25
    i = np.arange(n, dtype=np.float32)
    q = np.sin(i * np.float32(0.031) - np.float32(0.7), dtype=np.float32) * np.float32(0.85)
    k = np.cos(i * np.float32(0.047) + np.float32(0.2), dtype=np.float32) * np.float32(0.75)
    v = np.sin(i * np.float32(0.019) - np.float32(0.4), dtype=np.float32) * np.float32(1.2)
    return q, k, v


def half(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.float16)).cuda()


def run(kind, shp, cfg, q16, k16, v16, rot=None, layout=None):
    c = ctx()
    out = c.create_output_buffer(fa.F16, shp)
    out.fill_(0x7f)
    before = c.launch_count()
    args = (fa.F16, shp, cfg) + ((rot,) if rot is not None else ()) + (half(q16), half(k16), half(v16), out)
    getattr(c, kind)(*args)
    o, lse = c.split_output(out, fa.F16, shp, layout if layout is not None else fa.HEAD_MAJOR)
    assert o.dtype == torch.float16
    return o.float().cpu().numpy().reshape(-1), lse.cpu().numpy().reshape(-1), c.launch_count() - before


# tests/wgpu_f16.rs:68-137: the two reference shapes (generic kernel: seq_len < 32)
@pytest.mark.parametrize("B,H,N,D", [(1, 2, 17, 64), (1, 1, 9, 128)])
@pytest.mark.parametrize("causal", [False, True])
def test_packed_f16_reference_shapes(B, H, N, D, causal):
    q, k, v = fixture(B * H * N * D)
    q16, k16, v16 = ob.f16_from_f32(q), ob.f16_from_f32(k), ob.f16_from_f32(v)
    eo, el = ob.forward_reference(ob.f16_to_f32(q16), ob.f16_to_f32(k16), ob.f16_to_f32(v16), B, H, N, D, causal)
    o, l, _ = run("forward_mha", fa.shape(B, H, H, N, N, D), fa.config(causal), q16, k16, v16)
    assert_close("packed-f16 O", o, ob.f16_round(eo), O_ATOL, O_RTOL)
    assert_close("packed-f16 LSE", l, el, LSE_ATOL, LSE_RTOL)


@pytest.mark.parametrize("B,Hq,Hkv,N,D", [(1, 4, 2, 256, 128), (2, 2, 2, 128, 128), (1, 4, 1, 200, 128), (1, 2, 2, 333, 64),
                                          (1, 8, 2, 700, 64), (1, 2, 1, 640, 128), (1, 3, 3, 50, 80)])
@pytest.mark.parametrize("causal", [False, True])
def test_grouped_f16(B, Hq, Hkv, N, D, causal):
    """Tensor-core route (generic for head_dim 80): N(0,1) inputs quantised to binary16."""
    g = lambda n, s: torch.randn(n, generator=torch.Generator().manual_seed(s)).numpy()
    q16, k16, v16 = (ob.f16_from_f32(g(B * h * N * D, s)) for h, s in ((Hq, 1), (Hkv, 2), (Hkv, 3)))
    eo, el = ob.forward_reference_grouped(ob.f16_to_f32(q16), ob.f16_to_f32(k16), ob.f16_to_f32(v16), B, Hq, Hkv, N, D, causal)
    o, l, launches = run("forward_grouped", fa.shape(B, Hq, Hkv, N, N, D), fa.config(causal), q16, k16, v16)
    assert_close("f16 O", o, ob.f16_round(eo), O_ATOL, O_RTOL)
    assert_close("f16 LSE", l, el, LSE_ATOL, LSE_RTOL)
    assert launches == 1 and ctx().device_status() == 0


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nkv,D,causal,coff,qr,kr,rotate_k", [
    (1, 4, 2, 256, 256, 128, True, 0, 7, 7, True),
    (2, 4, 2, 100, 300, 128, True, 200, 200, 0, True),
    (1, 8, 2, 130, 517, 64, True, 387, 400, 13, True),
    (1, 4, 1, 64, 400, 128, False, 0, 50, 3, True),
    (1, 4, 2, 128, 384, 128, True, 256, 256, 0, False),  # K already rotated and stored in binary16
])
def test_projection_rope_asymmetric_f16(B, Hq, Hkv, Nq, Nkv, D, causal, coff, qr, kr, rotate_k):
    theta = 5e5
    g = lambda n, s: ob.f16_round(torch.randn(n, generator=torch.Generator().manual_seed(s)).numpy())
    q, k, v = g(B * Nq * Hq * D, 1), g(B * Nkv * Hkv * D, 2), g(B * Nkv * Hkv * D, 3)
    kpos = np.repeat(np.tile(np.arange(Nkv, dtype=np.uint64) + kr, B), Hkv)
    qpos = np.repeat(np.tile(np.arange(Nq, dtype=np.uint64) + qr, B), Hq)
    k_in = k
    if rotate_k:
        rk = ob.rotate_rows(k, D, kpos, theta)
    else:
        k_in = rk = ob.f16_round(ob.rotate_rows(k, D, kpos, theta))
    rq = ob.rotate_rows(q, D, qpos, theta)
    rows = [(b, h, r) for b in range(B) for h in range(Hq) for r in range(Nq)]
    eo, el = ob.forward_rows(rq, rk, v, ob._shape(B, Hq, Hkv, Nq, Nkv, D, coff), ob.PROJECTION, rows, causal, threads=8)
    o, l, launches = run("forward_projection_rope_asymmetric", fa.shape(B, Hq, Hkv, Nq, Nkv, D, coff), fa.config(causal),
                         ob.f16_from_f32(q), ob.f16_from_f32(k_in), ob.f16_from_f32(v), rot=fa.rotary(theta, qr, kr, rotate_k=rotate_k),
                         layout=fa.PROJECTION)
    o = o.reshape(B, Nq, Hq, D).transpose(0, 2, 1, 3).reshape(-1)
    assert_close("f16 rope O", o, ob.f16_round(eo), O_ATOL, O_RTOL)
    assert_close("f16 rope LSE", l, el, LSE_ATOL, LSE_RTOL)
    assert launches >= 2 and ctx().device_status() == 0  # tables / K rotation + the tensor-core kernel


def test_f16_only_on_forward_entry_points():
    c = ctx()
    shp = fa.shape(1, 2, 2, 64, 64, 64)
    L = fa.backward_layout(fa.BF16, shp)
    packed = c.empty_bytes(L.input_bytes)
    grads = c.empty_bytes(L.output_bytes)
    with pytest.raises(fa.FlatAttentionError) as e:
        c.backward_grouped(fa.F16, shp, fa.config(True), packed, grads)
    assert e.value.kind == "UnsupportedDtype"


def test_f16_host_slice_forward_validates_finiteness():
    # validate_f16_input (src/wgpu_f16_backend.rs:566-586): infinity and NaN patterns are rejected with their index
    c = ctx()
    B, H, N, D = 1, 2, 40, 64
    shp = fa.shape(B, H, H, N, N, D)
    q, k, v = fixture(B * H * N * D)
    hq, hk, hv = (torch.from_numpy(ob.f16_from_f32(x).view(np.float16).copy()) for x in (q, k, v))
    L = fa.forward_layout(fa.F16, shp)
    out = torch.empty(L.combined_bytes, dtype=torch.uint8)
    c.forward_host(fa.F16, fa.HEAD_MAJOR, shp, fa.config(True), None, hq, hk, hv, out, check_finite=True)
    o = out[:L.q_bytes].view(torch.float16).float().numpy()
    lse = out[L.lse_byte_offset:].view(torch.float32).numpy()
    eo, el = ob.forward_reference(ob.f16_round(q), ob.f16_round(k), ob.f16_round(v), B, H, N, D, True)
    assert_close("host f16 O", o, ob.f16_round(eo), O_ATOL, O_RTOL)
    assert_close("host f16 LSE", lse, el, LSE_ATOL, LSE_RTOL)
    hk.view(torch.int16)[5] = 0x7c00
    with pytest.raises(fa.FlatAttentionError) as e:
        c.forward_host(fa.F16, fa.HEAD_MAJOR, shp, fa.config(True), None, hq, hk, hv, out, check_finite=True)
    assert e.value.kind == "NonFiniteInput" and "K" in str(e.value) and "index 5" in str(e.value)


# ---- WgpuPreferredAttention (tests/wgpu_f16.rs:139-243) ----------------------------------------
def test_preferred_router_uses_packed_f16_only_for_qualified_shapes_and_never_cpu():
    router = fa.CudaPreferredAttention(0)
    assert router.io_precision_for_head_dim(80) == fa.IO_F32
    assert router.io_precision_for_head_dim(64) == fa.IO_PACKED_F16
    assert router.io_precision_for_head_dim(128) == fa.IO_PACKED_F16
    for D in (64, 80, 128):
        B, H, N = 1, 1, 9
        q, k, v = fixture(B * H * N * D)
        got = router.forward(q, k, v, fa.shape(B, H, H, N, N, D), fa.config(True))
        o, l = got.output.numpy().reshape(-1), got.lse.numpy().reshape(-1)
        if router.io_precision_for_head_dim(D) == fa.IO_F32:
            assert router.last_precision == fa.IO_F32
            eo, el = ob.forward_reference(q, k, v, B, H, N, D, True)
            assert_close("preferred f32 O", o, eo, 5e-5, 5e-4)
            assert_close("preferred f32 LSE", l, el, 5e-5, 5e-4)
        else:
            assert router.last_precision == fa.IO_PACKED_F16
            eo, el = ob.forward_reference(ob.f16_round(q), ob.f16_round(k), ob.f16_round(v), B, H, N, D, True)
            assert_close("preferred packed-f16 O", o, ob.f16_round(eo), O_ATOL, O_RTOL)
            assert_close("preferred packed-f16 LSE", l, el, LSE_ATOL, LSE_RTOL)


def test_preferred_router_tensor_core_shape_and_overflow_route():
    router = fa.CudaPreferredAttention(0)
    B, H, N, D = 2, 3, 300, 128
    g = lambda s: torch.randn(B * H * N * D, generator=torch.Generator().manual_seed(s)).numpy()
    q, k, v = g(1), g(2), g(3)
    got = router.forward(q, k, v, fa.shape(B, H, H, N, N, D), fa.config(True))
    assert router.last_precision == fa.IO_PACKED_F16
    eo, el = ob.forward_reference(ob.f16_round(q), ob.f16_round(k), ob.f16_round(v), B, H, N, D, True)
    assert_close("router O", got.output.numpy().reshape(-1), ob.f16_round(eo), O_ATOL, O_RTOL)
    assert_close("router LSE", got.lse.numpy().reshape(-1), el, LSE_ATOL, LSE_RTOL)
    # a finite f32 value beyond the binary16 range: the call runs in f32 (src/wgpu_f16_backend.rs:521-528)
    v2 = v.copy()
    v2[7] = 1.0e5
    got = router.forward(q, k, v2, fa.shape(B, H, H, N, N, D), fa.config(True))
    assert router.last_precision == fa.IO_F32
    rows = [(b, h, r) for b in range(B) for h in range(H) for r in (0, 1, 7, 150, 299)]
    eo, el = ob.forward_rows(q, k, v2, ob._shape(B, H, H, N, N, D, 0), ob.HEAD_MAJOR, rows, True, threads=4)
    go = np.stack([got.output.numpy()[b, h, r] for b, h, r in rows]).reshape(-1)
    gl = np.array([got.lse.numpy()[b, h, r] for b, h, r in rows])
    assert_close("overflow-route O", go, eo, 2e-3, 5e-4)  # rows that see the 1e5 value carry an f32 rounding of it
    assert_close("overflow-route LSE", gl, el, 5e-5, 5e-4)
    # non-finite f32 input is rejected before anything is quantised
    v2[9] = np.inf
    with pytest.raises(fa.FlatAttentionError) as e:
        router.forward(q, k, v2, fa.shape(B, H, H, N, N, D), fa.config(True))
    assert e.value.kind == "NonFiniteInput" and "index 9" in str(e.value)
    with pytest.raises(fa.FlatAttentionError) as e:
        router.forward(q, k[:-1], v, fa.shape(B, H, H, N, N, D), fa.config(True))
    assert e.value.kind == "LengthMismatch"


# ---- NumericalExecutor (tests/numerical_policy.rs, tests/wgpu_numerical_policy.rs) ------------------
def numerical_fixture(n):
    # tests/wgpu_numerical_policy.rs:26-43
    i = np.arange(n)
    f = i.astype(np.float32)
    q = np.where(i % 3 == 0, -1.0, 1.0).astype(np.float32) * (np.sin(f * np.float32(0.027), dtype=np.float32) * np.float32(3.5) + np.float32(0.125))
    k = np.where((i // 5) % 2 == 0, 1.0, -1.0).astype(np.float32) * (np.cos(f * np.float32(0.019), dtype=np.float32) * np.float32(2.75) - np.float32(0.0625))
    v = np.sin(f * np.float32(0.013), dtype=np.float32) * np.float32(4.0)
    return q, k, v


def test_mode_guarantees_are_explicit():
    # src/numerical.rs:283-311
    exact, fast, det = (fa.numerical_mode_guarantees(m) for m in (fa.EXACT_REFERENCE, fa.FAST_PORTABLE, fa.DETERMINISTIC_PORTABLE))
    assert (exact.accumulation, exact.reduction, exact.repeatable_same_backend_device, exact.allows_subgroup) == (0, 0, 1, 0)
    assert (fast.accumulation, fast.reduction, fast.repeatable_same_backend_device, fast.allows_subgroup) == (2, 1, 0, 1)
    assert (det.accumulation, det.reduction, det.repeatable_same_backend_device, det.allows_subgroup) == (1, 2, 1, 0)
    with pytest.raises(fa.FlatAttentionError) as e:
        fa.NumericalExecutor(fa.EXACT_REFERENCE)  # reference execution is never presented as a GPU result
    assert e.value.kind == "Unavailable"


def test_deterministic_mode_is_bit_repeatable_and_matches_reference():
    # tests/wgpu_numerical_policy.rs:88-128
    ex = fa.NumericalExecutor(fa.DETERMINISTIC_PORTABLE)
    for N, D in [(17, 64), (33, 80), (9, 128)]:
        q, k, v = numerical_fixture(2 * N * D)
        for causal in (False, True):
            shp, cfg = fa.shape(1, 2, 2, N, N, D), fa.config(causal, 0.125)
            first = ex.forward(q, k, v, shp, cfg)
            for _ in range(4):
                again = ex.forward(q, k, v, shp, cfg)
                assert torch.equal(again.output.view(torch.int32), first.output.view(torch.int32))
                assert torch.equal(again.lse.view(torch.int32), first.lse.view(torch.int32))
            eo, el = ob.forward_reference(q, k, v, 1, 2, N, D, causal, 0.125)
            assert_close("deterministic O", first.output.numpy().reshape(-1), eo, 5e-5, 5e-4)
            assert_close("deterministic LSE", first.lse.numpy().reshape(-1), el, 5e-5, 5e-4)
    fast = fa.NumericalExecutor(fa.FAST_PORTABLE)
    q, k, v = numerical_fixture(17 * 64)
    got = fast.forward(q, k, v, fa.shape(1, 1, 1, 17, 17, 64), fa.config(True))
    eo, el = ob.forward_reference(q, k, v, 1, 1, 17, 64, True)
    assert_close("fast O", got.output.numpy().reshape(-1), eo, 5e-5, 5e-4)
    assert_close("fast LSE", got.lse.numpy().reshape(-1), el, 5e-5, 5e-4)


def test_random_shapes_f16_tensor_core_against_f32_path():
    """Differential sweep: the binary16 instantiation of the tcgen05 kernel against the generic f32 kernel on the same
    binary16-rounded inputs: ragged and rectangular lengths, causal offsets, RoPE offsets, both head dims, raw and
    pre-rotated K, and padded variable-length batches."""
    from tests.gpu_util import run_forward
    rng = np.random.default_rng(1606)
    for case in range(16):
        D = int(rng.choice([64, 128]))
        Hkv = int(rng.choice([1, 2, 4]))
        Hq = Hkv * int(rng.choice([1, 2, 4]))
        B = int(rng.integers(1, 4))
        Nq = int(rng.integers(32, 600))
        extra = int(rng.integers(0, 400))
        Nkv = Nq + extra
        causal = bool(rng.integers(0, 2))
        coff = extra if causal else 0
        qr, kr = int(rng.integers(0, 5000)), int(rng.integers(0, 5000))
        rotate_k = bool(rng.integers(0, 2))
        varlen = case % 4 == 3
        g = lambda n, s: ob.f16_round(torch.randn(n, generator=torch.Generator().manual_seed(s)).numpy())
        q, k, v = g(B * Nq * Hq * D, 100 + case), g(B * Nkv * Hkv * D, 200 + case), g(B * Nkv * Hkv * D, 300 + case)
        if not rotate_k:
            kpos = np.repeat(np.tile(np.arange(Nkv, dtype=np.uint64) + kr, B), Hkv)
            k = ob.f16_round(ob.rotate_rows(k, D, kpos, 5e5))
        shp, cfg, rot = fa.shape(B, Hq, Hkv, Nq, Nkv, D, coff), fa.config(causal), fa.rotary(5e5, qr, kr, rotate_k=rotate_k)
        what = f"case {case}: B={B} Hq={Hq} Hkv={Hkv} Nq={Nq} Nkv={Nkv} D={D} causal={causal} rotate_k={rotate_k} varlen={varlen}"
        kind, kw = "projection_rope_asymmetric", {}
        if varlen:
            seqs = []
            for b in range(B):
                aq = int(rng.integers(1, Nq + 1))
                akv = int(rng.integers(aq, Nkv + 1))
                seqs.append(fa.VarlenSequence(aq, akv, akv - aq, int(rng.integers(0, 3000))))
            kind, kw = "projection_rope_varlen", {"sequences": seqs}
            shp = fa.shape(B, Hq, Hkv, Nq, Nkv, D, 0)
        # run_forward converts the (already binary16-exact) host values to the storage type of each route
        o, l = run_forward(kind, fa.F16, shp, cfg, q, k, v, rot=rot, **kw)
        eo, el = run_forward(kind, fa.F32, shp, cfg, q, k, v, rot=rot, **kw)
        live = np.isfinite(el)
        assert np.array_equal(np.isfinite(l), live), what  # padded rows: LSE = -inf on both routes
        assert_close("sweep O " + what, o, ob.f16_round(eo), O_ATOL, O_RTOL)
        assert_close("sweep LSE " + what, l[live], el[live], LSE_ATOL, LSE_RTOL)
        assert ctx().device_status() == 0, what
