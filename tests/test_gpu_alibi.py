"""ALiBi score bias on the CUDA forward (flat_forward_projection_rope_asymmetric_alibi) against the
additive-bias oracle (src/attention_bias.rs:193-339).  The f32 cases restate tests/m13_alibi_wgpu.rs
(ATOL 2e-4, RTOL 1e-3, raw and pre-rotated K); the bf16 cases run the tensor-core kernel at the bf16
budget (|dO| <= 2e-2, |dLSE| <= 2e-3)."""
import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.gpu_util import assert_close, bf16_round, ctx, dev, fa

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2.0e-4, 1.0e-3  # tests/m13_alibi_wgpu.rs:12-13


def fixture(n, phase):
    # tests/m13_alibi_wgpu.rs:47-54
    return ob.fixture(n, 0.019, phase, 1.625, 0.37, 0.3125)


def two_pass_biased(rq, rk, v, B, Hq, Hkv, Nq, Nkv, D, causal, coff, slopes, bq, bk):
    """Projection-layout attention over already rotated rows with the ALiBi bias, in f64."""
    rq = np.asarray(rq, np.float64).reshape(B, Nq, Hq, D)
    rk = np.asarray(rk, np.float64).reshape(B, Nkv, Hkv, D)
    vv = np.asarray(v, np.float64).reshape(B, Nkv, Hkv, D)
    o = np.zeros((B, Nq, Hq, D))
    lse = np.zeros((B, Hq, Nq))
    g = Hq // Hkv
    for b in range(B):
        for h in range(Hq):
            s = rq[b, :, h] @ rk[b, :, h // g].T / np.sqrt(D)
            s += np.float32(slopes[h]) * ((bk + np.arange(Nkv))[None, :] - (bq + np.arange(Nq))[:, None]).astype(np.float64)
            if causal:
                s = np.where(np.arange(Nkv)[None, :] <= coff + np.arange(Nq)[:, None], s, -np.inf)
            m = s.max(axis=1, keepdims=True)
            p = np.exp(s - m)
            den = p.sum(axis=1, keepdims=True)
            o[b, :, h] = (p / den) @ vv[b, :, h // g]
            lse[b, h] = (m + np.log(den))[:, 0]
    return o.reshape(-1).astype(np.float32), lse.reshape(-1).astype(np.float32)


def run_alibi(dtype, shp, cfg, rot, slopes, bq, bk, q, k, v):
    c = ctx()
    td = fa.torch_dtype(dtype)
    out = c.create_output_buffer(dtype, shp)
    out.fill_(0x7f)
    before = c.launch_count()
    c.forward_projection_rope_asymmetric_alibi(dtype, shp, cfg, rot, slopes, bq, bk, dev(q, td), dev(k, td), dev(v, td), out)
    launches = c.launch_count() - before
    o, lse = c.split_output(out, dtype, shp, fa.PROJECTION)
    return o.float().cpu().numpy().reshape(-1), lse.cpu().numpy().reshape(-1), launches


# tests/m13_alibi_wgpu.rs:160-272
@pytest.mark.parametrize("pre_rotated_k", [False, True])
def test_reference_alibi_case_f32(pre_rotated_k):
    Hq, Hkv, Nq, Nkv, D, theta = 8, 2, 3, 17, 64, 10000.0
    slopes = [0.03125, 0.0625, 0.09375, 0.125, 0.15625, 0.1875, 0.21875, 0.25]
    q, k, v = fixture(Nq * Hq * D, 0.2), fixture(Nkv * Hkv * D, 0.8), fixture(Nkv * Hkv * D, 1.4)
    eo, el = ob.forward_reference_projection_grouped_rope_asymmetric_biased(
        q, k, v, ob._shape(1, Hq, Hkv, Nq, Nkv, D, 14), theta, 41, 7, causal=True, alibi=(slopes, 103, 97))
    k_in = k
    if pre_rotated_k:
        k_in = ob.rotate_rows(k, D, np.repeat(np.arange(Nkv, dtype=np.uint64) + 7, Hkv), theta)
    o, l, _ = run_alibi(fa.F32, fa.shape(1, Hq, Hkv, Nq, Nkv, D, 14), fa.config(True),
                        fa.rotary(theta, 41, 7, rotate_k=not pre_rotated_k), slopes, 103, 97, q, k_in, v)
    assert_close("ALiBi O", o, eo, ATOL, RTOL)
    assert_close("ALiBi LSE", l, el, ATOL, RTOL)


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nkv,D,causal,coff,bq,bk", [
    (2, 4, 2, 40, 70, 32, True, 30, 30, 0),
    (1, 4, 1, 9, 33, 80, False, 0, 5, 1000),        # keys far ahead of the queries: large positive bias
    (1, 2, 2, 65, 65, 128, True, 0, 4000000000, 4000000000),  # bias positions near the top of u32
    (1, 3, 3, 17, 5, 16, False, 0, 0, 0),
])
def test_alibi_shapes_f32(B, Hq, Hkv, Nq, Nkv, D, causal, coff, bq, bk):
    rng = np.random.default_rng(Nq * 131 + Nkv)
    q = rng.standard_normal(B * Nq * Hq * D).astype(np.float32)
    k = rng.standard_normal(B * Nkv * Hkv * D).astype(np.float32)
    v = rng.standard_normal(B * Nkv * Hkv * D).astype(np.float32)
    slopes = [2.0 ** -(1 + h) * (-1.0 if h == 2 else 1.0) for h in range(Hq)]
    eo, el = ob.forward_reference_projection_grouped_rope_asymmetric_biased(
        q, k, v, ob._shape(B, Hq, Hkv, Nq, Nkv, D, coff), 5e5, 11, 3, causal=causal, alibi=(slopes, bq, bk))
    o, l, _ = run_alibi(fa.F32, fa.shape(B, Hq, Hkv, Nq, Nkv, D, coff), fa.config(causal), fa.rotary(5e5, 11, 3),
                        slopes, bq, bk, q, k, v)
    assert_close("ALiBi O", o, eo, ATOL, RTOL)
    assert_close("ALiBi LSE", l, el, ATOL, RTOL)


def test_zero_slopes_equal_unbiased_forward():
    B, Hq, Hkv, Nq, Nkv, D = 1, 4, 2, 50, 90, 64
    rng = np.random.default_rng(3)
    q = rng.standard_normal(B * Nq * Hq * D).astype(np.float32)
    k = rng.standard_normal(B * Nkv * Hkv * D).astype(np.float32)
    v = rng.standard_normal(B * Nkv * Hkv * D).astype(np.float32)
    shp, cfg, rot = fa.shape(B, Hq, Hkv, Nq, Nkv, D, 40), fa.config(True), fa.rotary(1e4, 40, 0)
    for dtype in (fa.F32, fa.BF16):
        c = ctx()
        td = fa.torch_dtype(dtype)
        a, b = c.create_output_buffer(dtype, shp), c.create_output_buffer(dtype, shp)
        dq, dk, dv = dev(q, td), dev(k, td), dev(v, td)
        c.forward_projection_rope_asymmetric(dtype, shp, cfg, rot, dq, dk, dv, a)
        c.forward_projection_rope_asymmetric_alibi(dtype, shp, cfg, rot, [0.0] * Hq, 7, 9, dq, dk, dv, b)
        c.synchronize()
        if dtype == fa.F32:
            assert torch.equal(a, b)
        else:
            # the tensor-core kernel rounds s*c before the bias FMA, so the two routes differ in the last bf16 bit at most
            oa, la = c.split_output(a, dtype, shp, fa.PROJECTION)
            ob_, lb = c.split_output(b, dtype, shp, fa.PROJECTION)
            assert (oa.float() - ob_.float()).abs().max().item() <= 2.0 ** -6
            assert (la - lb).abs().max().item() <= 1e-5


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nkv,D,causal,coff,qr,kr,bq,bk,rotate_k", [
    (1, 4, 2, 256, 256, 128, True, 0, 7, 7, 0, 0, True),
    (2, 4, 2, 100, 300, 128, True, 200, 200, 0, 1200, 1000, True),
    (1, 8, 2, 130, 517, 64, True, 387, 400, 13, 387, 0, True),
    (1, 4, 1, 64, 400, 128, False, 0, 50, 3, 350, 0, True),      # non-causal: keys on both sides of the queries
    (1, 4, 2, 128, 384, 128, True, 256, 256, 0, 256, 0, False),  # pre-rotated bf16 K
    (1, 8, 2, 130, 517, 64, True, 387, 400, 13, 5000387, 5000000, False),
    (1, 8, 2, 700, 700, 128, True, 0, 0, 0, 0, 0, True),         # several work items per head
])
def test_alibi_bf16_tensor_core(B, Hq, Hkv, Nq, Nkv, D, causal, coff, qr, kr, bq, bk, rotate_k):
    theta = 5e5
    g = lambda n, s: bf16_round(torch.randn(n, generator=torch.Generator().manual_seed(s)).numpy())
    q, k, v = g(B * Nq * Hq * D, 1), g(B * Nkv * Hkv * D, 2), g(B * Nkv * Hkv * D, 3)
    slopes = [2.0 ** -(1 + 8.0 * h / Hq) for h in range(Hq)]
    k_in = k
    if rotate_k:
        eo, el = ob.forward_reference_projection_grouped_rope_asymmetric_biased(
            q, k, v, ob._shape(B, Hq, Hkv, Nq, Nkv, D, coff), theta, qr, kr, causal=causal, alibi=(slopes, bq, bk))
    else:
        # the cache convention: K rotated once and stored in bf16.  The oracle always rotates, so the expected values
        # for these rows come from a two-pass f64 softmax over the host-rotated Q and the stored K.
        kpos = np.repeat(np.tile(np.arange(Nkv, dtype=np.uint64) + kr, B), Hkv)
        qpos = np.repeat(np.tile(np.arange(Nq, dtype=np.uint64) + qr, B), Hq)
        k_in = bf16_round(ob.rotate_rows(k, D, kpos, theta))
        rq = ob.rotate_rows(q, D, qpos, theta)
        eo, el = two_pass_biased(rq, k_in, v, B, Hq, Hkv, Nq, Nkv, D, causal, coff, slopes, bq, bk)
    o, l, launches = run_alibi(fa.BF16, fa.shape(B, Hq, Hkv, Nq, Nkv, D, coff), fa.config(causal),
                               fa.rotary(theta, qr, kr, rotate_k=rotate_k), slopes, bq, bk, q, k_in, v)
    assert np.isfinite(o).all() and np.isfinite(l).all()
    assert np.abs(o - eo).max() <= 2e-2, float(np.abs(o - eo).max())
    assert np.abs(l - el).max() <= 2e-3, float(np.abs(l - el).max())
    assert ctx().device_status() == 0
    assert launches >= 2  # tables / K rotation plus the attention kernel: the tensor-core route (the generic one is 1)


def test_alibi_validation_errors():
    # validate_alibi, src/wgpu_external_asymmetric.rs:512-545
    c = ctx()
    Hq, Hkv, Nq, Nkv, D = 4, 2, 3, 5, 8
    shp, cfg, rot = fa.shape(1, Hq, Hkv, Nq, Nkv, D, 2), fa.config(True), fa.rotary(1e4, 17, 13)
    q, k, v = dev(np.zeros(Nq * Hq * D)), dev(np.zeros(Nkv * Hkv * D)), dev(np.zeros(Nkv * Hkv * D))
    out = c.create_output_buffer(fa.F32, shp)

    def call(slopes, bq=0, bk=0, s=shp):
        c.forward_projection_rope_asymmetric_alibi(fa.F32, s, cfg, rot, slopes, bq, bk, q, k, v, out)

    with pytest.raises(fa.FlatAttentionError) as e:
        call([0.1, 0.2, 0.3])
    assert e.value.kind == "LengthMismatch" and "ALiBi slopes" in str(e.value)
    with pytest.raises(fa.FlatAttentionError) as e:
        call([0.0, float("nan"), 0.0, 0.0])
    assert e.value.kind == "NonFiniteInput" and "index 1" in str(e.value)
    with pytest.raises(fa.FlatAttentionError) as e:
        call([0.0] * 4, bq=2 ** 32 - 2)
    assert e.value.kind == "PositionOverflow"
    with pytest.raises(fa.FlatAttentionError) as e:
        call([0.0] * 4, bk=2 ** 64 - 1)
    assert e.value.kind == "PositionOverflow"
    call([0.0] * 4, bq=2 ** 32 - 3, bk=2 ** 32 - 5)  # the last positions are exactly u32::MAX
    big = fa.shape(1, 257, 1, 1, 1, 8, 0)
    with pytest.raises(fa.FlatAttentionError) as e:
        call([0.0] * 257, s=big)
    assert e.value.kind == "IndexSpaceExceeded"
    assert c.device_status() == 0


def test_random_shapes_alibi_tensor_core_against_f32_path():
    """Differential sweep: the ALIBI instantiation of the tcgen05 kernel (bf16) against the generic f32 kernel (pinned to
    the oracle above) on the same bf16-rounded inputs: ragged and rectangular lengths, causal offsets, bias origins on
    either side of each other, negative slopes, both head dims, rotated and pre-rotated K."""
    rng = np.random.default_rng(1312)
    c = ctx()
    for case in range(16):
        D = int(rng.choice([64, 128]))
        Hkv = int(rng.choice([1, 2, 4]))
        Hq = Hkv * int(rng.choice([1, 2, 4]))
        B = int(rng.integers(1, 3))
        Nq = int(rng.integers(32, 600))
        extra = int(rng.integers(0, 400))
        Nkv = Nq + extra
        causal = bool(rng.integers(0, 2))
        coff = extra if causal else 0
        qr, kr = int(rng.integers(0, 5000)), int(rng.integers(0, 5000))
        bq, bk = int(rng.integers(0, 100000)), int(rng.integers(0, 100000))
        if causal:
            bq = bk + extra  # the usual convention: bias positions are the causal positions
        rotate_k = bool(rng.integers(0, 2))
        slopes = [float(s) for s in rng.choice([-1.0, 1.0], Hq) * 2.0 ** -rng.integers(3, 9, Hq)]
        if not causal:
            slopes = [s * 2.0 ** -4 for s in slopes]  # keep the LSE magnitude inside the absolute 2e-3 budget
        g = lambda n, s: bf16_round(torch.randn(n, generator=torch.Generator().manual_seed(s)).numpy())
        q, k, v = g(B * Nq * Hq * D, 100 + case), g(B * Nkv * Hkv * D, 200 + case), g(B * Nkv * Hkv * D, 300 + case)
        if not rotate_k:
            kpos = np.repeat(np.tile(np.arange(Nkv, dtype=np.uint64) + kr, B), Hkv)
            k = bf16_round(ob.rotate_rows(k, D, kpos, 5e5))
        shp, cfg, rot = fa.shape(B, Hq, Hkv, Nq, Nkv, D, coff), fa.config(causal), fa.rotary(5e5, qr, kr, rotate_k=rotate_k)
        what = f"case {case}: B={B} Hq={Hq} Hkv={Hkv} Nq={Nq} Nkv={Nkv} D={D} causal={causal} rotate_k={rotate_k} bq={bq} bk={bk}"
        o, l, launches = run_alibi(fa.BF16, shp, cfg, rot, slopes, bq, bk, q, k, v)
        eo, el, one = run_alibi(fa.F32, shp, cfg, rot, slopes, bq, bk, q, k, v)
        assert one == 1 and launches >= 2, what
        assert np.isfinite(o).all() and np.isfinite(l).all(), what
        assert np.abs(o - eo).max() <= 2e-2, (what, float(np.abs(o - eo).max()))
        assert np.abs(l - el).max() <= 2e-3 + 2e-5 * np.abs(el).max(), (what, float(np.abs(l - el).max()))
        assert c.device_status() == 0, what
