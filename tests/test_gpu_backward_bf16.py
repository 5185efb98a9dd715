"""bf16 tensor-core backward (tcgen05) against the CPU oracle on de-quantised inputs: max-abs error
<= 2e-2 on dQ, dK, dV.  The forward O and LSE the backward consumes are inputs of the call; the oracle
is given the same (de-quantised) values."""
import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.gpu_util import bf16_round, ctx, fa
from tests.test_gpu_chunked_backward import run_backward

pytestmark = pytest.mark.gpu
TOL = 2e-2


def randn(n, seed):
    return bf16_round(torch.randn(n, generator=torch.Generator().manual_seed(seed)).numpy())


@pytest.fixture(params=["spill", "recompute"])
def dq_route(request):
    """Both routes of the tensor-core backward to dQ: from the dS tiles kept in scratch (the default while they fit the
    context's budget) and by recomputing the scores in a second kernel (budget 0)."""
    ctx().set_backward_scratch_budget(0 if request.param == "recompute" else 8 << 30)
    yield request.param
    ctx().set_backward_scratch_budget(8 << 30)


@pytest.mark.parametrize("B,Hq,Hkv,N,D", [(1, 4, 2, 256, 128), (2, 2, 2, 128, 64), (1, 8, 1, 384, 128), (1, 2, 1, 512, 64),
                                          # sequence lengths that are not whole 128-row tiles
                                          (2, 4, 2, 200, 128), (1, 4, 1, 333, 64), (1, 2, 2, 40, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_backward_bf16_small(B, Hq, Hkv, N, D, causal, dq_route):
    q, k, v, do = randn(B * Hq * N * D, 1), randn(B * Hkv * N * D, 2), randn(B * Hkv * N * D, 3), randn(B * Hq * N * D, 4)
    fo, fl = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, causal)
    fo = bf16_round(fo)
    edq, edk, edv = ob.backward_reference_grouped(q, k, v, do, fo, fl, B, Hq, Hkv, N, D, causal)
    dq, dk, dv = run_backward(fa.BF16, B, Hq, Hkv, N, D, causal, None, q, k, v, do, fo, fl)
    for name, a, e in (("dQ", dq, edq), ("dK", dk, edk), ("dV", dv, edv)):
        assert np.isfinite(a).all(), name
        assert np.abs(a - e).max() <= TOL, (name, float(np.abs(a - e).max()))
    again = run_backward(fa.BF16, B, Hq, Hkv, N, D, causal, None, q, k, v, do, fo, fl)
    assert all(np.array_equal(x, y) for x, y in zip((dq, dk, dv), again))  # bitwise repeatable
    assert ctx().device_status() == 0


def test_random_shapes_tensor_core_backward_against_f32_path(dq_route):
    """Differential sweep: the tcgen05 backward (bf16) against the generic f32 backward (pinned to the oracle at 1e-4)
    on the same bf16-rounded inputs and the same forward results, over seeded random shapes (ragged lengths, both
    head dims, GQA groups, causal and not)."""
    from tests.gpu_util import run_forward
    rng = np.random.default_rng(77)
    for case in range(12):
        D = int(rng.choice([64, 128]))
        Hkv = int(rng.choice([1, 2]))
        Hq = Hkv * int(rng.choice([1, 2, 4]))
        B = int(rng.integers(1, 3))
        N = int(rng.integers(20, 600))
        causal = bool(rng.integers(0, 2))
        q, k, v, do = (randn(B * Hq * N * D, 10 + case), randn(B * Hkv * N * D, 30 + case), randn(B * Hkv * N * D, 50 + case),
                       randn(B * Hq * N * D, 70 + case))
        fo, fl = run_forward("grouped", fa.F32, fa.shape(B, Hq, Hkv, N, N, D), fa.config(causal), q, k, v)
        fo = bf16_round(fo)
        what = f"case {case}: B={B} Hq={Hq} Hkv={Hkv} N={N} D={D} causal={causal}"
        got = run_backward(fa.BF16, B, Hq, Hkv, N, D, causal, None, q, k, v, do, fo, fl)
        exp = run_backward(fa.F32, B, Hq, Hkv, N, D, causal, None, q, k, v, do, fo, fl)
        for name, a, e in zip(("dQ", "dK", "dV"), got, exp):
            assert np.isfinite(a).all(), (what, name)
            assert np.abs(a - e).max() <= TOL, (what, name, float(np.abs(a - e).max()))
        assert ctx().device_status() == 0, what


def test_config5_grouped_backward_sampled_rows(dq_route):
    """B=2, Hq=32, Hkv=8, N=8192, D=128, causal: forward on the device, backward on the device, oracle
    on sampled dQ rows and dK/dV rows (first/last rows, tile boundaries, random)."""
    B, Hq, Hkv, N, D = 2, 32, 8, 8192, 128
    c = ctx()
    q = torch.randn(B, Hq, N, D, generator=torch.Generator().manual_seed(1)).bfloat16()
    k = torch.randn(B, Hkv, N, D, generator=torch.Generator().manual_seed(2)).bfloat16()
    v = torch.randn(B, Hkv, N, D, generator=torch.Generator().manual_seed(3)).bfloat16()
    do = torch.randn(B, Hq, N, D, generator=torch.Generator().manual_seed(4)).bfloat16()
    shp = fa.shape(B, Hq, Hkv, N, N, D)
    FL, L = fa.forward_layout(fa.BF16, shp), fa.backward_layout(fa.BF16, shp)
    dq_, dk_, dv_, ddo = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    fwd = c.create_output_buffer(fa.BF16, shp)
    c.forward_grouped(fa.BF16, shp, fa.config(True), dq_, dk_, dv_, fwd)
    packed = c.empty_bytes(L.input_bytes)
    for off, t in ((L.q_offset, dq_), (L.k_offset, dk_), (L.v_offset, dv_), (L.d_out_offset, ddo)):
        packed[off:off + t.numel() * 2] = t.view(torch.uint8).reshape(-1)
    packed[L.out_offset:L.out_offset + FL.q_bytes] = fwd[:FL.q_bytes]
    packed[L.lse_offset:L.lse_offset + 4 * FL.lse_elements] = fwd[FL.lse_byte_offset:FL.lse_byte_offset + 4 * FL.lse_elements]
    grads = c.empty_bytes(L.output_bytes)
    c.backward_grouped(fa.BF16, shp, fa.config(True), packed, grads)
    c.synchronize()
    assert c.device_status() == 0
    raw = grads.cpu()
    gq = raw[L.dq_offset:L.dq_offset + L.q_elements * 4].view(torch.float32).numpy().reshape(B, Hq, N, D)
    gk = raw[L.dk_offset:L.dk_offset + L.kv_elements * 4].view(torch.float32).numpy().reshape(B, Hkv, N, D)
    gv = raw[L.dv_offset:L.dv_offset + L.kv_elements * 4].view(torch.float32).numpy().reshape(B, Hkv, N, D)
    assert np.isfinite(gq).all() and np.isfinite(gk).all() and np.isfinite(gv).all()
    o, l = c.split_output(fwd, fa.BF16, shp)
    rng = np.random.default_rng(0)
    qr = [(0, 0, 0), (0, 0, 127), (0, 0, 128), (1, 31, N - 1), (1, 7, 4095), (0, 13, 4096)] + \
         [(int(rng.integers(B)), int(rng.integers(Hq)), int(rng.integers(N))) for _ in range(18)]
    kr = [(0, 0, 0), (0, 0, 127), (0, 0, 128), (1, 7, N - 1), (1, 3, N - 128), (0, 5, 4096)] + \
         [(int(rng.integers(B)), int(rng.integers(Hkv)), int(rng.integers(N))) for _ in range(10)]
    edq, edk, edv = ob.backward_rows(q.float().numpy(), k.float().numpy(), v.float().numpy(), do.float().numpy(),
                                     o.float().cpu().numpy(), l.cpu().numpy(), B, Hq, Hkv, N, D, qr, kr, True, threads=8)
    aq = np.stack([gq[b, h, r] for (b, h, r) in qr])
    ak = np.stack([gk[b, h, r] for (b, h, r) in kr])
    av = np.stack([gv[b, h, r] for (b, h, r) in kr])
    assert np.abs(aq - edq).max() <= TOL, float(np.abs(aq - edq).max())
    assert np.abs(ak - edk).max() <= TOL, float(np.abs(ak - edk).max())
    assert np.abs(av - edv).max() <= TOL, float(np.abs(av - edv).max())
