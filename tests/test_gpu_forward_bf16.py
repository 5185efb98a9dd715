"""bf16 tensor-core forward (tcgen05) against the CPU oracle evaluated on the de-quantised bf16
inputs (policy of docs/m8-precision.md:74-85): max-abs error <= 2e-2 on O and <= 2e-3 on LSE.
RoPE cases use the materialise-then-grouped oracle route, bit-identical to the fused oracle
(tests/rotary_grouped.rs:48-143)."""
import numpy as np
import pytest
import torch

from oracle import binding as ob
from tests.gpu_util import bf16_round, ctx, fa, run_forward

pytestmark = pytest.mark.gpu
O_TOL, LSE_TOL = 2e-2, 2e-3


def randn(n, seed):
    return bf16_round(torch.randn(n, generator=torch.Generator().manual_seed(seed)).numpy())


def check(o, l, eo, el, what=""):
    eo, el = np.asarray(eo).reshape(-1), np.asarray(el).reshape(-1)
    assert np.isfinite(o).all() and np.isfinite(l).all(), what
    assert np.abs(o - eo).max() <= O_TOL, (what, float(np.abs(o - eo).max()))
    assert np.abs(l - el).max() <= LSE_TOL, (what, float(np.abs(l - el).max()))


SHAPES = [(1, 4, 2, 256, 128), (2, 2, 2, 128, 128), (1, 4, 1, 200, 128), (1, 2, 2, 333, 64), (1, 8, 2, 512, 64),
          (1, 2, 1, 640, 128), (1, 4, 4, 40, 128)]


@pytest.mark.parametrize("B,Hq,Hkv,N,D", SHAPES)
@pytest.mark.parametrize("causal", [False, True])
def test_grouped_bf16(B, Hq, Hkv, N, D, causal):
    q, k, v = randn(B * Hq * N * D, 1), randn(B * Hkv * N * D, 2), randn(B * Hkv * N * D, 3)
    o, l = run_forward("grouped", fa.BF16, fa.shape(B, Hq, Hkv, N, N, D), fa.config(causal), q, k, v)
    eo, el = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, causal)
    check(o, l, eo, el)
    assert ctx().device_status() == 0


@pytest.mark.parametrize("B,Hq,Hkv,N,D,theta,off", [(1, 4, 2, 256, 128, 5e5, 0), (1, 2, 1, 300, 64, 1e4, 11),
                                                    (2, 4, 4, 160, 128, 5e5, 4000)])
def test_grouped_rope_bf16(B, Hq, Hkv, N, D, theta, off):
    q, k, v = randn(B * Hq * N * D, 1), randn(B * Hkv * N * D, 2), randn(B * Hkv * N * D, 3)
    for causal in (True, False):
        o, l = run_forward("grouped_rope", fa.BF16, fa.shape(B, Hq, Hkv, N, N, D), fa.config(causal), q, k, v,
                           rot=fa.rotary(theta, off))
        rq = ob.rotate_rows(q, D, np.tile(np.arange(N, dtype=np.uint64) + off, B * Hq), theta)
        rk = ob.rotate_rows(k, D, np.tile(np.arange(N, dtype=np.uint64) + off, B * Hkv), theta)
        eo, el = ob.forward_reference_grouped(rq, rk, v, B, Hq, Hkv, N, D, causal)
        check(o, l, eo, el)


@pytest.mark.parametrize("B,Hq,Hkv,N,D,rope", [(2, 48, 8, 300, 128, True), (3, 64, 8, 130, 64, True), (2, 40, 8, 520, 128, False)])
def test_persistent_grid_walks_several_items_per_cta(B, Hq, Hkv, N, D, rope):
    """More (query block, batch, head) items than SMs: every CTA of the persistent forward kernel walks several
    items, with ragged last blocks (an item whose second 128-row tile lies past q_len) in between.  Sampled rows
    (first / last rows, tile borders, random ones) of every head are checked against the oracle."""
    q, k, v = randn(B * Hq * N * D, 1), randn(B * Hkv * N * D, 2), randn(B * Hkv * N * D, 3)
    theta, off = 5e5, 17
    shp = fa.shape(B, Hq, Hkv, N, N, D)
    if rope:
        o, l = run_forward("grouped_rope", fa.BF16, shp, fa.config(True), q, k, v, rot=fa.rotary(theta, off))
        rq = ob.rotate_rows(q, D, np.tile(np.arange(N, dtype=np.uint64) + off, B * Hq), theta)
        rk = ob.rotate_rows(k, D, np.tile(np.arange(N, dtype=np.uint64) + off, B * Hkv), theta)
    else:
        o, l = run_forward("grouped", fa.BF16, shp, fa.config(True), q, k, v)
        rq, rk = q, k
    rng = np.random.default_rng(5)
    picks = sorted({0, 1, 127, 128, 255, 256, N - 1} & set(range(N)))
    rows = [(b, h, r) for b in range(B) for h in range(Hq) for r in picks + list(rng.integers(0, N, 3))]
    eo, el = ob.forward_rows(rq, rk, v, ob._shape(B, Hq, Hkv, N, N, D, 0), ob.HEAD_MAJOR, rows, True, threads=8)
    o = o.reshape(B, Hq, N, D)
    l = l.reshape(B, Hq, N)
    go = np.stack([o[b, h, r] for b, h, r in rows]).reshape(-1)
    gl = np.array([l[b, h, r] for b, h, r in rows])
    check(go, gl, eo, el)
    assert ctx().device_status() == 0


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nkv,D,causal,coff,qr,kr,rotate_k", [
    (1, 4, 2, 256, 256, 128, True, 0, 7, 7, True),
    (2, 4, 2, 100, 300, 128, True, 200, 200, 0, True),
    (1, 8, 2, 130, 517, 64, True, 387, 400, 13, True),
    (1, 4, 1, 64, 400, 128, False, 0, 50, 3, True),
    (1, 4, 2, 128, 384, 128, True, 256, 256, 0, False),   # pre-rotated bf16 K: converted to fp16 in shared memory
    (1, 8, 2, 130, 517, 64, True, 387, 400, 13, False),
])
def test_projection_rope_asymmetric_bf16(B, Hq, Hkv, Nq, Nkv, D, causal, coff, qr, kr, rotate_k):
    theta = 5e5
    q, k, v = randn(B * Nq * Hq * D, 1), randn(B * Nkv * Hkv * D, 2), randn(B * Nkv * Hkv * D, 3)
    kpos = np.repeat(np.tile(np.arange(Nkv, dtype=np.uint64) + kr, B), Hkv)
    qpos = np.repeat(np.tile(np.arange(Nq, dtype=np.uint64) + qr, B), Hq)
    k_in = k
    if not rotate_k:  # the cache convention: K rotated once, stored in bf16
        k_in = bf16_round(ob.rotate_rows(k, D, kpos, theta))
        rk = k_in
    else:
        rk = ob.rotate_rows(k, D, kpos, theta)
    rq = ob.rotate_rows(q, D, qpos, theta)
    o, l = run_forward("projection_rope_asymmetric", fa.BF16, fa.shape(B, Hq, Hkv, Nq, Nkv, D, coff), fa.config(causal),
                       q, k_in, v, rot=fa.rotary(theta, qr, kr, rotate_k=rotate_k))
    rows = [(b, h, r) for b in range(B) for h in range(Hq) for r in range(Nq)]
    eo, el = ob.forward_rows(rq, rk, v, ob._shape(B, Hq, Hkv, Nq, Nkv, D, coff), ob.PROJECTION, rows, causal, threads=8)
    o = o.reshape(B, Nq, Hq, D).transpose(0, 2, 1, 3).reshape(-1)
    check(o, l, eo, el)
    assert ctx().device_status() == 0


def test_config2_llama8b_prefill_sampled_rows():
    """B=4, Hq=32, Hkv=8, N=4096, D=128, causal, RoPE theta 5e5: oracle on sampled
    (batch, q_head, row) triples including tile and sequence boundaries; V = 1 gives O = 1."""
    B, Hq, Hkv, N, D, theta = 4, 32, 8, 4096, 128, 5e5
    g = torch.Generator().manual_seed(1)
    q = torch.randn(B, Hq, N, D, generator=torch.Generator().manual_seed(1)).bfloat16()
    k = torch.randn(B, Hkv, N, D, generator=torch.Generator().manual_seed(2)).bfloat16()
    v = torch.randn(B, Hkv, N, D, generator=torch.Generator().manual_seed(3)).bfloat16()
    c = ctx()
    shp = fa.shape(B, Hq, Hkv, N, N, D)
    out = c.create_output_buffer(fa.BF16, shp)
    dq, dk, dv = q.cuda(), k.cuda(), v.cuda()
    c.forward_grouped_rope(fa.BF16, shp, fa.config(True), fa.rotary(theta, 0), dq, dk, dv, out)
    o, l = c.split_output(out, fa.BF16, shp)
    o, l = o.float().cpu().numpy(), l.cpu().numpy()
    assert c.device_status() == 0
    rng = np.random.default_rng(0)
    rows = {(0, 0, 0), (0, 0, 1), (0, 0, 127), (0, 0, 128), (3, 31, 4095), (1, 5, 255), (1, 5, 256), (2, 17, 2047)}
    while len(rows) < 72:
        rows.add((int(rng.integers(B)), int(rng.integers(Hq)), int(rng.integers(N))))
    rows = sorted(rows)
    qf, kf, vf = q.float().numpy(), k.float().numpy(), v.float().numpy()
    pos_k = np.tile(np.arange(N, dtype=np.uint64), B * Hkv)
    rk = ob.rotate_rows(kf, D, pos_k, theta)
    rq = qf.copy().reshape(B, Hq, N, D)
    for (b, h, r) in rows:  # only the sampled query rows need rotating
        rq[b, h, r] = ob.rotate_rows(qf.reshape(B, Hq, N, D)[b, h, r], D, [r], theta)
    eo, el = ob.forward_rows(rq, rk, vf, ob._shape(B, Hq, Hkv, N, N, D), ob.HEAD_MAJOR, rows, True, threads=8)
    ao = np.stack([o[b, h, r] for (b, h, r) in rows])
    al = np.array([l[b, h, r] for (b, h, r) in rows])
    assert np.abs(ao - eo).max() <= O_TOL, float(np.abs(ao - eo).max())
    assert np.abs(al - el).max() <= LSE_TOL, float(np.abs(al - el).max())
    # size-independent properties on the whole output
    assert np.isfinite(o).all() and np.isfinite(l).all()
    c.forward_grouped_rope(fa.BF16, shp, fa.config(True), fa.rotary(theta, 0), dq, dk, torch.ones_like(dv), out)
    o1, l1 = c.split_output(out, fa.BF16, shp)
    assert (o1.float() - 1.0).abs().max().item() <= 8e-3
    assert torch.equal(l1.cpu(), torch.from_numpy(l))  # LSE does not depend on V; runs are bitwise repeatable


def test_host_slice_forward_pipelined_over_batch_matches_resident_call():
    """flat_forward_host overlaps upload / attention / download per batch element and KV-head group; the packed host
    result must equal the resident-buffer call bit for bit (bf16 tensor-core path and f32 path)."""
    c = ctx()
    for dtype, B, Hq, Hkv, N, D in ((fa.BF16, 3, 4, 2, 256, 128), (fa.F32, 3, 4, 2, 40, 32)):
        td = fa.torch_dtype(dtype)
        g = torch.Generator().manual_seed(5)
        q = torch.randn(B, Hq, N, D, generator=g).to(td)
        k = torch.randn(B, Hkv, N, D, generator=g).to(td)
        v = torch.randn(B, Hkv, N, D, generator=g).to(td)
        shp = fa.shape(B, Hq, Hkv, N, N, D)
        rot = fa.rotary(5e5, 3)
        L = fa.forward_layout(dtype, shp)
        host_out = torch.empty(L.combined_bytes, dtype=torch.uint8).pin_memory()
        c.forward_host(dtype, fa.HEAD_MAJOR, shp, fa.config(True), rot, q.pin_memory(), k.pin_memory(), v.pin_memory(), host_out)
        dev_out = c.create_output_buffer(dtype, shp)
        c.forward_grouped_rope(dtype, shp, fa.config(True), rot, q.cuda(), k.cuda(), v.cuda(), dev_out)
        assert torch.equal(host_out, dev_out.cpu())
        # projection layout [B, N, H*D]: one chunk per batch element
        qp, kp, vp = (t.transpose(1, 2).contiguous() for t in (q, k, v))
        host_out2 = torch.empty(L.combined_bytes, dtype=torch.uint8).pin_memory()
        c.forward_host(dtype, fa.PROJECTION, shp, fa.config(True), rot, qp.pin_memory(), kp.pin_memory(), vp.pin_memory(), host_out2)
        dev_out2 = c.create_output_buffer(dtype, shp)
        c.forward_projection_rope(dtype, shp, fa.config(True), rot, qp.cuda(), kp.cuda(), vp.cuda(), dev_out2)
        assert torch.equal(host_out2, dev_out2.cpu())


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nkv,D,causal,kvoff,meta", [
    (3, 8, 2, 300, 400, 128, True, 5, [(300, 400, 100, 105), (1, 33, 32, 37), (130, 129, 0, 900)]),
    (2, 4, 4, 260, 260, 64, False, 0, [(129, 260, 0, 0), (260, 64, 0, 7)]),
    (40, 4, 1, 256, 256, 128, True, 0, [(1 + (37 * i) % 256, 1 + (91 * i) % 256, 0, i) for i in range(40)]),
])
def test_variable_length_projection_bf16(B, Hq, Hkv, Nq, Nkv, D, causal, kvoff, meta):
    """Padded variable-length batch (tests/wgpu_external_variable.rs:160-387) on the tensor-core path: per-sequence
    active lengths, causal offsets and RoPE offsets; the padding is poisoned and must not leak; padded query rows
    come back as O = 0, LSE = -inf."""
    theta = 5e5
    q = randn(B * Nq * Hq * D, 1).reshape(B, Nq, Hq * D).copy()
    k = randn(B * Nkv * Hkv * D, 2).reshape(B, Nkv, Hkv * D).copy()
    v = randn(B * Nkv * Hkv * D, 3).reshape(B, Nkv, Hkv * D).copy()
    for b, (aq, akv, _, _) in enumerate(meta):
        q[b, aq:] = bf16_round(np.float32(1.0e20))
        k[b, akv:] = bf16_round(np.float32(-1.0e20))
        v[b, akv:] = bf16_round(np.float32(1.0e20))
    seqs = [fa.VarlenSequence(*m) for m in meta]
    launches = ctx().launch_count()
    o, l = run_forward("projection_rope_varlen", fa.BF16, fa.shape(B, Hq, Hkv, Nq, Nkv, D), fa.config(causal), q, k, v,
                       rot=fa.rotary(theta, 0, kvoff), sequences=seqs)
    # K rotation, padding fill and the tcgen05 kernel (plus the table kernels): the generic kernel is a single launch
    assert ctx().launch_count() - launches >= 3
    o, l = o.reshape(B, Nq, Hq, D), l.reshape(B, Hq, Nq)
    for b, (aq, akv, coff, qr) in enumerate(meta):
        eo, el = ob.forward_reference_projection_grouped_rope_asymmetric(
            q[b, :aq], k[b, :akv], v[b, :akv], ob._shape(1, Hq, Hkv, aq, akv, D, coff), theta, qr, kvoff, causal)
        check(o[b, :aq].reshape(-1), l[b, :, :aq].reshape(-1), eo, np.asarray(el).reshape(Hq, aq).reshape(-1), f"sequence {b}")
        assert np.all(o[b, aq:] == 0.0)
        assert np.all(l[b, :, aq:].view(np.uint32) == 0xFF800000)
    assert ctx().device_status() == 0


def test_random_shapes_tensor_core_path_against_f32_path():
    """Differential sweep: the tcgen05 kernel (bf16) against the generic f32 kernel (itself pinned to the oracle at
    1e-4) on the same bf16-rounded inputs, over seeded random shapes: ragged and rectangular lengths, causal offsets,
    RoPE offsets, both head dims, rotated and pre-rotated K, GQA groups, batches that give a CTA several items."""
    rng = np.random.default_rng(20240607)
    for case in range(24):
        D = int(rng.choice([64, 128]))
        Hkv = int(rng.choice([1, 2, 4]))
        Hq = Hkv * int(rng.choice([1, 2, 4]))
        B = int(rng.integers(1, 4))
        Nq = int(rng.integers(32, 700))
        extra = int(rng.integers(0, 500))
        Nkv = Nq + extra
        causal = bool(rng.integers(0, 2))
        coff = extra if causal else 0          # the last query row sees every key
        theta = float(rng.choice([1e4, 5e5]))
        qr, kr = int(rng.integers(0, 5000)), int(rng.integers(0, 5000))
        rotate_k = bool(rng.integers(0, 2))
        q, k, v = randn(B * Nq * Hq * D, 100 + case), randn(B * Nkv * Hkv * D, 200 + case), randn(B * Nkv * Hkv * D, 300 + case)
        if not rotate_k:  # the cache convention: K rotated once and stored in bf16
            kpos = np.repeat(np.tile(np.arange(Nkv, dtype=np.uint64) + kr, B), Hkv)
            k = bf16_round(ob.rotate_rows(k, D, kpos, theta))
        shp = fa.shape(B, Hq, Hkv, Nq, Nkv, D, coff)
        rot = fa.rotary(theta, qr, kr, rotate_k=rotate_k)
        what = f"case {case}: B={B} Hq={Hq} Hkv={Hkv} Nq={Nq} Nkv={Nkv} D={D} causal={causal} rotate_k={rotate_k}"
        o, l = run_forward("projection_rope_asymmetric", fa.BF16, shp, fa.config(causal), q, k, v, rot=rot)
        eo, el = run_forward("projection_rope_asymmetric", fa.F32, shp, fa.config(causal), q, k, v, rot=rot)
        check(o, l, eo, el, what)
        assert ctx().device_status() == 0, what


@pytest.mark.parametrize("B,Hq,Hkv,N,D", [(3, 6, 3, 300, 128), (5, 12, 4, 260, 64), (7, 9, 9, 130, 128), (1, 15, 5, 513, 128)])
def test_head_and_batch_counts_that_are_not_powers_of_two(B, Hq, Hkv, N, D):
    """The persistent kernel turns a work-item index into (query block, batch, head, kv head) with multiply-high
    constants made on the host instead of divisions: batch * heads, heads and group sizes that are not powers of two,
    against the generic f32 kernel on the same bf16-rounded inputs."""
    q, k, v = randn(B * N * Hq * D, 41), randn(B * N * Hkv * D, 42), randn(B * N * Hkv * D, 43)
    shp = fa.shape(B, Hq, Hkv, N, N, D)
    rot = fa.rotary(5e5, 0)
    o, l = run_forward("projection_rope", fa.BF16, shp, fa.config(True), q, k, v, rot=rot)
    eo, el = run_forward("projection_rope", fa.F32, shp, fa.config(True), q, k, v, rot=rot)
    check(o, l, eo, el, f"B={B} Hq={Hq} Hkv={Hkv} N={N} D={D}")
    assert ctx().device_status() == 0


@pytest.mark.parametrize("B,Hq,Hkv,Nq,Nkv,off,D,causal,rope", [
    (1, 4, 2, 2048, 8192, 0, 128, False, False),    # 32 items on 148 SMs: every item cut into 4 KV parts
    (1, 4, 2, 256, 8192, 7936, 128, True, True),    # 4 items, 4 parts of 16 KV tiles; the last part holds the diagonal
    (1, 8, 8, 384, 4736, 4352, 64, True, False),    # ragged: the second Q tile of the last block lies past q_len
    (2, 40, 8, 1024, 5120, 4096, 128, True, True),  # 320 items: two whole rounds, 24 left, each cut into 2 parts
])
def test_last_round_items_split_along_kv(B, Hq, Hkv, Nq, Nkv, off, D, causal, rope):
    """When the last round of the persistent forward holds few items, each is cut along KV into parts that run on
    different CTAs and a merge kernel finishes the rows.  Sampled rows of every (batch, head) - first / last rows,
    tile borders, random ones - against the oracle."""
    q, k, v = randn(B * Hq * Nq * D, 1), randn(B * Hkv * Nkv * D, 2), randn(B * Hkv * Nkv * D, 3)
    theta = 5e5
    shp = fa.shape(B, Hq, Hkv, Nq, Nkv, D, off)
    c = ctx()
    launches = c.launch_count()
    if rope:
        o, l = run_forward("projection_rope_asymmetric", fa.BF16, shp, fa.config(causal), q, k, v, rot=fa.rotary(theta, off, 0))
        rq = ob.rotate_rows(q, D, np.repeat(np.tile(np.arange(Nq, dtype=np.uint64) + off, B), Hq), theta)
        rk = ob.rotate_rows(k, D, np.repeat(np.tile(np.arange(Nkv, dtype=np.uint64), B), Hkv), theta)
        layout = ob.PROJECTION
        o, pick = o.reshape(B, Nq, Hq, D), (lambda b, h, r: (b, r, h))
    else:
        o, l = run_forward("grouped_asymmetric", fa.BF16, shp, fa.config(causal), q, k, v)
        rq, rk, layout = q, k, ob.HEAD_MAJOR
        o, pick = o.reshape(B, Hq, Nq, D), (lambda b, h, r: (b, h, r))
    rng = np.random.default_rng(7)
    picks = sorted({0, 1, 127, 128, 255, 256, Nq - 1} & set(range(Nq)))
    rows = [(b, h, r) for b in range(B) for h in range(Hq) for r in picks + [int(x) for x in rng.integers(0, Nq, 2)]]
    eo, el = ob.forward_rows(rq, rk, v, ob._shape(B, Hq, Hkv, Nq, Nkv, D, off), layout, rows, causal, threads=8)
    l = l.reshape(B, Hq, Nq)
    go = np.stack([o[pick(b, h, r)] for b, h, r in rows]).reshape(-1)
    gl = np.array([l[b, h, r] for b, h, r in rows])
    check(go, gl, eo, el)
    assert c.device_status() == 0
    # the split really ran: the call launched a merge kernel besides the attention kernel (and the K rotation / tables)
    assert c.launch_count() - launches >= 2


def test_prepared_forward_and_backward_only_enqueue():
    """prepare validates once and sizes the scratch; encode_prepared gives the same bits as the direct entry point
    and neither allocates nor re-validates (src/wgpu_forward_grouped.rs:352-529, src/wgpu_backward_grouped.rs:231-326)."""
    c = fa.Context(0)
    B, Hq, Hkv, N, D, theta = 1, 8, 2, 384, 128, 5e5
    g = torch.Generator().manual_seed(41)
    q, do = (torch.randn(B, Hq, N, D, generator=g).bfloat16().cuda() for _ in range(2))
    k, v = (torch.randn(B, Hkv, N, D, generator=g).bfloat16().cuda() for _ in range(2))
    shp, cfg, rot = fa.shape(B, Hq, Hkv, N, N, D), fa.config(True), fa.rotary(theta, 3)
    direct, out = c.create_output_buffer(fa.BF16, shp), c.create_output_buffer(fa.BF16, shp)
    c.forward_grouped_rope(fa.BF16, shp, cfg, rot, q, k, v, direct)
    c.reserve_rope_tables(N, D)
    prep = c.prepare_forward(fa.BF16, fa.HEAD_MAJOR, shp, cfg, rot, q, k, v, out)
    ws, launches = c.workspace_bytes(), c.launch_count()
    for _ in range(3):
        out.fill_(0x7f)
        prep.encode()
    c.synchronize()
    assert torch.equal(out, direct) and c.workspace_bytes() == ws and c.launch_count() - launches == 6  # K rotation + attention
    # errors surface at prepare time, with the direct entry point's variants
    with pytest.raises(fa.FlatAttentionError) as e:
        c.prepare_forward(fa.BF16, fa.HEAD_MAJOR, shp, cfg, rot, q, k, v, out[:-8])
    assert e.value.kind == "BufferTooSmall"
    with pytest.raises(fa.FlatAttentionError) as e:
        c.prepare_forward(fa.BF16, fa.HEAD_MAJOR, fa.shape(B, Hq, 3, N, N, D), cfg, rot, q, k, v, out)
    assert e.value.kind == "InvalidHeadGrouping"
    other = fa.Context(0)
    st = fa.lib().flat_forward_encode_prepared(other.h, prep.h)
    assert fa.STATUS[st] == "UnsupportedShape"
    # backward
    fwd = c.create_output_buffer(fa.BF16, shp)
    c.forward_grouped(fa.BF16, shp, cfg, q, k, v, fwd)
    FL, L = fa.forward_layout(fa.BF16, shp), fa.backward_layout(fa.BF16, shp)
    packed = c.empty_bytes(L.input_bytes)
    for off, t in ((L.q_offset, q), (L.k_offset, k), (L.v_offset, v), (L.d_out_offset, do)):
        packed[off:off + t.numel() * 2] = t.view(torch.uint8).reshape(-1)
    packed[L.out_offset:L.out_offset + FL.q_bytes] = fwd[:FL.q_bytes]
    packed[L.lse_offset:L.lse_offset + 4 * FL.lse_elements] = fwd[FL.lse_byte_offset:FL.lse_byte_offset + 4 * FL.lse_elements]
    g_direct, g_prep = c.empty_bytes(L.output_bytes), c.empty_bytes(L.output_bytes)
    c.backward_grouped(fa.BF16, shp, cfg, packed, g_direct)
    bprep = c.prepare_backward(fa.BF16, shp, cfg, packed, g_prep)
    ws = c.workspace_bytes()
    for _ in range(2):
        g_prep.fill_(0x7f)
        bprep.encode()
    c.synchronize()
    assert torch.equal(g_prep, g_direct) and c.workspace_bytes() == ws
    with pytest.raises(fa.FlatAttentionError) as e:
        c.prepare_backward(fa.BF16, shp, cfg, packed[:-4], g_prep)
    assert e.value.kind == "BufferTooSmall"
    assert c.device_status() == 0
