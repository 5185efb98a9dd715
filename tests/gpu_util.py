"""Shared helpers of the GPU parity tests: one context per process, fixtures in the style of the
reference tests (closed-form sin/cos ramps), tolerance checks `|a-e| <= atol + rtol*|e|`."""
import numpy as np
import torch

from __graft_entry__ import load_package
from oracle import binding as ob

fa = load_package()
_ctx = None


def ctx():
    global _ctx
    if _ctx is None:
        _ctx = fa.Context(0)
    return _ctx


def ramp(n, phase, step=0.021, a=1.1875, c=0.43, b=0.34375):
    """tests/m16_paged_decode.rs:49-56 style fixture."""
    return ob.fixture(n, step, phase, a, c, b)


def dev(x, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(x)).to(dtype).cuda()


def assert_close(name, actual, expected, atol, rtol):
    actual = np.asarray(actual, dtype=np.float32).reshape(-1)
    expected = np.asarray(expected, dtype=np.float32).reshape(-1)
    assert actual.shape == expected.shape, (name, actual.shape, expected.shape)
    tol = atol + rtol * np.abs(expected)
    err = np.abs(actual - expected)
    both_inf = np.isinf(actual) & np.isinf(expected) & (np.sign(actual) == np.sign(expected))
    bad = ~(err <= tol) & ~both_inf
    assert not bad.any(), "%s: %d/%d outside tolerance, worst |err|=%g at %d (actual %g expected %g)" % (
        name, int(bad.sum()), bad.size, float(np.nanmax(np.where(bad, err, 0))), int(np.argmax(np.where(bad, err, 0))),
        actual[int(np.argmax(np.where(bad, err, 0)))], expected[int(np.argmax(np.where(bad, err, 0)))])


def run_forward(kind, dtype, shp, cfg, q, k, v, rot=None, sequences=None, layout=None):
    """Launch one forward entry point on device copies of host arrays; returns (O, LSE) numpy."""
    c = ctx()
    td = fa.torch_dtype(dtype)
    dq, dk, dv = dev(q, td), dev(k, td), dev(v, td)
    out = c.create_output_buffer(dtype, shp)
    out.fill_(0x7f)  # poison
    if kind == "mha":
        c.forward_mha(dtype, shp, cfg, dq, dk, dv, out)
    elif kind == "grouped":
        c.forward_grouped(dtype, shp, cfg, dq, dk, dv, out)
    elif kind == "grouped_asymmetric":
        c.forward_grouped_asymmetric(dtype, shp, cfg, dq, dk, dv, out)
    elif kind == "grouped_rope":
        c.forward_grouped_rope(dtype, shp, cfg, rot, dq, dk, dv, out)
    elif kind == "projection_rope":
        c.forward_projection_rope(dtype, shp, cfg, rot, dq, dk, dv, out)
    elif kind == "projection_rope_asymmetric":
        c.forward_projection_rope_asymmetric(dtype, shp, cfg, rot, dq, dk, dv, out)
    elif kind == "projection_rope_varlen":
        c.forward_projection_rope_varlen(dtype, shp, cfg, rot, sequences, dq, dk, dv, out)
    else:
        raise ValueError(kind)
    lay = layout if layout is not None else (fa.PROJECTION if kind.startswith("projection") else fa.HEAD_MAJOR)
    o, lse = c.split_output(out, dtype, shp, lay)
    return o.float().cpu().numpy().reshape(-1), lse.cpu().numpy().reshape(-1)


def bf16_round(x):
    """Quantise to bf16 (RNE) and return the de-quantised f32 values the oracle consumes."""
    return torch.as_tensor(np.ascontiguousarray(x, dtype=np.float32)).bfloat16().float().numpy()
