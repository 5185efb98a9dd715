"""Writes tests/golden/oracle_pins.json: regression pins of the CPU oracle on fixed closed-form fixtures.

The reference ships no stored vectors and cannot be executed in this image (Rust), so these pins are NOT reference
outputs: they freeze what the restated oracle produced when its tests against the reference's own oracle tests were
green, so that a later edit of the oracle cannot drift unnoticed.  Each entry records the call, the SHA-256 of the raw
f32 output and LSE bytes, and the first four values of each as hex floats.

    python tests/golden/make_golden.py          # rewrite the file
"""
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
from oracle import binding as ob  # noqa: E402
from oracle import telemetry_oracle as to  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_pins.json")


def digest(a):
    a = np.ascontiguousarray(a)
    return {"sha256": hashlib.sha256(a.tobytes()).hexdigest(), "n": int(a.size),
            "head": [float(x).hex() for x in a.reshape(-1)[:4].astype(np.float64)]}


def fx(n, phase):
    return ob.fixture(n, 0.071, phase, 0.625)


def cases():
    out = {}
    B, H, N, D = 2, 3, 7, 8
    q, k, v = fx(B * H * N * D, 0.2), fx(B * H * N * D, 0.8), fx(B * H * N * D, 1.4)
    for causal in (False, True):
        o, l = ob.forward_reference(q, k, v, B, H, N, D, causal)
        out[f"forward_reference causal={causal}"] = {"o": digest(o), "lse": digest(l)}
    s = ob.Shape(1, 4, 2, 3, 5, 8, 2)
    q, k, v = fx(96, 0.3), fx(80, 0.9), fx(80, 1.5)
    o, l = ob.forward_reference_projection_grouped_rope_asymmetric(q, k, v, s, 10000.0, 17, 13, True)
    out["projection_rope_asymmetric causal"] = {"o": digest(o), "lse": digest(l)}
    o, l = ob.forward_reference_projection_grouped_rope_asymmetric_biased(q, k, v, s, 10000.0, 17, 13, causal=False,
                                                                           alibi=([0.25, 0.5, 0.75, 1.0], 31, 29))
    out["projection_rope_asymmetric alibi"] = {"o": digest(o), "lse": digest(l)}
    B, Hq, Hkv, N, D = 1, 4, 2, 6, 8
    q, do = fx(B * Hq * N * D, 0.1), fx(B * Hq * N * D, 2.1)
    k, v = fx(B * Hkv * N * D, 0.7), fx(B * Hkv * N * D, 1.3)
    fo, fl = ob.forward_reference_grouped(q, k, v, B, Hq, Hkv, N, D, True)
    dq, dk, dv = ob.backward_reference_grouped(q, k, v, do, fo, fl, B, Hq, Hkv, N, D, True)
    out["backward_grouped causal"] = {"dq": digest(dq), "dk": digest(dk), "dv": digest(dv)}
    bits = ob.f16_from_f32(ob.fixture(4096, 0.019, 0.4, 60000.0, 0.37, 1e-6))
    out["f16_from_f32 fixture"] = {"sha256": hashlib.sha256(bits.tobytes()).hexdigest(), "head": [int(x) for x in bits[:4]]}
    m = dict(commit_sha="0123456789abcdef0123456789abcdef01234567", benchmark_id="m40-test",
             command='cargo run --release --example bench -- --case \\"gqa\\"', device='Device "A"', backend="Vulkan",
             driver="driver-1", os="Linux", arch="aarch64", precision="f32", batch=1, q_heads=8, kv_heads=2, query_len=128,
             kv_len=128, head_dim=64, causal=True, warmup_iterations=3, measured_iterations=11, median_latency_ns=1234567,
             p95_latency_ns=1456789, tokens_per_second_milli=103680000)
    out["benchmark_manifest"] = {"canonical_json": to.canonical_json(m), "result_checksum": to.result_checksum(m)}
    rec = to.fingerprint_record("NVIDIA Tegra NVIDIA Thor", "Vulkan", "580.00", "test-driver-info", 0x10de, 1)
    out["device_fingerprint"] = {"record": rec, "fnv1a64": "%016x" % to.fnv1a64(rec.encode())}
    return out


if __name__ == "__main__":
    with open(OUT, "w") as f:
        json.dump(cases(), f, indent=1, sort_keys=True)
        f.write("\n")
    print("wrote", OUT)
