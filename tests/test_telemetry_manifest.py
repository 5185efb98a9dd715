"""Runtime-telemetry records and benchmark manifests: the library's host-only entry points against the
Python restatement, both pinned by the literals of the reference's unit tests
(src/runtime_telemetry.rs:179-291, src/benchmark_manifest.rs:249-316) and by the published FNV-1a-64
vectors.  Byte-exact throughout.  The context-bound calls are covered by the GPU tests at the end."""
import dataclasses
import importlib

import pytest

from __graft_entry__ import load_package
from oracle import telemetry_oracle as to

fa = load_package()
tel = importlib.import_module("flat_attention_b200.telemetry")


def test_fnv1a64_published_vectors():
    assert to.fnv1a64(b"") == 0xcbf29ce484222325
    assert to.fnv1a64(b"a") == 0xaf63dc4c8601ec8c
    assert to.fnv1a64(b"foobar") == 0x85944171f73967e8


FP = ("NVIDIA Tegra NVIDIA Thor", "Vulkan", "580.00", "test-driver-info", 0x10de, 0x0001)  # runtime_telemetry.rs:183-192


def test_device_fingerprint_is_deterministic_and_driver_sensitive():
    a = tel.fingerprint(*FP)
    assert tel.fingerprint_canonical_record(a) == to.fingerprint_record(*FP)
    assert tel.fingerprint_canonical_record(a) == ("name=NVIDIA Tegra NVIDIA Thor;backend=Vulkan;driver=580.00;"
                                                   "driver_info=test-driver-info;vendor=000010de;device=00000001")
    assert tel.fingerprint_stable(a) == tel.fingerprint_stable(tel.fingerprint(*FP)) == to.fnv1a64(
        to.fingerprint_record(*FP).encode())
    changed = tel.fingerprint(FP[0], FP[1], FP[2] + "-changed", *FP[3:])
    assert tel.fingerprint_stable(changed) != tel.fingerprint_stable(a)


def test_canonical_record_preserves_utf8_and_escapes_delimiters():
    # runtime_telemetry.rs:207-214
    name = "GPU été;a=b%"
    rec = tel.fingerprint_canonical_record(tel.fingerprint(name, *FP[1:]))
    assert "name=GPU été%3ba%3db%25;" in rec
    assert rec == to.fingerprint_record(name, *FP[1:])


CAPS = (65535, 1024, 1024, 64, 32768, 12, 1 << 30, 1, 32, 32, 1)  # runtime_telemetry.rs:251-265


def test_capabilities_record_is_deterministic_and_limit_sensitive():
    base = tel.DeviceCapabilities(*CAPS)
    assert tel.capabilities_canonical_record(base) == to.capabilities_record(CAPS) == (
        "wgpd=65535;wgsx=1024;wgsy=1024;wgsz=64;wgss=32768;bind=12;sbuf=1073741824;sub=1;submin=32;submax=32;f16=1")
    assert tel.capabilities_stable(base) == to.fnv1a64(to.capabilities_record(CAPS).encode())
    smaller = tel.DeviceCapabilities(*CAPS[:4], 16384, *CAPS[5:])
    no_f16 = tel.DeviceCapabilities(*CAPS[:10], 0)
    assert len({tel.capabilities_stable(x) for x in (base, smaller, no_f16)}) == 3


def test_autotuner_annotation_is_pure_metadata():
    # runtime_telemetry.rs:216-249
    t = tel.DispatchTelemetry()
    t.dispatch_count = 1
    hit = t.with_autotuner_cache(1)
    assert tel.AUTOTUNER_CACHE[hit.autotuner_cache] == "Hit" and hit.dispatch_count == 1
    assert tel.AUTOTUNER_CACHE[t.autotuner_cache] == "NotApplicable"


def manifest(**kw):
    # benchmark_manifest.rs:253-283
    m = tel.BenchmarkManifest(
        commit_sha="0123456789abcdef0123456789abcdef01234567", benchmark_id="m40-test",
        command='cargo run --release --example bench -- --case \\"gqa\\"', device='Device "A"', backend="Vulkan",
        driver="driver-1", os="Linux", arch="aarch64", precision="f32", batch=1, q_heads=8, kv_heads=2, query_len=128,
        kv_len=128, head_dim=64, causal=True, warmup_iterations=3, measured_iterations=11, median_latency_ns=1_234_567,
        p95_latency_ns=1_456_789, tokens_per_second_milli=103_680_000)
    return dataclasses.replace(m, **kw)


def test_canonical_record_is_bit_reproducible():
    a, b = manifest(), manifest()
    assert a.canonical_json() == b.canonical_json() == to.canonical_json(dataclasses.asdict(a))
    assert a.result_checksum() == b.result_checksum() == to.result_checksum(dataclasses.asdict(a))
    assert 'Device \\"A\\"' in a.canonical_json()
    assert a.canonical_json().startswith('{"schema_version":1,"commit_sha":"0123456789abcdef0123456789abcdef01234567",'
                                         '"benchmark_id":"m40-test","command":"cargo run --release --example bench -- '
                                         '--case \\\\\\"gqa\\\\\\"","environment":{"device":"Device \\"A\\"",')
    assert a.canonical_json().endswith('"protocol":{"warmup_iterations":3,"measured_iterations":11},"result":'
                                       '{"median_latency_ns":1234567,"p95_latency_ns":1456789,'
                                       '"tokens_per_second_milli":103680000},"result_checksum":{"algorithm":"fnv1a64",'
                                       '"value":"%s"}}' % a.result_checksum())
    import json
    assert json.loads(a.canonical_json())["problem"] == {"precision": "f32", "batch": 1, "q_heads": 8, "kv_heads": 2,
                                                         "query_len": 128, "kv_len": 128, "head_dim": 64, "causal": True}


def test_result_change_invalidates_checksum():
    a = manifest()
    assert a.result_checksum() != manifest(median_latency_ns=a.median_latency_ns + 1).result_checksum()


@pytest.mark.parametrize("change,kind,field", [
    (dict(commit_sha="main"), "ManifestInvalidCommitSha", ""),
    (dict(commit_sha="g" * 40), "ManifestInvalidCommitSha", ""),
    (dict(measured_iterations=0), "ManifestZeroMeasuredIterations", ""),
    (dict(kv_heads=3), "InvalidHeadGrouping", ""),
    (dict(os=" \t 　"), "ManifestEmptyField", "environment.os"),
    (dict(precision=""), "ManifestEmptyField", "problem.precision"),
    (dict(kv_len=0), "ZeroDimension", "kv_len"),
    (dict(p95_latency_ns=1), "ManifestInvalidPercentileOrdering", ""),
])
def test_malformed_provenance_fails_closed(change, kind, field):
    m = manifest(**change)
    with pytest.raises(fa.FlatAttentionError) as e:
        m.validate()
    assert e.value.kind == kind and e.value.detail == field
    with pytest.raises(fa.FlatAttentionError) as e:
        m.canonical_json()
    assert e.value.kind == kind
    expected = to.validate(dataclasses.asdict(m))
    assert expected is not None and expected[0] == kind.replace("Manifest", "") and (expected[1] or "") == field


def test_control_characters_and_unicode_in_json_strings():
    m = manifest(command="a\x01b\nc\td\\eé ", device="\x1f")
    assert m.canonical_json() == to.canonical_json(dataclasses.asdict(m))
    assert '"command":"a\\u0001b\\nc\\td\\\\eé "' in m.canonical_json()
    assert '"device":"\\u001f"' in m.canonical_json()


# ---- context-bound calls -----------------------------------------------------------------------
@pytest.mark.gpu
def test_context_fingerprint_and_capabilities():
    from tests.gpu_util import ctx
    c = ctx()
    fp = tel.device_fingerprint(c)
    assert fp.name and fp.backend == b"Cuda" and fp.vendor == 0x10de and fp.device == 100
    assert tel.fingerprint_stable(fp) == to.fnv1a64(tel.fingerprint_canonical_record(fp).encode())
    caps = tel.device_capabilities(c)
    assert caps.subgroup_min_size == caps.subgroup_max_size == 32 and caps.max_workgroup_storage_bytes >= 227 * 1024
    assert caps.max_workgroups_per_dimension >= 1 and caps.max_workgroup_size_x >= 1


@pytest.mark.gpu
def test_passive_snapshot_matches_selected_dispatch():
    # tests/m29_runtime_telemetry.rs:8-63: the snapshot names the kernel a real call then launches, and takes no launch
    import torch
    from tests.gpu_util import ctx
    c = ctx()
    before = c.launch_count()
    shp = fa.shape(2, 8, 2, 700, 700, 128)
    rot = fa.rotary(5e5, 0)
    t = tel.forward_runtime_telemetry(c, fa.BF16, fa.HEAD_MAJOR, shp, rot)
    assert c.launch_count() == before
    assert t.kernel == "ForwardTcgen05" and (t.query_rows, t.kv_rows) == (256, 128)
    assert list(t.workgroups) == [min(3 * 2 * 8, 148), 1, 1] and t.fallback_reason is None
    assert t.dispatch_count == 2 and t.temporary_allocation_count == 1
    assert t.temporary_allocation_bytes == 2 * 2 * 700 * 128 * 2
    assert tel.AUTOTUNER_CACHE[t.autotuner_cache] == "NotApplicable" and t.device.name
    q = torch.randn(2, 8, 700, 128, device="cuda").bfloat16()
    k = torch.randn(2, 2, 700, 128, device="cuda").bfloat16()
    out = c.create_output_buffer(fa.BF16, shp)
    c.forward_grouped_rope(fa.BF16, shp, fa.config(True), rot, q, k, k, out)  # cold (cos, sin) tables
    before = c.launch_count()
    c.forward_grouped_rope(fa.BF16, shp, fa.config(True), rot, q, k, k, out)
    assert c.launch_count() - before == t.dispatch_count
    # a shape without tensor-core specialization reports the selection reason without a dispatch
    t = tel.forward_runtime_telemetry(c, fa.BF16, fa.HEAD_MAJOR, fa.shape(1, 1, 1, 5, 5, 32))
    assert t.kernel == "ForwardGeneric" and t.fallback_reason == "tensor-core specialization unavailable for head_dim=32"
    assert (t.query_rows, t.kv_rows, list(t.workgroups)) == (32, 32, [1, 1, 1]) and t.dispatch_count == 1
    t = tel.forward_runtime_telemetry(c, fa.F32, fa.PROJECTION, fa.shape(2, 3, 3, 17, 17, 64))
    assert t.kernel == "ForwardGeneric" and list(t.workgroups) == [1, 3, 2] and "16-bit storage" in t.fallback_reason
    with pytest.raises(fa.FlatAttentionError) as e:
        tel.forward_runtime_telemetry(c, fa.BF16, fa.HEAD_MAJOR, fa.shape(1, 3, 2, 5, 5, 32))
    assert e.value.kind == "InvalidHeadGrouping"
    t = tel.forward_runtime_telemetry(c, fa.F16, fa.HEAD_MAJOR, fa.shape(1, 4, 2, 512, 512, 64))
    assert t.kernel == "ForwardTcgen05" and list(t.workgroups) == [8, 1, 1] and t.dispatch_count == 1
