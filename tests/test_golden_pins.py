"""The oracle against its committed regression pins (tests/golden/oracle_pins.json, written by
tests/golden/make_golden.py), and the library's host-only writers against the pinned strings."""
import importlib.util
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))


def load_maker():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_oracle_reproduces_its_pins_bit_for_bit():
    pins = json.load(open(os.path.join(HERE, "golden", "oracle_pins.json")))
    now = json.loads(json.dumps(load_maker().cases()))
    assert sorted(now) == sorted(pins)
    for name in pins:
        assert now[name] == pins[name], name


def test_library_writers_reproduce_the_pinned_strings():
    import dataclasses
    import importlib
    from __graft_entry__ import load_package
    load_package()
    tel = importlib.import_module("flat_attention_b200.telemetry")
    pins = json.load(open(os.path.join(HERE, "golden", "oracle_pins.json")))
    fp = tel.fingerprint("NVIDIA Tegra NVIDIA Thor", "Vulkan", "580.00", "test-driver-info", 0x10de, 1)
    assert tel.fingerprint_canonical_record(fp) == pins["device_fingerprint"]["record"]
    assert "%016x" % tel.fingerprint_stable(fp) == pins["device_fingerprint"]["fnv1a64"]
    j = json.loads(pins["benchmark_manifest"]["canonical_json"])
    m = tel.BenchmarkManifest(
        commit_sha=j["commit_sha"], benchmark_id=j["benchmark_id"], command=j["command"], **j["environment"], **j["problem"],
        warmup_iterations=j["protocol"]["warmup_iterations"], measured_iterations=j["protocol"]["measured_iterations"], **j["result"])
    assert m.canonical_json() == pins["benchmark_manifest"]["canonical_json"]
    assert m.result_checksum() == pins["benchmark_manifest"]["result_checksum"] == j["result_checksum"]["value"]
    assert dataclasses.asdict(m)["causal"] is True
