"""The Rust binding sources under rust/ cannot be compiled on a machine without a Rust toolchain; what can be checked
anywhere: the generated `extern "C"` block declares exactly the functions of the C header (and is not stale), and the
hand-written `#[repr(C)]` structs carry the header's fields in the header's order."""
import os
import re
import subprocess
import sys

from __graft_entry__ import load_package

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
fa = load_package()


def test_extern_block_matches_the_header_and_is_current():
    text = open(os.path.join(ROOT, "rust", "src", "cuda_ffi.rs")).read()
    declared = sorted(re.findall(r"pub fn (flat_[a-z0-9_]+)\(", text))
    assert declared == fa.exported_symbols_in_header()
    assert subprocess.run([sys.executable, os.path.join(ROOT, "rust", "gen_ffi.py"), "--check"]).returncode == 0


def test_repr_c_structs_follow_the_header_field_order():
    header = re.sub(r"/\*.*?\*/", "", open(fa.HEADER_PATH).read(), flags=re.S)
    rust = open(os.path.join(ROOT, "rust", "src", "cuda_types.rs")).read()
    pairs = {"flat_attention_shape": "FlatAttentionShape", "flat_attention_config": "FlatAttentionConfigRaw",
             "flat_rotary_config": "FlatRotaryConfig", "flat_buffer": "FlatBuffer", "flat_forward_layout": "FlatForwardLayout",
             "flat_decode_layout": "FlatDecodeLayout", "flat_backward_layout": "FlatBackwardLayout",
             "flat_varlen_sequence": "FlatVarlenSequence", "flat_paged_kv_telemetry": "FlatPagedKvTelemetry",
             "flat_paged_kv_address": "FlatPagedKvAddress", "flat_numerical_guarantees": "FlatNumericalGuarantees",
             "flat_device_fingerprint": "FlatDeviceFingerprint", "flat_device_capabilities": "FlatDeviceCapabilities",
             "flat_dispatch_telemetry": "FlatDispatchTelemetry", "flat_benchmark_manifest": "FlatBenchmarkManifest"}
    for c_name, r_name in pairs.items():
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (c_name, c_name), header, flags=re.S).group(1)
        c_fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            for part in decl.split(","):
                c_fields.append(re.sub(r"\[.*?\]", "", part).replace("*", " ").split()[-1])
        r_body = re.search(r"pub struct %s \{(.*?)\n\}" % r_name, rust, flags=re.S).group(1)
        r_fields = re.findall(r"pub ([a-z_0-9]+):", r_body)
        assert c_fields == r_fields, (c_name, c_fields, r_fields)
