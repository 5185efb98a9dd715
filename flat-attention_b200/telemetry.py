"""Python mirror of the passive telemetry records and benchmark manifests of the C ABI
(RuntimeDeviceFingerprint / RuntimeDeviceCapabilities / RuntimeDispatchTelemetry,
src/runtime_telemetry.rs:10-177; BenchmarkManifest, src/benchmark_manifest.rs:10-199).
Every string and checksum is produced by the library; nothing here touches a stream."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

KERNEL_IDS = {0: "ForwardTcgen05", 1: "ForwardGeneric"}
AUTOTUNER_CACHE = {0: "NotApplicable", 1: "Hit", 2: "Miss"}


class DeviceFingerprint(C.Structure):
    _fields_ = [("name", C.c_char * 256), ("backend", C.c_char * 32), ("driver", C.c_char * 64),
                ("driver_info", C.c_char * 128), ("vendor", C.c_uint32), ("device", C.c_uint32)]


class DeviceCapabilities(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "max_workgroups_per_dimension", "max_workgroup_size_x", "max_workgroup_size_y", "max_workgroup_size_z",
        "max_workgroup_storage_bytes", "max_binding_entries", "max_storage_buffer_binding_size", "subgroup_supported",
        "subgroup_min_size", "subgroup_max_size", "f16_supported")]


class DispatchTelemetry(C.Structure):
    _fields_ = [("kernel_id", C.c_int32), ("device", DeviceFingerprint), ("query_rows", C.c_uint32),
                ("kv_rows", C.c_uint32), ("workgroups", C.c_uint32 * 3), ("dispatch_count", C.c_uint32),
                ("temporary_allocation_count", C.c_uint32), ("temporary_allocation_bytes", C.c_uint64),
                ("has_fallback_reason", C.c_int32), ("_fallback_reason", C.c_char * 160), ("autotuner_cache", C.c_int32)]

    @property
    def kernel(self) -> str:
        return KERNEL_IDS.get(self.kernel_id, "Unknown")

    @property
    def fallback_reason(self):
        return self._fallback_reason.decode() if self.has_fallback_reason else None

    def with_autotuner_cache(self, status: int) -> "DispatchTelemetry":
        """with_autotuner_cache (src/runtime_telemetry.rs:169-176): a copy with the annotation changed."""
        out = DispatchTelemetry.from_buffer_copy(self)
        out.autotuner_cache = status
        return out


class _Manifest(C.Structure):
    _fields_ = ([(n, C.c_char_p) for n in ("commit_sha", "benchmark_id", "command", "device", "backend", "driver", "os",
                                           "arch", "precision")]
                + [(n, C.c_uint64) for n in ("batch", "q_heads", "kv_heads", "query_len", "kv_len", "head_dim")]
                + [("causal", C.c_int32), ("warmup_iterations", C.c_uint32), ("measured_iterations", C.c_uint32)]
                + [(n, C.c_uint64) for n in ("median_latency_ns", "p95_latency_ns", "tokens_per_second_milli")])


def _lib():
    from . import lib
    L = lib()
    L.flat_device_fingerprint_stable.restype = C.c_uint64
    L.flat_device_capabilities_stable.restype = C.c_uint64
    for name in ("flat_device_fingerprint_canonical_record", "flat_device_capabilities_canonical_record",
                 "flat_benchmark_manifest_canonical_json"):
        getattr(L, name).restype = C.c_int64
    return L


def _string_call(fn, record) -> str:
    from . import FlatAttentionError
    need = fn(C.byref(record), None, C.c_uint64(0))
    if need < 0:
        raise FlatAttentionError(int(-need))
    buf = C.create_string_buffer(need + 1)
    fn(C.byref(record), buf, C.c_uint64(need + 1))
    return buf.value.decode()


def fingerprint(name, backend, driver, driver_info, vendor, device) -> DeviceFingerprint:
    return DeviceFingerprint(name.encode(), backend.encode(), driver.encode(), driver_info.encode(), vendor, device)


def fingerprint_canonical_record(fp: DeviceFingerprint) -> str:
    return _string_call(_lib().flat_device_fingerprint_canonical_record, fp)


def fingerprint_stable(fp: DeviceFingerprint) -> int:
    return int(_lib().flat_device_fingerprint_stable(C.byref(fp)))


def capabilities_canonical_record(caps: DeviceCapabilities) -> str:
    return _string_call(_lib().flat_device_capabilities_canonical_record, caps)


def capabilities_stable(caps: DeviceCapabilities) -> int:
    return int(_lib().flat_device_capabilities_stable(C.byref(caps)))


def device_fingerprint(ctx) -> DeviceFingerprint:
    out = DeviceFingerprint()
    ctx.check(_lib().flat_ctx_device_fingerprint(ctx.h, C.byref(out)))
    return out


def device_capabilities(ctx) -> DeviceCapabilities:
    out = DeviceCapabilities()
    ctx.check(_lib().flat_ctx_device_capabilities(ctx.h, C.byref(out)))
    return out


def forward_runtime_telemetry(ctx, dtype, layout, shp, rot=None) -> DispatchTelemetry:
    """WgpuFlatAttention::runtime_telemetry (src/wgpu_backend.rs:370-416) for a forward call."""
    out = DispatchTelemetry()
    ctx.check(_lib().flat_forward_runtime_telemetry(ctx.h, C.c_int32(dtype), C.c_int32(layout), C.byref(shp),
                                                    C.byref(rot) if rot is not None else None, C.byref(out)))
    return out


@dataclass
class BenchmarkManifest:
    """BenchmarkManifest with BenchmarkEnvironment / BenchmarkProblem / BenchmarkResult flattened."""
    commit_sha: str
    benchmark_id: str
    command: str
    device: str
    backend: str
    driver: str
    os: str
    arch: str
    precision: str
    batch: int
    q_heads: int
    kv_heads: int
    query_len: int
    kv_len: int
    head_dim: int
    causal: bool
    warmup_iterations: int
    measured_iterations: int
    median_latency_ns: int
    p95_latency_ns: int
    tokens_per_second_milli: int

    def _raw(self) -> _Manifest:
        e = lambda s: s.encode()
        return _Manifest(e(self.commit_sha), e(self.benchmark_id), e(self.command), e(self.device), e(self.backend),
                         e(self.driver), e(self.os), e(self.arch), e(self.precision), self.batch, self.q_heads,
                         self.kv_heads, self.query_len, self.kv_len, self.head_dim, int(self.causal),
                         self.warmup_iterations, self.measured_iterations, self.median_latency_ns, self.p95_latency_ns,
                         self.tokens_per_second_milli)

    def validate(self):
        from . import FlatAttentionError
        field = C.c_char_p()
        st = _lib().flat_benchmark_manifest_validate(C.byref(self._raw()), C.byref(field))
        if st:
            raise FlatAttentionError(st, field.value.decode() if field.value else "")

    def canonical_json(self) -> str:
        return _string_call(_lib().flat_benchmark_manifest_canonical_json, self._raw())

    def result_checksum(self) -> str:
        out = C.create_string_buffer(17)
        _lib().flat_benchmark_manifest_result_checksum(C.byref(self._raw()), out)
        return out.value.decode()
