// Passive runtime telemetry records and benchmark manifests: host-only string and integer work, no kernel.
// Canonical records and the FNV-1a-64 fingerprints follow src/runtime_telemetry.rs:49-91,116-135; the manifest
// validation and schema-1 canonical JSON follow src/benchmark_manifest.rs:90-247.
#include <cstring>
#include <string>

#include "common.h"

namespace {

// src/runtime_telemetry.rs:84-91, src/benchmark_manifest.rs:218-225
uint64_t fnv1a64(const std::string &bytes) {
    uint64_t hash = 0xcbf29ce484222325ull;
    for (unsigned char byte : bytes) {
        hash ^= byte;
        hash *= 0x100000001b3ull;
    }
    return hash;
}

// escape_component (src/runtime_telemetry.rs:70-82): '%', ';' and '=' are percent-escaped, UTF-8 passes through
std::string escape_component(const char *value) {
    std::string out;
    for (const char *p = value; *p; ++p) {
        switch (*p) {
            case '%': out += "%25"; break;
            case ';': out += "%3b"; break;
            case '=': out += "%3d"; break;
            default: out += *p;
        }
    }
    return out;
}

std::string bounded(const char *field, size_t cap) {
    size_t n = 0;
    while (n < cap && field[n]) ++n;
    return std::string(field, n);
}

std::string fingerprint_record(const flat_device_fingerprint *fp) {
    char tail[64];
    std::snprintf(tail, sizeof tail, ";vendor=%08x;device=%08x", fp->vendor, fp->device);
    return "name=" + escape_component(bounded(fp->name, sizeof fp->name).c_str()) +
           ";backend=" + escape_component(bounded(fp->backend, sizeof fp->backend).c_str()) +
           ";driver=" + escape_component(bounded(fp->driver, sizeof fp->driver).c_str()) +
           ";driver_info=" + escape_component(bounded(fp->driver_info, sizeof fp->driver_info).c_str()) + tail;
}

std::string capabilities_record(const flat_device_capabilities *c) {
    char buf[256];
    std::snprintf(buf, sizeof buf, "wgpd=%u;wgsx=%u;wgsy=%u;wgsz=%u;wgss=%u;bind=%u;sbuf=%u;sub=%u;submin=%u;submax=%u;f16=%u",
                  c->max_workgroups_per_dimension, c->max_workgroup_size_x, c->max_workgroup_size_y,
                  c->max_workgroup_size_z, c->max_workgroup_storage_bytes, c->max_binding_entries,
                  c->max_storage_buffer_binding_size, c->subgroup_supported ? 1u : 0u, c->subgroup_min_size,
                  c->subgroup_max_size, c->f16_supported ? 1u : 0u);
    return buf;
}

// snprintf convention for the string-returning entry points
int64_t emit(const std::string &s, char *buf, uint64_t cap) {
    if (buf && cap) {
        const uint64_t n = s.size() < cap - 1 ? s.size() : cap - 1;
        std::memcpy(buf, s.data(), n);
        buf[n] = 0;
    }
    return (int64_t)s.size();
}

// Rust's str::trim removes Unicode White_Space; this decodes UTF-8 and tests that property.
bool is_white_space(uint32_t c) {
    return (c >= 0x09 && c <= 0x0d) || c == 0x20 || c == 0x85 || c == 0xa0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200a) ||
           c == 0x2028 || c == 0x2029 || c == 0x202f || c == 0x205f || c == 0x3000;
}

bool blank(const char *s) {
    if (!s) return true;
    const unsigned char *p = reinterpret_cast<const unsigned char *>(s);
    while (*p) {
        uint32_t c = *p;
        int extra = 0;
        if (c >= 0xf0) { c &= 0x07; extra = 3; }
        else if (c >= 0xe0) { c &= 0x0f; extra = 2; }
        else if (c >= 0xc0) { c &= 0x1f; extra = 1; }
        ++p;
        for (int i = 0; i < extra && (*p & 0xc0) == 0x80; ++i, ++p) c = (c << 6) | (*p & 0x3f);
        if (!is_white_space(c)) return false;
    }
    return true;
}

// json_string (src/benchmark_manifest.rs:227-247)
std::string json_string(const char *value) {
    std::string out = "\"";
    for (const unsigned char *p = reinterpret_cast<const unsigned char *>(value); *p; ++p) {
        switch (*p) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            default:
                if (*p <= 0x1f) {
                    char esc[8];
                    std::snprintf(esc, sizeof esc, "\\u%04x", (unsigned)*p);
                    out += esc;
                } else {
                    out += (char)*p;
                }
        }
    }
    out += '"';
    return out;
}

// result_json (src/benchmark_manifest.rs:211-216)
std::string result_json(const flat_benchmark_manifest *m) {
    char buf[192];
    std::snprintf(buf, sizeof buf, "{\"median_latency_ns\":%llu,\"p95_latency_ns\":%llu,\"tokens_per_second_milli\":%llu}",
                  (unsigned long long)m->median_latency_ns, (unsigned long long)m->p95_latency_ns,
                  (unsigned long long)m->tokens_per_second_milli);
    return buf;
}

std::string checksum_hex(const flat_benchmark_manifest *m) {
    char buf[24];
    std::snprintf(buf, sizeof buf, "%016llx", (unsigned long long)fnv1a64(result_json(m)));
    return buf;
}

}  // namespace

extern "C" {

int64_t flat_device_fingerprint_canonical_record(const flat_device_fingerprint *fp, char *buf, uint64_t cap) {
    if (!fp) return -FLAT_ERR_NULL_POINTER;
    return emit(fingerprint_record(fp), buf, cap);
}

int64_t flat_device_capabilities_canonical_record(const flat_device_capabilities *caps, char *buf, uint64_t cap) {
    if (!caps) return -FLAT_ERR_NULL_POINTER;
    return emit(capabilities_record(caps), buf, cap);
}

uint64_t flat_device_fingerprint_stable(const flat_device_fingerprint *fp) { return fp ? fnv1a64(fingerprint_record(fp)) : 0; }
uint64_t flat_device_capabilities_stable(const flat_device_capabilities *caps) {
    return caps ? fnv1a64(capabilities_record(caps)) : 0;
}

int32_t flat_ctx_device_fingerprint(const flat_ctx *ctx, flat_device_fingerprint *out) {
    if (!ctx || !out) return FLAT_ERR_NULL_POINTER;
    *out = ctx->fingerprint;
    return FLAT_OK;
}

int32_t flat_ctx_device_capabilities(const flat_ctx *ctx, flat_device_capabilities *out) {
    if (!ctx || !out) return FLAT_ERR_NULL_POINTER;
    *out = ctx->capabilities;
    return FLAT_OK;
}

int32_t flat_benchmark_manifest_validate(const flat_benchmark_manifest *m, const char **field) {
    if (field) *field = nullptr;
    if (!m) return FLAT_ERR_NULL_POINTER;
    // exactly 40 hex digits
    size_t sha_len = m->commit_sha ? std::strlen(m->commit_sha) : 0;
    bool sha_ok = sha_len == 40;
    for (size_t i = 0; sha_ok && i < 40; ++i) {
        const char c = m->commit_sha[i];
        sha_ok = (c >= '0' && c <= '9') || (c >= 'a' && c <= 'f') || (c >= 'A' && c <= 'F');
    }
    if (!sha_ok) return FLAT_ERR_MANIFEST_INVALID_COMMIT_SHA;
    const struct { const char *name, *value; } strings[] = {
        {"benchmark_id", m->benchmark_id},        {"command", m->command},
        {"environment.device", m->device},        {"environment.backend", m->backend},
        {"environment.driver", m->driver},        {"environment.os", m->os},
        {"environment.arch", m->arch},            {"problem.precision", m->precision},
    };
    for (const auto &s : strings)
        if (blank(s.value)) {
            if (field) *field = s.name;
            return FLAT_ERR_MANIFEST_EMPTY_FIELD;
        }
    const struct { const char *name; uint64_t value; } dims[] = {
        {"batch", m->batch},         {"q_heads", m->q_heads}, {"kv_heads", m->kv_heads},
        {"query_len", m->query_len}, {"kv_len", m->kv_len},   {"head_dim", m->head_dim},
    };
    for (const auto &d : dims)
        if (d.value == 0) {
            if (field) *field = d.name;
            return FLAT_ERR_ZERO_DIMENSION;
        }
    if (m->q_heads % m->kv_heads != 0) return FLAT_ERR_INVALID_HEAD_GROUPING;
    if (m->measured_iterations == 0) return FLAT_ERR_MANIFEST_ZERO_MEASURED_ITERATIONS;
    if (m->p95_latency_ns < m->median_latency_ns) return FLAT_ERR_MANIFEST_INVALID_PERCENTILE_ORDERING;
    return FLAT_OK;
}

int64_t flat_benchmark_manifest_canonical_json(const flat_benchmark_manifest *m, char *buf, uint64_t cap) {
    const int st = flat_benchmark_manifest_validate(m, nullptr);
    if (st) return -st;
    // field order is part of schema version 1 (src/benchmark_manifest.rs:144-197)
    std::string out = "{\"schema_version\":" + std::to_string(FLAT_BENCHMARK_MANIFEST_SCHEMA_VERSION);
    out += ",\"commit_sha\":" + json_string(m->commit_sha);
    out += ",\"benchmark_id\":" + json_string(m->benchmark_id);
    out += ",\"command\":" + json_string(m->command);
    out += ",\"environment\":{\"device\":" + json_string(m->device) + ",\"backend\":" + json_string(m->backend) +
           ",\"driver\":" + json_string(m->driver) + ",\"os\":" + json_string(m->os) + ",\"arch\":" + json_string(m->arch) + "}";
    out += ",\"problem\":{\"precision\":" + json_string(m->precision) + ",\"batch\":" + std::to_string(m->batch) +
           ",\"q_heads\":" + std::to_string(m->q_heads) + ",\"kv_heads\":" + std::to_string(m->kv_heads) +
           ",\"query_len\":" + std::to_string(m->query_len) + ",\"kv_len\":" + std::to_string(m->kv_len) +
           ",\"head_dim\":" + std::to_string(m->head_dim) + ",\"causal\":" + (m->causal ? "true" : "false") + "}";
    out += ",\"protocol\":{\"warmup_iterations\":" + std::to_string(m->warmup_iterations) +
           ",\"measured_iterations\":" + std::to_string(m->measured_iterations) + "}";
    out += ",\"result\":" + result_json(m);
    out += ",\"result_checksum\":{\"algorithm\":\"fnv1a64\",\"value\":\"" + checksum_hex(m) + "\"}}";
    return emit(out, buf, cap);
}

int32_t flat_benchmark_manifest_result_checksum(const flat_benchmark_manifest *m, char out[17]) {
    if (!m || !out) return FLAT_ERR_NULL_POINTER;
    std::memcpy(out, checksum_hex(m).c_str(), 17);
    return FLAT_OK;
}

}  // extern "C"
