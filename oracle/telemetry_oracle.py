"""CPU restatement (TEST INFRASTRUCTURE, not product code) of the reference's deterministic
host-side records: canonical telemetry records with their FNV-1a-64 fingerprints
(src/runtime_telemetry.rs:49-91, 116-135) and the schema-1 benchmark manifest
(src/benchmark_manifest.rs:90-247).  Pure string and integer work, so plain Python.

Pinned by the literals of the reference's own unit tests (escaped record fragment, escaped JSON
fragment, validation outcomes) and by the published FNV-1a-64 test vectors, see
tests/test_telemetry_manifest.py."""

MASK = (1 << 64) - 1


def fnv1a64(data: bytes) -> int:
    # src/runtime_telemetry.rs:84-91
    h = 0xcbf29ce484222325
    for b in data:
        h ^= b
        h = (h * 0x100000001b3) & MASK
    return h


def escape_component(value: str) -> str:
    # src/runtime_telemetry.rs:70-82
    return "".join({"%": "%25", ";": "%3b", "=": "%3d"}.get(ch, ch) for ch in value)


def fingerprint_record(name, backend, driver, driver_info, vendor, device) -> str:
    # src/runtime_telemetry.rs:49-59
    return "name=%s;backend=%s;driver=%s;driver_info=%s;vendor=%08x;device=%08x" % (
        escape_component(name), escape_component(backend), escape_component(driver), escape_component(driver_info),
        vendor, device)


CAP_KEYS = ("wgpd", "wgsx", "wgsy", "wgsz", "wgss", "bind", "sbuf", "sub", "submin", "submax", "f16")


def capabilities_record(values) -> str:
    # src/runtime_telemetry.rs:116-131; `values` in struct order, booleans as 0/1
    return ";".join("%s=%d" % (k, int(v)) for k, v in zip(CAP_KEYS, values))


def json_string(value: str) -> str:
    # src/benchmark_manifest.rs:227-247
    out = ['"']
    for ch in value:
        if ch == '"':
            out.append('\\"')
        elif ch == "\\":
            out.append("\\\\")
        elif ch == "\n":
            out.append("\\n")
        elif ch == "\r":
            out.append("\\r")
        elif ch == "\t":
            out.append("\\t")
        elif ord(ch) <= 0x1f:
            out.append("\\u%04x" % ord(ch))
        else:
            out.append(ch)
    out.append('"')
    return "".join(out)


def result_json(m) -> str:
    # src/benchmark_manifest.rs:211-216
    return '{"median_latency_ns":%d,"p95_latency_ns":%d,"tokens_per_second_milli":%d}' % (
        m["median_latency_ns"], m["p95_latency_ns"], m["tokens_per_second_milli"])


def result_checksum(m) -> str:
    return "%016x" % fnv1a64(result_json(m).encode())


# Unicode White_Space, the set Rust's str::trim removes (Python's str.strip also removes U+001C..U+001F)
WHITE_SPACE = set([*range(0x09, 0x0e), 0x20, 0x85, 0xa0, 0x1680, *range(0x2000, 0x200b), 0x2028, 0x2029, 0x202f, 0x205f,
                   0x3000])


def validate(m):
    """Returns None or (error name, field) in the order of src/benchmark_manifest.rs:90-137."""
    sha = m["commit_sha"]
    if len(sha.encode()) != 40 or any(c not in "0123456789abcdefABCDEF" for c in sha):
        return ("InvalidCommitSha", None)
    for name, key in (("benchmark_id", "benchmark_id"), ("command", "command"), ("environment.device", "device"),
                      ("environment.backend", "backend"), ("environment.driver", "driver"), ("environment.os", "os"),
                      ("environment.arch", "arch"), ("problem.precision", "precision")):
        if all(ord(ch) in WHITE_SPACE for ch in m[key]):
            return ("EmptyField", name)
    for name in ("batch", "q_heads", "kv_heads", "query_len", "kv_len", "head_dim"):
        if m[name] == 0:
            return ("ZeroDimension", name)
    if m["q_heads"] % m["kv_heads"] != 0:
        return ("InvalidHeadGrouping", None)
    if m["measured_iterations"] == 0:
        return ("ZeroMeasuredIterations", None)
    if m["p95_latency_ns"] < m["median_latency_ns"]:
        return ("InvalidPercentileOrdering", None)
    return None


def canonical_json(m) -> str:
    # src/benchmark_manifest.rs:140-199
    assert validate(m) is None
    return ('{"schema_version":1,"commit_sha":%s,"benchmark_id":%s,"command":%s,'
            '"environment":{"device":%s,"backend":%s,"driver":%s,"os":%s,"arch":%s},'
            '"problem":{"precision":%s,"batch":%d,"q_heads":%d,"kv_heads":%d,"query_len":%d,"kv_len":%d,"head_dim":%d,"causal":%s},'
            '"protocol":{"warmup_iterations":%d,"measured_iterations":%d},'
            '"result":%s,"result_checksum":{"algorithm":"fnv1a64","value":"%s"}}') % (
        json_string(m["commit_sha"]), json_string(m["benchmark_id"]), json_string(m["command"]),
        json_string(m["device"]), json_string(m["backend"]), json_string(m["driver"]), json_string(m["os"]),
        json_string(m["arch"]), json_string(m["precision"]), m["batch"], m["q_heads"], m["kv_heads"], m["query_len"],
        m["kv_len"], m["head_dim"], "true" if m["causal"] else "false", m["warmup_iterations"],
        m["measured_iterations"], result_json(m), result_checksum(m))
