"""Host-API fuzz in the spirit of tests/m39_host_api_fuzz.rs:54-188: 4096 xorshift cases of hostile
shapes through the pure C-ABI functions; nothing may crash, every outcome is a typed status, and the
status agrees with an independent big-integer model of the validation rules (src/api.rs:36-59)."""
import ctypes as C

from __graft_entry__ import load_package

fa = load_package()
U64 = (1 << 64) - 1


class XorShift:
    def __init__(self, seed):
        self.s = seed

    def next(self):
        x = self.s
        x ^= (x << 13) & U64
        x ^= x >> 7
        x ^= (x << 17) & U64
        self.s = x
        return x


def hostile(rng):
    r = rng.next() % 10
    if r == 0:
        return 0
    if r == 1:
        return U64
    if r == 2:
        return (1 << 32) + rng.next() % 5
    if r == 3:
        return (1 << 63) + rng.next() % 3
    if r == 4:
        return (1 << 31) - 1 + rng.next() % 3
    if r == 5:
        return 1 + rng.next() % 5000
    return 1 + rng.next() % 130


def model(b, hq, hkv, nq, nkv, d, off):
    """Expected status of flat_forward_layout_for."""
    if 0 in (b, hq, hkv, nq, nkv, d):
        return "ZeroDimension"
    if hq % hkv:
        return "InvalidHeadGrouping"
    lse = b * hq * nq
    if lse > U64 or lse * d > U64 or b * hkv * nkv * d > U64:
        return "ShapeOverflow"
    if off + nq - 1 > U64:
        return "PositionOverflow"
    if d > 128:
        return "UnsupportedHeadDim"
    lim = (1 << 31) - 1
    if b > lim or hq > lim or nq > lim or nkv > lim or off + nq - 1 > lim or lse * d > 1 << 46 or b * hkv * nkv * d > 1 << 46:
        return "IndexSpaceExceeded"
    return "OK"


def test_layout_functions_never_crash_and_match_the_model():
    rng = XorShift(0x39F0_5EED_1234_ABCD)
    lib = fa.lib()
    seen = set()
    for _ in range(4096):
        dims = [hostile(rng) for _ in range(6)]
        off = hostile(rng) if rng.next() % 4 == 0 else rng.next() % 1000
        shp = fa.Shape(*dims, off)
        out = fa.ForwardLayout()
        st = lib.flat_forward_layout_for(C.c_int32(rng.next() % 2), C.byref(shp), C.byref(out))
        kind = fa.STATUS.get(st)
        assert kind is not None, st
        assert kind == model(*dims, off), (dims, off, kind)
        seen.add(kind)
        bl = fa.BackwardLayout()
        st2 = lib.flat_backward_layout_for(C.c_int32(rng.next() % 2), C.byref(shp), C.byref(bl))
        assert st2 in fa.STATUS
        if st == 0:
            es = 4
            assert out.q_elements == dims[0] * dims[1] * dims[3] * dims[5]
            assert out.kv_elements == dims[0] * dims[2] * dims[4] * dims[5]
            assert out.combined_bytes >= out.lse_byte_offset + 4 * out.lse_elements
    assert {"OK", "ZeroDimension", "InvalidHeadGrouping", "ShapeOverflow"} <= seen
    assert lib.flat_forward_layout_for(C.c_int32(0), C.byref(fa.shape(1, 2, 1, 3, 3, 130)), C.byref(fa.ForwardLayout())) == 20
    assert lib.flat_forward_layout_for(C.c_int32(7), C.byref(fa.shape(1, 1, 1, 1, 1, 2)), C.byref(fa.ForwardLayout())) == 26
    assert lib.flat_forward_layout_for(C.c_int32(0), None, C.byref(fa.ForwardLayout())) == 27


def test_decode_layout_fuzz_matches_the_model():
    """flat_decode_layout_for (the *DecodePipeline::layout functions, src/wgpu_paged_decode.rs:268-283): hostile
    geometry gives a typed status that agrees with a big-integer model; valid geometry gives the packed offsets."""
    rng = XorShift(0x0DEC_0DE5_EED5_1234)
    lib = fa.lib()
    seen = set()
    for _ in range(2048):
        batch, hq, d = hostile(rng), hostile(rng), hostile(rng)
        dtype = rng.next() % 2
        out = fa.DecodeLayout()
        st = lib.flat_decode_layout_for(C.c_int32(dtype), C.c_uint64(batch), C.c_uint64(hq), C.c_uint64(d), C.byref(out))
        kind = fa.STATUS.get(st)
        if 0 in (batch, hq, d):
            want = "ZeroDimension"
        elif d % 2:
            want = "InvalidRotaryHeadDim"
        elif d > 128:
            want = "UnsupportedHeadDim"
        elif batch * hq > U64 or batch * hq * d > U64 or batch * hq * (d + 1) > U64 or batch * hq * d > 1 << 46:
            want = "ShapeOverflow"
        else:
            want = "OK"
        assert kind == want, (batch, hq, d, kind, want)
        seen.add(kind)
        if st == 0:
            es = 4 if dtype == 0 else 2
            assert out.q_elements == out.output_elements == batch * hq * d and out.lse_elements == batch * hq
            assert out.combined_elements == batch * hq * (d + 1) and out.q_bytes == batch * hq * d * es
            assert out.lse_byte_offset == (out.q_bytes + 3) // 4 * 4 and out.combined_bytes == out.lse_byte_offset + 4 * batch * hq
    assert {"OK", "ZeroDimension", "ShapeOverflow", "UnsupportedHeadDim", "InvalidRotaryHeadDim"} <= seen
    assert lib.flat_decode_layout_for(C.c_int32(2), C.c_uint64(1), C.c_uint64(1), C.c_uint64(2), C.byref(fa.DecodeLayout())) == 26
    assert lib.flat_decode_layout_for(C.c_int32(0), C.c_uint64(1), C.c_uint64(1), C.c_uint64(2), None) == 27
    L = fa.decode_layout(fa.BF16, 64, 32, 128)  # the paged-decode benchmark shape
    assert (L.q_bytes, L.lse_byte_offset, L.combined_bytes) == (64 * 32 * 128 * 2, 64 * 32 * 128 * 2, 64 * 32 * 128 * 2 + 64 * 32 * 4)


def test_paged_table_fuzz_never_crashes():
    rng = XorShift(0x1357_9BDF_2468_ACE0)
    lib = fa.lib()
    for _ in range(512):
        ps, pages = hostile(rng), hostile(rng)
        h = C.c_void_p()
        st = lib.flat_paged_kv_table_create(C.c_uint64(ps), C.c_uint64(pages), C.byref(h))
        assert st in fa.STATUS
        if pages > 1 << 28:
            assert st in (1, 40)   # ZeroDimension (page_size 0) or CapacityOverflow: refused, never allocated
        if st:
            continue
        for _ in range(8):
            st = lib.flat_paged_kv_table_append(h, C.c_uint64(hostile(rng)))
            assert st in fa.STATUS
            addr = fa.PagedKvAddress()
            st = lib.flat_paged_kv_table_address(h, C.c_uint64(hostile(rng)), C.byref(addr))
            assert st in (0, 34)
            tel = fa.PagedKvTelemetry()
            assert lib.flat_paged_kv_table_telemetry(h, C.byref(tel)) == 0
            assert tel.live_tokens <= tel.capacity_tokens and tel.mapped_pages + tel.free_pages == pages
        lib.flat_paged_kv_table_destroy(h)


def test_null_context_is_an_error_not_a_crash():
    lib = fa.lib()
    z = fa.Buffer(None, 0)
    shp, cfg = fa.shape(1, 1, 1, 1, 1, 2), fa.config()
    assert lib.flat_forward_grouped(None, C.c_int32(0), C.byref(shp), C.byref(cfg), z, z, z, z) == 27
    assert lib.flat_backward_grouped(None, C.c_int32(0), C.byref(shp), C.byref(cfg), z, z) == 27
    assert lib.flat_synchronize(None) == 27
    assert lib.flat_forward_host(None, C.c_int32(0), C.c_int32(0), C.byref(shp), C.byref(cfg), None, None, C.c_uint64(0), None,
                                 C.c_uint64(0), None, C.c_uint64(0), C.c_int32(1), None, C.c_uint64(0)) == 27
    assert lib.flat_forward_projection_rope_asymmetric_alibi(None, C.c_int32(1), C.byref(shp), C.byref(cfg), None, None,
                                                             C.c_uint64(0), C.c_uint64(0), C.c_uint64(0), z, z, z, z) == 27
    assert lib.flat_forward_runtime_telemetry(None, C.c_int32(1), C.c_int32(0), C.byref(shp), None, None) == 27
    assert lib.flat_preferred_forward_host(None, C.byref(shp), C.byref(cfg), None, C.c_uint64(0), None, C.c_uint64(0), None,
                                           C.c_uint64(0), None, C.c_uint64(0), None) == 27
    assert lib.flat_numerical_forward_host(None, C.c_int32(1), C.byref(shp), C.byref(cfg), None, C.c_uint64(0), None,
                                           C.c_uint64(0), None, C.c_uint64(0), None, C.c_uint64(0)) == 27
    assert lib.flat_decode_paged_batched_static_scratch(
        None, C.c_int32(1), C.c_uint64(1 << 62), C.c_uint64(1 << 62), C.c_uint64(1 << 62), C.c_uint64(64), C.c_uint64(16),
        C.c_uint64(1), C.c_uint64(1), None, None, None, None, None, C.byref(cfg), C.c_float(1e4), C.c_uint32(0), z, z, z, z) == 27
    assert lib.flat_splitkv_merge_nccl(None, None, C.c_int32(0), C.c_int32(1), C.c_int32(1), C.c_uint64(1), C.c_uint64(2), z, z) == 27
    assert lib.flat_splitkv_decode_nccl(None, None, C.c_int32(0), C.c_int32(1), C.c_int32(1), C.c_uint64(1), C.c_uint64(1),
                                        C.c_uint64(1), C.c_uint64(2), C.c_uint64(16), C.c_uint64(1), C.c_uint64(1), None, None, None,
                                        None, None, C.byref(cfg), C.c_float(1e4), z, z, z, z, z) == 27
    assert lib.flat_splitkv_exchange_create(None, C.c_int32(0), C.c_int32(2), C.c_uint64(64), C.c_uint64(128), None) == 27
    assert lib.flat_splitkv_exchange_handle(None, None) == 27 and lib.flat_splitkv_exchange_connect(None, None, C.c_uint64(0)) == 27
    lib.flat_splitkv_exchange_destroy(None)
    assert lib.flat_splitkv_decode_peer(None, None, C.c_int32(1), C.c_uint64(1), C.c_uint64(1), C.c_uint64(1), C.c_uint64(2),
                                        C.c_uint64(16), C.c_uint64(1), C.c_uint64(1), None, None, None, None, None,
                                        C.byref(cfg), C.c_float(1e4), z, z, z, z) == 27
    assert lib.flat_forward_prepare(None, C.c_int32(1), C.c_int32(0), C.byref(shp), C.byref(cfg), None, z, z, z, z, None) == 27
    assert lib.flat_forward_encode_prepared(None, None) == 27 and lib.flat_backward_encode_prepared(None, None) == 27
    assert lib.flat_backward_prepare(None, C.c_int32(1), C.byref(shp), C.byref(cfg), z, z, None) == 27
    assert lib.flat_ctx_reserve_rope_tables(None, C.c_uint64(1), C.c_uint64(2)) == 27
    lib.flat_prepared_forward_destroy(None)
    lib.flat_prepared_backward_destroy(None)
    assert lib.flat_ctx_device_fingerprint(None, None) == 27 and lib.flat_ctx_device_capabilities(None, None) == 27
    assert lib.flat_benchmark_manifest_validate(None, None) == 27
    lib.flat_benchmark_manifest_canonical_json.restype = C.c_int64
    assert lib.flat_benchmark_manifest_canonical_json(None, None, C.c_uint64(0)) == -27
    lib.flat_device_fingerprint_canonical_record.restype = C.c_int64
    assert lib.flat_device_fingerprint_canonical_record(None, None, C.c_uint64(0)) == -27


def test_manifest_and_record_fuzz_matches_the_restatement():
    """Random byte soup (valid UTF-8, control characters, delimiters, quotes) through the canonical-record and
    canonical-JSON writers: library and restatement agree byte for byte, small buffers truncate without overrun."""
    import dataclasses
    import importlib
    from oracle import telemetry_oracle as to
    tel = importlib.import_module("flat_attention_b200.telemetry")
    rng = XorShift(0x9E3779B97F4A7C15)
    alphabet = ['"', "\\", "\n", "\r", "\t", "\x01", "\x1f", ";", "=", "%", " ", "a", "Z", "é", "漢", "😀", " ", "\xa0", "7"]

    def text(max_len):
        return "".join(alphabet[rng.next() % len(alphabet)] for _ in range(rng.next() % max_len))

    for _ in range(300):
        name, backend, driver, info = text(40), text(12), text(20), text(30)
        vendor, device = rng.next() & 0xffffffff, rng.next() & 0xffffffff
        fp = tel.fingerprint(name, backend, driver, info, vendor, device)
        # the struct fields are NUL-terminated fixed arrays: the restatement sees the same truncation
        cut = lambda s, cap: s.encode()[:cap].decode(errors="ignore") if len(s.encode()) >= cap else s
        if any(len(s.encode()) >= cap for s, cap in ((name, 256), (backend, 32), (driver, 64), (info, 128))):
            continue
        expect = to.fingerprint_record(name, backend, driver, info, vendor, device)
        assert tel.fingerprint_canonical_record(fp) == expect
        assert tel.fingerprint_stable(fp) == to.fnv1a64(expect.encode())
        m = tel.BenchmarkManifest(
            commit_sha="%040x" % (rng.next() << 64 | rng.next()), benchmark_id="b" + text(10), command="c" + text(60),
            device="d" + text(20), backend="x" + text(5), driver="r" + text(9), os="o" + text(4), arch="a" + text(4),
            precision="p" + text(4), batch=1 + rng.next() % 9, q_heads=8, kv_heads=1 + rng.next() % 2 * 3, query_len=1 + rng.next() % 99,
            kv_len=1 + rng.next() % 99, head_dim=64, causal=bool(rng.next() & 1), warmup_iterations=rng.next() % 9,
            measured_iterations=rng.next() % 5, median_latency_ns=rng.next() >> 20, p95_latency_ns=rng.next() >> 20,
            tokens_per_second_milli=rng.next())
        want = to.validate(dataclasses.asdict(m))
        if want is None:
            assert m.canonical_json() == to.canonical_json(dataclasses.asdict(m))
        else:
            try:
                m.canonical_json()
                raise AssertionError("expected " + want[0])
            except fa.FlatAttentionError as e:
                assert e.kind.replace("Manifest", "") == want[0]
    # snprintf convention: a short buffer receives a NUL-terminated prefix and the call still reports the full length
    fp = tel.fingerprint("abc", "Cuda", "d", "i", 1, 2)
    lib = fa.lib()
    buf = C.create_string_buffer(b"\xff" * 16, 16)
    full = lib.flat_device_fingerprint_canonical_record(C.byref(fp), buf, C.c_uint64(8))
    assert full == len(to.fingerprint_record("abc", "Cuda", "d", "i", 1, 2)) and buf.raw[:8] == b"name=ab\x00" and buf.raw[8:] == b"\xff" * 8
