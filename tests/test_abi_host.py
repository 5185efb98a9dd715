"""CPU-side checks of the C ABI library: it loads, exports every symbol the header declares, and
its host-only logic (PagedKvTable, layouts, no-device behaviour) matches the reference contract.
No compute call is made."""
import ctypes as C

import pytest

from __graft_entry__ import load_package

fa = load_package()


def test_library_exports_every_declared_symbol():
    lib = fa.lib()
    names = fa.exported_symbols_in_header()
    assert len(names) >= 50
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_status_strings():
    lib = fa.lib()
    assert lib.flat_status_str(0) == b"ok"
    for code in fa.STATUS:
        assert lib.flat_status_str(code) != b"unknown status", code


def test_no_device_means_unavailable_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = C.c_void_p()
    assert fa.lib().flat_ctx_create(C.c_int32(0), None, C.byref(h)) == 23
    with pytest.raises(fa.FlatAttentionError) as e:
        fa.Context(0)
    assert e.value.kind == "Unavailable"


# ---- PagedKvTable through the C ABI: src/paged_kv.rs:200-270 ----------------------------------
def test_mapping_is_stable_across_page_boundaries():
    t = fa.PagedKvTable(4, 3)
    t.append(9)
    assert t.address(0)[0] == 0
    assert t.address(3)[1] == 3
    assert t.address(4)[0] == 1
    assert t.address(8)[0] == 2
    assert t.address(9) is None
    assert t.export() == [0, 1, 2]


def test_telemetry_reports_exact_internal_fragmentation():
    t = fa.PagedKvTable(8, 4)
    t.append(9)
    assert t.telemetry() == dict(live_tokens=9, capacity_tokens=32, mapped_pages=2, free_pages=2,
                                 internal_fragmentation_tokens=7, generation=0)


def test_reset_invalidates_old_generation_before_page_reuse():
    t = fa.PagedKvTable(2, 2)
    t.append(1)
    old = t.address(0)
    t.reset()
    assert t.address(0) is None
    t.append(1)
    new = t.address(0)
    assert old[0] == new[0] and old[2] != new[2]
    assert t.generation() == 1


def test_capacity_overflow_is_explicit_and_non_mutating():
    t = fa.PagedKvTable(4, 2)
    t.append(7)
    before = t.telemetry()
    with pytest.raises(fa.FlatAttentionError) as e:
        t.append(2)
    assert e.value.kind == "CapacityExceeded"
    assert t.telemetry() == before
    with pytest.raises(fa.FlatAttentionError) as e:
        fa.PagedKvTable(0, 2)
    assert e.value.kind == "ZeroDimension"
    with pytest.raises(fa.FlatAttentionError) as e:
        fa.PagedKvTable(2**40, 2**40)
    assert e.value.kind == "CapacityOverflow"
    empty = fa.PagedKvTable(2, 2)
    with pytest.raises(fa.FlatAttentionError) as e:
        empty.export()
    assert e.value.kind == "EmptyTable"


def test_table_matches_oracle_table_on_random_walk():
    from oracle import binding as ob
    import random
    rnd = random.Random(7)
    a, b = fa.PagedKvTable(5, 9), ob.PagedKvTable(5, 9)
    for _ in range(200):
        if rnd.random() < 0.1:
            a.reset(), b.reset()
        n = rnd.randrange(0, 9)
        ea = eb = None
        try:
            a.append(n)
        except fa.FlatAttentionError as e:
            ea = e.status
        try:
            b.append(n)
        except ob.OracleError as e:
            eb = e.status
        assert ea == eb
        assert a.telemetry() == b.telemetry()
        for tok in range(0, 46):
            assert a.address(tok) == b.address(tok)


# ---- layouts (pure functions): src/wgpu_forward_grouped.rs:306-334, wgpu_backward_grouped.rs:181-215
def test_forward_layout():
    L = fa.forward_layout(fa.F32, fa.shape(2, 8, 2, 17, 17, 64))
    assert L.q_elements == 2 * 8 * 17 * 64 and L.kv_elements == 2 * 2 * 17 * 64 and L.lse_elements == 2 * 8 * 17
    assert L.lse_byte_offset == 4 * L.q_elements and L.combined_bytes == 4 * (L.q_elements + L.lse_elements)
    L = fa.forward_layout(fa.BF16, fa.shape(1, 4, 2, 3, 7, 16))
    assert L.q_bytes == 2 * 4 * 3 * 16 and L.lse_byte_offset == L.q_bytes and L.kv_elements == 2 * 7 * 16
    for bad, kind in ((fa.shape(0, 1, 1, 1, 1, 2), "ZeroDimension"), (fa.shape(1, 6, 4, 1, 1, 2), "InvalidHeadGrouping"),
                      (fa.shape(1, 1, 1, 1, 1, 256), "UnsupportedHeadDim"),
                      (fa.shape(2**40, 2**30, 1, 1, 1, 2), "ShapeOverflow"),
                      (fa.shape(1, 1, 1, 4, 4, 2, 2**64 - 2), "PositionOverflow")):
        with pytest.raises(fa.FlatAttentionError) as e:
            fa.forward_layout(fa.F32, bad)
        assert e.value.kind == kind, (e.value.kind, kind)


def test_backward_layout_matches_reference_packing():
    s = fa.shape(2, 8, 2, 5, 5, 16)
    L = fa.backward_layout(fa.F32, s)
    q, kv, lse = 2 * 8 * 5 * 16, 2 * 2 * 5 * 16, 2 * 8 * 5
    assert (L.q_offset, L.k_offset, L.v_offset, L.d_out_offset, L.out_offset, L.lse_offset) == (
        0, 4 * q, 4 * (q + kv), 4 * (q + 2 * kv), 4 * (2 * q + 2 * kv), 4 * (3 * q + 2 * kv))
    assert L.input_bytes == 4 * (3 * q + 2 * kv + lse)
    assert (L.dq_offset, L.dk_offset, L.dv_offset, L.output_bytes) == (0, 4 * q, 4 * (q + kv), 4 * (q + 2 * kv))


def test_cpp_host_mirror_compiles_and_runs(tmp_path):
    """The header-only C++ mirror (flat-attention_b200/host/flat_attention.hpp) builds against the C ABI
    with plain g++ and its host-only logic gives the reference's known answers."""
    import os
    import subprocess
    import torch
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "host_mirror_check")
    libdir = os.path.join(root, "flat-attention_b200")
    subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", os.path.join(root, "tests", "host_mirror_check.cpp"), "-o", exe,
                    "-L" + libdir, "-lflat_attention_b200", "-Wl,-rpath," + libdir], check=True, capture_output=True, timeout=300)
    env = dict(os.environ)
    if not torch.cuda.is_available():
        env["FLAT_EXPECT_NO_DEVICE"] = "1"
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0 and "host mirror ok" in r.stdout, r.stdout + r.stderr
