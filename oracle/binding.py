"""ctypes binding of the CPU oracle (TEST INFRASTRUCTURE, not product code).

Only tests, the smoke check and the benchmark's CPU-baseline / reference legs import this
module.  Function names follow the reference oracle they restate (see flat_oracle.cpp for the
file:line citations).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libflat_oracle.so")

HEAD_MAJOR = 0
PROJECTION = 1


class Shape(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("batch", "q_heads", "kv_heads", "query_len", "kv_len",
                                            "head_dim", "query_position_offset")]


class Config(C.Structure):
    _fields_ = [("causal", C.c_int32), ("has_softmax_scale", C.c_int32), ("softmax_scale", C.c_float)]


def make_config(causal: bool, softmax_scale=None) -> Config:
    return Config(int(bool(causal)), 0 if softmax_scale is None else 1,
                  0.0 if softmax_scale is None else float(softmax_scale))


def build(force: bool = False) -> str:
    """Compile libflat_oracle.so with the recipe in oracle/Makefile."""
    src = os.path.join(_HERE, "flat_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "libflat_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.flat_oracle_last_error.restype = C.c_char_p
    return _lib


class OracleError(Exception):
    def __init__(self, status: int):
        self.status = status
        self.detail = lib().flat_oracle_last_error().decode()
        super().__init__(f"oracle status {status}: {self.detail}")


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _u64p(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_uint64))


def _check(st: int):
    if st != 0:
        raise OracleError(st)


def _shape(batch, q_heads, kv_heads, query_len, kv_len, head_dim, offset=0) -> Shape:
    return Shape(batch, q_heads, kv_heads, query_len, kv_len, head_dim, offset)


def forward_reference(q, k, v, batch, heads, seq_len, head_dim, causal=False, softmax_scale=None):
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty(batch * heads * seq_len * head_dim, np.float32)
    lse = np.empty(batch * heads * seq_len, np.float32)
    cfg = make_config(causal, softmax_scale)
    _check(lib().flat_oracle_forward_reference(_p(q), C.c_uint64(q.size), _p(k), C.c_uint64(k.size), _p(v),
                                               C.c_uint64(v.size), C.c_uint64(batch), C.c_uint64(heads),
                                               C.c_uint64(seq_len), C.c_uint64(head_dim), C.byref(cfg),
                                               _p(out), _p(lse)))
    return out, lse


def forward_reference_grouped_asymmetric(q, k, v, shape: Shape, causal=False, softmax_scale=None):
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty(max(q.size, 1), np.float32)
    lse = np.empty(max(shape.batch * shape.q_heads * shape.query_len, 1), np.float32)
    cfg = make_config(causal, softmax_scale)
    _check(lib().flat_oracle_forward_grouped_asymmetric(_p(q), C.c_uint64(q.size), _p(k), C.c_uint64(k.size),
                                                        _p(v), C.c_uint64(v.size), C.byref(shape),
                                                        C.byref(cfg), _p(out), _p(lse)))
    return out[:q.size], lse


def forward_reference_grouped(q, k, v, batch, q_heads, kv_heads, seq_len, head_dim, causal=False,
                              softmax_scale=None):
    return forward_reference_grouped_asymmetric(
        q, k, v, _shape(batch, q_heads, kv_heads, seq_len, seq_len, head_dim), causal, softmax_scale)


def forward_reference_grouped_rope(q, k, v, batch, q_heads, kv_heads, seq_len, head_dim, theta,
                                   position_offset, causal=False, softmax_scale=None):
    q, k, v = _f32(q), _f32(k), _f32(v)
    shape = _shape(batch, q_heads, kv_heads, seq_len, seq_len, head_dim)
    out = np.empty(max(q.size, 1), np.float32)
    lse = np.empty(batch * q_heads * seq_len, np.float32)
    cfg = make_config(causal, softmax_scale)
    _check(lib().flat_oracle_forward_grouped_rope(_p(q), C.c_uint64(q.size), _p(k), C.c_uint64(k.size), _p(v),
                                                  C.c_uint64(v.size), C.byref(shape), C.byref(cfg),
                                                  C.c_float(theta), C.c_uint64(position_offset), _p(out),
                                                  _p(lse)))
    return out[:q.size], lse


def forward_reference_projection_grouped_rope_asymmetric(q, k, v, shape: Shape, theta,
                                                         query_rope_offset, kv_rope_offset,
                                                         causal=False, softmax_scale=None):
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty(max(q.size, 1), np.float32)
    lse = np.empty(max(shape.batch * shape.q_heads * shape.query_len, 1), np.float32)
    cfg = make_config(causal, softmax_scale)
    _check(lib().flat_oracle_forward_projection_rope_asymmetric(
        _p(q), C.c_uint64(q.size), _p(k), C.c_uint64(k.size), _p(v), C.c_uint64(v.size), C.byref(shape),
        C.byref(cfg), C.c_float(theta), C.c_uint64(query_rope_offset), C.c_uint64(kv_rope_offset), _p(out),
        _p(lse)))
    return out[:q.size], lse


def forward_reference_projection_grouped_rope_asymmetric_biased(q, k, v, shape: Shape, theta,
                                                                query_rope_offset, kv_rope_offset,
                                                                causal=False, softmax_scale=None, dense=None,
                                                                alibi=None):
    """src/attention_bias.rs:193-339.  `dense` is the [batch, q_heads, query_len, kv_len] bias;
    `alibi` is (slopes, query_position_offset, kv_position_offset); neither means AttentionBias::None."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty(max(q.size, 1), np.float32)
    lse = np.empty(max(shape.batch * shape.q_heads * shape.query_len, 1), np.float32)
    cfg = make_config(causal, softmax_scale)
    mode, values, q_off, kv_off = 0, np.zeros(1, np.float32), 0, 0
    n = 0
    if dense is not None:
        mode, values = 1, _f32(dense)
        n = values.size
    elif alibi is not None:
        mode, values, q_off, kv_off = 2, _f32(alibi[0]), alibi[1], alibi[2]
        n = values.size
    if values.size == 0:
        values = np.zeros(1, np.float32)
    _check(lib().flat_oracle_forward_projection_rope_asymmetric_biased(
        _p(q), C.c_uint64(q.size), _p(k), C.c_uint64(k.size), _p(v), C.c_uint64(v.size), C.byref(shape),
        C.byref(cfg), C.c_float(theta), C.c_uint64(query_rope_offset), C.c_uint64(kv_rope_offset),
        C.c_int32(mode), _p(values), C.c_uint64(n), C.c_uint64(q_off), C.c_uint64(kv_off), _p(out), _p(lse)))
    return out[:q.size], lse


def forward_reference_projection_grouped_rope(q, k, v, batch, q_heads, kv_heads, seq_len, head_dim,
                                              theta, position_offset, causal=False,
                                              softmax_scale=None):
    return forward_reference_projection_grouped_rope_asymmetric(
        q, k, v, _shape(batch, q_heads, kv_heads, seq_len, seq_len, head_dim), theta, position_offset,
        position_offset, causal, softmax_scale)


def forward_reference_variable_lengths(q, k, v, shape: Shape, active, causal=False,
                                       softmax_scale=None):
    """`active` is a list of (active_q, active_kv, query_position_offset) per batch element."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    act = np.ascontiguousarray(np.array(active, dtype=np.uint64).reshape(-1))
    out = np.empty(max(q.size, 1), np.float32)
    lse = np.empty(shape.batch * shape.q_heads * shape.query_len, np.float32)
    cfg = make_config(causal, softmax_scale)
    _check(lib().flat_oracle_forward_variable_lengths(_p(q), C.c_uint64(q.size), _p(k), C.c_uint64(k.size),
                                                      _p(v), C.c_uint64(v.size), C.byref(shape), _u64p(act),
                                                      C.c_uint64(len(active)), C.byref(cfg), _p(out),
                                                      _p(lse)))
    return out[:q.size], lse


def forward_reference_projection_grouped_rope_chunked_prefill(q, k, v, batch, q_heads, kv_heads,
                                                              seq_len, head_dim, theta,
                                                              position_offset, query_chunk_size,
                                                              causal=False, softmax_scale=None):
    q, k, v = _f32(q), _f32(k), _f32(v)
    shape = _shape(batch, q_heads, kv_heads, seq_len, seq_len, head_dim)
    out = np.empty(max(q.size, 1), np.float32)
    lse = np.empty(batch * q_heads * seq_len, np.float32)
    cfg = make_config(causal, softmax_scale)
    _check(lib().flat_oracle_chunked_prefill(_p(q), C.c_uint64(q.size), _p(k), C.c_uint64(k.size), _p(v),
                                             C.c_uint64(v.size), C.byref(shape), C.byref(cfg),
                                             C.c_float(theta), C.c_uint64(position_offset),
                                             C.c_uint64(query_chunk_size), _p(out), _p(lse)))
    return out[:q.size], lse


def backward_reference_grouped(q, k, v, d_out, fwd_out, fwd_lse, batch, q_heads, kv_heads, seq_len,
                               head_dim, causal=False, softmax_scale=None):
    q, k, v, d_out, fwd_out, fwd_lse = map(_f32, (q, k, v, d_out, fwd_out, fwd_lse))
    dq = np.empty(max(q.size, 1), np.float32)
    dk = np.empty(max(k.size, 1), np.float32)
    dv = np.empty(max(k.size, 1), np.float32)
    cfg = make_config(causal, softmax_scale)
    _check(lib().flat_oracle_backward_grouped(
        _p(q), C.c_uint64(q.size), _p(k), C.c_uint64(k.size), _p(v), C.c_uint64(v.size), _p(d_out),
        C.c_uint64(d_out.size), _p(fwd_out), C.c_uint64(fwd_out.size), _p(fwd_lse), C.c_uint64(fwd_lse.size),
        C.c_uint64(batch), C.c_uint64(q_heads), C.c_uint64(kv_heads), C.c_uint64(seq_len),
        C.c_uint64(head_dim), C.byref(cfg), _p(dq), _p(dk), _p(dv)))
    return dq[:q.size], dk[:k.size], dv[:k.size]


def backward_reference(q, k, v, d_out, fwd_out, fwd_lse, batch, heads, seq_len, head_dim,
                       causal=False, softmax_scale=None):
    return backward_reference_grouped(q, k, v, d_out, fwd_out, fwd_lse, batch, heads, heads, seq_len,
                                      head_dim, causal, softmax_scale)


def forward_rows(q, k, v, shape: Shape, layout, rows, causal=False, softmax_scale=None, threads=1):
    """Oracle on sampled (batch, q_head, query_pos) rows; no RoPE (materialise it first)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    rows = np.ascontiguousarray(np.array(rows, dtype=np.uint64).reshape(-1, 3))
    n = rows.shape[0]
    out = np.empty((n, shape.head_dim), np.float32)
    lse = np.empty(n, np.float32)
    cfg = make_config(causal, softmax_scale)
    _check(lib().flat_oracle_forward_rows(_p(q), _p(k), _p(v), C.byref(shape), C.c_int32(layout),
                                          C.byref(cfg), _u64p(rows), C.c_uint64(n), C.c_int32(threads),
                                          _p(out), _p(lse)))
    return out, lse


def forward_rows_alibi(q, k, v, shape: Shape, layout, rows, slopes, bias_q_offset=0, bias_kv_offset=0, causal=False,
                       softmax_scale=None, threads=1):
    """forward_rows with an ALiBi score bias (one slope per query head); no RoPE (materialise it first)."""
    q, k, v, slopes = _f32(q), _f32(k), _f32(v), _f32(slopes)
    assert slopes.size == shape.q_heads
    rows = np.ascontiguousarray(np.array(rows, dtype=np.uint64).reshape(-1, 3))
    n = rows.shape[0]
    out = np.empty((n, shape.head_dim), np.float32)
    lse = np.empty(n, np.float32)
    cfg = make_config(causal, softmax_scale)
    _check(lib().flat_oracle_forward_rows_alibi(_p(q), _p(k), _p(v), C.byref(shape), C.c_int32(layout), C.byref(cfg),
                                                _p(slopes), C.c_uint64(bias_q_offset), C.c_uint64(bias_kv_offset),
                                                _u64p(rows), C.c_uint64(n), C.c_int32(threads), _p(out), _p(lse)))
    return out, lse


def backward_units(q, k, v, d_out, fwd_out, fwd_lse, batch, q_heads, kv_heads, seq_len, head_dim,
                   units, causal=False, softmax_scale=None, threads=1):
    """Oracle backward for whole (batch, kv_head) units."""
    q, k, v, d_out, fwd_out, fwd_lse = map(_f32, (q, k, v, d_out, fwd_out, fwd_lse))
    units = np.ascontiguousarray(np.array(units, dtype=np.uint64).reshape(-1, 2))
    n = units.shape[0]
    group = q_heads // kv_heads
    dq = np.empty((n, group, seq_len, head_dim), np.float32)
    dk = np.empty((n, seq_len, head_dim), np.float32)
    dv = np.empty((n, seq_len, head_dim), np.float32)
    cfg = make_config(causal, softmax_scale)
    _check(lib().flat_oracle_backward_units(_p(q), _p(k), _p(v), _p(d_out), _p(fwd_out), _p(fwd_lse),
                                            C.c_uint64(batch), C.c_uint64(q_heads), C.c_uint64(kv_heads),
                                            C.c_uint64(seq_len), C.c_uint64(head_dim), C.byref(cfg),
                                            _u64p(units), C.c_uint64(n), C.c_int32(threads), _p(dq),
                                            _p(dk), _p(dv)))
    return dq, dk, dv


def backward_rows(q, k, v, d_out, fwd_out, fwd_lse, batch, q_heads, kv_heads, seq_len, head_dim, dq_rows, dkv_rows,
                  causal=False, softmax_scale=None, threads=1):
    """Oracle backward on sampled rows: dq_rows = (batch, q_head, query), dkv_rows = (batch, kv_head, key)."""
    q, k, v, d_out, fwd_out, fwd_lse = map(_f32, (q, k, v, d_out, fwd_out, fwd_lse))
    a = np.ascontiguousarray(np.array(dq_rows, dtype=np.uint64).reshape(-1, 3))
    b = np.ascontiguousarray(np.array(dkv_rows, dtype=np.uint64).reshape(-1, 3))
    dq = np.empty((max(a.shape[0], 1), head_dim), np.float32)
    dk = np.empty((max(b.shape[0], 1), head_dim), np.float32)
    dv = np.empty((max(b.shape[0], 1), head_dim), np.float32)
    cfg = make_config(causal, softmax_scale)
    _check(lib().flat_oracle_backward_rows(_p(q), _p(k), _p(v), _p(d_out), _p(fwd_out), _p(fwd_lse), C.c_uint64(batch),
                                           C.c_uint64(q_heads), C.c_uint64(kv_heads), C.c_uint64(seq_len),
                                           C.c_uint64(head_dim), C.byref(cfg), _u64p(a), C.c_uint64(a.shape[0]), _u64p(b),
                                           C.c_uint64(b.shape[0]), C.c_int32(threads), _p(dq), _p(dk), _p(dv)))
    return dq[:a.shape[0]], dk[:b.shape[0]], dv[:b.shape[0]]


def rotate_rows(src, head_dim, positions, theta):
    """Materialised RoPE of rows [row_count, head_dim] at the given absolute positions."""
    src = _f32(src)
    pos = np.ascontiguousarray(np.array(positions, dtype=np.uint64).reshape(-1))
    assert src.size == pos.size * head_dim
    dst = np.empty_like(src)
    lib().flat_oracle_rotate_rows(_p(src), _p(dst), C.c_uint64(pos.size), C.c_uint64(head_dim), _u64p(pos),
                                  C.c_float(theta))
    return dst


def rope_frequencies(theta, head_dim):
    out = np.empty(head_dim // 2, np.float32)
    lib().flat_oracle_rope_frequencies(C.c_float(theta), C.c_uint64(head_dim), _p(out))
    return out


def fixture(length, step, phase, a, c=0.0, b=0.0):
    """sin(x)*a + cos(x*c)*b with x = i*step + phase in f32 libm arithmetic."""
    out = np.empty(length, np.float32)
    lib().flat_oracle_fixture(_p(out), C.c_uint64(length), C.c_float(step), C.c_float(phase), C.c_float(a),
                              C.c_float(c), C.c_float(b))
    return out


def f16_from_f32(values) -> np.ndarray:
    """F16::from_f32 (src/f16.rs:26-82) element-wise; returns the binary16 bit patterns."""
    a = _f32(values)
    out = np.empty(a.size, np.uint16)
    lib().flat_oracle_f16_from_f32(_p(a), C.c_uint64(a.size), out.ctypes.data_as(C.POINTER(C.c_uint16)))
    return out


def f16_to_f32(bits) -> np.ndarray:
    """F16::to_f32 (src/f16.rs:85-110) element-wise."""
    a = np.ascontiguousarray(bits, dtype=np.uint16).reshape(-1)
    out = np.empty(a.size, np.float32)
    lib().flat_oracle_f16_to_f32(a.ctypes.data_as(C.POINTER(C.c_uint16)), C.c_uint64(a.size), _p(out))
    return out


def f16_round(values) -> np.ndarray:
    """Quantise to binary16 and expand again: the values a binary16 kernel consumes."""
    return f16_to_f32(f16_from_f32(values))


class PagedKvTable:
    """PagedKvTable restatement (src/paged_kv.rs:75-188)."""

    def __init__(self, page_size, physical_pages):
        h = C.c_void_p()
        _check(lib().flat_oracle_paged_table_new(C.c_uint64(page_size), C.c_uint64(physical_pages), C.byref(h)))
        self._h = h
        self.page_size, self.physical_pages = page_size, physical_pages

    def __del__(self):
        if getattr(self, "_h", None):
            lib().flat_oracle_paged_table_free(self._h)
            self._h = None

    def append(self, tokens):
        _check(lib().flat_oracle_paged_table_append(self._h, C.c_uint64(tokens)))

    def address(self, logical_token):
        out = (C.c_uint64 * 3)()
        if not lib().flat_oracle_paged_table_address(self._h, C.c_uint64(logical_token), out):
            return None
        return tuple(out)  # (physical_page, offset_in_page, generation)

    def telemetry(self):
        out = (C.c_uint64 * 6)()
        lib().flat_oracle_paged_table_telemetry(self._h, out)
        keys = ("live_tokens", "capacity_tokens", "mapped_pages", "free_pages",
                "internal_fragmentation_tokens", "generation")
        return dict(zip(keys, out))

    def reset(self):
        _check(lib().flat_oracle_paged_table_reset(self._h))
