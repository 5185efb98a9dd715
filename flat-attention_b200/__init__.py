"""Host-side mirror of FLAT-ATTENTION's backend interface over the sm_100a C ABI.

The product is the shared library (`libflat_attention_b200.so`, C ABI in
`include/flat_attention_b200.h`).  This module binds it with ctypes and mirrors the reference's
struct families so tests read like the reference's own: owning executors (`CudaFlatAttention`,
`CudaGroupedAttention`, `CudaRotaryGroupedAttention`), caller-owned pipelines
(`CudaGroupedForwardPipeline`, `CudaExternal*Pipeline`, `Cuda*DecodePipeline`,
`CudaGroupedBackwardRecomputePipeline`, `CudaChunkedProjectionPrefillPipeline`), the KV caches and
`PagedKvTable`.  torch is used only for device memory and streams.  There is no CPU fallback: if the
library or a B200 is missing, construction raises.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libflat_attention_b200.so")
HEADER_PATH = os.path.join(HERE, "..", "include", "flat_attention_b200.h")

F32 = 0
BF16 = 1
F16 = 2  # IEEE binary16 storage: forward entry points only
HEAD_MAJOR = 0
PROJECTION = 1

STATUS = {
    0: "OK", 1: "ZeroDimension", 2: "ShapeOverflow", 3: "InvalidHeadGrouping", 4: "InvalidRotaryHeadDim",
    5: "InvalidRotaryTheta", 6: "PositionOverflow", 7: "LengthMismatch", 8: "InvalidScale", 9: "NonFiniteInput",
    20: "UnsupportedHeadDim", 21: "IndexSpaceExceeded", 22: "BufferTooSmall", 23: "Unavailable", 24: "Execution",
    25: "DispatchLimit", 26: "UnsupportedDtype", 27: "NullPointer", 28: "MisalignedBuffer", 29: "UnsupportedShape",
    30: "EmptyCache", 31: "InvalidCacheLength", 32: "InvalidQueryLen", 33: "CausalVisibilityMismatch",
    34: "EmptyTable", 35: "PageOutOfRange", 36: "PageShared", 37: "InvalidTheta", 40: "CapacityOverflow",
    41: "CapacityExceeded", 42: "GenerationOverflow", 50: "ZeroQueryChunkSize", 60: "DeviceWaitTimeout",
    70: "ManifestInvalidCommitSha", 71: "ManifestEmptyField", 72: "ManifestZeroMeasuredIterations",
    73: "ManifestInvalidPercentileOrdering",
}


class FlatAttentionError(Exception):
    """Typed error: `.status` is the flat_status code, `.kind` its variant name."""

    def __init__(self, status: int, detail: str = ""):
        self.status = status
        self.kind = STATUS.get(status, "Unknown")
        self.detail = detail
        super().__init__(f"{self.kind} ({status}): {detail}")


class Shape(C.Structure):
    """api::v1::AttentionShape (src/api.rs:24-33)."""
    _fields_ = [(n, C.c_uint64) for n in ("batch", "q_heads", "kv_heads", "query_len", "kv_len", "head_dim",
                                            "query_position_offset")]


def shape(batch, q_heads, kv_heads, query_len, kv_len=None, head_dim=0, query_position_offset=0) -> Shape:
    return Shape(batch, q_heads, kv_heads, query_len, query_len if kv_len is None else kv_len, head_dim,
                 query_position_offset)


class Config(C.Structure):
    """FlatAttentionConfig (src/lib.rs:248-269)."""
    _fields_ = [("causal", C.c_int32), ("has_softmax_scale", C.c_int32), ("softmax_scale", C.c_float)]


def config(causal: bool = False, softmax_scale: Optional[float] = None) -> Config:
    return Config(int(bool(causal)), 0 if softmax_scale is None else 1,
                  0.0 if softmax_scale is None else float(softmax_scale))


class Rotary(C.Structure):
    """AsymmetricRotaryEmbeddingConfig + rotate_k (src/projection_asymmetric.rs:18-23)."""
    _fields_ = [("theta", C.c_float), ("rotate_k", C.c_int32), ("query_position_offset", C.c_uint64),
                ("kv_position_offset", C.c_uint64)]


def rotary(theta: float, query_position_offset: int = 0, kv_position_offset: Optional[int] = None,
           rotate_k: bool = True) -> Rotary:
    return Rotary(float(theta), int(bool(rotate_k)), query_position_offset,
                  query_position_offset if kv_position_offset is None else kv_position_offset)


class Buffer(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("bytes", C.c_uint64)]


class ForwardLayout(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("q_elements", "kv_elements", "lse_elements", "q_bytes", "kv_bytes",
                                            "lse_byte_offset", "combined_bytes")]


class DecodeLayout(C.Structure):
    """ResidentDecodeLayout / PagedDecodeLayout (src/wgpu_decode.rs:437-455, src/wgpu_paged_decode.rs:221-235)."""
    _fields_ = [(n, C.c_uint64) for n in ("q_elements", "output_elements", "lse_elements", "combined_elements", "q_bytes",
                                            "lse_byte_offset", "combined_bytes")]


class VarlenSequence(C.Structure):
    """VariableLengthSequenceMetadata (src/wgpu_external_variable.rs:21-33)."""
    _fields_ = [(n, C.c_uint32) for n in ("active_query_len", "active_kv_len", "causal_query_offset",
                                            "query_rope_offset")]


class PagedKvTelemetry(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("live_tokens", "capacity_tokens", "mapped_pages", "free_pages",
                                            "internal_fragmentation_tokens", "generation")]


class PagedKvAddress(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("physical_page", "offset_in_page", "generation")]


class BackwardLayout(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("q_elements", "kv_elements", "lse_elements", "q_offset", "k_offset",
                                            "v_offset", "d_out_offset", "out_offset", "lse_offset", "input_bytes",
                                            "dq_offset", "dk_offset", "dv_offset", "output_bytes")]


_lib = None


def lib() -> C.CDLL:
    """Loads the CUDA library; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FlatAttentionError(23, f"{LIB_PATH} is missing: run `python flat-attention_b200/build.py`")
        _lib = C.CDLL(LIB_PATH)
        _lib.flat_status_str.restype = C.c_char_p
        _lib.flat_last_error_detail.restype = C.c_char_p
        _lib.flat_last_error_detail.argtypes = [C.c_void_p]
        for name in ("flat_ctx_workspace_bytes", "flat_ctx_launch_count", "flat_paged_kv_table_len",
                     "flat_paged_kv_table_generation", "flat_paged_kv_cache_len", "flat_paged_kv_cache_generation",
                     "flat_resident_kv_cache_len", "flat_resident_kv_cache_capacity"):
            getattr(_lib, name).restype = C.c_uint64
            getattr(_lib, name).argtypes = [C.c_void_p]
        for name in ("flat_paged_kv_cache_k_buffer", "flat_paged_kv_cache_v_buffer", "flat_resident_kv_cache_k_buffer",
                     "flat_resident_kv_cache_v_buffer"):
            getattr(_lib, name).restype = Buffer
            getattr(_lib, name).argtypes = [C.c_void_p]
        _lib.flat_paged_kv_cache_table.restype = C.c_void_p
        _lib.flat_paged_kv_cache_table.argtypes = [C.c_void_p]
        for name in ("flat_ctx_destroy", "flat_paged_kv_table_destroy", "flat_paged_kv_cache_destroy",
                     "flat_resident_kv_cache_destroy", "flat_resident_kv_cache_reset", "flat_prepared_forward_destroy",
                     "flat_prepared_backward_destroy", "flat_splitkv_exchange_destroy"):
            getattr(_lib, name).restype = None
            getattr(_lib, name).argtypes = [C.c_void_p]
    return _lib


def _torch():
    import torch
    return torch


def buf(t) -> Buffer:
    """A torch CUDA tensor viewed as a flat_buffer (pointer + size in bytes)."""
    if t is None:
        return Buffer(None, 0)
    return Buffer(t.data_ptr(), t.numel() * t.element_size())


def _dtype_of(t) -> int:
    torch = _torch()
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype == torch.float16:
        return F16
    raise FlatAttentionError(26, f"unsupported tensor dtype {t.dtype}")


def torch_dtype(dtype: int):
    torch = _torch()
    return {BF16: torch.bfloat16, F16: torch.float16}.get(dtype, torch.float32)


def forward_layout(dtype: int, shp: Shape) -> ForwardLayout:
    out = ForwardLayout()
    st = lib().flat_forward_layout_for(C.c_int32(dtype), C.byref(shp), C.byref(out))
    if st:
        raise FlatAttentionError(st, lib().flat_status_str(st).decode())
    return out


def decode_layout(dtype: int, batch: int, q_heads: int, head_dim: int) -> DecodeLayout:
    """*DecodePipeline::layout: offsets of the packed decode output [O | LSE] for `batch` decoded rows."""
    out = DecodeLayout()
    st = lib().flat_decode_layout_for(C.c_int32(dtype), C.c_uint64(batch), C.c_uint64(q_heads), C.c_uint64(head_dim),
                                      C.byref(out))
    if st:
        raise FlatAttentionError(st, lib().flat_status_str(st).decode())
    return out


def backward_layout(dtype: int, shp: Shape) -> BackwardLayout:
    out = BackwardLayout()
    st = lib().flat_backward_layout_for(C.c_int32(dtype), C.byref(shp), C.byref(out))
    if st:
        raise FlatAttentionError(st, lib().flat_status_str(st).decode())
    return out


class Context:
    """One device + stream (the wgpu device/queue pair of the reference executors)."""

    def __init__(self, device: int = 0, stream=None):
        torch = _torch()
        if not torch.cuda.is_available():
            raise FlatAttentionError(23, "no CUDA device: this backend has no CPU fallback")
        self.device = device
        torch.cuda.set_device(device)
        self._stream = stream if stream is not None else torch.cuda.current_stream(device)
        h = C.c_void_p()
        st = lib().flat_ctx_create(C.c_int32(device), C.c_void_p(self._stream.cuda_stream), C.byref(h))
        if st:
            raise FlatAttentionError(st, lib().flat_status_str(st).decode())
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            lib().flat_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, st: int):
        if st:
            raise FlatAttentionError(st, lib().flat_last_error_detail(self.h).decode())

    def set_stream(self, stream):
        self._stream = stream
        self.check(lib().flat_ctx_set_stream(self.h, C.c_void_p(stream.cuda_stream)))

    @property
    def stream(self):
        return self._stream

    def synchronize(self):
        self.check(lib().flat_synchronize(self.h))

    def launch_count(self) -> int:
        return int(lib().flat_ctx_launch_count(self.h))

    def workspace_bytes(self) -> int:
        return int(lib().flat_ctx_workspace_bytes(self.h))

    def reserve_workspace(self, nbytes: int):
        self.check(lib().flat_ctx_reserve_workspace(self.h, C.c_uint64(nbytes)))

    def set_backward_scratch_budget(self, nbytes: int):
        """Bytes the bf16 backward may use to keep its dS tiles (O(N^2)) instead of recomputing the scores for dQ; 0 = never."""
        self.check(lib().flat_ctx_set_backward_scratch_budget(self.h, C.c_uint64(nbytes)))

    def reserve_rope_tables(self, rows: int, head_dim: int):
        """Pre-size the cached (cos, sin) tables so RoPE calls with moving positions never allocate."""
        self.check(lib().flat_ctx_reserve_rope_tables(self.h, C.c_uint64(rows), C.c_uint64(head_dim)))

    def prepare_forward(self, dtype, layout, shp, cfg, rot, q, k, v, out) -> "PreparedForward":
        """*Pipeline::prepare (src/wgpu_forward_grouped.rs:352-493): validate once, then `encode()` only enqueues."""
        return PreparedForward(self, dtype, layout, shp, cfg, rot, q, k, v, out)

    def prepare_backward(self, dtype, shp, cfg, packed_inputs, packed_grads) -> "PreparedBackward":
        """WgpuGroupedBackwardRecomputePipeline::prepare (src/wgpu_backward_grouped.rs:231-300)."""
        return PreparedBackward(self, dtype, shp, cfg, packed_inputs, packed_grads)

    def set_kernel_timing(self, enabled: bool):
        self.check(lib().flat_ctx_set_kernel_timing(self.h, C.c_int32(int(enabled))))

    def take_kernel_time(self):
        """(summed milliseconds, launches) of the dominant kernels timed since the last call."""
        ms, n = C.c_double(), C.c_uint64()
        self.check(lib().flat_ctx_take_kernel_time(self.h, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def device_status(self) -> int:
        return int(lib().flat_ctx_device_status(self.h))

    # ---- allocation helpers (create_output_buffer of the reference pipelines) ----
    def empty_bytes(self, nbytes: int):
        torch = _torch()
        return torch.empty(int(nbytes), dtype=torch.uint8, device=f"cuda:{self.device}")

    def create_output_buffer(self, dtype: int, shp: Shape):
        return self.empty_bytes(forward_layout(dtype, shp).combined_bytes)

    def create_decode_output_buffer(self, dtype: int, batch: int, q_heads: int, head_dim: int):
        """*DecodePipeline::create_output_buffer (src/wgpu_paged_decode.rs:285-298)."""
        return self.empty_bytes(decode_layout(dtype, batch, q_heads, head_dim).combined_bytes)

    def split_decode_output(self, out_and_lse, dtype: int, batch: int, q_heads: int, head_dim: int):
        """Views of a packed decode output: (O [batch, q_heads, head_dim], LSE [batch, q_heads] f32)."""
        L = decode_layout(dtype, batch, q_heads, head_dim)
        raw = out_and_lse.view(_torch().uint8).reshape(-1)
        o = raw[:L.q_bytes].view(torch_dtype(dtype)).view(batch, q_heads, head_dim)
        lse = raw[L.lse_byte_offset:L.lse_byte_offset + 4 * L.lse_elements].view(_torch().float32).view(batch, q_heads)
        return o, lse

    def split_output(self, out_and_lse, dtype: int, shp: Shape, layout: int = HEAD_MAJOR):
        """Views of the packed [O | LSE] buffer: (O in its layout, LSE [B, Hq, Nq] f32)."""
        L = forward_layout(dtype, shp)
        raw = out_and_lse.view(_torch().uint8).reshape(-1)
        o = raw[:L.q_bytes].view(torch_dtype(dtype))
        lse = raw[L.lse_byte_offset:L.lse_byte_offset + 4 * L.lse_elements].view(_torch().float32)
        B, Hq, Nq, D = shp.batch, shp.q_heads, shp.query_len, shp.head_dim
        o = o.view(B, Hq, Nq, D) if layout == HEAD_MAJOR else o.view(B * Nq, Hq * D)
        return o, lse.view(B, Hq, Nq)

    # ---- raw entry points ----
    def _fwd(self, name, dtype, shp, cfg, rot, q, k, v, out):
        fn = getattr(lib(), name)
        if rot is None:
            self.check(fn(self.h, C.c_int32(dtype), C.byref(shp), C.byref(cfg), buf(q), buf(k), buf(v), buf(out)))
        else:
            self.check(fn(self.h, C.c_int32(dtype), C.byref(shp), C.byref(cfg), C.byref(rot), buf(q), buf(k), buf(v),
                          buf(out)))

    def forward_mha(self, dtype, shp, cfg, q, k, v, out):
        self._fwd("flat_forward_mha", dtype, shp, cfg, None, q, k, v, out)

    def forward_grouped(self, dtype, shp, cfg, q, k, v, out):
        self._fwd("flat_forward_grouped", dtype, shp, cfg, None, q, k, v, out)

    def forward_grouped_asymmetric(self, dtype, shp, cfg, q, k, v, out):
        self._fwd("flat_forward_grouped_asymmetric", dtype, shp, cfg, None, q, k, v, out)

    def forward_grouped_rope(self, dtype, shp, cfg, rot, q, k, v, out):
        self._fwd("flat_forward_grouped_rope", dtype, shp, cfg, rot, q, k, v, out)

    def forward_projection_rope(self, dtype, shp, cfg, rot, q, k, v, out):
        self._fwd("flat_forward_projection_rope", dtype, shp, cfg, rot, q, k, v, out)

    def forward_projection_rope_asymmetric(self, dtype, shp, cfg, rot, q, k, v, out):
        self._fwd("flat_forward_projection_rope_asymmetric", dtype, shp, cfg, rot, q, k, v, out)

    def forward_projection_rope_asymmetric_alibi(self, dtype, shp, cfg, rot, slopes, bias_query_offset,
                                                 bias_kv_offset, q, k, v, out):
        """encode_alibi / encode_pre_rotated_k_alibi (src/wgpu_external_asymmetric.rs:245-282); `slopes` is a
        host sequence of one f32 per query head, rot.rotate_k selects raw or pre-rotated K."""
        arr = (C.c_float * max(len(slopes), 1))(*[float(x) for x in slopes])
        self.check(lib().flat_forward_projection_rope_asymmetric_alibi(
            self.h, C.c_int32(dtype), C.byref(shp), C.byref(cfg), C.byref(rot), arr, C.c_uint64(len(slopes)),
            C.c_uint64(bias_query_offset), C.c_uint64(bias_kv_offset), buf(q), buf(k), buf(v), buf(out)))

    def forward_projection_rope_varlen(self, dtype, shp, cfg, rot, sequences: Sequence[VarlenSequence], q, k, v, out):
        arr = (VarlenSequence * max(len(sequences), 1))(*sequences)
        self.check(lib().flat_forward_projection_rope_varlen(self.h, C.c_int32(dtype), C.byref(shp), C.byref(cfg),
                                                             C.byref(rot), arr, C.c_uint64(len(sequences)), buf(q),
                                                             buf(k), buf(v), buf(out)))

    def forward_host(self, dtype, layout, shp, cfg, rot, q, k, v, out, check_finite=True):
        """Host tensors in (torch CPU, ideally pinned), host packed [O | LSE] out; blocks.  Like the reference's
        `forward`, the call rejects non-finite Q/K/V (validate_input, src/lib.rs:428-447); the scan runs on the
        device as the chunks land.  check_finite=False skips it."""
        self.check(lib().flat_forward_host(self.h, C.c_int32(dtype), C.c_int32(layout), C.byref(shp), C.byref(cfg),
                                           C.byref(rot) if rot is not None else None, C.c_void_p(q.data_ptr()),
                                           C.c_uint64(q.numel()), C.c_void_p(k.data_ptr()), C.c_uint64(k.numel()),
                                           C.c_void_p(v.data_ptr()), C.c_uint64(v.numel()), C.c_int32(int(check_finite)),
                                           C.c_void_p(out.data_ptr()), C.c_uint64(out.numel() * out.element_size())))

    def decode_resident(self, dtype, batch, q_heads, kv_heads, head_dim, kv_len, kv_capacity, cfg, theta,
                        q_rope_position, q, k, v, out):
        self.check(lib().flat_decode_resident(self.h, C.c_int32(dtype), C.c_uint64(batch), C.c_uint64(q_heads),
                                              C.c_uint64(kv_heads), C.c_uint64(head_dim), C.c_uint64(kv_len),
                                              C.c_uint64(kv_capacity), C.byref(cfg), C.c_float(theta),
                                              C.c_uint64(q_rope_position), buf(q), _b(k), _b(v), buf(out)))

    def decode_paged(self, dtype, table: "PagedKvTable", q_heads, kv_heads, head_dim, cfg, theta, q_rope_position,
                     q, k, v, out):
        self.check(lib().flat_decode_paged(self.h, C.c_int32(dtype), table.h, C.c_uint64(q_heads), C.c_uint64(kv_heads),
                                           C.c_uint64(head_dim), C.byref(cfg), C.c_float(theta),
                                           C.c_uint64(q_rope_position), buf(q), _b(k), _b(v), buf(out)))

    def decode_paged_batched(self, dtype, num_seqs, q_heads, kv_heads, head_dim, page_size, physical_pages,
                             max_pages_per_seq, page_tables_dev, context_lens_dev, q_rope_positions_dev,
                             host_page_tables, host_context_lens, host_q_rope_positions, cfg, theta, q, k, v, out,
                             kv_splits: int = 0):
        def ip(a):
            return None if a is None else a.ctypes.data_as(C.POINTER(C.c_int32))
        self.check(lib().flat_decode_paged_batched(
            self.h, C.c_int32(dtype), C.c_uint64(num_seqs), C.c_uint64(q_heads), C.c_uint64(kv_heads),
            C.c_uint64(head_dim), C.c_uint64(page_size), C.c_uint64(physical_pages), C.c_uint64(max_pages_per_seq),
            C.c_void_p(page_tables_dev.data_ptr()), C.c_void_p(context_lens_dev.data_ptr()),
            C.c_void_p(q_rope_positions_dev.data_ptr()), ip(host_page_tables), ip(host_context_lens),
            ip(host_q_rope_positions), C.byref(cfg), C.c_float(theta), C.c_uint32(kv_splits), buf(q), _b(k), _b(v),
            buf(out)))

    def decode_paged_batched_static_scratch(self, dtype, num_seqs, q_heads, kv_heads, head_dim, page_size,
                                            physical_pages, max_pages_per_seq, page_tables_dev, context_lens_dev,
                                            q_rope_positions_dev, host_context_lens, host_q_rope_positions, cfg, theta,
                                            q, k, v, out, kv_splits: int = 0):
        """Split-KV paged decode whose partials live in the library's fixed 8 MiB device array: the
        call allocates nothing (for callers that cannot call cudaMalloc at that point)."""
        def ip(a):
            return None if a is None else a.ctypes.data_as(C.POINTER(C.c_int32))
        self.check(lib().flat_decode_paged_batched_static_scratch(
            self.h, C.c_int32(dtype), C.c_uint64(num_seqs), C.c_uint64(q_heads), C.c_uint64(kv_heads),
            C.c_uint64(head_dim), C.c_uint64(page_size), C.c_uint64(physical_pages), C.c_uint64(max_pages_per_seq),
            C.c_void_p(page_tables_dev.data_ptr()), C.c_void_p(context_lens_dev.data_ptr()),
            C.c_void_p(q_rope_positions_dev.data_ptr()), ip(host_context_lens), ip(host_q_rope_positions),
            C.byref(cfg), C.c_float(theta), C.c_uint32(kv_splits), buf(q), _b(k), _b(v), buf(out)))

    def decode_paged_batched_partial(self, dtype, num_seqs, q_heads, kv_heads, head_dim, page_size, physical_pages,
                                     max_pages_per_seq, page_tables_dev, context_lens_dev, q_rope_positions_dev,
                                     host_page_tables, host_context_lens, cfg, theta, q, k, v, out):
        """Per-GPU leg of KV-split decode: f32 [O | LSE] of this cache slice."""
        def ip(a):
            return None if a is None else a.ctypes.data_as(C.POINTER(C.c_int32))
        self.check(lib().flat_decode_paged_batched_partial(
            self.h, C.c_int32(dtype), C.c_uint64(num_seqs), C.c_uint64(q_heads), C.c_uint64(kv_heads),
            C.c_uint64(head_dim), C.c_uint64(page_size), C.c_uint64(physical_pages), C.c_uint64(max_pages_per_seq),
            C.c_void_p(page_tables_dev.data_ptr()), C.c_void_p(context_lens_dev.data_ptr()),
            C.c_void_p(q_rope_positions_dev.data_ptr()), ip(host_page_tables), ip(host_context_lens), C.byref(cfg),
            C.c_float(theta), buf(q), _b(k), _b(v), buf(out)))

    def splitkv_decode_nccl(self, comm_ptr: int, rank: int, world: int, dtype, num_seqs, q_heads, kv_heads, head_dim,
                            page_size, physical_pages, max_pages_per_seq, page_tables_dev, context_lens_dev,
                            q_rope_positions_dev, host_page_tables, host_context_lens, cfg, theta, q, k, v, gathered, out):
        """One KV-split decode step over an NCCL communicator (`comm_ptr` = the ncclComm_t as an integer): partial of
        this rank's slice into its block of `gathered`, in-place all-gather, local merge.  Enqueues only."""
        def ip(a):
            return None if a is None else a.ctypes.data_as(C.POINTER(C.c_int32))
        self.check(lib().flat_splitkv_decode_nccl(
            self.h, C.c_void_p(comm_ptr), C.c_int32(rank), C.c_int32(world), C.c_int32(dtype), C.c_uint64(num_seqs),
            C.c_uint64(q_heads), C.c_uint64(kv_heads), C.c_uint64(head_dim), C.c_uint64(page_size), C.c_uint64(physical_pages),
            C.c_uint64(max_pages_per_seq), C.c_void_p(page_tables_dev.data_ptr()), C.c_void_p(context_lens_dev.data_ptr()),
            C.c_void_p(q_rope_positions_dev.data_ptr()), ip(host_page_tables), ip(host_context_lens), C.byref(cfg),
            C.c_float(theta), buf(q), _b(k), _b(v), buf(gathered), buf(out)))

    def splitkv_decode_peer(self, exchange: "SplitKvPeerExchange", dtype, num_seqs, q_heads, kv_heads, head_dim, page_size,
                            physical_pages, max_pages_per_seq, page_tables_dev, context_lens_dev, q_rope_positions_dev,
                            host_page_tables, host_context_lens, cfg, theta, q, k, v, out):
        """One KV-split decode step over NVLink peer memory: partial of this rank's slice, then one kernel that
        stores it into every rank's buffer, waits for theirs and merges.  Enqueues only; every rank must call."""
        def ip(a):
            return None if a is None else a.ctypes.data_as(C.POINTER(C.c_int32))
        self.check(lib().flat_splitkv_decode_peer(
            self.h, exchange.h, C.c_int32(dtype), C.c_uint64(num_seqs), C.c_uint64(q_heads), C.c_uint64(kv_heads),
            C.c_uint64(head_dim), C.c_uint64(page_size), C.c_uint64(physical_pages), C.c_uint64(max_pages_per_seq),
            C.c_void_p(page_tables_dev.data_ptr()), C.c_void_p(context_lens_dev.data_ptr()),
            C.c_void_p(q_rope_positions_dev.data_ptr()), ip(host_page_tables), ip(host_context_lens), C.byref(cfg),
            C.c_float(theta), buf(q), _b(k), _b(v), buf(out)))

    def splitkv_merge_nccl(self, comm_ptr: int, rank: int, world: int, dtype, rows, head_dim, gathered, out):
        self.check(lib().flat_splitkv_merge_nccl(self.h, C.c_void_p(comm_ptr), C.c_int32(rank), C.c_int32(world),
                                                 C.c_int32(dtype), C.c_uint64(rows), C.c_uint64(head_dim), buf(gathered),
                                                 buf(out)))

    def splitkv_merge_packed(self, dtype, parts, rows, head_dim, gathered, out):
        self.check(lib().flat_splitkv_merge_packed(self.h, C.c_int32(dtype), C.c_uint64(parts), C.c_uint64(rows),
                                                   C.c_uint64(head_dim), buf(gathered), buf(out)))

    def splitkv_merge(self, dtype, parts, rows, head_dim, partial_o, partial_lse, out):
        self.check(lib().flat_splitkv_merge(self.h, C.c_int32(dtype), C.c_uint64(parts), C.c_uint64(rows),
                                            C.c_uint64(head_dim), buf(partial_o), buf(partial_lse), buf(out)))

    def chunked_prefill(self, dtype, shp, cfg, rot, query_chunk_size, q, k, v, out):
        self.check(lib().flat_chunked_prefill(self.h, C.c_int32(dtype), C.byref(shp), C.byref(cfg), C.byref(rot),
                                              C.c_uint64(query_chunk_size), buf(q), buf(k), buf(v), buf(out)))

    def chunked_prefill_paged(self, cache: "CudaPagedKvCache", q_heads, chunk_len, cfg, theta, position_offset,
                              q_chunk, k_chunk, v_chunk, out):
        self.check(lib().flat_chunked_prefill_paged(self.h, cache.h, C.c_uint64(q_heads), C.c_uint64(chunk_len),
                                                    C.byref(cfg), C.c_float(theta), C.c_uint64(position_offset),
                                                    buf(q_chunk), buf(k_chunk), buf(v_chunk), buf(out)))

    def backward_grouped(self, dtype, shp, cfg, packed_inputs, packed_grads):
        self.check(lib().flat_backward_grouped(self.h, C.c_int32(dtype), C.byref(shp), C.byref(cfg),
                                               buf(packed_inputs), buf(packed_grads)))

    def backward_mha(self, dtype, shp, cfg, packed_inputs, packed_grads):
        self.check(lib().flat_backward_mha(self.h, C.c_int32(dtype), C.byref(shp), C.byref(cfg), buf(packed_inputs),
                                           buf(packed_grads)))


class SplitKvPeerExchange:
    """The peer-memory exchange object of KV-split decode (flat_splitkv_exchange_*): one device allocation per rank
    that the other ranks of the box map through CUDA IPC.  `handle()` is what a rank gives the others;
    `connect(all_handles)` maps theirs (see `distributed.connect_peer_exchange`)."""

    def __init__(self, ctx: "Context", rank: int, world: int, rows: int, head_dim: int):
        self.ctx = ctx
        h = C.c_void_p()
        ctx.check(lib().flat_splitkv_exchange_create(ctx.h, C.c_int32(rank), C.c_int32(world), C.c_uint64(rows),
                                                     C.c_uint64(head_dim), C.byref(h)))
        self.h, self.world = h, world

    def handle(self) -> bytes:
        out = (C.c_uint8 * 64)()
        self.ctx.check(lib().flat_splitkv_exchange_handle(self.h, out))
        return bytes(out)

    def connect(self, handles: bytes):
        arr = (C.c_uint8 * len(handles)).from_buffer_copy(handles)
        self.ctx.check(lib().flat_splitkv_exchange_connect(self.h, arr, C.c_uint64(len(handles))))

    def close(self):
        if getattr(self, "h", None):
            lib().flat_splitkv_exchange_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown: the module's globals may be gone already
            pass


class PreparedForward:
    """PreparedGroupedForward (src/wgpu_forward_grouped.rs:54-91): a validated forward pass; keeps the tensors alive."""

    def __init__(self, ctx: Context, dtype, layout, shp, cfg, rot, q, k, v, out):
        self.ctx, self._keep = ctx, (q, k, v, out)
        h = C.c_void_p()
        ctx.check(lib().flat_forward_prepare(ctx.h, C.c_int32(dtype), C.c_int32(layout), C.byref(shp), C.byref(cfg),
                                             C.byref(rot) if rot is not None else None, buf(q), buf(k), buf(v), buf(out),
                                             C.byref(h)))
        self.h = h

    def encode(self):
        self.ctx.check(lib().flat_forward_encode_prepared(self.ctx.h, self.h))

    def __del__(self):
        if getattr(self, "h", None):
            try:
                lib().flat_prepared_forward_destroy(self.h)
            except Exception:  # interpreter shutdown: the module's globals may be gone already
                pass
            self.h = None


class PreparedBackward:
    """PreparedGroupedBackwardRecompute (src/wgpu_backward_grouped.rs:124-129)."""

    def __init__(self, ctx: Context, dtype, shp, cfg, packed_inputs, packed_grads):
        self.ctx, self._keep = ctx, (packed_inputs, packed_grads)
        h = C.c_void_p()
        ctx.check(lib().flat_backward_prepare(ctx.h, C.c_int32(dtype), C.byref(shp), C.byref(cfg), buf(packed_inputs),
                                              buf(packed_grads), C.byref(h)))
        self.h = h

    def encode(self):
        self.ctx.check(lib().flat_backward_encode_prepared(self.ctx.h, self.h))

    def __del__(self):
        if getattr(self, "h", None):
            try:
                lib().flat_prepared_backward_destroy(self.h)
            except Exception:  # interpreter shutdown: the module's globals may be gone already
                pass
            self.h = None


def _b(x) -> Buffer:
    return x if isinstance(x, Buffer) else buf(x)


# ---- PagedKvTable (src/paged_kv.rs:75-188) -----------------------------------------------------
class PagedKvTable:
    def __init__(self, page_size: int, physical_pages: int, _borrowed=None):
        self._owned = _borrowed is None
        if _borrowed is not None:
            self.h = C.c_void_p(_borrowed)
            return
        h = C.c_void_p()
        st = lib().flat_paged_kv_table_create(C.c_uint64(page_size), C.c_uint64(physical_pages), C.byref(h))
        if st:
            raise FlatAttentionError(st, lib().flat_status_str(st).decode())
        self.h = h

    def __del__(self):
        if getattr(self, "_owned", False) and getattr(self, "h", None):
            try:
                lib().flat_paged_kv_table_destroy(self.h)
            except Exception:  # interpreter shutdown: the module's globals may be gone already
                pass
            self.h = None

    def append(self, tokens: int):
        st = lib().flat_paged_kv_table_append(self.h, C.c_uint64(tokens))
        if st:
            raise FlatAttentionError(st, lib().flat_status_str(st).decode())

    def address(self, logical_token: int):
        out = PagedKvAddress()
        st = lib().flat_paged_kv_table_address(self.h, C.c_uint64(logical_token), C.byref(out))
        return None if st else (out.physical_page, out.offset_in_page, out.generation)

    def telemetry(self) -> dict:
        out = PagedKvTelemetry()
        lib().flat_paged_kv_table_telemetry(self.h, C.byref(out))
        return {n: getattr(out, n) for n, _ in PagedKvTelemetry._fields_}

    def reset(self):
        st = lib().flat_paged_kv_table_reset(self.h)
        if st:
            raise FlatAttentionError(st, lib().flat_status_str(st).decode())

    def __len__(self):
        return int(lib().flat_paged_kv_table_len(self.h))

    def generation(self) -> int:
        return int(lib().flat_paged_kv_table_generation(self.h))

    def export(self):
        """WgpuPagedKvTable::from_table: the flattened logical -> physical u32 entries."""
        n = C.c_uint64()
        st = lib().flat_paged_kv_table_export(self.h, None, C.c_uint64(0), C.byref(n))
        if st:
            raise FlatAttentionError(st, lib().flat_status_str(st).decode())
        arr = (C.c_uint32 * n.value)()
        st = lib().flat_paged_kv_table_export(self.h, arr, n, C.byref(n))
        if st:
            raise FlatAttentionError(st, lib().flat_status_str(st).decode())
        return list(arr)


class CudaPagedKvCache:
    """WgpuPagedKvCache (src/wgpu_paged_kv_cache.rs:76-279)."""

    def __init__(self, ctx: Context, dtype: int, page_size: int, physical_pages: int, kv_heads: int, head_dim: int):
        self.ctx, self.dtype = ctx, dtype
        self.page_size, self.physical_pages, self.kv_heads, self.head_dim = page_size, physical_pages, kv_heads, head_dim
        h = C.c_void_p()
        ctx.check(lib().flat_paged_kv_cache_create(ctx.h, C.c_int32(dtype), C.c_uint64(page_size),
                                                   C.c_uint64(physical_pages), C.c_uint64(kv_heads),
                                                   C.c_uint64(head_dim), C.byref(h)))
        self.h = h

    def __del__(self):
        if getattr(self, "h", None) and getattr(self.ctx, "h", None):
            try:
                lib().flat_paged_kv_cache_destroy(self.h)
            except Exception:  # interpreter shutdown: the module's globals may be gone already
                pass
            self.h = None

    def record_append(self, k_source, v_source, append_len: int) -> int:
        n = C.c_uint64()
        self.ctx.check(lib().flat_paged_kv_cache_append(self.h, buf(k_source), buf(v_source), C.c_uint64(append_len),
                                                        C.byref(n)))
        return n.value

    def record_append_rotating(self, k_source, v_source, append_len: int, theta: float, kv_position_offset: int = 0) -> int:
        n = C.c_uint64()
        self.ctx.check(lib().flat_paged_kv_cache_append_rotating(self.h, buf(k_source), buf(v_source),
                                                                 C.c_uint64(append_len), C.c_float(theta),
                                                                 C.c_uint64(kv_position_offset), C.byref(n)))
        return n.value

    def enable_prefill_shadow(self):
        """Keep a binary16 copy of K for the tensor-core chunked prefill (bf16 caches; one more K-sized allocation)."""
        self.ctx.check(lib().flat_paged_kv_cache_enable_prefill_shadow(self.h))

    def reset(self):
        self.ctx.check(lib().flat_paged_kv_cache_reset(self.h))

    def __len__(self):
        return int(lib().flat_paged_kv_cache_len(self.h))

    def is_empty(self):
        return len(self) == 0

    def generation(self):
        return int(lib().flat_paged_kv_cache_generation(self.h))

    def k_buffer(self) -> Buffer:
        return lib().flat_paged_kv_cache_k_buffer(self.h)

    def v_buffer(self) -> Buffer:
        return lib().flat_paged_kv_cache_v_buffer(self.h)

    def table(self) -> PagedKvTable:
        return PagedKvTable(0, 0, _borrowed=lib().flat_paged_kv_cache_table(self.h))

    def download(self):
        """Host copies of K and V as [physical_pages*page_size, kv_heads*head_dim] (test helper)."""
        torch = _torch()
        outs = []
        for b in (self.k_buffer(), self.v_buffer()):
            t = torch.empty(b.bytes, dtype=torch.uint8)
            self.ctx.check(lib().flat_download(self.ctx.h, C.c_void_p(t.data_ptr()), b, C.c_uint64(b.bytes)))
            outs.append(t.view(torch_dtype(self.dtype)).view(self.physical_pages * self.page_size,
                                                             self.kv_heads * self.head_dim))
        return outs


class CudaResidentKvCache:
    """WgpuResidentKvCache (src/wgpu_kv_cache.rs:79-262)."""

    def __init__(self, ctx: Context, dtype: int, batch: int, kv_heads: int, capacity: int, head_dim: int):
        self.ctx, self.dtype = ctx, dtype
        self.batch, self.kv_heads, self.capacity, self.head_dim = batch, kv_heads, capacity, head_dim
        h = C.c_void_p()
        ctx.check(lib().flat_resident_kv_cache_create(ctx.h, C.c_int32(dtype), C.c_uint64(batch), C.c_uint64(kv_heads),
                                                      C.c_uint64(capacity), C.c_uint64(head_dim), C.byref(h)))
        self.h = h

    def __del__(self):
        if getattr(self, "h", None) and getattr(self.ctx, "h", None):
            try:
                lib().flat_resident_kv_cache_destroy(self.h)
            except Exception:  # interpreter shutdown: the module's globals may be gone already
                pass
            self.h = None

    def record_append(self, k_source, v_source, append_len: int) -> int:
        n = C.c_uint64()
        self.ctx.check(lib().flat_resident_kv_cache_append(self.h, buf(k_source), buf(v_source), C.c_uint64(append_len),
                                                           C.byref(n)))
        return n.value

    def reset(self):
        lib().flat_resident_kv_cache_reset(self.h)

    def __len__(self):
        return int(lib().flat_resident_kv_cache_len(self.h))

    def remaining_capacity(self):
        return self.capacity - len(self)

    def k_buffer(self) -> Buffer:
        return lib().flat_resident_kv_cache_k_buffer(self.h)

    def v_buffer(self) -> Buffer:
        return lib().flat_resident_kv_cache_v_buffer(self.h)

    def download(self):
        torch = _torch()
        outs = []
        for b in (self.k_buffer(), self.v_buffer()):
            t = torch.empty(b.bytes, dtype=torch.uint8)
            self.ctx.check(lib().flat_download(self.ctx.h, C.c_void_p(t.data_ptr()), b, C.c_uint64(b.bytes)))
            outs.append(t.view(torch_dtype(self.dtype)).view(self.batch, self.capacity, self.kv_heads * self.head_dim))
        return outs


# ---- owning executors (host slices in, host results out) ----------------------------------------
@dataclass
class FlatAttentionOutput:
    """FlatAttentionOutput (src/lib.rs:354-360): `output` in Q's layout, `lse` [B, Hq, Nq] f32."""
    output: "object"
    lse: "object"


class CudaFlatAttention:
    """WgpuFlatAttention / WgpuGroupedAttention / WgpuRotaryGroupedAttention
    (src/wgpu_backend.rs:170-608, src/wgpu_grouped_backend.rs:126-146,
    src/wgpu_rotary_grouped_backend.rs:117-293): owns its context; `forward` takes host tensors,
    uploads, launches and downloads; `upload` / `forward_resident` / `download_attention` split
    those steps."""

    def __init__(self, device: int = 0, dtype: int = F32):
        self.ctx = Context(device)
        self.dtype = dtype

    def upload(self, host):
        torch = _torch()
        t = torch.as_tensor(host)
        if t.dtype != torch_dtype(self.dtype):
            t = t.to(torch_dtype(self.dtype))
        return t.contiguous().to(f"cuda:{self.ctx.device}", non_blocking=True)

    def forward_resident(self, q, k, v, shp: Shape, cfg: Config, rot: Optional[Rotary] = None,
                         layout: int = HEAD_MAJOR, out=None):
        if out is None:
            out = self.ctx.create_output_buffer(self.dtype, shp)
        if layout == HEAD_MAJOR:
            if rot is None:
                self.ctx.forward_grouped_asymmetric(self.dtype, shp, cfg, q, k, v, out)
            else:
                self.ctx.forward_grouped_rope(self.dtype, shp, cfg, rot, q, k, v, out)
        else:
            self.ctx.forward_projection_rope_asymmetric(self.dtype, shp, cfg, rot, q, k, v, out)
        return out

    def download_attention(self, out, shp: Shape, layout: int = HEAD_MAJOR) -> FlatAttentionOutput:
        o, lse = self.ctx.split_output(out, self.dtype, shp, layout)
        return FlatAttentionOutput(o.cpu(), lse.cpu())

    def forward(self, q, k, v, shp: Shape, cfg: Config, rot: Optional[Rotary] = None,
                layout: int = HEAD_MAJOR) -> FlatAttentionOutput:
        """Host slices in, host result out, inputs validated like the reference's validate_input."""
        torch = _torch()
        td = torch_dtype(self.dtype)
        hq, hk, hv = (torch.as_tensor(x).to(td).contiguous().reshape(-1) for x in (q, k, v))
        L = forward_layout(self.dtype, shp)
        out = torch.empty(L.combined_bytes, dtype=torch.uint8)
        self.ctx.forward_host(self.dtype, layout, shp, cfg, rot, hq, hk, hv, out, check_finite=True)
        o = out[:L.q_bytes].view(td)
        lse = out[L.lse_byte_offset:L.lse_byte_offset + 4 * L.lse_elements].view(torch.float32)
        B, Hq, Nq, D = shp.batch, shp.q_heads, shp.query_len, shp.head_dim
        o = o.view(B, Hq, Nq, D) if layout == HEAD_MAJOR else o.view(B * Nq, Hq * D)
        return FlatAttentionOutput(o, lse.view(B, Hq, Nq))


IO_F32, IO_PACKED_F16 = 0, 1
EXACT_REFERENCE, FAST_PORTABLE, DETERMINISTIC_PORTABLE = 0, 1, 2


class NumericalGuarantees(C.Structure):
    """NumericalGuarantees (src/numerical.rs:56-66); policies are the integer codes of the C header."""
    _fields_ = [(n, C.c_int32) for n in ("accumulation", "reduction", "softmax_update", "repeatable_same_backend_device",
                                           "allows_subgroup")]


def numerical_mode_guarantees(mode: int) -> NumericalGuarantees:
    out = NumericalGuarantees()
    st = lib().flat_numerical_mode_guarantees(C.c_int32(mode), C.byref(out))
    if st:
        raise FlatAttentionError(st, "unknown numerical mode")
    return out


def _host_f32_call(ctx, fn, shp, cfg, q, k, v, pre=(), post=()):
    torch = _torch()
    hq, hk, hv = (torch.as_tensor(x, dtype=torch.float32).contiguous().reshape(-1) for x in (q, k, v))
    L = forward_layout(F32, shp)
    out = torch.empty(L.combined_bytes // 4, dtype=torch.float32)
    fp = lambda t: C.cast(C.c_void_p(t.data_ptr()), C.POINTER(C.c_float))
    ctx.check(fn(ctx.h, *pre, C.byref(shp), C.byref(cfg), fp(hq), C.c_uint64(hq.numel()), fp(hk), C.c_uint64(hk.numel()),
                 fp(hv), C.c_uint64(hv.numel()), fp(out), C.c_uint64(out.numel() * 4), *post))
    B, H, N, D = shp.batch, shp.q_heads, shp.query_len, shp.head_dim
    return FlatAttentionOutput(out[:L.q_elements].view(B, H, N, D), out[L.lse_byte_offset // 4:].view(B, H, N))


class CudaPreferredAttention:
    """WgpuPreferredAttention (src/wgpu_f16_backend.rs:474-544): routes by head_dim between binary16 and f32
    storage; host f32 in, host f32 out; never a CPU path."""

    def __init__(self, device: int = 0):
        self.ctx = Context(device)
        self.last_precision = None

    @staticmethod
    def io_precision_for_head_dim(head_dim: int) -> int:
        return int(lib().flat_preferred_io_precision_for_head_dim(C.c_uint64(head_dim)))

    def forward(self, q, k, v, shp: Shape, cfg: Config) -> "FlatAttentionOutput":
        used = C.c_int32(-1)
        out = _host_f32_call(self.ctx, lib().flat_preferred_forward_host, shp, cfg, q, k, v, post=(C.byref(used),))
        self.last_precision = used.value
        return out


class NumericalExecutor:
    """NumericalExecutor (src/numerical.rs:135-256).  ExactReference is CPU execution in the reference; this library
    has no CPU path, so constructing it raises Unavailable."""

    def __init__(self, mode: int = FAST_PORTABLE, device: int = 0):
        self.guarantees = numerical_mode_guarantees(mode)
        if mode == EXACT_REFERENCE:
            raise FlatAttentionError(23, "exact-reference execution is CPU-only and is not part of this library")
        self.mode = mode
        self.ctx = Context(device)

    def forward(self, q, k, v, shp: Shape, cfg: Config) -> "FlatAttentionOutput":
        return _host_f32_call(self.ctx, lib().flat_numerical_forward_host, shp, cfg, q, k, v, pre=(C.c_int32(self.mode),))


def exported_symbols_in_header() -> list[str]:
    """Names of every function the C header declares (used by the symbol-export test)."""
    import re
    text = open(HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(flat_[a-z0-9_]+)\s*\(", text)))
