//! sm_100a CUDA backend for FLAT-ATTENTION.
//!
//! A family of `Cuda*` structs with the method names and semantics of the reference's wgpu backends
//! (`WgpuGroupedForwardPipeline`, `WgpuPagedKvCache`, `WgpuPagedDecodePipeline`, ...), over the C ABI of
//! `libflat_attention_b200` (declared in `cuda_ffi`, generated from the C header).  Shapes, configurations and
//! errors are the reference crate's own types; device buffers are `(pointer, bytes)` pairs the caller owns, the
//! command encoder is the context's CUDA stream.  There is no CPU fallback: without an sm_100 device
//! `CudaContext::new` returns `CudaError::Unavailable`.
pub mod cuda_ffi;
pub mod cuda_types;

use core::ffi::c_void;
use std::ffi::CStr;

use cuda_types::*;
use flat_attention::{FlatAttentionConfig, GroupedAttentionShape};

/// A status code of the C ABI with the library's detail message (tensor name, sizes, CUDA text): the payload of
/// the reference's error variants.  `code` maps 1:1 onto `FlatAttentionError` / `GroupedForwardError` /
/// `PagedDecodeError` variants (the table is in include/flat_attention_b200.h).
#[derive(Debug, Clone, PartialEq, Eq)]
pub struct CudaError {
    pub code: i32,
    pub detail: String,
}

impl std::fmt::Display for CudaError {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        let name = unsafe { CStr::from_ptr(cuda_ffi::flat_status_str(self.code)) }.to_string_lossy();
        write!(f, "{name} ({}): {}", self.code, self.detail)
    }
}
impl std::error::Error for CudaError {}

/// Storage type of Q/K/V/O on the device (LSE is always f32).
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum DType {
    F32 = 0,
    Bf16 = 1,
    F16 = 2,
}

/// A caller-owned device allocation: what `&wgpu::Buffer` is in the reference's passes.
#[derive(Clone, Copy, Debug)]
pub struct DeviceBuffer {
    pub ptr: *mut c_void,
    pub bytes: u64,
}
impl DeviceBuffer {
    fn raw(self) -> FlatBuffer {
        FlatBuffer { ptr: self.ptr, bytes: self.bytes }
    }
}

fn raw_config(c: FlatAttentionConfig) -> FlatAttentionConfigRaw {
    FlatAttentionConfigRaw {
        causal: c.causal as i32,
        has_softmax_scale: c.softmax_scale.is_some() as i32,
        softmax_scale: c.softmax_scale.unwrap_or(0.0),
    }
}

fn raw_grouped(s: GroupedAttentionShape) -> FlatAttentionShape {
    FlatAttentionShape {
        batch: s.batch as u64,
        q_heads: s.q_heads as u64,
        kv_heads: s.kv_heads as u64,
        query_len: s.seq_len as u64,
        kv_len: s.seq_len as u64,
        head_dim: s.head_dim as u64,
        query_position_offset: 0,
    }
}

/// One device and one stream: the `wgpu::Device` + `wgpu::Queue` pair of the reference executors.
pub struct CudaContext {
    raw: *mut FlatCtx,
}

impl CudaContext {
    /// `stream` is a `cudaStream_t` (null = the legacy default stream); the caller owns it.
    pub fn new(device: i32, stream: *mut c_void) -> Result<Self, CudaError> {
        let mut raw = core::ptr::null_mut();
        let code = unsafe { cuda_ffi::flat_ctx_create(device, stream, &mut raw) };
        if code != 0 {
            return Err(CudaError { code, detail: String::new() });
        }
        Ok(Self { raw })
    }
    fn check(&self, code: i32) -> Result<(), CudaError> {
        if code == 0 {
            return Ok(());
        }
        let detail = unsafe { CStr::from_ptr(cuda_ffi::flat_last_error_detail(self.raw)) }.to_string_lossy().into_owned();
        Err(CudaError { code, detail })
    }
    pub fn synchronize(&self) -> Result<(), CudaError> {
        self.check(unsafe { cuda_ffi::flat_synchronize(self.raw) })
    }
    pub fn reserve_workspace(&self, bytes: u64) -> Result<(), CudaError> {
        self.check(unsafe { cuda_ffi::flat_ctx_reserve_workspace(self.raw, bytes) })
    }
    pub fn device_status(&self) -> i32 {
        unsafe { cuda_ffi::flat_ctx_device_status(self.raw) }
    }
}

impl Drop for CudaContext {
    fn drop(&mut self) {
        unsafe { cuda_ffi::flat_ctx_destroy(self.raw) }
    }
}

/// `GroupedForwardPass` (src/wgpu_forward_grouped.rs:93-102).
#[derive(Clone, Copy, Debug)]
pub struct CudaGroupedForwardPass {
    pub q: DeviceBuffer,
    pub k: DeviceBuffer,
    pub v: DeviceBuffer,
    pub output: DeviceBuffer,
    pub shape: GroupedAttentionShape,
    pub config: FlatAttentionConfig,
}

/// `WgpuGroupedForwardPipeline` (src/wgpu_forward_grouped.rs:170-539): caller-owned buffers, packed `[O | LSE]`
/// output, `layout` / `encode` / `prepare` / `encode_prepared`.
pub struct CudaGroupedForwardPipeline<'a> {
    ctx: &'a CudaContext,
    dtype: DType,
}

/// `PreparedGroupedForward`: a validated pass; `encode_prepared` only enqueues.
pub struct CudaPreparedGroupedForward {
    raw: *mut FlatPreparedForward,
}
impl Drop for CudaPreparedGroupedForward {
    fn drop(&mut self) {
        unsafe { cuda_ffi::flat_prepared_forward_destroy(self.raw) }
    }
}

impl<'a> CudaGroupedForwardPipeline<'a> {
    pub fn new(ctx: &'a CudaContext, dtype: DType) -> Self {
        Self { ctx, dtype }
    }
    /// Pure and allocation-free, like the reference's `layout`.
    pub fn layout(dtype: DType, shape: GroupedAttentionShape) -> Result<FlatForwardLayout, CudaError> {
        let mut out = FlatForwardLayout::default();
        let code = unsafe { cuda_ffi::flat_forward_layout_for(dtype as i32, &raw_grouped(shape), &mut out) };
        if code != 0 {
            return Err(CudaError { code, detail: String::new() });
        }
        Ok(out)
    }
    /// Records the dispatch on the context's stream; never synchronises.
    pub fn encode(&self, pass: CudaGroupedForwardPass) -> Result<FlatForwardLayout, CudaError> {
        let (shape, cfg) = (raw_grouped(pass.shape), raw_config(pass.config));
        self.ctx.check(unsafe {
            cuda_ffi::flat_forward_grouped(self.ctx.raw, self.dtype as i32, &shape, &cfg, pass.q.raw(), pass.k.raw(), pass.v.raw(),
                                           pass.output.raw())
        })?;
        Self::layout(self.dtype, pass.shape)
    }
    pub fn prepare(&self, pass: CudaGroupedForwardPass) -> Result<CudaPreparedGroupedForward, CudaError> {
        let (shape, cfg) = (raw_grouped(pass.shape), raw_config(pass.config));
        let mut raw = core::ptr::null_mut();
        self.ctx.check(unsafe {
            cuda_ffi::flat_forward_prepare(self.ctx.raw, self.dtype as i32, FLAT_LAYOUT_HEAD_MAJOR, &shape, &cfg, core::ptr::null(),
                                           pass.q.raw(), pass.k.raw(), pass.v.raw(), pass.output.raw(), &mut raw)
        })?;
        Ok(CudaPreparedGroupedForward { raw })
    }
    pub fn encode_prepared(&self, prepared: &CudaPreparedGroupedForward) -> Result<(), CudaError> {
        self.ctx.check(unsafe { cuda_ffi::flat_forward_encode_prepared(self.ctx.raw, prepared.raw) })
    }
}

/// `GroupedBackwardRecomputePass` (src/wgpu_backward_grouped.rs:104-112): one packed input buffer
/// `[Q | K | V | dO | O | LSE]` and one packed f32 gradient buffer `[dQ | dK | dV]`, offsets from `layout`.
#[derive(Clone, Copy, Debug)]
pub struct CudaGroupedBackwardRecomputePass {
    pub packed_inputs: DeviceBuffer,
    pub packed_grads: DeviceBuffer,
    pub shape: GroupedAttentionShape,
    pub config: FlatAttentionConfig,
}

/// `WgpuGroupedBackwardRecomputePipeline` (src/wgpu_backward_grouped.rs:181-326): `layout` / `encode` /
/// `prepare` / `encode_prepared`; gradients are bitwise repeatable.
pub struct CudaGroupedBackwardRecomputePipeline<'a> {
    ctx: &'a CudaContext,
    dtype: DType,
}

/// `PreparedGroupedBackwardRecompute` (src/wgpu_backward_grouped.rs:231-326): a validated pass with its scratch
/// sized; `encode_prepared` only enqueues.
pub struct CudaPreparedGroupedBackwardRecompute {
    raw: *mut FlatPreparedBackward,
}
impl Drop for CudaPreparedGroupedBackwardRecompute {
    fn drop(&mut self) {
        unsafe { cuda_ffi::flat_prepared_backward_destroy(self.raw) }
    }
}

impl<'a> CudaGroupedBackwardRecomputePipeline<'a> {
    pub fn new(ctx: &'a CudaContext, dtype: DType) -> Self {
        Self { ctx, dtype }
    }
    pub fn layout(dtype: DType, shape: GroupedAttentionShape) -> Result<FlatBackwardLayout, CudaError> {
        let mut out = FlatBackwardLayout::default();
        let code = unsafe { cuda_ffi::flat_backward_layout_for(dtype as i32, &raw_grouped(shape), &mut out) };
        if code != 0 {
            return Err(CudaError { code, detail: String::new() });
        }
        Ok(out)
    }
    /// Records the two kernels on the context's stream; never synchronises.
    pub fn encode(&self, pass: CudaGroupedBackwardRecomputePass) -> Result<FlatBackwardLayout, CudaError> {
        let (shape, cfg) = (raw_grouped(pass.shape), raw_config(pass.config));
        self.ctx.check(unsafe {
            cuda_ffi::flat_backward_grouped(self.ctx.raw, self.dtype as i32, &shape, &cfg, pass.packed_inputs.raw(),
                                            pass.packed_grads.raw())
        })?;
        Self::layout(self.dtype, pass.shape)
    }
    pub fn prepare(&self, pass: CudaGroupedBackwardRecomputePass) -> Result<CudaPreparedGroupedBackwardRecompute, CudaError> {
        let (shape, cfg) = (raw_grouped(pass.shape), raw_config(pass.config));
        let mut raw = core::ptr::null_mut();
        self.ctx.check(unsafe {
            cuda_ffi::flat_backward_prepare(self.ctx.raw, self.dtype as i32, &shape, &cfg, pass.packed_inputs.raw(),
                                            pass.packed_grads.raw(), &mut raw)
        })?;
        Ok(CudaPreparedGroupedBackwardRecompute { raw })
    }
    pub fn encode_prepared(&self, prepared: &CudaPreparedGroupedBackwardRecompute) -> Result<(), CudaError> {
        self.ctx.check(unsafe { cuda_ffi::flat_backward_encode_prepared(self.ctx.raw, prepared.raw) })
    }
    /// Bound of the dS scratch between the two kernels; 0 selects the recompute route.
    pub fn set_scratch_budget(&self, bytes: u64) -> Result<(), CudaError> {
        self.ctx.check(unsafe { cuda_ffi::flat_ctx_set_backward_scratch_budget(self.ctx.raw, bytes) })
    }
}

/// `WgpuPagedKvCache` (src/wgpu_paged_kv_cache.rs:76-279): owns K and V `[pages * page_size, kv_heads * head_dim]`.
pub struct CudaPagedKvCache<'a> {
    ctx: &'a CudaContext,
    raw: *mut FlatPagedKvCache,
}

impl<'a> CudaPagedKvCache<'a> {
    pub fn new(ctx: &'a CudaContext, dtype: DType, page_size: usize, physical_pages: usize, kv_heads: usize,
               head_dim: usize) -> Result<Self, CudaError> {
        let mut raw = core::ptr::null_mut();
        ctx.check(unsafe {
            cuda_ffi::flat_paged_kv_cache_create(ctx.raw, dtype as i32, page_size as u64, physical_pages as u64, kv_heads as u64,
                                                 head_dim as u64, &mut raw)
        })?;
        Ok(Self { ctx, raw })
    }
    /// Sources are `[append_len, kv_heads * head_dim]`, K already rotated; returns the new live length.
    pub fn record_append(&mut self, k_source: DeviceBuffer, v_source: DeviceBuffer, append_len: usize) -> Result<usize, CudaError> {
        let mut new_len = 0u64;
        self.ctx.check(unsafe {
            cuda_ffi::flat_paged_kv_cache_append(self.raw, k_source.raw(), v_source.raw(), append_len as u64, &mut new_len)
        })?;
        Ok(new_len as usize)
    }
    pub fn reset(&mut self) -> Result<(), CudaError> {
        self.ctx.check(unsafe { cuda_ffi::flat_paged_kv_cache_reset(self.raw) })
    }
    pub fn len(&self) -> usize {
        unsafe { cuda_ffi::flat_paged_kv_cache_len(self.raw) as usize }
    }
    pub fn is_empty(&self) -> bool {
        self.len() == 0
    }
    pub fn generation(&self) -> u64 {
        unsafe { cuda_ffi::flat_paged_kv_cache_generation(self.raw) }
    }
    pub fn k_buffer(&self) -> DeviceBuffer {
        let b = unsafe { cuda_ffi::flat_paged_kv_cache_k_buffer(self.raw) };
        DeviceBuffer { ptr: b.ptr, bytes: b.bytes }
    }
    pub fn v_buffer(&self) -> DeviceBuffer {
        let b = unsafe { cuda_ffi::flat_paged_kv_cache_v_buffer(self.raw) };
        DeviceBuffer { ptr: b.ptr, bytes: b.bytes }
    }
    pub fn table(&self) -> *const FlatPagedKvTable {
        unsafe { cuda_ffi::flat_paged_kv_cache_table(self.raw) }
    }
}

impl Drop for CudaPagedKvCache<'_> {
    fn drop(&mut self) {
        unsafe { cuda_ffi::flat_paged_kv_cache_destroy(self.raw) }
    }
}

/// `PagedDecodePass` (src/wgpu_paged_decode.rs:200-219).
#[derive(Clone, Copy, Debug)]
pub struct CudaPagedDecodePass {
    pub q: DeviceBuffer,
    pub k: DeviceBuffer,
    pub v: DeviceBuffer,
    pub page_table: *const FlatPagedKvTable,
    pub out_and_lse: DeviceBuffer,
    pub q_heads: usize,
    pub kv_heads: usize,
    pub head_dim: usize,
    pub config: FlatAttentionConfig,
    pub theta: f32,
    pub q_rope_position: usize,
}

/// `WgpuPagedDecodePipeline` (src/wgpu_paged_decode.rs:237-437).
pub struct CudaPagedDecodePipeline<'a> {
    ctx: &'a CudaContext,
    dtype: DType,
}

impl<'a> CudaPagedDecodePipeline<'a> {
    pub fn new(ctx: &'a CudaContext, dtype: DType) -> Self {
        Self { ctx, dtype }
    }
    pub fn layout(dtype: DType, q_heads: usize, head_dim: usize) -> Result<FlatDecodeLayout, CudaError> {
        let mut out = FlatDecodeLayout::default();
        let code = unsafe { cuda_ffi::flat_decode_layout_for(dtype as i32, 1, q_heads as u64, head_dim as u64, &mut out) };
        if code != 0 {
            return Err(CudaError { code, detail: String::new() });
        }
        Ok(out)
    }
    pub fn encode(&self, pass: CudaPagedDecodePass) -> Result<FlatDecodeLayout, CudaError> {
        let cfg = raw_config(pass.config);
        self.ctx.check(unsafe {
            cuda_ffi::flat_decode_paged(self.ctx.raw, self.dtype as i32, pass.page_table, pass.q_heads as u64, pass.kv_heads as u64,
                                        pass.head_dim as u64, &cfg, pass.theta, pass.q_rope_position as u64, pass.q.raw(),
                                        pass.k.raw(), pass.v.raw(), pass.out_and_lse.raw())
        })?;
        Self::layout(self.dtype, pass.q_heads, pass.head_dim)
    }
}

/// The peer-memory exchange of KV-split decode (no counterpart in the reference, which is single-device): one device
/// allocation per rank that the other ranks of the box map through CUDA IPC.  `handle` is what a rank gives the
/// others, `connect` maps theirs; `flat_splitkv_decode_peer` then runs a step (the rank's partial, then one kernel that
/// stores it into every rank's buffer, waits for the others' flags and merges).
pub struct CudaSplitKvPeerExchange<'a> {
    ctx: &'a CudaContext,
    raw: *mut FlatSplitKvExchange,
}

impl<'a> CudaSplitKvPeerExchange<'a> {
    pub fn new(ctx: &'a CudaContext, rank: i32, world: i32, rows: u64, head_dim: u64) -> Result<Self, CudaError> {
        let mut raw = core::ptr::null_mut();
        ctx.check(unsafe { cuda_ffi::flat_splitkv_exchange_create(ctx.raw, rank, world, rows, head_dim, &mut raw) })?;
        Ok(Self { ctx, raw })
    }
    pub fn handle(&self) -> Result<[u8; 64], CudaError> {
        let mut out = [0u8; 64];
        self.ctx.check(unsafe { cuda_ffi::flat_splitkv_exchange_handle(self.raw, out.as_mut_ptr()) })?;
        Ok(out)
    }
    /// `all_handles`: every rank's handle in rank order (the own entry is ignored).
    pub fn connect(&mut self, all_handles: &[u8]) -> Result<(), CudaError> {
        self.ctx.check(unsafe { cuda_ffi::flat_splitkv_exchange_connect(self.raw, all_handles.as_ptr(), all_handles.len() as u64) })
    }
    pub fn raw(&self) -> *mut FlatSplitKvExchange {
        self.raw
    }
}

impl Drop for CudaSplitKvPeerExchange<'_> {
    fn drop(&mut self) {
        unsafe { cuda_ffi::flat_splitkv_exchange_destroy(self.raw) }
    }
}
