//! `#[repr(C)]` mirrors of the structs of include/flat_attention_b200.h (field for field, same order).
use core::ffi::{c_char, c_void};

/// Opaque handles of the C ABI.
macro_rules! opaque {
    ($($name:ident),*) => { $(#[repr(C)] pub struct $name { _private: [u8; 0] })* };
}
opaque!(FlatCtx, FlatPagedKvTable, FlatPagedKvCache, FlatResidentKvCache, FlatPreparedForward, FlatPreparedBackward,
        FlatSplitKvExchange);

pub const FLAT_F32: i32 = 0;
pub const FLAT_BF16: i32 = 1;
pub const FLAT_F16: i32 = 2;
pub const FLAT_LAYOUT_HEAD_MAJOR: i32 = 0;
pub const FLAT_LAYOUT_PROJECTION: i32 = 1;

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct FlatAttentionShape {
    pub batch: u64,
    pub q_heads: u64,
    pub kv_heads: u64,
    pub query_len: u64,
    pub kv_len: u64,
    pub head_dim: u64,
    pub query_position_offset: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq)]
pub struct FlatAttentionConfigRaw {
    pub causal: i32,
    pub has_softmax_scale: i32,
    pub softmax_scale: f32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq)]
pub struct FlatRotaryConfig {
    pub theta: f32,
    pub rotate_k: i32,
    pub query_position_offset: u64,
    pub kv_position_offset: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct FlatBuffer {
    pub ptr: *mut c_void,
    pub bytes: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct FlatForwardLayout {
    pub q_elements: u64,
    pub kv_elements: u64,
    pub lse_elements: u64,
    pub q_bytes: u64,
    pub kv_bytes: u64,
    pub lse_byte_offset: u64,
    pub combined_bytes: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct FlatDecodeLayout {
    pub q_elements: u64,
    pub output_elements: u64,
    pub lse_elements: u64,
    pub combined_elements: u64,
    pub q_bytes: u64,
    pub lse_byte_offset: u64,
    pub combined_bytes: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct FlatBackwardLayout {
    pub q_elements: u64,
    pub kv_elements: u64,
    pub lse_elements: u64,
    pub q_offset: u64,
    pub k_offset: u64,
    pub v_offset: u64,
    pub d_out_offset: u64,
    pub out_offset: u64,
    pub lse_offset: u64,
    pub input_bytes: u64,
    pub dq_offset: u64,
    pub dk_offset: u64,
    pub dv_offset: u64,
    pub output_bytes: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct FlatVarlenSequence {
    pub active_query_len: u32,
    pub active_kv_len: u32,
    pub causal_query_offset: u32,
    pub query_rope_offset: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct FlatPagedKvTelemetry {
    pub live_tokens: u64,
    pub capacity_tokens: u64,
    pub mapped_pages: u64,
    pub free_pages: u64,
    pub internal_fragmentation_tokens: u64,
    pub generation: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct FlatPagedKvAddress {
    pub physical_page: u64,
    pub offset_in_page: u64,
    pub generation: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct FlatNumericalGuarantees {
    pub accumulation: i32,
    pub reduction: i32,
    pub softmax_update: i32,
    pub repeatable_same_backend_device: i32,
    pub allows_subgroup: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct FlatDeviceFingerprint {
    pub name: [c_char; 256],
    pub backend: [c_char; 32],
    pub driver: [c_char; 64],
    pub driver_info: [c_char; 128],
    pub vendor: u32,
    pub device: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct FlatDeviceCapabilities {
    pub max_workgroups_per_dimension: u32,
    pub max_workgroup_size_x: u32,
    pub max_workgroup_size_y: u32,
    pub max_workgroup_size_z: u32,
    pub max_workgroup_storage_bytes: u32,
    pub max_binding_entries: u32,
    pub max_storage_buffer_binding_size: u32,
    pub subgroup_supported: u32,
    pub subgroup_min_size: u32,
    pub subgroup_max_size: u32,
    pub f16_supported: u32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct FlatDispatchTelemetry {
    pub kernel_id: i32,
    pub device: FlatDeviceFingerprint,
    pub query_rows: u32,
    pub kv_rows: u32,
    pub workgroups: [u32; 3],
    pub dispatch_count: u32,
    pub temporary_allocation_count: u32,
    pub temporary_allocation_bytes: u64,
    pub has_fallback_reason: i32,
    pub fallback_reason: [c_char; 160],
    pub autotuner_cache: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct FlatBenchmarkManifest {
    pub commit_sha: *const c_char,
    pub benchmark_id: *const c_char,
    pub command: *const c_char,
    pub device: *const c_char,
    pub backend: *const c_char,
    pub driver: *const c_char,
    pub os: *const c_char,
    pub arch: *const c_char,
    pub precision: *const c_char,
    pub batch: u64,
    pub q_heads: u64,
    pub kv_heads: u64,
    pub query_len: u64,
    pub kv_len: u64,
    pub head_dim: u64,
    pub causal: i32,
    pub warmup_iterations: u32,
    pub measured_iterations: u32,
    pub median_latency_ns: u64,
    pub p95_latency_ns: u64,
    pub tokens_per_second_milli: u64,
}
