// Internal declarations shared by the host layer (abi.cu) and the kernel translation units.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <algorithm>
#include <cstdio>
#include <string>
#include <utility>
#include <vector>

#include "../../include/flat_attention_b200.h"

namespace flat {

constexpr int kMaxHeadDim = 128;  // WGSL_MAX_HEAD_DIM, src/lib.rs:60

// Device status word written by bounded waits.
struct DeviceStatus {
    int code;    // FLAT_OK or FLAT_ERR_DEVICE_WAIT_TIMEOUT
    int where;   // which wait gave up (kernel-specific tag)
};

}  // namespace flat

struct flat_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    flat_device_fingerprint fingerprint{};    // captured once at creation, like the reference's owned context
    flat_device_capabilities capabilities{};
    void *workspace = nullptr;
    uint64_t workspace_bytes = 0;
    flat::DeviceStatus *dev_status = nullptr;  // device memory
    uint64_t launches = 0;
    std::string detail;
    void *host_stage = nullptr;       // device staging of the host-slice entry points (Q | K | V | O|LSE)
    uint64_t host_stage_bytes = 0;
    cudaStream_t copy_in = nullptr, copy_out = nullptr;  // upload / download streams of the host-slice entry points
    unsigned long long *finite_first = nullptr;       // device [3]: first non-finite index of Q, K, V (device-side scan)
    unsigned long long *finite_first_host = nullptr;  // pinned host mirror, read once per call
    std::vector<cudaEvent_t> pipe_events;
    // (cos, sin) tables of recent RoPE calls, kept on the device: a serving or training loop calls with the same
    // theta, head_dim and positions every step, and the table is then computed once instead of per call
    struct RopeTable {
        void *dev = nullptr;
        uint64_t bytes = 0;
        float inv_freq[64] = {};
        int half_dim = 0, rows = 0;
        int64_t pos_off = 0;
        uint64_t last_use = 0;
    };
    RopeTable rope_tables[2];
    uint64_t rope_clock = 0;
    // The tensor-core backward may keep every bf16 dS^T tile in scratch (O(N^2) bytes) so that dQ needs no second score
    // recompute; it does so while that spill fits this budget (flat_ctx_set_backward_scratch_budget).
    uint64_t backward_scratch_budget = 8ull << 30;
    cudaEvent_t stream_switch = nullptr;  // orders the old and the new stream in flat_ctx_set_stream
    // sequence offsets of the last balanced decode plan and where they were uploaded (skips identical re-uploads)
    std::vector<int32_t> plan_offsets;
    const void *plan_offsets_at = nullptr;
    // optional timing of the dominant kernel of each call (CUDA events on the launch stream)
    bool timing = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> timed;
};

namespace flat {

// printf-style error recording; returns `status` so call sites can `return fail(...)`.
int fail(flat_ctx *ctx, int status, const char *fmt, ...);

inline bool mul_ok(uint64_t a, uint64_t b, uint64_t *out) { return !__builtin_mul_overflow(a, b, out); }
inline bool add_ok(uint64_t a, uint64_t b, uint64_t *out) { return !__builtin_add_overflow(a, b, out); }

// Brackets the dominant kernel of a call with CUDA events when timing is enabled.
struct KernelTimer {
    flat_ctx *ctx;
    cudaEvent_t start = nullptr, stop = nullptr;
    explicit KernelTimer(flat_ctx *c) : ctx(c) {
        if (!ctx->timing) return;
        if (cudaEventCreate(&start) != cudaSuccess || cudaEventCreate(&stop) != cudaSuccess) {
            start = stop = nullptr;
            return;
        }
        cudaEventRecord(start, ctx->stream);
    }
    ~KernelTimer() {
        if (!start) return;
        cudaEventRecord(stop, ctx->stream);
        ctx->timed.emplace_back(start, stop);
    }
};

inline size_t dtype_size(int dtype) { return dtype == FLAT_F32 ? 4 : 2; }

// Grows (never shrinks) the context scratch; synchronises the stream when it reallocates, so it
// must be called before anything of the current call is copied into the scratch.
int ensure_workspace(flat_ctx *ctx, uint64_t bytes);
// Grows the device staging area of the host-slice entry points (synchronises the stream when it reallocates).
int ensure_host_stage(flat_ctx *ctx, uint64_t bytes);
// Scratch convention: the first kWorkspaceMeta bytes hold small host-provided tables of the
// current call (variable-length metadata, a single-sequence page table); kernel scratch (split-KV
// partials, rotated operands, backward accumulators) starts behind it.
constexpr uint64_t kWorkspaceMeta = 1 << 16;
inline char *scratch_ptr(flat_ctx *ctx) { return static_cast<char *>(ctx->workspace) + kWorkspaceMeta; }

#define FLAT_CUDA_OK(ctx, expr)                                                            \
    do {                                                                                   \
        cudaError_t e__ = (expr);                                                          \
        if (e__ != cudaSuccess)                                                            \
            return ::flat::fail((ctx), FLAT_ERR_EXECUTION, "%s: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

// ---- forward ---------------------------------------------------------------------------------
// One parameter block serves every forward flavour: layouts are element strides, RoPE is two
// switches plus three position domains, variable-length batches and paged K/V are optional
// pointers.  (The reference kernels' uniform blocks: src/wgpu_external_asymmetric.rs:319-339,
// src/wgpu_external_variable.rs:148-171.)
struct FwdParams {
    const void *q, *k, *v;
    void *o;
    float *lse;
    int64_t q_bs, q_hs, q_rs;     // Q element strides: batch, head, row
    int64_t kv_bs, kv_hs, kv_rs;  // K/V element strides (ignored for paged K/V except kv_hs)
    int64_t o_bs, o_hs, o_rs;
    int64_t lse_hs;               // LSE elements between consecutive (batch, q_head) rows
    int batch, q_heads, kv_heads, q_len, kv_len, head_dim, group;
    int causal;
    int64_t causal_off;
    float scale;
    int rope_q, rope_k;
    int64_t q_rope_off, k_rope_off;
    const flat_varlen_sequence *varlen;  // device, [batch] or null
    int64_t varlen_rope_min, varlen_rope_max;  // smallest / largest query_rope_offset of the batch (host-side copy)
    const int32_t *page_table;           // device, [batch, max_pages] or null
    int page_size, max_pages;
    int64_t page_row_stride;             // elements per physical row (kv_heads*head_dim)
    float inv_freq[kMaxHeadDim / 2];     // theta^(-2j/D), host-computed in f32
    // ALiBi (src/attention_bias.rs:82-95): score += slopes[q_head] * ((kv_off + key) - (q_off + query row))
    const float *alibi_slopes;           // device, [q_heads] or null
    int64_t alibi_q_off, alibi_kv_off;
    float alibi_max_abs_slope;           // host-side copy of max |slope|
    int f16_io;                          // 16-bit storage is IEEE binary16 instead of bf16 (forward only)
    int k_f16;                           // K alone is binary16 (the prefill shadow of a bf16 paged cache): no in-kernel conversion
};

// Generic SIMT forward (f32 arithmetic; T = float or __nv_bfloat16 storage).
int launch_forward_simt(flat_ctx *ctx, int dtype, const FwdParams &p);
// tile geometry and grid of the two forward kernels for a parameter block (telemetry; nothing is launched)
void forward_simt_geometry(const FwdParams &p, uint32_t *query_rows, uint32_t *kv_rows, uint32_t grid[3]);
void forward_sm100_geometry(const flat_ctx *ctx, const FwdParams &p, uint32_t *query_rows, uint32_t *kv_rows, uint32_t grid[3],
                            uint32_t *dispatches);
// tcgen05 forward for bf16, head_dim 64/128; returns FLAT_ERR_UNSUPPORTED_SHAPE when the shape
// does not fit it (the caller then uses the SIMT kernel).
bool forward_sm100_supported(const FwdParams &p);
uint64_t forward_sm100_workspace_bytes(const flat_ctx *ctx, const FwdParams &p);
int launch_forward_sm100(flat_ctx *ctx, const FwdParams &p);

// ---- decode ----------------------------------------------------------------------------------
struct DecodeParams {
    const void *q;       // [num_seqs, q_heads*head_dim]
    const void *k, *v;   // paged: [pages, page_size, kv_heads*head_dim]; resident: [batch, capacity, ...]
    void *o;             // [num_seqs, q_heads*head_dim]
    float *lse;          // [num_seqs, q_heads]
    int num_seqs, q_heads, kv_heads, head_dim, group;
    int page_size, max_pages;            // page_size == 0 -> resident (contiguous) addressing
    int physical_pages;                  // paged: entries outside [0, physical_pages) are masked and flagged, never read
    DeviceStatus *status;                // device status word of the context (page-table range violations)
    const int32_t *page_table;           // device [num_seqs, max_pages]
    const int32_t *context_lens;         // device [num_seqs] or null (-> uniform_len)
    const int32_t *q_rope_positions;     // device [num_seqs] or null (-> uniform_q_pos)
    int uniform_len;
    int64_t uniform_q_pos;
    int64_t seq_stride_rows;             // resident: capacity (rows per batch element)
    float scale;
    int rope_q;
    float inv_freq[kMaxHeadDim / 2];
    int kv_splits;                       // >= 1
    float *partial_o;                    // [splits, num_seqs*q_heads, head_dim] f32 (splits > 1)
    float *partial_lse;                  // [splits, num_seqs*q_heads]
    int chunk_tokens;                    // tokens per split chunk (splits > 1)
    // Balanced mode (tensor-core decode only): sequences, each padded to a multiple of 16 tokens,
    // are laid end to end and CTA i streams tokens [i*span, (i+1)*span) of that line, whatever
    // sequences they belong to.  seq_offsets[s] is where sequence s starts (device, num_seqs+1
    // entries).  Partial slot of (sequence, CTA) = CTA index - first CTA touching the sequence;
    // kv_splits then holds the maximum number of slots per sequence.
    int out_f32;                         // write the final O as f32 whatever the storage type (cross-GPU partials)
    int balanced;
    int span_tokens;
    int num_ctas;
    const int32_t *seq_offsets;
};
uint64_t decode_workspace_bytes(const DecodeParams &p);
// Fixed scratch of the allocation-free decode entry point: a file-scope device array of the library image.
constexpr uint64_t kDecodeStaticScratchBytes = 8ull << 20;  // 8 MiB per device that loads the library
// Device address of that array on the context's device (looked up once per device with cudaGetSymbolAddress).
int decode_static_scratch(flat_ctx *ctx, float **out);
bool decode_fast_path_ok(int dtype, int head_dim, int group);
int launch_decode(flat_ctx *ctx, int dtype, const DecodeParams &p);
// bf16 tensor-core decode (mma.sync), head_dim 64/128, group <= 8, pages of a multiple of 16 tokens
bool decode_mma_supported(int dtype, const DecodeParams &p);
int launch_decode_mma(flat_ctx *ctx, const DecodeParams &p);
// part i of the partial O / LSE starts part_stride_o / part_stride_lse floats after part i-1
int launch_splitkv_merge(flat_ctx *ctx, int dtype, int parts, int64_t rows, int head_dim,
                         const float *partial_o, const float *partial_lse, int64_t part_stride_o,
                         int64_t part_stride_lse, void *o, float *lse);

// ---- input validation on the device ----------------------------------------------------------
// Up to three segments (Q, K, V chunks) scanned for non-finite values in one launch; first[slot] receives the
// smallest absolute element index of an offending value (atomicMin; ~0 = none found).
struct FiniteScan {
    struct Segment {
        const void *data;     // device, 16-byte aligned
        uint64_t elements;
        uint64_t base_index;  // index of data[0] inside the caller's tensor
        int slot;             // which entry of `first` the segment reports to
    } seg[3];
    unsigned long long *first;  // device, [3]
    int elem_size;              // 4 (f32) or 2 (bf16 / binary16)
    uint32_t mask16;            // exponent mask of the 16-bit type (0x7f80 bf16, 0x7c00 binary16)
};
int launch_finite_scan(flat_ctx *ctx, const FiniteScan &scan, cudaStream_t stream);

// ---- KV cache --------------------------------------------------------------------------------
// Copies `rows` source rows of `row_elems` elements to destination rows dst_rows[i] (device
// array of int64), optionally rotating each head_dim-wide head slice at positions pos0 + i.
// k_shadow: optional binary16 copy of the stored K (bf16 caches), same row layout as k_dst.
int launch_shadow_fill(flat_ctx *ctx, const void *k, void *shadow, int64_t elements);
int launch_append_rows(flat_ctx *ctx, int dtype, const void *k_src, const void *v_src, void *k_dst,
                       void *v_dst, void *k_shadow, int64_t rows, int row_elems, int head_dim,
                       const int32_t *page_table, int page_size, int64_t first_logical,
                       int64_t dst_row0, int rotate, int64_t pos0, const float *inv_freq);

// ---- backward --------------------------------------------------------------------------------
struct BwdParams {
    const void *q, *k, *v, *d_out, *out;
    const float *lse;
    void *dq, *dk, *dv;
    int batch, q_heads, kv_heads, seq_len, head_dim, group;
    int causal;
    float scale;
};
int launch_backward_simt(flat_ctx *ctx, int dtype, const BwdParams &p);
bool backward_sm100_supported(const BwdParams &p);
uint64_t backward_sm100_workspace_bytes(const flat_ctx *ctx, const BwdParams &p);
int launch_backward_sm100(flat_ctx *ctx, const BwdParams &p);

}  // namespace flat
