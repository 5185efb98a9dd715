/*
 * flat_attention_b200.h — C ABI of the B200 (sm_100a) fused-attention backend.
 *
 * This is the boundary a Rust `Cuda*` backend would bind (one `extern "C"` block, plain
 * pointers and sizes).  Every entry point names the FLAT-ATTENTION interface it stands in
 * for (`file:line` in that project).  Conventions kept from the reference backends:
 *
 *  - all validation happens before any launch; the result is a typed status, never an
 *    abort and never a CPU result (src/lib.rs:362, src/numerical.rs:150-153);
 *  - `flat_*` calls that launch work are "encode"-style: they enqueue on the context's
 *    CUDA stream and return without synchronising (src/wgpu_decode.rs:1-8,
 *    src/wgpu_paged_kv_cache.rs:8-9); only flat_synchronize / flat_download block;
 *  - buffers may be larger than required, too-small buffers are rejected with the exact
 *    byte counts (src/wgpu_forward_grouped.rs:565-579);
 *  - outputs are packed `[O | LSE]` in one buffer, O first (src/wgpu_forward_grouped.rs:34-42).
 *    f32 mode: LSE starts at element q_elements.  bf16 mode: O is bf16, LSE is f32 at byte
 *    offset 2*q_elements (the 16-bit packing of src/wgpu_f16_backend.rs:273-277).
 */
#ifndef FLAT_ATTENTION_B200_H
#define FLAT_ATTENTION_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes -------------------------------------------------------------------- */
/* 1..9 mirror FlatAttentionError (src/lib.rs:363-386) and api::v1::ApiError
 * (src/api.rs:203-222); the other blocks mirror the per-component error enums. */
typedef enum flat_status {
    FLAT_OK = 0,
    FLAT_ERR_ZERO_DIMENSION = 1,
    FLAT_ERR_SHAPE_OVERFLOW = 2,
    FLAT_ERR_INVALID_HEAD_GROUPING = 3,
    FLAT_ERR_INVALID_ROTARY_HEAD_DIM = 4,
    FLAT_ERR_INVALID_ROTARY_THETA = 5,
    FLAT_ERR_POSITION_OVERFLOW = 6,
    FLAT_ERR_LENGTH_MISMATCH = 7,
    FLAT_ERR_INVALID_SCALE = 8,
    FLAT_ERR_NON_FINITE_INPUT = 9,
    /* backend errors (src/wgpu_backend.rs:39-63, src/wgpu_forward_grouped.rs:104-125) */
    FLAT_ERR_UNSUPPORTED_HEAD_DIM = 20,
    FLAT_ERR_INDEX_SPACE_EXCEEDED = 21,
    FLAT_ERR_BUFFER_TOO_SMALL = 22,
    FLAT_ERR_UNAVAILABLE = 23,      /* no CUDA device / not an sm_100 device */
    FLAT_ERR_EXECUTION = 24,        /* a CUDA call failed; detail carries the CUDA message */
    FLAT_ERR_DISPATCH_LIMIT = 25,
    FLAT_ERR_UNSUPPORTED_DTYPE = 26,
    FLAT_ERR_NULL_POINTER = 27,
    FLAT_ERR_MISALIGNED_BUFFER = 28,
    FLAT_ERR_UNSUPPORTED_SHAPE = 29, /* shape valid for the contract, not for this kernel */
    /* decode errors (src/wgpu_decode.rs:104-142, src/wgpu_paged_decode.rs:27-71) */
    FLAT_ERR_EMPTY_CACHE = 30,
    FLAT_ERR_INVALID_CACHE_LENGTH = 31,
    FLAT_ERR_INVALID_QUERY_LEN = 32,
    FLAT_ERR_CAUSAL_VISIBILITY_MISMATCH = 33,
    FLAT_ERR_EMPTY_TABLE = 34,
    FLAT_ERR_PAGE_OUT_OF_RANGE = 35,
    FLAT_ERR_PAGE_SHARED = 36,
    FLAT_ERR_INVALID_THETA = 37,
    /* paged-KV metadata errors (src/paged_kv.rs:37-43) and cache errors
     * (src/wgpu_kv_cache.rs:21-38, src/wgpu_paged_kv_cache.rs:16-33) */
    FLAT_ERR_CAPACITY_OVERFLOW = 40,
    FLAT_ERR_CAPACITY_EXCEEDED = 41,
    FLAT_ERR_GENERATION_OVERFLOW = 42,
    /* chunked prefill (src/chunked_projection_prefill.rs:23-27) */
    FLAT_ERR_ZERO_QUERY_CHUNK_SIZE = 50,
    /* a bounded device-side wait expired; the kernel returned early and the context is
     * still usable (outputs of that launch are undefined) */
    FLAT_ERR_DEVICE_WAIT_TIMEOUT = 60,
    /* BenchmarkManifestError (src/benchmark_manifest.rs:56-63); ZeroDimension and
     * InvalidHeadGrouping reuse the codes above */
    FLAT_ERR_MANIFEST_INVALID_COMMIT_SHA = 70,
    FLAT_ERR_MANIFEST_EMPTY_FIELD = 71,
    FLAT_ERR_MANIFEST_ZERO_MEASURED_ITERATIONS = 72,
    FLAT_ERR_MANIFEST_INVALID_PERCENTILE_ORDERING = 73
} flat_status;

/* Storage/arithmetic mode.  F32: f32 I/O, f32 SIMT arithmetic (parity mode, <=1e-4).
 * BF16: bf16 Q/K/V/dO/O, f32 LSE, tcgen05 tensor-core arithmetic with f32 accumulation. */
/* FLAT_F16 is IEEE binary16 storage (F16, src/f16.rs:9-115; the packed-f16 executor
 * src/wgpu_f16_backend.rs:168-430): accepted by the forward entry points and
 * flat_forward_layout_for only; arithmetic, softmax and LSE stay f32 as in the reference. */
typedef enum flat_dtype { FLAT_F32 = 0, FLAT_BF16 = 1, FLAT_F16 = 2 } flat_dtype;

/* HEAD_MAJOR: Q/O [B,Hq,Nq,D], K/V [B,Hkv,Nkv,D] (src/grouped.rs:11-16).
 * PROJECTION: Q/O [B*Nq, Hq*D], K/V [B*Nkv, Hkv*D] (src/projection_grouped.rs:3-8).
 * LSE is [B,Hq,Nq] in both. */
typedef enum flat_layout { FLAT_LAYOUT_HEAD_MAJOR = 0, FLAT_LAYOUT_PROJECTION = 1 } flat_layout;

/* api::v1::AttentionShape (src/api.rs:24-33); for equal-length calls query_len == kv_len
 * and query_position_offset == 0. */
typedef struct flat_attention_shape {
    uint64_t batch;
    uint64_t q_heads;
    uint64_t kv_heads;
    uint64_t query_len;
    uint64_t kv_len;
    uint64_t head_dim;
    uint64_t query_position_offset; /* causal domain: row q sits at offset + q */
} flat_attention_shape;

/* FlatAttentionConfig (src/lib.rs:248-269). has_softmax_scale == 0 -> 1/sqrt(head_dim). */
typedef struct flat_attention_config {
    int32_t causal;
    int32_t has_softmax_scale;
    float softmax_scale;
} flat_attention_config;

/* AsymmetricRotaryEmbeddingConfig (src/projection_asymmetric.rs:18-23) plus the
 * `rotate_k` switch of encode_pre_rotated_k (src/wgpu_external_asymmetric.rs:203-211):
 * rotate_k == 0 means K in memory is already rotated and only Q is rotated in-kernel. */
typedef struct flat_rotary_config {
    float theta;
    int32_t rotate_k;
    uint64_t query_position_offset;
    uint64_t kv_position_offset;
} flat_rotary_config;

/* A device allocation: the wgpu::Buffer analogue (pointer + size in bytes). */
typedef struct flat_buffer {
    void *ptr;
    uint64_t bytes;
} flat_buffer;

/* GroupedForwardLayout / ExternalProjectionLayout (src/wgpu_forward_grouped.rs:23-42). */
typedef struct flat_forward_layout {
    uint64_t q_elements;
    uint64_t kv_elements;
    uint64_t lse_elements;
    uint64_t q_bytes;
    uint64_t kv_bytes;
    uint64_t lse_byte_offset; /* where LSE starts inside the packed output */
    uint64_t combined_bytes;  /* size of the packed [O | LSE] buffer */
} flat_forward_layout;

/* VariableLengthSequenceMetadata (src/wgpu_external_variable.rs:21-33). */
typedef struct flat_varlen_sequence {
    uint32_t active_query_len;
    uint32_t active_kv_len;
    uint32_t causal_query_offset;
    uint32_t query_rope_offset;
} flat_varlen_sequence;

/* PagedKvTelemetry (src/paged_kv.rs:27-35). */
typedef struct flat_paged_kv_telemetry {
    uint64_t live_tokens;
    uint64_t capacity_tokens;
    uint64_t mapped_pages;
    uint64_t free_pages;
    uint64_t internal_fragmentation_tokens;
    uint64_t generation;
} flat_paged_kv_telemetry;

/* PagedKvAddress (src/paged_kv.rs:20-25). */
typedef struct flat_paged_kv_address {
    uint64_t physical_page;
    uint64_t offset_in_page;
    uint64_t generation;
} flat_paged_kv_address;

/* GroupedBackwardRecomputeLayout (src/wgpu_backward_grouped.rs:17-56): packed input
 * Q|K|V|dO|O|LSE and packed output dQ|dK|dV, offsets in bytes. */
typedef struct flat_backward_layout {
    uint64_t q_elements;
    uint64_t kv_elements;
    uint64_t lse_elements;
    uint64_t q_offset, k_offset, v_offset, d_out_offset, out_offset, lse_offset;
    uint64_t input_bytes;
    uint64_t dq_offset, dk_offset, dv_offset;
    uint64_t output_bytes;
} flat_backward_layout;

typedef struct flat_ctx flat_ctx;
typedef struct flat_paged_kv_table flat_paged_kv_table;
typedef struct flat_paged_kv_cache flat_paged_kv_cache;
typedef struct flat_resident_kv_cache flat_resident_kv_cache;

/* ---- context ------------------------------------------------------------------------- */

/* WgpuFlatAttention::new (src/wgpu_backend.rs:177-255): bind to one device.  `stream` is a
 * cudaStream_t (NULL = legacy default stream); the caller owns it, like the wgpu queue. */
int32_t flat_ctx_create(int32_t device, void *stream, flat_ctx **out);
void flat_ctx_destroy(flat_ctx *ctx);
/* Replace the stream later launches are enqueued on.  The new stream is made to wait (on the
 * device, by an event) for everything the context queued on the old one, because consecutive
 * calls share the context's scratch; the host is not blocked. */
int32_t flat_ctx_set_stream(flat_ctx *ctx, void *stream);
const char *flat_status_str(int32_t status);
/* Human-readable detail of the last error on this context (tensor name, actual/expected
 * sizes, CUDA message): the payload of the reference's error variants. */
const char *flat_last_error_detail(const flat_ctx *ctx);
/* Pre-size the context's device scratch (split-KV partials, rotated-operand staging,
 * backward accumulators) so later encode calls do not allocate. */
int32_t flat_ctx_reserve_workspace(flat_ctx *ctx, uint64_t bytes);
uint64_t flat_ctx_workspace_bytes(const flat_ctx *ctx);
/* The bf16 tensor-core backward has two routes to dQ.  With scratch to spare it keeps every bf16
 * dS tile of the dK/dV kernel (32 KiB per visible 128 x 128 (key, query) tile pair:
 * batch * q_heads * N^2 bytes for a causal call, twice that otherwise) and forms dQ from the tiles
 * with one more GEMM, five GEMM units in all; otherwise it recomputes the scores in a second
 * kernel, seven GEMM units and no O(N^2) scratch.  The spill route is taken while its scratch fits
 * `bytes` (default 8 GiB; 0 = never).  Results are bitwise repeatable on either route. */
int32_t flat_ctx_set_backward_scratch_budget(flat_ctx *ctx, uint64_t bytes);
/* Pre-size the context's two cached (cos, sin) tables for calls of up to `rows` positions at
 * `head_dim`, so that RoPE entry points whose positions change from call to call (chunked
 * prefill) recompute into memory that exists instead of freeing and allocating.  Together with
 * flat_ctx_reserve_workspace this makes the encode-style entry points allocation-free, the
 * contract of the reference's encode functions (src/wgpu_decode.rs:1-8). */
int32_t flat_ctx_reserve_rope_tables(flat_ctx *ctx, uint64_t rows, uint64_t head_dim);
/* Number of kernel launches this context has enqueued since creation. */
uint64_t flat_ctx_launch_count(const flat_ctx *ctx);
/* Reads the device status word written by kernels: FLAT_OK, FLAT_ERR_DEVICE_WAIT_TIMEOUT (a
 * bounded wait gave up) or FLAT_ERR_PAGE_OUT_OF_RANGE (a decode kernel met a page-table entry
 * outside the pool and masked its tokens); synchronises the stream and clears the word. */
int32_t flat_ctx_device_status(flat_ctx *ctx);

/* Kernel timing for benchmarks (the reference benches time encode+submit+poll on the host,
 * examples/m15_decode_bench.rs:181-203; here the dominant kernel of each call is bracketed with
 * CUDA events on the context stream).  take: synchronises, returns the summed duration in
 * milliseconds and the number of timed launches since the last take, and clears the record. */
int32_t flat_ctx_set_kernel_timing(flat_ctx *ctx, int32_t enabled);
int32_t flat_ctx_take_kernel_time(flat_ctx *ctx, double *total_ms, uint64_t *timed_launches);

/* WgpuFlatAttention::upload / download_attention (src/wgpu_backend.rs:465-482,588-608):
 * explicit host<->device copies on the context stream; download blocks. */
int32_t flat_upload(flat_ctx *ctx, flat_buffer dst, const void *host_src, uint64_t bytes);
int32_t flat_download(flat_ctx *ctx, void *host_dst, flat_buffer src, uint64_t bytes);
int32_t flat_synchronize(flat_ctx *ctx);

/* ---- forward ------------------------------------------------------------------------- */

/* *Pipeline::layout (src/wgpu_forward_grouped.rs:306-334, src/wgpu_external.rs:153-173):
 * pure, allocation-free. */
int32_t flat_forward_layout_for(int32_t dtype, const flat_attention_shape *shape,
                                flat_forward_layout *out);

/* WgpuFlatAttention::forward_resident (src/wgpu_backend.rs:484-586): MHA, head-major;
 * requires q_heads == kv_heads and query_len == kv_len. */
int32_t flat_forward_mha(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                         const flat_attention_config *config, flat_buffer q, flat_buffer k,
                         flat_buffer v, flat_buffer out_and_lse);

/* WgpuGroupedForwardPipeline::encode (src/wgpu_forward_grouped.rs:531-539): GQA/MQA,
 * head-major, equal length. */
int32_t flat_forward_grouped(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                             const flat_attention_config *config, flat_buffer q, flat_buffer k,
                             flat_buffer v, flat_buffer out_and_lse);

/* Head-major rectangular GQA without RoPE: forward_reference_grouped_asymmetric
 * (src/asymmetric_grouped.rs:230-304). */
int32_t flat_forward_grouped_asymmetric(flat_ctx *ctx, int32_t dtype,
                                        const flat_attention_shape *shape,
                                        const flat_attention_config *config, flat_buffer q,
                                        flat_buffer k, flat_buffer v, flat_buffer out_and_lse);

/* WgpuRotaryGroupedAttention::forward_resident (src/wgpu_rotary_grouped_backend.rs:163-271):
 * head-major GQA with fused RoPE; rotary->query_position_offset == kv_position_offset. */
int32_t flat_forward_grouped_rope(flat_ctx *ctx, int32_t dtype,
                                  const flat_attention_shape *shape,
                                  const flat_attention_config *config,
                                  const flat_rotary_config *rotary, flat_buffer q, flat_buffer k,
                                  flat_buffer v, flat_buffer out_and_lse);

/* ExternalProjectionRotaryGroupedPipeline::encode (src/wgpu_external.rs:198-211):
 * projection layout, equal length, fused RoPE. */
int32_t flat_forward_projection_rope(flat_ctx *ctx, int32_t dtype,
                                     const flat_attention_shape *shape,
                                     const flat_attention_config *config,
                                     const flat_rotary_config *rotary, flat_buffer q,
                                     flat_buffer k, flat_buffer v, flat_buffer out_and_lse);

/* ExternalAsymmetricProjectionRotaryGroupedPipeline::encode / encode_pre_rotated_k
 * (src/wgpu_external_asymmetric.rs:192-211): rectangular projection layout, three position
 * domains, optional pre-rotated K. */
int32_t flat_forward_projection_rope_asymmetric(flat_ctx *ctx, int32_t dtype,
                                                const flat_attention_shape *shape,
                                                const flat_attention_config *config,
                                                const flat_rotary_config *rotary, flat_buffer q,
                                                flat_buffer k, flat_buffer v,
                                                flat_buffer out_and_lse);

/* ExternalAsymmetricProjectionRotaryGroupedPipeline::encode_alibi / encode_pre_rotated_k_alibi
 * (src/wgpu_external_asymmetric.rs:245-282; rotary->rotate_k selects which): the rectangular
 * projection-layout forward with an additive ALiBi score bias,
 *   score = dot * scale + slopes[q_head] * ((bias_kv_offset + key) - (bias_query_offset + query)),
 * added before the online-softmax update (src/attention_bias.rs:82-95, 284-285).
 * `slopes` is a HOST array of slope_count f32 values, one per query head (validated, then copied
 * to the device).  Errors follow validate_alibi (src/wgpu_external_asymmetric.rs:512-545):
 * LENGTH_MISMATCH "ALiBi slopes", NON_FINITE_INPUT with the first bad index,
 * INDEX_SPACE_EXCEEDED above FLAT_ALIBI_MAX_HEADS query heads, POSITION_OVERFLOW when the last
 * query or key position leaves u32. */
#define FLAT_ALIBI_MAX_HEADS 256
int32_t flat_forward_projection_rope_asymmetric_alibi(flat_ctx *ctx, int32_t dtype,
                                                      const flat_attention_shape *shape,
                                                      const flat_attention_config *config,
                                                      const flat_rotary_config *rotary,
                                                      const float *slopes, uint64_t slope_count,
                                                      uint64_t bias_query_offset,
                                                      uint64_t bias_kv_offset, flat_buffer q,
                                                      flat_buffer k, flat_buffer v,
                                                      flat_buffer out_and_lse);

/* ExternalVariableProjectionRotaryGroupedPipeline::encode
 * (src/wgpu_external_variable.rs:190-223): padded variable-length batch; `sequences` is a
 * HOST array of shape->batch entries (validated, then copied to the device); padded query
 * rows get O = 0 and LSE = -inf.  rotary->query_position_offset is ignored (per-sequence). */
int32_t flat_forward_projection_rope_varlen(flat_ctx *ctx, int32_t dtype,
                                            const flat_attention_shape *shape,
                                            const flat_attention_config *config,
                                            const flat_rotary_config *rotary,
                                            const flat_varlen_sequence *sequences,
                                            uint64_t sequence_count, flat_buffer q,
                                            flat_buffer k, flat_buffer v,
                                            flat_buffer out_and_lse);

/* WgpuGroupedForwardPipeline::prepare / encode_prepared (src/wgpu_forward_grouped.rs:352-529;
 * PreparedGroupedForward :54-91): validate a forward pass once - shape, configuration, rotary
 * (NULL = none), buffer sizes - size the scratch it needs, and keep the launch parameters; later
 * flat_forward_encode_prepared calls only enqueue (no validation, no allocation, no
 * synchronisation) on the context's current stream, for as long as the four buffers stay where
 * they were.  `layout` selects head-major or projection tensors; rectangular shapes and
 * pre-rotated K (rotary->rotate_k = 0) are accepted like in the direct entry points.  The handle
 * belongs to the context it was prepared on. */
typedef struct flat_prepared_forward flat_prepared_forward;
int32_t flat_forward_prepare(flat_ctx *ctx, int32_t dtype, int32_t layout, const flat_attention_shape *shape,
                             const flat_attention_config *config, const flat_rotary_config *rotary,
                             flat_buffer q, flat_buffer k, flat_buffer v, flat_buffer out_and_lse,
                             flat_prepared_forward **out);
int32_t flat_forward_encode_prepared(flat_ctx *ctx, const flat_prepared_forward *prepared);
void flat_prepared_forward_destroy(flat_prepared_forward *prepared);

/* WgpuFlatAttention::forward / WgpuGroupedAttention::forward / WgpuRotaryGroupedAttention::forward
 * (src/wgpu_backend.rs:445-463, src/wgpu_grouped_backend.rs:126-146,
 * src/wgpu_rotary_grouped_backend.rs:117-139): host slices in, host [O | LSE] out.  Validates
 * like validate_input (src/lib.rs:428-447: exact element counts, and with check_finite != 0 the
 * first non-finite element of Q, then K, then V, by tensor name and index), uploads into staging
 * owned by the context, launches the forward of `layout` (with RoPE when rotary != NULL,
 * rectangular shapes allowed), downloads and blocks.  The finiteness scan runs on the device,
 * chunk by chunk as the upload lands, and its verdict is read back once before the call returns:
 * a call that returns FLAT_ERR_NON_FINITE_INPUT has no result (the contents of out_and_lse are
 * then unspecified).  Pinned host memory makes the copies asynchronous to the host. */
int32_t flat_forward_host(flat_ctx *ctx, int32_t dtype, int32_t layout, const flat_attention_shape *shape,
                          const flat_attention_config *config, const flat_rotary_config *rotary,
                          const void *q, uint64_t q_elements, const void *k, uint64_t k_elements,
                          const void *v, uint64_t v_elements, int32_t check_finite,
                          void *out_and_lse, uint64_t out_bytes);

/* ---- paged-KV metadata (host only) --------------------------------------------------- */

/* PagedKvTable::new / append / address / telemetry / reset (src/paged_kv.rs:84-188). */
int32_t flat_paged_kv_table_create(uint64_t page_size, uint64_t physical_pages,
                                   flat_paged_kv_table **out);
void flat_paged_kv_table_destroy(flat_paged_kv_table *table);
int32_t flat_paged_kv_table_append(flat_paged_kv_table *table, uint64_t tokens);
/* returns FLAT_OK and fills *out, or FLAT_ERR_EMPTY_TABLE when the reference returns None */
int32_t flat_paged_kv_table_address(const flat_paged_kv_table *table, uint64_t logical_token,
                                    flat_paged_kv_address *out);
int32_t flat_paged_kv_table_telemetry(const flat_paged_kv_table *table,
                                      flat_paged_kv_telemetry *out);
int32_t flat_paged_kv_table_reset(flat_paged_kv_table *table);
uint64_t flat_paged_kv_table_len(const flat_paged_kv_table *table);
uint64_t flat_paged_kv_table_generation(const flat_paged_kv_table *table);
/* WgpuPagedKvTable::from_table (src/wgpu_paged_decode.rs:162-198): flatten the logical ->
 * physical map into u32 entries; *count receives mapped_pages (entries may be NULL to query). */
int32_t flat_paged_kv_table_export(const flat_paged_kv_table *table, uint32_t *entries,
                                   uint64_t capacity, uint64_t *count);

/* ---- KV caches ----------------------------------------------------------------------- */

/* WgpuPagedKvCache::new (src/wgpu_paged_kv_cache.rs:99-146): owns K and V
 * [physical_pages*page_size, kv_heads*head_dim] in device memory. */
int32_t flat_paged_kv_cache_create(flat_ctx *ctx, int32_t dtype, uint64_t page_size,
                                   uint64_t physical_pages, uint64_t kv_heads,
                                   uint64_t head_dim, flat_paged_kv_cache **out);
void flat_paged_kv_cache_destroy(flat_paged_kv_cache *cache);
/* WgpuPagedKvCache::record_append (src/wgpu_paged_kv_cache.rs:206-279): sources are
 * [append_len, kv_heads*head_dim], K already rotated; metadata commits only if every copy
 * was enqueued; *new_len receives the live length. */
int32_t flat_paged_kv_cache_append(flat_paged_kv_cache *cache, flat_buffer k_source,
                                   flat_buffer v_source, uint64_t append_len,
                                   uint64_t *new_len);
/* Same append with RoPE fused into the copy: K rows are raw projections and are rotated
 * at positions kv_position_offset + old_len + i while being written (V copied as is). */
int32_t flat_paged_kv_cache_append_rotating(flat_paged_kv_cache *cache, flat_buffer k_source,
                                            flat_buffer v_source, uint64_t append_len,
                                            float theta, uint64_t kv_position_offset,
                                            uint64_t *new_len);
/* Optional, bf16 caches: keep a binary16 copy of K beside the bf16 K (one more K-sized device
 * allocation, made by this call; existing contents are converted, later appends write both).
 * The chunked prefill rotates Q to binary16, and the tensor core takes both score operands in one
 * format: without the copy every K tile is converted in shared memory inside the attention kernel,
 * with it K tiles are used as they arrive.  The copy holds exactly the bf16 values of the cache
 * (saturated beyond the binary16 range), so results do not change.  Writes made to k_buffer()
 * behind the cache's back are not mirrored.  No counterpart in the reference (its cache is f32). */
int32_t flat_paged_kv_cache_enable_prefill_shadow(flat_paged_kv_cache *cache);
int32_t flat_paged_kv_cache_reset(flat_paged_kv_cache *cache);
uint64_t flat_paged_kv_cache_len(const flat_paged_kv_cache *cache);
uint64_t flat_paged_kv_cache_generation(const flat_paged_kv_cache *cache);
flat_buffer flat_paged_kv_cache_k_buffer(const flat_paged_kv_cache *cache);
flat_buffer flat_paged_kv_cache_v_buffer(const flat_paged_kv_cache *cache);
const flat_paged_kv_table *flat_paged_kv_cache_table(const flat_paged_kv_cache *cache);

/* WgpuResidentKvCache (src/wgpu_kv_cache.rs:104-262): [batch, capacity, kv_heads*head_dim]. */
int32_t flat_resident_kv_cache_create(flat_ctx *ctx, int32_t dtype, uint64_t batch,
                                      uint64_t kv_heads, uint64_t capacity, uint64_t head_dim,
                                      flat_resident_kv_cache **out);
void flat_resident_kv_cache_destroy(flat_resident_kv_cache *cache);
/* sources are [batch, append_len, kv_heads*head_dim] (src/wgpu_kv_cache.rs:212-262) */
int32_t flat_resident_kv_cache_append(flat_resident_kv_cache *cache, flat_buffer k_source,
                                      flat_buffer v_source, uint64_t append_len,
                                      uint64_t *new_len);
void flat_resident_kv_cache_reset(flat_resident_kv_cache *cache);
uint64_t flat_resident_kv_cache_len(const flat_resident_kv_cache *cache);
uint64_t flat_resident_kv_cache_capacity(const flat_resident_kv_cache *cache);
flat_buffer flat_resident_kv_cache_k_buffer(const flat_resident_kv_cache *cache);
flat_buffer flat_resident_kv_cache_v_buffer(const flat_resident_kv_cache *cache);

/* ---- decode -------------------------------------------------------------------------- */

/* ResidentDecodeLayout / PagedDecodeLayout (src/wgpu_decode.rs:437-455,
 * src/wgpu_paged_decode.rs:221-235) of the packed decode output
 * [O(batch*q_heads*head_dim) | LSE(batch*q_heads)]: O in `dtype`, LSE f32 at lse_byte_offset
 * (= q_bytes rounded up to 4).  combined_elements counts values (O and LSE together), the
 * reference's f32 element count. */
typedef struct flat_decode_layout {
    uint64_t q_elements;
    uint64_t output_elements;
    uint64_t lse_elements;
    uint64_t combined_elements;
    uint64_t q_bytes;
    uint64_t lse_byte_offset;
    uint64_t combined_bytes;
} flat_decode_layout;
/* WgpuResidentDecodePipeline::layout / WgpuPagedDecodePipeline::layout
 * (src/wgpu_decode.rs:245-261, src/wgpu_paged_decode.rs:268-283): pure, allocation-free.  `batch`
 * is the number of decoded rows (1 for the single-sequence paged pipeline, num_seqs for the
 * batched entry points).  Errors: ZERO_DIMENSION, INVALID_ROTARY_HEAD_DIM (odd head_dim),
 * UNSUPPORTED_HEAD_DIM (> 128), SHAPE_OVERFLOW. */
int32_t flat_decode_layout_for(int32_t dtype, uint64_t batch, uint64_t q_heads, uint64_t head_dim,
                               flat_decode_layout *out);

/* WgpuResidentDecodePipeline::encode_external_pre_rotated_k (src/wgpu_decode.rs:263-322,
 * 419-435): q_len = 1 per batch row over [batch, kv_capacity, kv_heads*head_dim] with live
 * prefix kv_len; Q [batch, q_heads*head_dim] is raw and rotated at q_rope_position, K is
 * pre-rotated.  Output packed [O(batch*q_heads*head_dim) | LSE(batch*q_heads)]. */
int32_t flat_decode_resident(flat_ctx *ctx, int32_t dtype, uint64_t batch, uint64_t q_heads,
                             uint64_t kv_heads, uint64_t head_dim, uint64_t kv_len,
                             uint64_t kv_capacity, const flat_attention_config *config,
                             float theta, uint64_t q_rope_position, flat_buffer q,
                             flat_buffer k, flat_buffer v, flat_buffer out_and_lse);

/* WgpuPagedDecodePipeline::encode (src/wgpu_paged_decode.rs:300-436): one sequence, page
 * table taken from a PagedKvTable.  K/V physical layout
 * [physical_pages, page_size, kv_heads*head_dim]; output [O(q_heads*head_dim) | LSE(q_heads)]. */
int32_t flat_decode_paged(flat_ctx *ctx, int32_t dtype, const flat_paged_kv_table *table,
                          uint64_t q_heads, uint64_t kv_heads, uint64_t head_dim,
                          const flat_attention_config *config, float theta,
                          uint64_t q_rope_position, flat_buffer q, flat_buffer k, flat_buffer v,
                          flat_buffer out_and_lse);

/* Batched generalisation of the same kernel: num_seqs independent sequences sharing one
 * physical pool.  page_tables is a DEVICE array [num_seqs, max_pages_per_seq] of int32,
 * context_lens / q_rope_positions are DEVICE arrays [num_seqs] of int32.  host_context_lens
 * (and host_page_tables, optional) let the call validate before launch: every used entry
 * < physical_pages, no page shared between sequences, causal visibility per sequence.
 * Q is [num_seqs, q_heads*head_dim]; output [O(num_seqs*q_heads*head_dim) | LSE(num_seqs*q_heads)].
 * kv_splits = 0 lets the library choose the split along KV. */
int32_t flat_decode_paged_batched(flat_ctx *ctx, int32_t dtype, uint64_t num_seqs,
                                  uint64_t q_heads, uint64_t kv_heads, uint64_t head_dim,
                                  uint64_t page_size, uint64_t physical_pages,
                                  uint64_t max_pages_per_seq, const int32_t *page_tables_dev,
                                  const int32_t *context_lens_dev,
                                  const int32_t *q_rope_positions_dev,
                                  const int32_t *host_page_tables,
                                  const int32_t *host_context_lens,
                                  const int32_t *host_q_rope_positions,
                                  const flat_attention_config *config, float theta,
                                  uint32_t kv_splits, flat_buffer q, flat_buffer k,
                                  flat_buffer v, flat_buffer out_and_lse);

/* Per-GPU leg of single-sequence (or few-sequence) long-context decode split along KV across
 * GPUs: this cache holds a slice of each sequence; the result is the slice's normalised O and
 * LSE, both f32, packed [O(num_seqs*q_heads*head_dim) | LSE(num_seqs*q_heads)] - exactly the
 * block a rank contributes to the all-gather.  q_rope_positions are global positions.  The
 * reference never splits KV; there is no counterpart. */
int32_t flat_decode_paged_batched_partial(flat_ctx *ctx, int32_t dtype, uint64_t num_seqs,
                                          uint64_t q_heads, uint64_t kv_heads, uint64_t head_dim,
                                          uint64_t page_size, uint64_t physical_pages,
                                          uint64_t max_pages_per_seq, const int32_t *page_tables_dev,
                                          const int32_t *context_lens_dev,
                                          const int32_t *q_rope_positions_dev,
                                          const int32_t *host_page_tables,
                                          const int32_t *host_context_lens,
                                          const flat_attention_config *config, float theta,
                                          flat_buffer q, flat_buffer k, flat_buffer v,
                                          flat_buffer partial_out_and_lse);

/* Merge of `parts` such blocks laid end to end (the all-gather output): part i starts
 * rows*(head_dim+1) floats after part i-1.  Output packed [O | LSE] in `dtype`. */
int32_t flat_splitkv_merge_packed(flat_ctx *ctx, int32_t dtype, uint64_t parts, uint64_t rows,
                                  uint64_t head_dim, flat_buffer gathered, flat_buffer out_and_lse);

/* The exchange step of KV-split decode over an NCCL communicator (one process per GPU, NVLink /
 * NVSwitch underneath): `gathered` is a DEVICE buffer of world_size blocks of rows*(head_dim+1)
 * f32 whose block `rank` already holds this rank's partial [O | LSE] (as written by
 * flat_decode_paged_batched_partial); the blocks are all-gathered in place with ncclAllGather on
 * the context's stream and merged into out_and_lse on every rank.  nccl_comm is the caller's
 * ncclComm_t; NCCL is looked up in the process at the first call (the library is not linked
 * against it), FLAT_ERR_UNAVAILABLE when it is absent.  Enqueues only; no allocation, no
 * synchronisation.  The reference is single-device (src/wgpu_backend.rs:208-217): no counterpart. */
int32_t flat_splitkv_merge_nccl(flat_ctx *ctx, void *nccl_comm, int32_t rank, int32_t world_size,
                                int32_t dtype, uint64_t rows, uint64_t head_dim, flat_buffer gathered,
                                flat_buffer out_and_lse);

/* One whole KV-split decode step: this rank's partial of its cache slice (arguments as
 * flat_decode_paged_batched_partial; a rank whose host_context_lens are all zero contributes
 * weight zero) written into block `rank` of `gathered`, then flat_splitkv_merge_nccl.  Every rank
 * of the communicator must make the call.  No counterpart in the reference. */
int32_t flat_splitkv_decode_nccl(flat_ctx *ctx, void *nccl_comm, int32_t rank, int32_t world_size,
                                 int32_t dtype, uint64_t num_seqs, uint64_t q_heads, uint64_t kv_heads,
                                 uint64_t head_dim, uint64_t page_size, uint64_t physical_pages,
                                 uint64_t max_pages_per_seq, const int32_t *page_tables_dev,
                                 const int32_t *context_lens_dev, const int32_t *q_rope_positions_dev,
                                 const int32_t *host_page_tables, const int32_t *host_context_lens,
                                 const flat_attention_config *config, float theta, flat_buffer q,
                                 flat_buffer k, flat_buffer v, flat_buffer gathered,
                                 flat_buffer out_and_lse);

/* The same KV-split decode step without a collective library: exchange and merge in ONE kernel over
 * NVLink peer memory.  Each rank owns an exchange object (one device allocation: a staging block,
 * two receive buffers of world_size blocks of rows*(head_dim+1) f32, flags and a step counter) that
 * the other ranks of the box map through CUDA IPC:
 *   flat_splitkv_exchange_create   allocates it for `rows` = num_seqs*q_heads rows of head_dim;
 *   flat_splitkv_exchange_handle   gives the 64-byte handle the host passes to the other ranks by
 *                                  whatever channel it has (a torch.distributed all-gather, MPI, a file);
 *   flat_splitkv_exchange_connect  takes all ranks' handles (world_size * 64 bytes, in rank order; the
 *                                  own entry is ignored) and maps them; FLAT_ERR_UNAVAILABLE when a
 *                                  peer cannot be mapped (no peer access between the two GPUs); an entry
 *                                  equal to the own handle stands for this process's own buffer (a
 *                                  single-process harness in which a rank is absent);
 *   flat_splitkv_decode_peer       one step: this rank's partial into the staging block, then a kernel
 *                                  that stores the block into every rank's receive buffer with plain peer
 *                                  stores, raises this rank's flag there, waits until all ranks' flags
 *                                  of this step have arrived here and merges (same arithmetic and the
 *                                  same bits as flat_splitkv_merge_packed).  Every rank must make the
 *                                  call, once per step, in the same order.  Enqueues only, can be
 *                                  captured in a CUDA graph and replayed (the step counter is on the
 *                                  device).  A rank that waits longer than about a second gives up:
 *                                  flat_ctx_device_status then reports FLAT_ERR_DEVICE_WAIT_TIMEOUT,
 *                                  the output of that step is unspecified and the context stays usable;
 *   flat_splitkv_exchange_destroy  synchronises the context's stream, unmaps and frees.
 * At most 16 ranks.  No counterpart in the reference (single-device, src/wgpu_backend.rs:208-217). */
typedef struct flat_splitkv_exchange flat_splitkv_exchange;
int32_t flat_splitkv_exchange_create(flat_ctx *ctx, int32_t rank, int32_t world_size, uint64_t rows,
                                     uint64_t head_dim, flat_splitkv_exchange **out);
int32_t flat_splitkv_exchange_handle(const flat_splitkv_exchange *exchange, uint8_t out[64]);
int32_t flat_splitkv_exchange_connect(flat_splitkv_exchange *exchange, const uint8_t *handles,
                                      uint64_t handle_bytes);
void flat_splitkv_exchange_destroy(flat_splitkv_exchange *exchange);
int32_t flat_splitkv_decode_peer(flat_ctx *ctx, flat_splitkv_exchange *exchange, int32_t dtype,
                                 uint64_t num_seqs, uint64_t q_heads, uint64_t kv_heads,
                                 uint64_t head_dim, uint64_t page_size, uint64_t physical_pages,
                                 uint64_t max_pages_per_seq, const int32_t *page_tables_dev,
                                 const int32_t *context_lens_dev, const int32_t *q_rope_positions_dev,
                                 const int32_t *host_page_tables, const int32_t *host_context_lens,
                                 const flat_attention_config *config, float theta, flat_buffer q,
                                 flat_buffer k, flat_buffer v, flat_buffer out_and_lse);

/* The same batched split-KV decode for callers that cannot allocate device memory when the
 * call is made (a latency-critical serving loop where an allocation would stall the device, a
 * plug-in under a framework allocator that forbids side allocations, or a process whose memory
 * budget was fixed at start-up).  It has no
 * counterpart in the reference.  The per-chunk (O, LSE) partials live in an 8 MiB array that
 * is part of the library image (every GPU that loads the library holds it until exit) instead
 * of the growable context workspace; the call issues no cudaMalloc / cudaFree.
 *  - limit: kv_splits * num_seqs * q_heads * (head_dim + 1) * 4 bytes <= 8 MiB, head_dim a
 *    multiple of 16 bytes, a query-head group of 1, 2, 4 or 8 and 16-byte aligned buffers; an
 *    explicit kv_splits beyond the limit is refused with FLAT_ERR_UNSUPPORTED_SHAPE and a message
 *    giving both sizes.  kv_splits = 0 picks a split that fits.  Whenever the plan comes down to a
 *    single chunk (short contexts, kv_splits = 1, or an explicit split that the 64-token chunk
 *    rounding collapses) the kernel writes O and LSE directly and the array is not touched, so
 *    the first tokens of a sequence decode through this entry point as well.
 *  - the first call on a device that needs the array looks its device address up once
 *    (cudaGetSymbolAddress); make that first call before any stream capture.
 *  - all calls on a device share the array and it keeps the previous call's partials; nothing
 *    in it needs clearing (every live chunk is written before it is read), but two calls that
 *    overlap on the GPU (different streams) race on it.
 *  - arguments are validated like flat_decode_paged_batched (same helper).  There is no host
 *    copy of the page tables here, so sharing of a page between sequences is not checked, and
 *    entries are range-checked on the device instead: an entry outside [0, physical_pages) is
 *    never dereferenced, its tokens are left out of the softmax, and flat_ctx_device_status
 *    then returns FLAT_ERR_PAGE_OUT_OF_RANGE (the regular entry points do the same when they
 *    are called without host_page_tables). */
int32_t flat_decode_paged_batched_static_scratch(
    flat_ctx *ctx, int32_t dtype, uint64_t num_seqs, uint64_t q_heads, uint64_t kv_heads,
    uint64_t head_dim, uint64_t page_size, uint64_t physical_pages, uint64_t max_pages_per_seq,
    const int32_t *page_tables_dev, const int32_t *context_lens_dev,
    const int32_t *q_rope_positions_dev, const int32_t *host_context_lens,
    const int32_t *host_q_rope_positions, const flat_attention_config *config, float theta,
    uint32_t kv_splits, flat_buffer q, flat_buffer k, flat_buffer v, flat_buffer out_and_lse);

/* Split-KV merge over `parts` partial results laid out [parts, rows, head_dim] (O, f32,
 * each normalised within its part) and [parts, rows] (LSE, f32):
 * LSE = log(sum_i exp(LSE_i)), O = sum_i exp(LSE_i - LSE) O_i.  This is the consumer of the
 * all-gathered per-GPU partials of single-sequence long-context decode; the reference has
 * no counterpart (it never splits KV).  Output packed [O | LSE] in `dtype`. */
int32_t flat_splitkv_merge(flat_ctx *ctx, int32_t dtype, uint64_t parts, uint64_t rows,
                           uint64_t head_dim, flat_buffer partial_o, flat_buffer partial_lse,
                           flat_buffer out_and_lse);

/* ---- chunked prefill ----------------------------------------------------------------- */

/* WgpuChunkedProjectionPrefillPipeline::encode (src/wgpu_chunked_prefill.rs:156-299):
 * projection-layout prefill with Q/O/LSE processed in query chunks of query_chunk_size;
 * result identical to the contiguous call (src/chunked_projection_prefill.rs:63-169). */
int32_t flat_chunked_prefill(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                             const flat_attention_config *config,
                             const flat_rotary_config *rotary, uint64_t query_chunk_size,
                             flat_buffer q, flat_buffer k, flat_buffer v,
                             flat_buffer out_and_lse);

/* One prefill chunk against the growing paged cache (chunked prefill composed with
 * WgpuPagedKvCache::record_append, src/wgpu_paged_kv_cache.rs:206-279): the chunk's K rows
 * (raw) are rotated at their absolute positions and appended with V, then the chunk's
 * queries [chunk_len, q_heads*head_dim] attend causally to the whole cache through the page
 * table with query_position_offset = old cache length.  Output packed
 * [O(chunk_len*q_heads*head_dim) | LSE(q_heads*chunk_len)]. */
int32_t flat_chunked_prefill_paged(flat_ctx *ctx, flat_paged_kv_cache *cache, uint64_t q_heads,
                                   uint64_t chunk_len, const flat_attention_config *config,
                                   float theta, uint64_t position_offset, flat_buffer q_chunk,
                                   flat_buffer k_chunk, flat_buffer v_chunk,
                                   flat_buffer out_and_lse);

/* ---- backward ------------------------------------------------------------------------ */

/* GroupedBackwardRecomputePipeline::layout (src/wgpu_backward_grouped.rs:181-215). */
int32_t flat_backward_layout_for(int32_t dtype, const flat_attention_shape *shape,
                                 flat_backward_layout *out);

/* WgpuGroupedBackwardRecomputePipeline::encode (src/wgpu_backward_grouped.rs:318-326) and
 * WgpuBackwardRecomputePipeline::encode (src/wgpu_backward.rs:286-308; the q_heads ==
 * kv_heads case): head-major, equal length, inputs Q,K,V,dO,O,LSE packed per the layout,
 * outputs dQ|dK|dV with dK/dV reduced over each KV head's query-head group.  Gradients are f32
 * in both dtypes (bf16 mode: bf16 Q,K,V,dO,O in, f32 dQ,dK,dV out). */
int32_t flat_backward_grouped(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                              const flat_attention_config *config, flat_buffer packed_inputs,
                              flat_buffer packed_grads);
int32_t flat_backward_mha(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                          const flat_attention_config *config, flat_buffer packed_inputs,
                          flat_buffer packed_grads);

/* WgpuGroupedBackwardRecomputePipeline::prepare / encode_prepared and
 * PreparedGroupedBackwardRecompute (src/wgpu_backward_grouped.rs:231-326): the backward pass
 * validated once, its scratch sized, the launch parameters kept; encode_prepared only enqueues. */
typedef struct flat_prepared_backward flat_prepared_backward;
int32_t flat_backward_prepare(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                              const flat_attention_config *config, flat_buffer packed_inputs,
                              flat_buffer packed_grads, flat_prepared_backward **out);
int32_t flat_backward_encode_prepared(flat_ctx *ctx, const flat_prepared_backward *prepared);
void flat_prepared_backward_destroy(flat_prepared_backward *prepared);

/* ---- precision routing and numerical modes -------------------------------------------- */

/* WgpuIoPrecision (src/wgpu_f16_backend.rs:19-23). */
typedef enum flat_io_precision { FLAT_IO_F32 = 0, FLAT_IO_PACKED_F16 = 1 } flat_io_precision;

/* WgpuPreferredAttention::io_precision_for_head_dim (src/wgpu_f16_backend.rs:491-497):
 * binary16 storage for head_dim 64 and 128, f32 otherwise. */
int32_t flat_preferred_io_precision_for_head_dim(uint64_t head_dim);

/* WgpuPreferredAttention::forward (src/wgpu_f16_backend.rs:505-544): host f32 slices of an MHA
 * shape (q_heads == kv_heads, query_len == kv_len, head-major) in, host f32 [O | LSE] out.
 * Qualified head dims are quantised to binary16 on the device (round to nearest even,
 * F16::from_f32, src/f16.rs:26-82), run through the binary16 forward and expanded again; if any
 * quantised value is not finite the call runs in f32 instead.  Never a CPU path.  Blocks.
 * `*used_precision` (optional) receives the flat_io_precision that ran. */
int32_t flat_preferred_forward_host(flat_ctx *ctx, const flat_attention_shape *shape,
                                    const flat_attention_config *config, const float *q,
                                    uint64_t q_elements, const float *k, uint64_t k_elements,
                                    const float *v, uint64_t v_elements, float *out_and_lse,
                                    uint64_t out_bytes, int32_t *used_precision);

/* NumericalMode and NumericalGuarantees (src/numerical.rs:17-96). */
typedef enum flat_numerical_mode {
    FLAT_NUMERICAL_EXACT_REFERENCE = 0,
    FLAT_NUMERICAL_FAST_PORTABLE = 1,
    FLAT_NUMERICAL_DETERMINISTIC_PORTABLE = 2
} flat_numerical_mode;
typedef enum flat_accumulation_policy {
    FLAT_ACC_SERIAL_FP32 = 0, FLAT_ACC_FIXED_TREE_FP32 = 1, FLAT_ACC_CAPABILITY_OPTIMIZED_FP32 = 2
} flat_accumulation_policy;
typedef enum flat_reduction_policy {
    FLAT_RED_SERIAL_REFERENCE = 0, FLAT_RED_CAPABILITY_OPTIMIZED = 1, FLAT_RED_FIXED_WORKGROUP_TREE = 2
} flat_reduction_policy;
typedef struct flat_numerical_guarantees {
    int32_t accumulation;   /* flat_accumulation_policy */
    int32_t reduction;      /* flat_reduction_policy */
    int32_t softmax_update; /* 0 = StableOnlineFp32, the only policy */
    int32_t repeatable_same_backend_device;
    int32_t allows_subgroup;
} flat_numerical_guarantees;
int32_t flat_numerical_mode_guarantees(int32_t mode, flat_numerical_guarantees *out);

/* NumericalExecutor::forward (src/numerical.rs:154-256) for host f32 slices of an MHA shape.
 * FAST_PORTABLE and DETERMINISTIC_PORTABLE run the f32-arithmetic generic kernel, whose
 * reduction tree is fixed (bitwise repeatable on one device); EXACT_REFERENCE is CPU execution
 * in the reference and is never presented as a GPU result: it returns FLAT_ERR_UNAVAILABLE
 * here, the library has no CPU path. */
int32_t flat_numerical_forward_host(flat_ctx *ctx, int32_t mode, const flat_attention_shape *shape,
                                    const flat_attention_config *config, const float *q,
                                    uint64_t q_elements, const float *k, uint64_t k_elements,
                                    const float *v, uint64_t v_elements, float *out_and_lse,
                                    uint64_t out_bytes);

/* ---- runtime telemetry (src/runtime_telemetry.rs:10-177) ------------------------------ */
/* Passive host-side metadata: none of these calls launches a kernel, touches the stream or
 * synchronises.  Strings are NUL-terminated UTF-8. */

/* RuntimeDeviceFingerprint (src/runtime_telemetry.rs:35-68).  backend is "Cuda"; driver is the
 * CUDA driver API version, driver_info the runtime version, compute capability and SM count;
 * vendor is the PCI vendor id 0x10de; device is compute capability major * 10 + minor. */
typedef struct flat_device_fingerprint {
    char name[256];
    char backend[32];
    char driver[64];
    char driver_info[128];
    uint32_t vendor;
    uint32_t device;
} flat_device_fingerprint;

/* RuntimeDeviceCapabilities (src/runtime_telemetry.rs:99-135) with the CUDA counterparts of the
 * limits: grid x extent, block extents, opt-in shared memory per block, kernel parameter
 * pointers (bind groups have no CUDA counterpart: 0), largest single allocation (clamped to
 * u32), warp size as the subgroup range, f16 arithmetic. */
typedef struct flat_device_capabilities {
    uint32_t max_workgroups_per_dimension;
    uint32_t max_workgroup_size_x, max_workgroup_size_y, max_workgroup_size_z;
    uint32_t max_workgroup_storage_bytes;
    uint32_t max_binding_entries;
    uint32_t max_storage_buffer_binding_size;
    uint32_t subgroup_supported;
    uint32_t subgroup_min_size, subgroup_max_size;
    uint32_t f16_supported;
} flat_device_capabilities;

int32_t flat_ctx_device_fingerprint(const flat_ctx *ctx, flat_device_fingerprint *out);
int32_t flat_ctx_device_capabilities(const flat_ctx *ctx, flat_device_capabilities *out);
/* canonical_record (src/runtime_telemetry.rs:49-59, 116-131): writes at most cap bytes
 * including the NUL and returns the full length without the NUL (snprintf convention), or
 * a negative flat_status. */
int64_t flat_device_fingerprint_canonical_record(const flat_device_fingerprint *fp, char *buf,
                                                 uint64_t cap);
int64_t flat_device_capabilities_canonical_record(const flat_device_capabilities *caps,
                                                  char *buf, uint64_t cap);
/* stable_fingerprint: FNV-1a-64 of the canonical record (src/runtime_telemetry.rs:65-67,
 * 84-91, 133-135). */
uint64_t flat_device_fingerprint_stable(const flat_device_fingerprint *fp);
uint64_t flat_device_capabilities_stable(const flat_device_capabilities *caps);

/* RuntimeKernelId (src/runtime_telemetry.rs:10-20) for this library's kernel families. */
typedef enum flat_kernel_id {
    FLAT_KERNEL_FORWARD_TCGEN05 = 0,  /* fwd_sm100_kernel: bf16, head_dim 64/128 */
    FLAT_KERNEL_FORWARD_GENERIC = 1   /* fwd_simt_kernel: f32 arithmetic, any shape */
} flat_kernel_id;

/* AutotunerCacheStatus (src/runtime_telemetry.rs:138-145). */
typedef enum flat_autotuner_cache {
    FLAT_AUTOTUNER_NOT_APPLICABLE = 0,
    FLAT_AUTOTUNER_HIT = 1,
    FLAT_AUTOTUNER_MISS = 2
} flat_autotuner_cache;

/* RuntimeDispatchTelemetry + RuntimeTileGeometry (src/runtime_telemetry.rs:147-176). */
typedef struct flat_dispatch_telemetry {
    int32_t kernel_id;                   /* flat_kernel_id */
    flat_device_fingerprint device;
    uint32_t query_rows, kv_rows;        /* tile geometry of one work item */
    uint32_t workgroups[3];              /* grid of the attention kernel */
    uint32_t dispatch_count;             /* kernels of one call with warm (cos, sin) tables */
    uint32_t temporary_allocation_count; /* scratch regions of the context workspace used */
    uint64_t temporary_allocation_bytes;
    int32_t has_fallback_reason;
    char fallback_reason[160];           /* why the generic kernel was selected */
    int32_t autotuner_cache;             /* flat_autotuner_cache */
} flat_dispatch_telemetry;

/* WgpuFlatAttention::runtime_telemetry (src/wgpu_backend.rs:370-416): metadata of the dispatch
 * that a forward call of this dtype / layout / shape would select (rotary may be null: no
 * RoPE).  The shape is validated like the forward entry points. */
int32_t flat_forward_runtime_telemetry(flat_ctx *ctx, int32_t dtype, int32_t layout,
                                       const flat_attention_shape *shape,
                                       const flat_rotary_config *rotary,
                                       flat_dispatch_telemetry *out);

/* ---- benchmark manifests (src/benchmark_manifest.rs:10-199) --------------------------- */

/* BenchmarkManifest with its environment, problem and result flattened
 * (src/benchmark_manifest.rs:13-54); strings are NUL-terminated UTF-8. */
typedef struct flat_benchmark_manifest {
    const char *commit_sha, *benchmark_id, *command;
    const char *device, *backend, *driver, *os, *arch; /* BenchmarkEnvironment */
    const char *precision;                             /* BenchmarkProblem */
    uint64_t batch, q_heads, kv_heads, query_len, kv_len, head_dim;
    int32_t causal;
    uint32_t warmup_iterations, measured_iterations;
    uint64_t median_latency_ns, p95_latency_ns, tokens_per_second_milli; /* BenchmarkResult */
} flat_benchmark_manifest;

#define FLAT_BENCHMARK_MANIFEST_SCHEMA_VERSION 1

/* BenchmarkManifest::validate (src/benchmark_manifest.rs:90-137); `*field` (optional) receives
 * the name of the offending field for EMPTY_FIELD / ZERO_DIMENSION (static storage). */
int32_t flat_benchmark_manifest_validate(const flat_benchmark_manifest *m, const char **field);
/* canonical_json (src/benchmark_manifest.rs:140-199): validates, then writes the schema-1
 * payload (snprintf convention: returns the full length without the NUL, or a negative
 * flat_status). */
int64_t flat_benchmark_manifest_canonical_json(const flat_benchmark_manifest *m, char *buf,
                                               uint64_t cap);
/* result_checksum (src/benchmark_manifest.rs:205-209): 16 lower-case hex digits + NUL. */
int32_t flat_benchmark_manifest_result_checksum(const flat_benchmark_manifest *m, char out[17]);

#ifdef __cplusplus
}
#endif
#endif /* FLAT_ATTENTION_B200_H */
