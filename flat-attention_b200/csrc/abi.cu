// Host layer behind the C ABI: contexts, validation (all of it before any launch), the paged-KV
// metadata table, the KV caches and the entry points.  Every entry point mirrors a method of the
// reference's backends; the citations are in include/flat_attention_b200.h.
#include <cmath>
#include <cstring>
#include <limits>
#include <new>

#include "common.h"

namespace flat {

int fail(flat_ctx *ctx, int status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) ctx->detail = buf;
    return status;
}

int ensure_workspace(flat_ctx *ctx, uint64_t bytes) {
    if (bytes <= ctx->workspace_bytes) return FLAT_OK;
    FLAT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->workspace) FLAT_CUDA_OK(ctx, cudaFree(ctx->workspace));
    ctx->workspace = nullptr;
    ctx->workspace_bytes = 0;
    ctx->plan_offsets_at = nullptr;  // whatever the old allocation held is gone
    uint64_t rounded = (bytes + 255) & ~uint64_t(255);
    FLAT_CUDA_OK(ctx, cudaMalloc(&ctx->workspace, rounded));
    ctx->workspace_bytes = rounded;
    return FLAT_OK;
}

int ensure_host_stage(flat_ctx *ctx, uint64_t need) {
    if (need <= ctx->host_stage_bytes) return FLAT_OK;
    FLAT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->host_stage) FLAT_CUDA_OK(ctx, cudaFree(ctx->host_stage));
    ctx->host_stage = nullptr;
    ctx->host_stage_bytes = 0;
    FLAT_CUDA_OK(ctx, cudaMalloc(&ctx->host_stage, need));
    ctx->host_stage_bytes = need;
    return FLAT_OK;
}

namespace {

struct Dims {
    uint64_t q_elements, kv_elements, lse_elements;
};

// api::v1::AttentionShape::validate (src/api.rs:36-59) + the backend limits
// (src/wgpu_backend.rs:626-646): zero dimensions, head grouping, checked products, position
// overflow, head_dim <= 128, every dimension inside the kernels' 32-bit index space.
int validate_shape(flat_ctx *ctx, const flat_attention_shape *s, Dims *d) {
    if (!s) return fail(ctx, FLAT_ERR_NULL_POINTER, "shape is null");
    if (s->batch == 0 || s->q_heads == 0 || s->kv_heads == 0 || s->query_len == 0 || s->kv_len == 0 ||
        s->head_dim == 0)
        return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "attention dimensions must all be non-zero");
    if (s->q_heads % s->kv_heads != 0)
        return fail(ctx, FLAT_ERR_INVALID_HEAD_GROUPING, "q_heads (%llu) must be exactly divisible by kv_heads (%llu)",
                    (unsigned long long)s->q_heads, (unsigned long long)s->kv_heads);
    uint64_t t;
    if (!mul_ok(s->batch, s->q_heads, &t) || !mul_ok(t, s->query_len, &t))
        return fail(ctx, FLAT_ERR_SHAPE_OVERFLOW, "attention shape overflows the address space");
    d->lse_elements = t;
    if (!mul_ok(t, s->head_dim, &d->q_elements))
        return fail(ctx, FLAT_ERR_SHAPE_OVERFLOW, "attention shape overflows the address space");
    if (!mul_ok(s->batch, s->kv_heads, &t) || !mul_ok(t, s->kv_len, &t) || !mul_ok(t, s->head_dim, &d->kv_elements))
        return fail(ctx, FLAT_ERR_SHAPE_OVERFLOW, "attention shape overflows the address space");
    if (!add_ok(s->query_position_offset, s->query_len - 1, &t))
        return fail(ctx, FLAT_ERR_POSITION_OVERFLOW, "query position offset overflows the index space");
    if (s->head_dim > (uint64_t)kMaxHeadDim)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_HEAD_DIM, "head_dim %llu exceeds maximum %d",
                    (unsigned long long)s->head_dim, kMaxHeadDim);
    const uint64_t lim = (uint64_t)std::numeric_limits<int32_t>::max();
    if (s->batch > lim || s->q_heads > lim || s->query_len > lim || s->kv_len > lim || t > lim ||
        d->q_elements > (uint64_t)1 << 46 || d->kv_elements > (uint64_t)1 << 46)
        return fail(ctx, FLAT_ERR_INDEX_SPACE_EXCEEDED, "shape exceeds the kernel index space at %llu elements",
                    (unsigned long long)d->q_elements);
    return FLAT_OK;
}

// FlatAttentionConfig::resolved_scale (src/lib.rs:257-268).
int resolve_scale(flat_ctx *ctx, const flat_attention_config *c, uint64_t head_dim, float *scale) {
    if (!c) return fail(ctx, FLAT_ERR_NULL_POINTER, "config is null");
    float s = c->has_softmax_scale ? c->softmax_scale : 1.0f / std::sqrt((float)head_dim);
    if (!std::isfinite(s) || s <= 0.0f)
        return fail(ctx, FLAT_ERR_INVALID_SCALE, "softmax scale must be finite and positive, got %g", (double)s);
    *scale = s;
    return FLAT_OK;
}

// RotaryEmbeddingConfig::validate (src/rotary_grouped.rs:21-33).
int validate_rotary(flat_ctx *ctx, float theta, uint64_t offset, uint64_t head_dim, uint64_t len) {
    if (head_dim == 0 || head_dim % 2 != 0)
        return fail(ctx, FLAT_ERR_INVALID_ROTARY_HEAD_DIM, "rotary attention head_dim must be non-zero and even, got %llu",
                    (unsigned long long)head_dim);
    if (!std::isfinite(theta) || theta <= 0.0f)
        return fail(ctx, FLAT_ERR_INVALID_ROTARY_THETA, "rotary theta must be finite and positive, got %g", (double)theta);
    uint64_t t;
    if (!add_ok(offset, len ? len - 1 : 0, &t) || t > (uint64_t)std::numeric_limits<uint32_t>::max())
        return fail(ctx, FLAT_ERR_POSITION_OVERFLOW, "rotary position offset overflows the index space");
    return FLAT_OK;
}

// theta^(-2j/D) in f32, exactly the expression of rotated_pair (src/rotary_grouped.rs:44-45).
void fill_inv_freq(float theta, int head_dim, float *out) {
    for (int pair = 0; pair < head_dim / 2; ++pair) {
        float exponent = -2.0f * (float)pair / (float)head_dim;
        out[pair] = powf(theta, exponent);
    }
}

// validate_buffer (src/wgpu_forward_grouped.rs:565-579).
int check_buffer(flat_ctx *ctx, const char *name, flat_buffer b, uint64_t required) {
    if (!b.ptr) return fail(ctx, FLAT_ERR_NULL_POINTER, "%s buffer is null", name);
    if (b.bytes < required)
        return fail(ctx, FLAT_ERR_BUFFER_TOO_SMALL, "%s buffer has %llu bytes, requires %llu", name,
                    (unsigned long long)b.bytes, (unsigned long long)required);
    return FLAT_OK;
}

int check_dtype(flat_ctx *ctx, int dtype) {
    if (dtype == FLAT_F16)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_DTYPE, "binary16 storage is supported by the forward entry points only");
    if (dtype != FLAT_F32 && dtype != FLAT_BF16) return fail(ctx, FLAT_ERR_UNSUPPORTED_DTYPE, "unknown dtype %d", dtype);
    return FLAT_OK;
}

// forward entry points also take IEEE binary16 storage
int check_forward_dtype(flat_ctx *ctx, int dtype) { return dtype == FLAT_F16 ? FLAT_OK : check_dtype(ctx, dtype); }
inline bool storage16(int dtype) { return dtype == FLAT_BF16 || dtype == FLAT_F16; }

uint64_t lse_offset_bytes(int dtype, uint64_t q_elements) {
    uint64_t o = q_elements * dtype_size(dtype);
    return (o + 3) & ~uint64_t(3);
}

struct ForwardCall {
    int dtype;
    int layout;
    bool rope;
    const flat_rotary_config *rotary;
    const flat_varlen_sequence *varlen_host;
    uint64_t varlen_count;
    bool varlen;
    const float *alibi_slopes = nullptr;  // host, [alibi_count]; null = no bias
    uint64_t alibi_count = 0, alibi_q_off = 0, alibi_kv_off = 0;
};

int launch_forward(flat_ctx *ctx, int dtype, const FwdParams &p) {
    if (storage16(dtype) && forward_sm100_supported(p)) return launch_forward_sm100(ctx, p);
    return launch_forward_simt(ctx, dtype, p);
}

// Validates the call and builds the kernel parameters; launches unless `params_out` is given.
int forward_common(flat_ctx *ctx, const ForwardCall &call, const flat_attention_shape *shape,
                   const flat_attention_config *config, flat_buffer q, flat_buffer k, flat_buffer v,
                   flat_buffer out_and_lse, FwdParams *params_out = nullptr) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    int st;
    if ((st = check_forward_dtype(ctx, call.dtype))) return st;
    Dims d;
    if ((st = validate_shape(ctx, shape, &d))) return st;
    float theta = 0.f;
    uint64_t q_rope = 0, kv_rope = 0;
    int rotate_k = 0;
    if (call.rope) {
        if (!call.rotary) return fail(ctx, FLAT_ERR_NULL_POINTER, "rotary config is null");
        theta = call.rotary->theta;
        q_rope = call.rotary->query_position_offset;
        kv_rope = call.rotary->kv_position_offset;
        rotate_k = call.rotary->rotate_k;
        if ((st = validate_rotary(ctx, theta, call.varlen ? 0 : q_rope, shape->head_dim, shape->query_len))) return st;
        if ((st = validate_rotary(ctx, theta, kv_rope, shape->head_dim, shape->kv_len))) return st;
    }
    float scale;
    if ((st = resolve_scale(ctx, config, shape->head_dim, &scale))) return st;
    if (call.varlen) {
        // src/wgpu_external_variable.rs:251-304
        if (!call.varlen_host) return fail(ctx, FLAT_ERR_NULL_POINTER, "sequence metadata is null");
        if (call.varlen_count != shape->batch)
            return fail(ctx, FLAT_ERR_LENGTH_MISMATCH, "tensor active sequence metadata contains %llu elements, expected %llu",
                        (unsigned long long)call.varlen_count, (unsigned long long)shape->batch);
        for (uint64_t b = 0; b < shape->batch; ++b) {
            const flat_varlen_sequence &m = call.varlen_host[b];
            if (m.active_query_len == 0 || m.active_kv_len == 0)
                return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "sequence %llu has a zero active length", (unsigned long long)b);
            if (m.active_query_len > shape->query_len)
                return fail(ctx, FLAT_ERR_LENGTH_MISMATCH, "tensor active query length contains %u elements, expected %llu",
                            m.active_query_len, (unsigned long long)shape->query_len);
            if (m.active_kv_len > shape->kv_len)
                return fail(ctx, FLAT_ERR_LENGTH_MISMATCH, "tensor active KV length contains %u elements, expected %llu",
                            m.active_kv_len, (unsigned long long)shape->kv_len);
            uint64_t lim = std::numeric_limits<uint32_t>::max();
            if ((uint64_t)m.causal_query_offset + m.active_query_len - 1 > lim ||
                (uint64_t)m.query_rope_offset + m.active_query_len - 1 > lim)
                return fail(ctx, FLAT_ERR_POSITION_OVERFLOW, "sequence %llu position overflows u32", (unsigned long long)b);
        }
    }
    if (call.alibi_slopes) {
        // validate_alibi (src/wgpu_external_asymmetric.rs:512-545)
        if (call.alibi_count != shape->q_heads)
            return fail(ctx, FLAT_ERR_LENGTH_MISMATCH, "tensor ALiBi slopes contains %llu elements, expected %llu",
                        (unsigned long long)call.alibi_count, (unsigned long long)shape->q_heads);
        for (uint64_t i = 0; i < call.alibi_count; ++i)
            if (!std::isfinite(call.alibi_slopes[i]))
                return fail(ctx, FLAT_ERR_NON_FINITE_INPUT, "tensor ALiBi slopes contains a non-finite value at index %llu",
                            (unsigned long long)i);
        if (shape->q_heads > FLAT_ALIBI_MAX_HEADS)
            return fail(ctx, FLAT_ERR_INDEX_SPACE_EXCEEDED, "ALiBi supports at most %d query heads, got %llu",
                        FLAT_ALIBI_MAX_HEADS, (unsigned long long)shape->q_heads);
        const uint64_t lim = std::numeric_limits<uint32_t>::max();
        uint64_t q_final, kv_final;
        if (__builtin_add_overflow(call.alibi_q_off, shape->query_len - 1, &q_final) ||
            __builtin_add_overflow(call.alibi_kv_off, shape->kv_len - 1, &kv_final) || q_final > lim || kv_final > lim)
            return fail(ctx, FLAT_ERR_POSITION_OVERFLOW, "ALiBi position offset overflows u32");
    }
    const uint64_t es = dtype_size(call.dtype);
    const uint64_t lse_off = lse_offset_bytes(call.dtype, d.q_elements);
    if ((st = check_buffer(ctx, "Q", q, d.q_elements * es))) return st;
    if ((st = check_buffer(ctx, "K", k, d.kv_elements * es))) return st;
    if ((st = check_buffer(ctx, "V", v, d.kv_elements * es))) return st;
    if ((st = check_buffer(ctx, "O|LSE", out_and_lse, lse_off + d.lse_elements * 4))) return st;

    FwdParams p{};
    p.f16_io = call.dtype == FLAT_F16 ? 1 : 0;
    p.q = q.ptr;
    p.k = k.ptr;
    p.v = v.ptr;
    p.o = out_and_lse.ptr;
    p.lse = reinterpret_cast<float *>(static_cast<char *>(out_and_lse.ptr) + lse_off);
    p.batch = (int)shape->batch;
    p.q_heads = (int)shape->q_heads;
    p.kv_heads = (int)shape->kv_heads;
    p.q_len = (int)shape->query_len;
    p.kv_len = (int)shape->kv_len;
    p.head_dim = (int)shape->head_dim;
    p.group = p.q_heads / p.kv_heads;
    const int64_t D = p.head_dim;
    if (call.layout == FLAT_LAYOUT_HEAD_MAJOR) {
        p.q_rs = D; p.q_hs = (int64_t)p.q_len * D; p.q_bs = p.q_hs * p.q_heads;
        p.kv_rs = D; p.kv_hs = (int64_t)p.kv_len * D; p.kv_bs = p.kv_hs * p.kv_heads;
    } else {
        p.q_hs = D; p.q_rs = (int64_t)p.q_heads * D; p.q_bs = p.q_rs * p.q_len;
        p.kv_hs = D; p.kv_rs = (int64_t)p.kv_heads * D; p.kv_bs = p.kv_rs * p.kv_len;
    }
    p.o_rs = p.q_rs; p.o_hs = p.q_hs; p.o_bs = p.q_bs;
    p.lse_hs = p.q_len;
    p.causal = config->causal ? 1 : 0;
    p.causal_off = (int64_t)shape->query_position_offset;
    p.scale = scale;
    if (call.rope) {
        p.rope_q = 1;
        p.rope_k = rotate_k ? 1 : 0;
        p.q_rope_off = (int64_t)q_rope;
        p.k_rope_off = (int64_t)kv_rope;
        fill_inv_freq(theta, p.head_dim, p.inv_freq);
    }
    if (call.varlen) {
        uint64_t bytes = shape->batch * sizeof(flat_varlen_sequence);
        if (bytes > kWorkspaceMeta)
            return fail(ctx, FLAT_ERR_DISPATCH_LIMIT, "variable-length batch of %llu exceeds %llu sequences",
                        (unsigned long long)shape->batch, (unsigned long long)(kWorkspaceMeta / sizeof(flat_varlen_sequence)));
        p.varlen_rope_min = p.varlen_rope_max = call.varlen_host[0].query_rope_offset;
        for (uint64_t b = 1; b < shape->batch; ++b) {
            p.varlen_rope_min = std::min<int64_t>(p.varlen_rope_min, call.varlen_host[b].query_rope_offset);
            p.varlen_rope_max = std::max<int64_t>(p.varlen_rope_max, call.varlen_host[b].query_rope_offset);
        }
        // the metadata sits at the start of the workspace: size it for the kernel first, a later growth would move it
        p.varlen = reinterpret_cast<const flat_varlen_sequence *>(call.varlen_host);  // non-null for the capability test
        const bool tensor_path = storage16(call.dtype) && forward_sm100_supported(p);
        if ((st = ensure_workspace(ctx, kWorkspaceMeta + (tensor_path ? forward_sm100_workspace_bytes(ctx, p) : 0)))) return st;
        ctx->plan_offsets_at = nullptr;  // the metadata may reach into the part that holds a cached decode plan
        FLAT_CUDA_OK(ctx, cudaMemcpyAsync(ctx->workspace, call.varlen_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
        p.varlen = static_cast<const flat_varlen_sequence *>(ctx->workspace);
        return tensor_path ? launch_forward_sm100(ctx, p) : launch_forward_simt(ctx, call.dtype, p);
    }
    if (call.alibi_slopes) {
        // the slopes take the start of the workspace; size it for the kernel first, a later growth would move them
        p.alibi_slopes = call.alibi_slopes;  // non-null for the capability test
        p.alibi_q_off = (int64_t)call.alibi_q_off;
        p.alibi_kv_off = (int64_t)call.alibi_kv_off;
        for (uint64_t i = 0; i < call.alibi_count; ++i)
            p.alibi_max_abs_slope = std::max(p.alibi_max_abs_slope, std::fabs(call.alibi_slopes[i]));
        const bool tensor_path = storage16(call.dtype) && forward_sm100_supported(p);
        if ((st = ensure_workspace(ctx, kWorkspaceMeta + (tensor_path ? forward_sm100_workspace_bytes(ctx, p) : 0)))) return st;
        FLAT_CUDA_OK(ctx, cudaMemcpyAsync(ctx->workspace, call.alibi_slopes, call.alibi_count * sizeof(float),
                                          cudaMemcpyHostToDevice, ctx->stream));
        p.alibi_slopes = static_cast<const float *>(ctx->workspace);
        return tensor_path ? launch_forward_sm100(ctx, p) : launch_forward_simt(ctx, call.dtype, p);
    }
    if (params_out) {
        *params_out = p;
        return FLAT_OK;
    }
    return launch_forward(ctx, call.dtype, p);
}

}  // namespace
}  // namespace flat

using namespace flat;

// ---- PagedKvTable (src/paged_kv.rs:75-188) ----------------------------------------------------
struct flat_paged_kv_table {
    uint64_t page_size = 0, physical_pages = 0;
    uint64_t live_tokens = 0;
    uint64_t generation = 0;
    std::vector<uint64_t> logical_pages;       // physical page of each logical page
    std::vector<uint64_t> logical_generation;  // generation each entry was mapped in
    std::vector<uint64_t> free_pages;          // popped from the back: lowest page first
};

struct flat_paged_kv_cache {
    flat_ctx *ctx = nullptr;
    int dtype = FLAT_F32;
    uint64_t kv_heads = 0, head_dim = 0;
    uint64_t tensor_bytes = 0;
    void *k = nullptr, *v = nullptr;
    void *k_f16 = nullptr;         // optional binary16 shadow of K for the tensor-core prefill (bf16 caches)
    int32_t *dev_table = nullptr;  // device mirror of the logical -> physical map
    flat_paged_kv_table table;
};

struct flat_resident_kv_cache {
    flat_ctx *ctx = nullptr;
    int dtype = FLAT_F32;
    uint64_t batch = 0, kv_heads = 0, capacity = 0, head_dim = 0, len = 0;
    uint64_t tensor_bytes = 0;
    void *k = nullptr, *v = nullptr;
};

namespace {

int table_init(flat_paged_kv_table *t, uint64_t page_size, uint64_t physical_pages) {
    if (page_size == 0 || physical_pages == 0) return FLAT_ERR_ZERO_DIMENSION;
    uint64_t cap;
    if (!mul_ok(page_size, physical_pages, &cap)) return FLAT_ERR_CAPACITY_OVERFLOW;
    // the free list is materialised and device page tables hold int32 entries: pools beyond 2^28 pages
    // (far more than 180 GB of HBM can back) are refused instead of being allocated
    if (physical_pages > (uint64_t(1) << 28)) return FLAT_ERR_CAPACITY_OVERFLOW;
    t->page_size = page_size;
    t->physical_pages = physical_pages;
    t->free_pages.clear();
    t->free_pages.reserve(physical_pages);
    for (uint64_t p = physical_pages; p-- > 0;) t->free_pages.push_back(p);
    return FLAT_OK;
}

int table_append(flat_paged_kv_table *t, uint64_t tokens) {
    if (tokens == 0) return FLAT_OK;
    uint64_t new_len;
    if (!add_ok(t->live_tokens, tokens, &new_len)) return FLAT_ERR_CAPACITY_OVERFLOW;
    const uint64_t capacity = t->page_size * t->physical_pages;
    if (new_len > capacity) return FLAT_ERR_CAPACITY_EXCEEDED;
    const uint64_t required = (new_len + t->page_size - 1) / t->page_size;
    while (t->logical_pages.size() < required) {
        t->logical_pages.push_back(t->free_pages.back());
        t->logical_generation.push_back(t->generation);
        t->free_pages.pop_back();
    }
    t->live_tokens = new_len;
    return FLAT_OK;
}

bool table_address(const flat_paged_kv_table *t, uint64_t token, flat_paged_kv_address *out) {
    if (token >= t->live_tokens) return false;
    const uint64_t lp = token / t->page_size;
    if (lp >= t->logical_pages.size() || t->logical_generation[lp] != t->generation) return false;
    out->physical_page = t->logical_pages[lp];
    out->offset_in_page = token % t->page_size;
    out->generation = t->logical_generation[lp];
    return true;
}

int table_reset(flat_paged_kv_table *t) {
    if (t->generation == std::numeric_limits<uint64_t>::max()) return FLAT_ERR_GENERATION_OVERFLOW;
    t->generation += 1;
    t->live_tokens = 0;
    t->logical_pages.clear();
    t->logical_generation.clear();
    t->free_pages.clear();
    for (uint64_t p = t->physical_pages; p-- > 0;) t->free_pages.push_back(p);
    return FLAT_OK;
}

// Geometry checks shared by the decode entry points (src/wgpu_decode.rs:457-489,
// src/wgpu_paged_decode.rs:439-470).
int validate_decode_geometry(flat_ctx *ctx, uint64_t q_heads, uint64_t kv_heads, uint64_t head_dim, float theta) {
    if (q_heads == 0 || kv_heads == 0 || head_dim == 0)
        return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "decode dimensions must all be non-zero");
    if (q_heads % kv_heads != 0)
        return fail(ctx, FLAT_ERR_INVALID_HEAD_GROUPING, "q_heads (%llu) must be exactly divisible by kv_heads (%llu)",
                    (unsigned long long)q_heads, (unsigned long long)kv_heads);
    if (head_dim % 2 != 0)
        return fail(ctx, FLAT_ERR_INVALID_ROTARY_HEAD_DIM, "rotary attention head_dim must be non-zero and even, got %llu",
                    (unsigned long long)head_dim);
    if (head_dim > (uint64_t)kMaxHeadDim)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_HEAD_DIM, "head_dim %llu exceeds maximum %d", (unsigned long long)head_dim,
                    kMaxHeadDim);
    if (!std::isfinite(theta) || theta <= 0.0f)
        return fail(ctx, FLAT_ERR_INVALID_THETA, "decode RoPE theta must be finite and positive, got %g", (double)theta);
    if (q_heads > (uint64_t)1 << 20) return fail(ctx, FLAT_ERR_DISPATCH_LIMIT, "q_heads %llu too large", (unsigned long long)q_heads);
    return FLAT_OK;
}

// Chooses the split along KV for the streaming decode kernels and returns the scratch bytes the
// launch needs (behind the metadata region).  With kv_splits == 0 and the tensor-core decode
// available the work is balanced: sequences padded to 16 tokens are laid end to end and cut into
// equal spans, one per resident CTA (two per SM); `offsets` receives the start of every sequence
// on that line (num_seqs + 1 entries) and has to be copied to the metadata region by the caller.
// Otherwise every sequence is cut into kv_splits chunks of equal token count.
constexpr uint64_t kSeqOffsetsAt = 48 << 10;  // byte offset of the sequence offsets inside the metadata region

uint64_t plan_decode(flat_ctx *ctx, int dtype, DecodeParams &p, const int32_t *host_lens, uint64_t total_tokens_hint,
                     int max_len_hint, uint32_t kv_splits, std::vector<int32_t> *offsets, uint64_t max_splits = 0) {
    p.kv_splits = 1;
    p.chunk_tokens = 0;
    p.balanced = 0;
    if (!decode_fast_path_ok(dtype, p.head_dim, p.group)) return 0;
    if (kv_splits == 0 && offsets && decode_mma_supported(dtype, p) &&
        (uint64_t)(p.num_seqs + 1) * sizeof(int32_t) <= kWorkspaceMeta - kSeqOffsetsAt) {
        offsets->resize(p.num_seqs + 1);
        int64_t at = 0;
        int max16 = 0;
        for (int s = 0; s < p.num_seqs; ++s) {
            (*offsets)[s] = (int32_t)at;
            const int len = host_lens ? host_lens[s] : p.uniform_len;
            const int len16 = (len + 15) / 16 * 16;
            at += len16;
            if (len16 > max16) max16 = len16;
        }
        if (at < 0x7fffffff) {
            (*offsets)[p.num_seqs] = (int32_t)at;
            const int64_t head_blocks = (p.kv_heads + 7) / 8;
            int64_t ctas = (int64_t)ctx->sm_count * 2 / head_blocks;
            if (ctas < 1) ctas = 1;
            int64_t span = (at + ctas - 1) / ctas;
            span = (span + 15) / 16 * 16;
            if (span < 64) span = 64;
            ctas = (at + span - 1) / span;
            p.balanced = 1;
            p.span_tokens = (int)span;
            p.num_ctas = (int)ctas;
            p.kv_splits = (int)((max16 + span - 1) / span + 1);  // slots per sequence
            return decode_workspace_bytes(p);
        }
    }
    int splits = 1, chunk = 0;
    if (kv_splits > 1) {
        splits = (int)kv_splits;
    } else if (kv_splits == 0) {
        const uint64_t slots = (uint64_t)ctx->sm_count * 2;
        const uint64_t ctas_per_unit = (p.kv_heads + 7) / 8;
        uint64_t want = 4 * slots / ctas_per_unit;
        if (want < 1) want = 1;
        uint64_t c = (total_tokens_hint + want - 1) / want;
        c = (c + 63) / 64 * 64;
        if (c < 64) c = 64;
        splits = (int)((max_len_hint + c - 1) / c);
        if (max_splits && (uint64_t)splits > max_splits) splits = (int)max_splits;  // what a fixed scratch holds
    }
    if (splits > 1) {
        chunk = (max_len_hint + splits - 1) / splits;
        chunk = (chunk + 63) / 64 * 64;
        splits = (max_len_hint + chunk - 1) / chunk;
    }
    if (splits > 1) {
        p.kv_splits = splits;
        p.chunk_tokens = chunk;
    }
    return decode_workspace_bytes(p);
}

// Copies the sequence offsets of a balanced plan into the metadata region (after ensure_workspace).
int upload_decode_plan(flat_ctx *ctx, DecodeParams &p, const std::vector<int32_t> &offsets) {
    if (!p.balanced) return FLAT_OK;
    char *dst = static_cast<char *>(ctx->workspace) + kSeqOffsetsAt;
    // a serving loop decodes the same batch step after step: while the lengths stay inside their 16-token
    // paddings the offsets do not change, and only decode plans write this part of the metadata region
    if (ctx->plan_offsets_at != dst || ctx->plan_offsets != offsets) {
        FLAT_CUDA_OK(ctx, cudaMemcpyAsync(dst, offsets.data(), offsets.size() * sizeof(int32_t), cudaMemcpyHostToDevice,
                                          ctx->stream));
        ctx->plan_offsets = offsets;
        ctx->plan_offsets_at = dst;
    }
    p.seq_offsets = reinterpret_cast<const int32_t *>(dst);
    return FLAT_OK;
}

// Runs the streaming decode kernel, or the generic forward kernel (q_len = 1) for head
// dimensions / group sizes the streaming kernel does not cover.  The scratch must already be
// large enough (plan_decode + ensure_workspace).
int run_decode(flat_ctx *ctx, int dtype, DecodeParams &p) {
    if (!decode_fast_path_ok(dtype, p.head_dim, p.group) ||
        ((uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.o) % 16 != 0) {
        if (p.context_lens || p.q_rope_positions)
            return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE,
                        "batched decode needs head_dim %% %d == 0, group in {1,2,4,8} and 16-byte aligned buffers",
                        dtype == FLAT_BF16 ? 8 : 4);
        FwdParams f{};
        f.q = p.q; f.k = p.k; f.v = p.v; f.o = p.o; f.lse = p.lse;
        f.batch = p.num_seqs; f.q_heads = p.q_heads; f.kv_heads = p.kv_heads; f.q_len = 1; f.kv_len = p.uniform_len;
        f.head_dim = p.head_dim; f.group = p.group;
        const int64_t D = p.head_dim;
        f.q_hs = D; f.q_rs = (int64_t)p.q_heads * D; f.q_bs = f.q_rs;
        f.o_hs = f.q_hs; f.o_rs = f.q_rs; f.o_bs = f.q_bs;
        f.kv_hs = D; f.kv_rs = (int64_t)p.kv_heads * D; f.kv_bs = f.kv_rs * p.seq_stride_rows;
        f.lse_hs = 1;
        f.causal = 0; f.scale = p.scale;
        f.rope_q = p.rope_q; f.rope_k = 0; f.q_rope_off = p.uniform_q_pos;
        std::memcpy(f.inv_freq, p.inv_freq, sizeof f.inv_freq);
        if (p.page_size > 0) {
            f.page_table = p.page_table; f.page_size = p.page_size; f.max_pages = p.max_pages;
            f.page_row_stride = f.kv_rs;
        }
        return launch_forward_simt(ctx, dtype, f);
    }
    if (p.kv_splits > 1) {
        const uint64_t rows = (uint64_t)p.num_seqs * p.q_heads;
        const uint64_t o_bytes = (uint64_t)p.kv_splits * rows * p.head_dim * sizeof(float);
        p.partial_o = reinterpret_cast<float *>(scratch_ptr(ctx));
        p.partial_lse = reinterpret_cast<float *>(scratch_ptr(ctx) + o_bytes);
    }
    return launch_decode(ctx, dtype, p);
}

}  // namespace

extern "C" {

// ---- context ---------------------------------------------------------------------------------
int32_t flat_ctx_create(int32_t device, void *stream, flat_ctx **out) {
    if (!out) return FLAT_ERR_NULL_POINTER;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        cudaGetLastError();
        return FLAT_ERR_UNAVAILABLE;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return FLAT_ERR_UNAVAILABLE;
    if (prop.major != 10) return FLAT_ERR_UNAVAILABLE;  // built for sm_100a only; no fallback
    if (cudaSetDevice(device) != cudaSuccess) return FLAT_ERR_UNAVAILABLE;
    flat_ctx *ctx = new (std::nothrow) flat_ctx;
    if (!ctx) return FLAT_ERR_EXECUTION;
    ctx->device = device;
    ctx->stream = static_cast<cudaStream_t>(stream);
    ctx->sm_count = prop.multiProcessorCount;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    {
        // RuntimeDeviceFingerprint / RuntimeDeviceCapabilities, captured once (src/wgpu_backend.rs:239-316)
        int driver = 0, runtime = 0;
        cudaDriverGetVersion(&driver);
        cudaRuntimeGetVersion(&runtime);
        flat_device_fingerprint &fp = ctx->fingerprint;
        std::snprintf(fp.name, sizeof fp.name, "%s", prop.name);
        std::snprintf(fp.backend, sizeof fp.backend, "Cuda");
        std::snprintf(fp.driver, sizeof fp.driver, "cuda-driver-api %d.%d", driver / 1000, (driver % 1000) / 10);
        std::snprintf(fp.driver_info, sizeof fp.driver_info, "cuda-runtime %d.%d sm_%d%d %d SMs", runtime / 1000,
                      (runtime % 1000) / 10, prop.major, prop.minor, prop.multiProcessorCount);
        fp.vendor = 0x10de;
        fp.device = (uint32_t)(prop.major * 10 + prop.minor);
        flat_device_capabilities &c = ctx->capabilities;
        c.max_workgroups_per_dimension = (uint32_t)prop.maxGridSize[0];
        c.max_workgroup_size_x = (uint32_t)prop.maxThreadsDim[0];
        c.max_workgroup_size_y = (uint32_t)prop.maxThreadsDim[1];
        c.max_workgroup_size_z = (uint32_t)prop.maxThreadsDim[2];
        c.max_workgroup_storage_bytes = (uint32_t)prop.sharedMemPerBlockOptin;
        c.max_binding_entries = 0;
        c.max_storage_buffer_binding_size = (uint32_t)std::min<uint64_t>(prop.totalGlobalMem, 0xffffffffull);
        c.subgroup_supported = 1;
        c.subgroup_min_size = c.subgroup_max_size = (uint32_t)prop.warpSize;
        c.f16_supported = 1;
    }
    if (cudaMalloc(&ctx->dev_status, sizeof(DeviceStatus)) != cudaSuccess ||
        cudaMemset(ctx->dev_status, 0, sizeof(DeviceStatus)) != cudaSuccess) {
        delete ctx;
        return FLAT_ERR_EXECUTION;
    }
    *out = ctx;
    return FLAT_OK;
}

void flat_ctx_destroy(flat_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto &pr : ctx->timed) {
        cudaEventDestroy(pr.first);
        cudaEventDestroy(pr.second);
    }
    if (ctx->workspace) cudaFree(ctx->workspace);
    if (ctx->host_stage) cudaFree(ctx->host_stage);
    for (auto &t : ctx->rope_tables)
        if (t.dev) cudaFree(t.dev);
    for (cudaEvent_t e : ctx->pipe_events) cudaEventDestroy(e);
    if (ctx->stream_switch) cudaEventDestroy(ctx->stream_switch);
    if (ctx->copy_in) cudaStreamDestroy(ctx->copy_in);
    if (ctx->copy_out) cudaStreamDestroy(ctx->copy_out);
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->finite_first) cudaFree(ctx->finite_first);
    if (ctx->finite_first_host) cudaFreeHost(ctx->finite_first_host);
    delete ctx;
}

int32_t flat_ctx_set_stream(flat_ctx *ctx, void *stream) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    cudaStream_t next = static_cast<cudaStream_t>(stream);
    if (ctx->stream != next) {
        // The context's scratch (workspace, metadata region, cached RoPE tables, host staging, the static decode
        // array) is shared by consecutive calls: work queued on the old stream may still read what the first call
        // on the new stream overwrites.  The new stream waits for the old one; the host does not.
        if (!ctx->stream_switch) FLAT_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->stream_switch, cudaEventDisableTiming));
        FLAT_CUDA_OK(ctx, cudaEventRecord(ctx->stream_switch, ctx->stream));
        FLAT_CUDA_OK(ctx, cudaStreamWaitEvent(next, ctx->stream_switch, 0));
    }
    ctx->stream = next;
    return FLAT_OK;
}

const char *flat_status_str(int32_t status) {
    switch (status) {
        case FLAT_OK: return "ok";
        case FLAT_ERR_ZERO_DIMENSION: return "attention dimensions must all be non-zero";
        case FLAT_ERR_SHAPE_OVERFLOW: return "attention shape overflows the address space";
        case FLAT_ERR_INVALID_HEAD_GROUPING: return "q_heads must be exactly divisible by kv_heads";
        case FLAT_ERR_INVALID_ROTARY_HEAD_DIM: return "rotary attention head_dim must be non-zero and even";
        case FLAT_ERR_INVALID_ROTARY_THETA: return "rotary theta must be finite and positive";
        case FLAT_ERR_POSITION_OVERFLOW: return "position offset overflows the index space";
        case FLAT_ERR_LENGTH_MISMATCH: return "tensor length mismatch";
        case FLAT_ERR_INVALID_SCALE: return "softmax scale must be finite and positive";
        case FLAT_ERR_NON_FINITE_INPUT: return "tensor contains a non-finite value";
        case FLAT_ERR_UNSUPPORTED_HEAD_DIM: return "head_dim exceeds the supported maximum";
        case FLAT_ERR_INDEX_SPACE_EXCEEDED: return "shape exceeds the kernel index space";
        case FLAT_ERR_BUFFER_TOO_SMALL: return "buffer too small";
        case FLAT_ERR_UNAVAILABLE: return "no usable sm_100 CUDA device";
        case FLAT_ERR_EXECUTION: return "CUDA execution error";
        case FLAT_ERR_DISPATCH_LIMIT: return "launch grid limit exceeded";
        case FLAT_ERR_UNSUPPORTED_DTYPE: return "unsupported dtype";
        case FLAT_ERR_NULL_POINTER: return "null pointer";
        case FLAT_ERR_MISALIGNED_BUFFER: return "buffer is not sufficiently aligned";
        case FLAT_ERR_UNSUPPORTED_SHAPE: return "shape not supported by this kernel";
        case FLAT_ERR_EMPTY_CACHE: return "decode requires at least one live KV token";
        case FLAT_ERR_INVALID_CACHE_LENGTH: return "KV length exceeds cache capacity";
        case FLAT_ERR_INVALID_QUERY_LEN: return "decode requires query_len == 1";
        case FLAT_ERR_CAUSAL_VISIBILITY_MISMATCH: return "causal decode query cannot see all live KV tokens";
        case FLAT_ERR_EMPTY_TABLE: return "paged decode requires at least one live KV token";
        case FLAT_ERR_PAGE_OUT_OF_RANGE: return "page table entry outside the physical pool";
        case FLAT_ERR_PAGE_SHARED: return "physical page mapped by more than one sequence";
        case FLAT_ERR_INVALID_THETA: return "decode RoPE theta must be finite and positive";
        case FLAT_ERR_CAPACITY_OVERFLOW: return "paged KV capacity overflows";
        case FLAT_ERR_CAPACITY_EXCEEDED: return "KV cache capacity exceeded";
        case FLAT_ERR_GENERATION_OVERFLOW: return "paged KV generation counter overflowed";
        case FLAT_ERR_ZERO_QUERY_CHUNK_SIZE: return "chunked prefill requires a non-zero query chunk size";
        case FLAT_ERR_DEVICE_WAIT_TIMEOUT: return "a bounded device-side wait expired";
        case FLAT_ERR_MANIFEST_INVALID_COMMIT_SHA: return "commit_sha must contain exactly 40 hex digits";
        case FLAT_ERR_MANIFEST_EMPTY_FIELD: return "benchmark manifest field must not be empty";
        case FLAT_ERR_MANIFEST_ZERO_MEASURED_ITERATIONS: return "measured_iterations must be non-zero";
        case FLAT_ERR_MANIFEST_INVALID_PERCENTILE_ORDERING: return "p95 latency must be greater than or equal to median latency";
    }
    return "unknown status";
}

const char *flat_last_error_detail(const flat_ctx *ctx) { return ctx ? ctx->detail.c_str() : ""; }

int32_t flat_ctx_reserve_workspace(flat_ctx *ctx, uint64_t bytes) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    return ensure_workspace(ctx, bytes);
}
uint64_t flat_ctx_workspace_bytes(const flat_ctx *ctx) { return ctx ? ctx->workspace_bytes : 0; }

int32_t flat_ctx_set_backward_scratch_budget(flat_ctx *ctx, uint64_t bytes) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    ctx->backward_scratch_budget = bytes;
    return FLAT_OK;
}

int32_t flat_ctx_reserve_rope_tables(flat_ctx *ctx, uint64_t rows, uint64_t head_dim) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    if (head_dim == 0 || head_dim % 2 != 0 || head_dim > (uint64_t)kMaxHeadDim)
        return fail(ctx, FLAT_ERR_INVALID_ROTARY_HEAD_DIM, "rotary attention head_dim must be non-zero, even and at most %d", kMaxHeadDim);
    if (rows == 0 || rows > ((uint64_t)1 << 31)) return fail(ctx, FLAT_ERR_INDEX_SPACE_EXCEEDED, "table rows out of range");
    const uint64_t bytes = rows * (head_dim / 2) * 2 * sizeof(float);
    for (auto &t : ctx->rope_tables) {
        if (t.bytes >= bytes) continue;
        FLAT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));  // kernels in flight may still read the old table
        if (t.dev) FLAT_CUDA_OK(ctx, cudaFree(t.dev));
        t.dev = nullptr;
        t.bytes = 0;
        t.rows = 0;
        FLAT_CUDA_OK(ctx, cudaMalloc(&t.dev, bytes));
        t.bytes = bytes;
    }
    return FLAT_OK;
}
uint64_t flat_ctx_launch_count(const flat_ctx *ctx) { return ctx ? ctx->launches : 0; }

int32_t flat_ctx_device_status(flat_ctx *ctx) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    DeviceStatus h{};
    FLAT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    FLAT_CUDA_OK(ctx, cudaMemcpy(&h, ctx->dev_status, sizeof h, cudaMemcpyDeviceToHost));
    if (h.code != 0) {
        if (h.code == FLAT_ERR_PAGE_OUT_OF_RANGE)
            fail(ctx, h.code, "a page-table entry of sequence %d lies outside the physical pool; its tokens were masked", h.where);
        else if (h.code == FLAT_ERR_NON_FINITE_INPUT)
            fail(ctx, h.code, "a device-side input scan found a non-finite value (tensor %d)", h.where);
        else
            fail(ctx, h.code, "device wait expired at site %d", h.where);
        cudaMemset(ctx->dev_status, 0, sizeof(DeviceStatus));
    }
    return h.code;
}

int32_t flat_ctx_set_kernel_timing(flat_ctx *ctx, int32_t enabled) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    ctx->timing = enabled != 0;
    return FLAT_OK;
}

int32_t flat_ctx_take_kernel_time(flat_ctx *ctx, double *total_ms, uint64_t *timed_launches) {
    if (!ctx || !total_ms || !timed_launches) return FLAT_ERR_NULL_POINTER;
    FLAT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    double sum = 0.0;
    for (auto &pr : ctx->timed) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, pr.first, pr.second) == cudaSuccess) sum += ms;
        cudaEventDestroy(pr.first);
        cudaEventDestroy(pr.second);
    }
    *total_ms = sum;
    *timed_launches = ctx->timed.size();
    ctx->timed.clear();
    return FLAT_OK;
}

int32_t flat_upload(flat_ctx *ctx, flat_buffer dst, const void *host_src, uint64_t bytes) {
    if (!ctx || !host_src) return FLAT_ERR_NULL_POINTER;
    int st = check_buffer(ctx, "upload destination", dst, bytes);
    if (st) return st;
    FLAT_CUDA_OK(ctx, cudaMemcpyAsync(dst.ptr, host_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return FLAT_OK;
}

int32_t flat_download(flat_ctx *ctx, void *host_dst, flat_buffer src, uint64_t bytes) {
    if (!ctx || !host_dst) return FLAT_ERR_NULL_POINTER;
    int st = check_buffer(ctx, "download source", src, bytes);
    if (st) return st;
    FLAT_CUDA_OK(ctx, cudaMemcpyAsync(host_dst, src.ptr, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    FLAT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    return FLAT_OK;
}

int32_t flat_synchronize(flat_ctx *ctx) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    FLAT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    return FLAT_OK;
}

// ---- forward ---------------------------------------------------------------------------------
int32_t flat_forward_layout_for(int32_t dtype, const flat_attention_shape *shape, flat_forward_layout *out) {
    if (!out) return FLAT_ERR_NULL_POINTER;
    if (dtype != FLAT_F32 && dtype != FLAT_BF16 && dtype != FLAT_F16) return FLAT_ERR_UNSUPPORTED_DTYPE;
    Dims d;
    int st = validate_shape(nullptr, shape, &d);
    if (st) return st;
    const uint64_t es = dtype_size(dtype);
    out->q_elements = d.q_elements;
    out->kv_elements = d.kv_elements;
    out->lse_elements = d.lse_elements;
    out->q_bytes = d.q_elements * es;
    out->kv_bytes = d.kv_elements * es;
    out->lse_byte_offset = lse_offset_bytes(dtype, d.q_elements);
    out->combined_bytes = out->lse_byte_offset + d.lse_elements * 4;
    return FLAT_OK;
}

int32_t flat_forward_mha(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                         const flat_attention_config *config, flat_buffer q, flat_buffer k, flat_buffer v,
                         flat_buffer out_and_lse) {
    if (ctx && shape && shape->q_heads != shape->kv_heads)
        return fail(ctx, FLAT_ERR_INVALID_HEAD_GROUPING, "MHA requires q_heads == kv_heads, got %llu and %llu",
                    (unsigned long long)shape->q_heads, (unsigned long long)shape->kv_heads);
    return flat_forward_grouped(ctx, dtype, shape, config, q, k, v, out_and_lse);
}

int32_t flat_forward_grouped(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                             const flat_attention_config *config, flat_buffer q, flat_buffer k, flat_buffer v,
                             flat_buffer out_and_lse) {
    if (ctx && shape && (shape->query_len != shape->kv_len || shape->query_position_offset != 0))
        return fail(ctx, FLAT_ERR_LENGTH_MISMATCH, "equal-length forward requires query_len == kv_len and offset 0");
    ForwardCall c{dtype, FLAT_LAYOUT_HEAD_MAJOR, false, nullptr, nullptr, 0, false};
    return forward_common(ctx, c, shape, config, q, k, v, out_and_lse);
}

int32_t flat_forward_grouped_asymmetric(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                                        const flat_attention_config *config, flat_buffer q, flat_buffer k,
                                        flat_buffer v, flat_buffer out_and_lse) {
    ForwardCall c{dtype, FLAT_LAYOUT_HEAD_MAJOR, false, nullptr, nullptr, 0, false};
    return forward_common(ctx, c, shape, config, q, k, v, out_and_lse);
}

int32_t flat_forward_grouped_rope(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                                  const flat_attention_config *config, const flat_rotary_config *rotary,
                                  flat_buffer q, flat_buffer k, flat_buffer v, flat_buffer out_and_lse) {
    if (ctx && shape && (shape->query_len != shape->kv_len || shape->query_position_offset != 0))
        return fail(ctx, FLAT_ERR_LENGTH_MISMATCH, "equal-length forward requires query_len == kv_len and offset 0");
    ForwardCall c{dtype, FLAT_LAYOUT_HEAD_MAJOR, true, rotary, nullptr, 0, false};
    return forward_common(ctx, c, shape, config, q, k, v, out_and_lse);
}

int32_t flat_forward_projection_rope(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                                     const flat_attention_config *config, const flat_rotary_config *rotary,
                                     flat_buffer q, flat_buffer k, flat_buffer v, flat_buffer out_and_lse) {
    if (ctx && shape && (shape->query_len != shape->kv_len || shape->query_position_offset != 0))
        return fail(ctx, FLAT_ERR_LENGTH_MISMATCH, "equal-length forward requires query_len == kv_len and offset 0");
    ForwardCall c{dtype, FLAT_LAYOUT_PROJECTION, true, rotary, nullptr, 0, false};
    return forward_common(ctx, c, shape, config, q, k, v, out_and_lse);
}

int32_t flat_forward_projection_rope_asymmetric(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                                                const flat_attention_config *config,
                                                const flat_rotary_config *rotary, flat_buffer q, flat_buffer k,
                                                flat_buffer v, flat_buffer out_and_lse) {
    ForwardCall c{dtype, FLAT_LAYOUT_PROJECTION, true, rotary, nullptr, 0, false};
    return forward_common(ctx, c, shape, config, q, k, v, out_and_lse);
}

// ---- prepared passes (PreparedGroupedForward, src/wgpu_forward_grouped.rs:352-529) ---------------
struct flat_prepared_forward {
    flat_ctx *ctx;
    int dtype;
    FwdParams params;  // validated once; encode_prepared launches from it
};

int32_t flat_forward_prepare(flat_ctx *ctx, int32_t dtype, int32_t layout, const flat_attention_shape *shape,
                             const flat_attention_config *config, const flat_rotary_config *rotary, flat_buffer q,
                             flat_buffer k, flat_buffer v, flat_buffer out_and_lse, flat_prepared_forward **out) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    if (!out) return fail(ctx, FLAT_ERR_NULL_POINTER, "prepared-pass output is null");
    *out = nullptr;
    if (layout != FLAT_LAYOUT_HEAD_MAJOR && layout != FLAT_LAYOUT_PROJECTION)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "unknown layout %d", layout);
    ForwardCall c{dtype, layout, rotary != nullptr, rotary, nullptr, 0, false};
    FwdParams p{};
    int st = forward_common(ctx, c, shape, config, q, k, v, out_and_lse, &p);
    if (st) return st;
    // everything encode_prepared needs is made ready now: the scratch is sized, so encoding never allocates
    if (storage16(dtype) && forward_sm100_supported(p) &&
        (st = ensure_workspace(ctx, kWorkspaceMeta + forward_sm100_workspace_bytes(ctx, p))))
        return st;
    auto *prep = new (std::nothrow) flat_prepared_forward{ctx, dtype, p};
    if (!prep) return fail(ctx, FLAT_ERR_EXECUTION, "out of host memory");
    *out = prep;
    return FLAT_OK;
}

int32_t flat_forward_encode_prepared(flat_ctx *ctx, const flat_prepared_forward *prepared) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    if (!prepared) return fail(ctx, FLAT_ERR_NULL_POINTER, "prepared pass is null");
    if (prepared->ctx != ctx) return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "the pass was prepared on another context");
    return launch_forward(ctx, prepared->dtype, prepared->params);
}

void flat_prepared_forward_destroy(flat_prepared_forward *prepared) { delete prepared; }

int32_t flat_forward_runtime_telemetry(flat_ctx *ctx, int32_t dtype, int32_t layout, const flat_attention_shape *shape,
                                       const flat_rotary_config *rotary, flat_dispatch_telemetry *out) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    if (!out) return fail(ctx, FLAT_ERR_NULL_POINTER, "telemetry output is null");
    if (layout != FLAT_LAYOUT_HEAD_MAJOR && layout != FLAT_LAYOUT_PROJECTION)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "unknown layout %d", layout);
    // the parameter block of the call, built with stand-in buffers (any 256-byte aligned address of sufficient size)
    ForwardCall c{dtype, layout, rotary != nullptr, rotary, nullptr, 0, false};
    const flat_buffer stand_in{reinterpret_cast<void *>(uintptr_t(1) << 20), ~uint64_t(0)};
    const flat_attention_config cfg{1, 0, 0.f};
    FwdParams p{};
    int st = forward_common(ctx, c, shape, &cfg, stand_in, stand_in, stand_in, stand_in, &p);
    if (st) return st;
    std::memset(out, 0, sizeof *out);
    out->device = ctx->fingerprint;
    out->autotuner_cache = FLAT_AUTOTUNER_NOT_APPLICABLE;
    if (storage16(dtype) && forward_sm100_supported(p)) {
        out->kernel_id = FLAT_KERNEL_FORWARD_TCGEN05;
        forward_sm100_geometry(ctx, p, &out->query_rows, &out->kv_rows, out->workgroups, &out->dispatch_count);
        out->temporary_allocation_bytes = forward_sm100_workspace_bytes(ctx, p);
        out->temporary_allocation_count = out->temporary_allocation_bytes ? 1 : 0;
        return FLAT_OK;
    }
    out->kernel_id = FLAT_KERNEL_FORWARD_GENERIC;
    forward_simt_geometry(p, &out->query_rows, &out->kv_rows, out->workgroups);
    out->dispatch_count = 1;
    out->has_fallback_reason = 1;
    if (!storage16(dtype))
        std::snprintf(out->fallback_reason, sizeof out->fallback_reason, "tensor-core specialization requires 16-bit storage");
    else if (p.head_dim != 64 && p.head_dim != 128)
        std::snprintf(out->fallback_reason, sizeof out->fallback_reason,
                      "tensor-core specialization unavailable for head_dim=%d", p.head_dim);
    else if (p.q_len < 32 || p.kv_len < 32)
        std::snprintf(out->fallback_reason, sizeof out->fallback_reason,
                      "tensor-core specialization unavailable for query_len=%d kv_len=%d", p.q_len, p.kv_len);
    else
        std::snprintf(out->fallback_reason, sizeof out->fallback_reason,
                      "tensor-core specialization unavailable for this layout or position range");
    return FLAT_OK;
}

int32_t flat_forward_projection_rope_asymmetric_alibi(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                                                      const flat_attention_config *config,
                                                      const flat_rotary_config *rotary, const float *slopes,
                                                      uint64_t slope_count, uint64_t bias_query_offset,
                                                      uint64_t bias_kv_offset, flat_buffer q, flat_buffer k,
                                                      flat_buffer v, flat_buffer out_and_lse) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    if (!slopes) return fail(ctx, FLAT_ERR_NULL_POINTER, "ALiBi slopes is null");
    ForwardCall c{dtype, FLAT_LAYOUT_PROJECTION, true, rotary, nullptr, 0, false};
    c.alibi_slopes = slopes;
    c.alibi_count = slope_count;
    c.alibi_q_off = bias_query_offset;
    c.alibi_kv_off = bias_kv_offset;
    return forward_common(ctx, c, shape, config, q, k, v, out_and_lse);
}

int32_t flat_forward_projection_rope_varlen(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                                            const flat_attention_config *config, const flat_rotary_config *rotary,
                                            const flat_varlen_sequence *sequences, uint64_t sequence_count,
                                            flat_buffer q, flat_buffer k, flat_buffer v, flat_buffer out_and_lse) {
    ForwardCall c{dtype, FLAT_LAYOUT_PROJECTION, true, rotary, sequences, sequence_count, true};
    return forward_common(ctx, c, shape, config, q, k, v, out_and_lse);
}

// validate_input (src/lib.rs:428-447), host part: the exact length.  Finiteness is scanned on the device, chunk by
// chunk as the upload lands (validate.cu), and reported with the same tensor name and first index.
static int validate_host_tensor(flat_ctx *ctx, const char *name, const void *data, uint64_t actual, uint64_t expected) {
    if (!data) return fail(ctx, FLAT_ERR_NULL_POINTER, "%s is null", name);
    if (actual != expected)
        return fail(ctx, FLAT_ERR_LENGTH_MISMATCH, "tensor %s contains %llu elements, expected %llu", name,
                    (unsigned long long)actual, (unsigned long long)expected);
    return FLAT_OK;
}

int32_t flat_forward_host(flat_ctx *ctx, int32_t dtype, int32_t layout, const flat_attention_shape *shape,
                          const flat_attention_config *config, const flat_rotary_config *rotary, const void *q,
                          uint64_t q_elements, const void *k, uint64_t k_elements, const void *v, uint64_t v_elements,
                          int32_t check_finite, void *out_and_lse, uint64_t out_bytes) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    int st;
    if ((st = check_forward_dtype(ctx, dtype))) return st;
    if (layout != FLAT_LAYOUT_HEAD_MAJOR && layout != FLAT_LAYOUT_PROJECTION)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "unknown layout %d", layout);
    Dims d;
    if ((st = validate_shape(ctx, shape, &d))) return st;
    if (rotary) {
        if ((st = validate_rotary(ctx, rotary->theta, rotary->query_position_offset, shape->head_dim, shape->query_len))) return st;
        if ((st = validate_rotary(ctx, rotary->theta, rotary->kv_position_offset, shape->head_dim, shape->kv_len))) return st;
    }
    if ((st = validate_host_tensor(ctx, "Q", q, q_elements, d.q_elements))) return st;
    if ((st = validate_host_tensor(ctx, "K", k, k_elements, d.kv_elements))) return st;
    if ((st = validate_host_tensor(ctx, "V", v, v_elements, d.kv_elements))) return st;
    float scale;
    if ((st = resolve_scale(ctx, config, shape->head_dim, &scale))) return st;
    const uint64_t es = dtype_size(dtype);
    const uint64_t combined = lse_offset_bytes(dtype, d.q_elements) + d.lse_elements * 4;
    if (!out_and_lse) return fail(ctx, FLAT_ERR_NULL_POINTER, "output is null");
    if (out_bytes < combined)
        return fail(ctx, FLAT_ERR_BUFFER_TOO_SMALL, "O|LSE buffer has %llu bytes, requires %llu", (unsigned long long)out_bytes,
                    (unsigned long long)combined);
    auto up = [](uint64_t x) { return (x + 255) & ~uint64_t(255); };
    const uint64_t qb = up(d.q_elements * es), kb = up(d.kv_elements * es), ob = up(combined);
    const uint64_t need = qb + 2 * kb + ob;
    if ((st = ensure_host_stage(ctx, need))) return st;
    char *base = static_cast<char *>(ctx->host_stage);
    flat_buffer dq{base, qb}, dk{base + qb, kb}, dv{base + qb + kb, kb}, dout{base + qb + 2 * kb, ob};
    ForwardCall c{dtype, layout, rotary != nullptr, rotary, nullptr, 0, false};
    FwdParams p;
    if ((st = forward_common(ctx, c, shape, config, dq, dk, dv, dout, &p))) return st;

    // Batch elements, and in the head-major layout groups of KV heads, are independent: upload, attention and
    // download of consecutive chunks overlap on three streams (PCIe is full duplex), which is where the
    // host-to-host time goes.  Eight chunks measured best on the Llama-3-8B prefill shape (4: 4.87 ms, 8: 4.78 ms,
    // 16: 5.35 ms, 32: 5.87 ms): more chunks shorten fill and drain, but mixed-direction PCIe traffic and the
    // per-chunk enqueue cost grow.
    if (!ctx->copy_in) {
        FLAT_CUDA_OK(ctx, cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
        FLAT_CUDA_OK(ctx, cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
    }
    const int B = p.batch;
    int heads_per_chunk = p.kv_heads;
    if (layout == FLAT_LAYOUT_HEAD_MAJOR) {
        while (heads_per_chunk % 2 == 0 && (int64_t)B * (p.kv_heads / heads_per_chunk) < 8) heads_per_chunk /= 2;
    }
    const int chunks_per_b = p.kv_heads / heads_per_chunk;
    const int n_chunks = B * chunks_per_b;
    while ((int)ctx->pipe_events.size() < 2 * n_chunks + 1) {
        cudaEvent_t e;
        FLAT_CUDA_OK(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        ctx->pipe_events.push_back(e);
    }
    if (check_finite) {
        if (!ctx->finite_first) {
            FLAT_CUDA_OK(ctx, cudaMalloc(reinterpret_cast<void **>(&ctx->finite_first), 3 * sizeof(unsigned long long)));
            FLAT_CUDA_OK(ctx, cudaHostAlloc(reinterpret_cast<void **>(&ctx->finite_first_host), 3 * sizeof(unsigned long long),
                                            cudaHostAllocDefault));
        }
        FLAT_CUDA_OK(ctx, cudaMemsetAsync(ctx->finite_first, 0xff, 3 * sizeof(unsigned long long), ctx->stream));
    }
    // the staging buffers may still be read by earlier work on the context stream
    FLAT_CUDA_OK(ctx, cudaEventRecord(ctx->pipe_events[2 * n_chunks], ctx->stream));
    FLAT_CUDA_OK(ctx, cudaStreamWaitEvent(ctx->copy_in, ctx->pipe_events[2 * n_chunks], 0));
    const uint64_t lse_off = lse_offset_bytes(dtype, d.q_elements);
    const char *hq = static_cast<const char *>(q), *hk = static_cast<const char *>(k), *hv = static_cast<const char *>(v);
    char *ho = static_cast<char *>(out_and_lse);
    for (int c = 0; c < n_chunks; ++c) {
        const int b = c / chunks_per_b, kvh0 = (c % chunks_per_b) * heads_per_chunk;
        // byte offsets and sizes of this chunk; with one chunk per batch element the whole element is contiguous
        // in both layouts, a group of heads is contiguous only in the head-major one
        const uint64_t q_off = ((uint64_t)b * p.q_bs + (uint64_t)kvh0 * p.group * p.q_hs) * es;
        const uint64_t kv_off = ((uint64_t)b * p.kv_bs + (uint64_t)kvh0 * p.kv_hs) * es;
        const uint64_t q_sz = chunks_per_b == 1 ? (uint64_t)p.q_bs * es : (uint64_t)heads_per_chunk * p.group * p.q_hs * es;
        const uint64_t kv_sz = chunks_per_b == 1 ? (uint64_t)p.kv_bs * es : (uint64_t)heads_per_chunk * p.kv_hs * es;
        const uint64_t lse_row0 = ((uint64_t)b * p.q_heads + (uint64_t)kvh0 * p.group) * p.lse_hs;
        const uint64_t lse_sz = (uint64_t)heads_per_chunk * p.group * p.lse_hs * sizeof(float);
        FLAT_CUDA_OK(ctx, cudaMemcpyAsync((char *)dq.ptr + q_off, hq + q_off, q_sz, cudaMemcpyHostToDevice, ctx->copy_in));
        FLAT_CUDA_OK(ctx, cudaMemcpyAsync((char *)dk.ptr + kv_off, hk + kv_off, kv_sz, cudaMemcpyHostToDevice, ctx->copy_in));
        FLAT_CUDA_OK(ctx, cudaMemcpyAsync((char *)dv.ptr + kv_off, hv + kv_off, kv_sz, cudaMemcpyHostToDevice, ctx->copy_in));
        FLAT_CUDA_OK(ctx, cudaEventRecord(ctx->pipe_events[c], ctx->copy_in));
        FLAT_CUDA_OK(ctx, cudaStreamWaitEvent(ctx->stream, ctx->pipe_events[c], 0));
        if (check_finite) {
            FiniteScan scan{};
            scan.seg[0] = {(const char *)dq.ptr + q_off, q_sz / es, q_off / es, 0};
            scan.seg[1] = {(const char *)dk.ptr + kv_off, kv_sz / es, kv_off / es, 1};
            scan.seg[2] = {(const char *)dv.ptr + kv_off, kv_sz / es, kv_off / es, 2};
            scan.first = ctx->finite_first;
            scan.elem_size = (int)es;
            scan.mask16 = dtype == FLAT_F16 ? 0x7c00u : 0x7f80u;  // F16::is_finite (src/f16.rs:112-115); bf16: 8 exponent bits
            if ((st = launch_finite_scan(ctx, scan, ctx->stream))) return st;
        }
        FwdParams pb = p;
        pb.batch = 1;
        pb.q_heads = heads_per_chunk * p.group;
        pb.kv_heads = heads_per_chunk;
        pb.q = (const char *)p.q + q_off;
        pb.k = (const char *)p.k + kv_off;
        pb.v = (const char *)p.v + kv_off;
        pb.o = (char *)p.o + q_off;
        pb.lse = p.lse + lse_row0;
        if ((st = launch_forward(ctx, dtype, pb))) return st;
        FLAT_CUDA_OK(ctx, cudaEventRecord(ctx->pipe_events[n_chunks + c], ctx->stream));
        FLAT_CUDA_OK(ctx, cudaStreamWaitEvent(ctx->copy_out, ctx->pipe_events[n_chunks + c], 0));
        FLAT_CUDA_OK(ctx, cudaMemcpyAsync(ho + q_off, (char *)p.o + q_off, q_sz, cudaMemcpyDeviceToHost, ctx->copy_out));
        FLAT_CUDA_OK(ctx, cudaMemcpyAsync(ho + lse_off + lse_row0 * sizeof(float), (char *)(p.lse + lse_row0), lse_sz,
                                          cudaMemcpyDeviceToHost, ctx->copy_out));
    }
    if (check_finite)
        FLAT_CUDA_OK(ctx, cudaMemcpyAsync(ctx->finite_first_host, ctx->finite_first, 3 * sizeof(unsigned long long),
                                          cudaMemcpyDeviceToHost, ctx->stream));
    FLAT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->copy_out));
    FLAT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    if (check_finite) {
        // the reference validates Q, then K, then V, and names the first offender; an input that fails has no result
        // (what the output buffer received meanwhile is unspecified)
        static const char *const names[3] = {"Q", "K", "V"};
        for (int t = 0; t < 3; ++t)
            if (ctx->finite_first_host[t] != ~0ull)
                return fail(ctx, FLAT_ERR_NON_FINITE_INPUT, "tensor %s contains a non-finite value at index %llu", names[t],
                            ctx->finite_first_host[t]);
    }
    return FLAT_OK;
}

// ---- paged-KV metadata -----------------------------------------------------------------------
int32_t flat_paged_kv_table_create(uint64_t page_size, uint64_t physical_pages, flat_paged_kv_table **out) {
    if (!out) return FLAT_ERR_NULL_POINTER;
    *out = nullptr;
    auto *t = new (std::nothrow) flat_paged_kv_table;
    if (!t) return FLAT_ERR_EXECUTION;
    int st = table_init(t, page_size, physical_pages);
    if (st) {
        delete t;
        return st;
    }
    *out = t;
    return FLAT_OK;
}
void flat_paged_kv_table_destroy(flat_paged_kv_table *table) { delete table; }
int32_t flat_paged_kv_table_append(flat_paged_kv_table *table, uint64_t tokens) {
    return table ? table_append(table, tokens) : FLAT_ERR_NULL_POINTER;
}
int32_t flat_paged_kv_table_address(const flat_paged_kv_table *table, uint64_t logical_token,
                                    flat_paged_kv_address *out) {
    if (!table || !out) return FLAT_ERR_NULL_POINTER;
    return table_address(table, logical_token, out) ? FLAT_OK : FLAT_ERR_EMPTY_TABLE;
}
int32_t flat_paged_kv_table_telemetry(const flat_paged_kv_table *table, flat_paged_kv_telemetry *out) {
    if (!table || !out) return FLAT_ERR_NULL_POINTER;
    out->live_tokens = table->live_tokens;
    out->capacity_tokens = table->page_size * table->physical_pages;
    out->mapped_pages = table->logical_pages.size();
    out->free_pages = table->free_pages.size();
    out->internal_fragmentation_tokens = table->logical_pages.size() * table->page_size - table->live_tokens;
    out->generation = table->generation;
    return FLAT_OK;
}
int32_t flat_paged_kv_table_reset(flat_paged_kv_table *table) {
    return table ? table_reset(table) : FLAT_ERR_NULL_POINTER;
}
uint64_t flat_paged_kv_table_len(const flat_paged_kv_table *table) { return table ? table->live_tokens : 0; }
uint64_t flat_paged_kv_table_generation(const flat_paged_kv_table *table) { return table ? table->generation : 0; }

int32_t flat_paged_kv_table_export(const flat_paged_kv_table *table, uint32_t *entries, uint64_t capacity,
                                   uint64_t *count) {
    if (!table || !count) return FLAT_ERR_NULL_POINTER;
    if (table->live_tokens == 0 || table->logical_pages.empty()) return FLAT_ERR_EMPTY_TABLE;
    *count = table->logical_pages.size();
    if (!entries) return FLAT_OK;
    if (capacity < *count) return FLAT_ERR_BUFFER_TOO_SMALL;
    for (uint64_t i = 0; i < *count; ++i) {
        if (table->logical_pages[i] >= table->physical_pages) return FLAT_ERR_INDEX_SPACE_EXCEEDED;
        entries[i] = (uint32_t)table->logical_pages[i];
    }
    return FLAT_OK;
}

// ---- paged cache -----------------------------------------------------------------------------
int32_t flat_paged_kv_cache_create(flat_ctx *ctx, int32_t dtype, uint64_t page_size, uint64_t physical_pages,
                                   uint64_t kv_heads, uint64_t head_dim, flat_paged_kv_cache **out) {
    if (!ctx || !out) return FLAT_ERR_NULL_POINTER;
    *out = nullptr;
    int st;
    if ((st = check_dtype(ctx, dtype))) return st;
    if (kv_heads == 0 || head_dim == 0) return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "paged cache dimensions must be non-zero");
    auto *c = new (std::nothrow) flat_paged_kv_cache;
    if (!c) return FLAT_ERR_EXECUTION;
    if ((st = table_init(&c->table, page_size, physical_pages))) {
        delete c;
        return fail(ctx, st, "paged KV dimensions invalid");
    }
    uint64_t row, bytes;
    if (!mul_ok(kv_heads, head_dim, &row) || !mul_ok(row, dtype_size(dtype), &row) ||
        !mul_ok(row, page_size * physical_pages, &bytes) || physical_pages > (uint64_t)std::numeric_limits<int32_t>::max()) {
        delete c;
        return fail(ctx, FLAT_ERR_SHAPE_OVERFLOW, "paged cache size overflows");
    }
    c->ctx = ctx;
    c->dtype = dtype;
    c->kv_heads = kv_heads;
    c->head_dim = head_dim;
    c->tensor_bytes = bytes;
    cudaError_t e = cudaMalloc(&c->k, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&c->v, bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&c->dev_table), physical_pages * sizeof(int32_t));
    // Rows of a mapped page that were never appended reach the tensor core with probability 0;
    // they must hold finite values (0 * NaN is NaN), so the storage starts zeroed.
    if (e == cudaSuccess) e = cudaMemsetAsync(c->k, 0, bytes, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(c->v, 0, bytes, ctx->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        flat_paged_kv_cache_destroy(c);
        return fail(ctx, FLAT_ERR_EXECUTION, "cudaMalloc of %llu bytes failed: %s", (unsigned long long)bytes,
                    cudaGetErrorString(e));
    }
    *out = c;
    return FLAT_OK;
}

void flat_paged_kv_cache_destroy(flat_paged_kv_cache *c) {
    if (!c) return;
    if (c->ctx) cudaStreamSynchronize(c->ctx->stream);
    if (c->k) cudaFree(c->k);
    if (c->v) cudaFree(c->v);
    if (c->dev_table) cudaFree(c->dev_table);
    if (c->k_f16) cudaFree(c->k_f16);
    delete c;
}

static int paged_append_impl(flat_paged_kv_cache *c, flat_buffer k_source, flat_buffer v_source, uint64_t append_len,
                             int rotate, float theta, uint64_t kv_position_offset, uint64_t *new_len) {
    if (!c) return FLAT_ERR_NULL_POINTER;
    flat_ctx *ctx = c->ctx;
    if (append_len == 0) return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "append length must be non-zero");
    const uint64_t row_elems = c->kv_heads * c->head_dim;
    uint64_t need;
    if (!mul_ok(append_len, row_elems * dtype_size(c->dtype), &need))
        return fail(ctx, FLAT_ERR_SHAPE_OVERFLOW, "append size overflows");
    int st;
    if ((st = check_buffer(ctx, "K", k_source, need))) return st;
    if ((st = check_buffer(ctx, "V", v_source, need))) return st;
    float inv_freq[kMaxHeadDim / 2] = {};
    if (rotate) {
        if (c->head_dim > (uint64_t)kMaxHeadDim)
            return fail(ctx, FLAT_ERR_UNSUPPORTED_HEAD_DIM, "head_dim %llu exceeds maximum %d",
                        (unsigned long long)c->head_dim, kMaxHeadDim);
        if ((st = validate_rotary(ctx, theta, kv_position_offset + c->table.live_tokens, c->head_dim, append_len))) return st;
        fill_inv_freq(theta, (int)c->head_dim, inv_freq);
    }
    // stage the metadata; commit only once the copy is enqueued (src/wgpu_paged_kv_cache.rs:224-277)
    flat_paged_kv_table staged = c->table;
    st = table_append(&staged, append_len);
    if (st == FLAT_ERR_CAPACITY_EXCEEDED)
        return fail(ctx, st, "paged KV append requires %llu tokens, capacity is %llu",
                    (unsigned long long)(c->table.live_tokens + append_len),
                    (unsigned long long)(c->table.page_size * c->table.physical_pages));
    if (st) return fail(ctx, st, "paged KV append failed");
    const uint64_t old_pages = c->table.logical_pages.size();
    const uint64_t new_pages = staged.logical_pages.size();
    if (new_pages > old_pages) {
        std::vector<int32_t> fresh(new_pages - old_pages);
        for (uint64_t i = old_pages; i < new_pages; ++i) fresh[i - old_pages] = (int32_t)staged.logical_pages[i];
        FLAT_CUDA_OK(ctx, cudaMemcpyAsync(c->dev_table + old_pages, fresh.data(), fresh.size() * sizeof(int32_t),
                                          cudaMemcpyHostToDevice, ctx->stream));
    }
    st = launch_append_rows(ctx, c->dtype, k_source.ptr, v_source.ptr, c->k, c->v, c->k_f16, (int64_t)append_len, (int)row_elems,
                            (int)c->head_dim, c->dev_table, (int)c->table.page_size, (int64_t)c->table.live_tokens, 0,
                            rotate, (int64_t)(kv_position_offset + c->table.live_tokens), inv_freq);
    if (st) return st;
    c->table = std::move(staged);
    if (new_len) *new_len = c->table.live_tokens;
    return FLAT_OK;
}

int32_t flat_paged_kv_cache_append(flat_paged_kv_cache *cache, flat_buffer k_source, flat_buffer v_source,
                                   uint64_t append_len, uint64_t *new_len) {
    return paged_append_impl(cache, k_source, v_source, append_len, 0, 0.f, 0, new_len);
}

int32_t flat_paged_kv_cache_append_rotating(flat_paged_kv_cache *cache, flat_buffer k_source, flat_buffer v_source,
                                            uint64_t append_len, float theta, uint64_t kv_position_offset,
                                            uint64_t *new_len) {
    return paged_append_impl(cache, k_source, v_source, append_len, 1, theta, kv_position_offset, new_len);
}

int32_t flat_paged_kv_cache_enable_prefill_shadow(flat_paged_kv_cache *c) {
    if (!c) return FLAT_ERR_NULL_POINTER;
    flat_ctx *ctx = c->ctx;
    if (c->dtype != FLAT_BF16)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_DTYPE, "the prefill shadow exists for bf16 caches only (an f32 cache needs none)");
    if (c->k_f16) return FLAT_OK;
    cudaError_t e = cudaMalloc(&c->k_f16, c->tensor_bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        c->k_f16 = nullptr;
        return fail(ctx, FLAT_ERR_EXECUTION, "cudaMalloc of %llu bytes failed: %s", (unsigned long long)c->tensor_bytes,
                    cudaGetErrorString(e));
    }
    // what the cache already holds (zeros where nothing was appended yet)
    return launch_shadow_fill(ctx, c->k, c->k_f16, (int64_t)(c->tensor_bytes / 2));
}

int32_t flat_paged_kv_cache_reset(flat_paged_kv_cache *cache) {
    return cache ? table_reset(&cache->table) : FLAT_ERR_NULL_POINTER;
}
uint64_t flat_paged_kv_cache_len(const flat_paged_kv_cache *cache) { return cache ? cache->table.live_tokens : 0; }
uint64_t flat_paged_kv_cache_generation(const flat_paged_kv_cache *cache) { return cache ? cache->table.generation : 0; }
flat_buffer flat_paged_kv_cache_k_buffer(const flat_paged_kv_cache *cache) {
    return cache ? flat_buffer{cache->k, cache->tensor_bytes} : flat_buffer{nullptr, 0};
}
flat_buffer flat_paged_kv_cache_v_buffer(const flat_paged_kv_cache *cache) {
    return cache ? flat_buffer{cache->v, cache->tensor_bytes} : flat_buffer{nullptr, 0};
}
const flat_paged_kv_table *flat_paged_kv_cache_table(const flat_paged_kv_cache *cache) {
    return cache ? &cache->table : nullptr;
}

// ---- resident cache --------------------------------------------------------------------------
int32_t flat_resident_kv_cache_create(flat_ctx *ctx, int32_t dtype, uint64_t batch, uint64_t kv_heads,
                                      uint64_t capacity, uint64_t head_dim, flat_resident_kv_cache **out) {
    if (!ctx || !out) return FLAT_ERR_NULL_POINTER;
    *out = nullptr;
    int st;
    if ((st = check_dtype(ctx, dtype))) return st;
    if (batch == 0 || kv_heads == 0 || capacity == 0 || head_dim == 0)
        return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "resident cache dimensions must be non-zero");
    uint64_t row, bytes;
    if (!mul_ok(kv_heads, head_dim, &row) || !mul_ok(row, dtype_size(dtype), &row) || !mul_ok(batch, capacity, &bytes) ||
        !mul_ok(bytes, row, &bytes))
        return fail(ctx, FLAT_ERR_SHAPE_OVERFLOW, "resident cache size overflows");
    auto *c = new (std::nothrow) flat_resident_kv_cache;
    if (!c) return FLAT_ERR_EXECUTION;
    c->ctx = ctx; c->dtype = dtype; c->batch = batch; c->kv_heads = kv_heads; c->capacity = capacity;
    c->head_dim = head_dim; c->tensor_bytes = bytes;
    cudaError_t e = cudaMalloc(&c->k, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&c->v, bytes);
    if (e == cudaSuccess) e = cudaMemsetAsync(c->k, 0, bytes, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(c->v, 0, bytes, ctx->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        flat_resident_kv_cache_destroy(c);
        return fail(ctx, FLAT_ERR_EXECUTION, "cudaMalloc of %llu bytes failed: %s", (unsigned long long)bytes,
                    cudaGetErrorString(e));
    }
    *out = c;
    return FLAT_OK;
}

void flat_resident_kv_cache_destroy(flat_resident_kv_cache *c) {
    if (!c) return;
    if (c->ctx) cudaStreamSynchronize(c->ctx->stream);
    if (c->k) cudaFree(c->k);
    if (c->v) cudaFree(c->v);
    delete c;
}

int32_t flat_resident_kv_cache_append(flat_resident_kv_cache *c, flat_buffer k_source, flat_buffer v_source,
                                      uint64_t append_len, uint64_t *new_len) {
    if (!c) return FLAT_ERR_NULL_POINTER;
    flat_ctx *ctx = c->ctx;
    if (append_len == 0) return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "append length must be non-zero");
    uint64_t nl;
    if (!add_ok(c->len, append_len, &nl)) return fail(ctx, FLAT_ERR_SHAPE_OVERFLOW, "cache length overflows");
    if (nl > c->capacity)
        return fail(ctx, FLAT_ERR_CAPACITY_EXCEEDED, "append of %llu rows at length %llu exceeds capacity %llu",
                    (unsigned long long)append_len, (unsigned long long)c->len, (unsigned long long)c->capacity);
    const uint64_t row_bytes = c->kv_heads * c->head_dim * dtype_size(c->dtype);
    const uint64_t src_batch_bytes = append_len * row_bytes;
    int st;
    if ((st = check_buffer(ctx, "K", k_source, c->batch * src_batch_bytes))) return st;
    if ((st = check_buffer(ctx, "V", v_source, c->batch * src_batch_bytes))) return st;
    // one strided copy per tensor: source [batch, append_len, row] -> rows len.. of [batch, capacity, row]
    char *kd = static_cast<char *>(c->k) + c->len * row_bytes;
    char *vd = static_cast<char *>(c->v) + c->len * row_bytes;
    FLAT_CUDA_OK(ctx, cudaMemcpy2DAsync(kd, c->capacity * row_bytes, k_source.ptr, src_batch_bytes, src_batch_bytes,
                                        c->batch, cudaMemcpyDeviceToDevice, ctx->stream));
    FLAT_CUDA_OK(ctx, cudaMemcpy2DAsync(vd, c->capacity * row_bytes, v_source.ptr, src_batch_bytes, src_batch_bytes,
                                        c->batch, cudaMemcpyDeviceToDevice, ctx->stream));
    c->len = nl;
    if (new_len) *new_len = nl;
    return FLAT_OK;
}

void flat_resident_kv_cache_reset(flat_resident_kv_cache *cache) {
    if (cache) cache->len = 0;
}
uint64_t flat_resident_kv_cache_len(const flat_resident_kv_cache *cache) { return cache ? cache->len : 0; }
uint64_t flat_resident_kv_cache_capacity(const flat_resident_kv_cache *cache) { return cache ? cache->capacity : 0; }
flat_buffer flat_resident_kv_cache_k_buffer(const flat_resident_kv_cache *cache) {
    return cache ? flat_buffer{cache->k, cache->tensor_bytes} : flat_buffer{nullptr, 0};
}
flat_buffer flat_resident_kv_cache_v_buffer(const flat_resident_kv_cache *cache) {
    return cache ? flat_buffer{cache->v, cache->tensor_bytes} : flat_buffer{nullptr, 0};
}

// ---- decode ----------------------------------------------------------------------------------
int32_t flat_decode_layout_for(int32_t dtype, uint64_t batch, uint64_t q_heads, uint64_t head_dim, flat_decode_layout *out) {
    if (!out) return FLAT_ERR_NULL_POINTER;
    if (dtype != FLAT_F32 && dtype != FLAT_BF16) return FLAT_ERR_UNSUPPORTED_DTYPE;
    // validate_geometry (src/wgpu_paged_decode.rs:439-458) / validate_kv_view (src/wgpu_decode.rs:466-489)
    if (batch == 0 || q_heads == 0 || head_dim == 0) return FLAT_ERR_ZERO_DIMENSION;
    if (head_dim % 2 != 0) return FLAT_ERR_INVALID_ROTARY_HEAD_DIM;
    if (head_dim > (uint64_t)kMaxHeadDim) return FLAT_ERR_UNSUPPORTED_HEAD_DIM;
    uint64_t rows, q_elements, combined;
    if (!mul_ok(batch, q_heads, &rows) || !mul_ok(rows, head_dim, &q_elements) || !add_ok(q_elements, rows, &combined) ||
        q_elements > (uint64_t)1 << 46)
        return FLAT_ERR_SHAPE_OVERFLOW;
    out->q_elements = q_elements;
    out->output_elements = q_elements;
    out->lse_elements = rows;
    out->combined_elements = combined;
    out->q_bytes = q_elements * dtype_size(dtype);
    out->lse_byte_offset = lse_offset_bytes(dtype, q_elements);
    out->combined_bytes = out->lse_byte_offset + rows * 4;
    return FLAT_OK;
}

int32_t flat_decode_resident(flat_ctx *ctx, int32_t dtype, uint64_t batch, uint64_t q_heads, uint64_t kv_heads,
                             uint64_t head_dim, uint64_t kv_len, uint64_t kv_capacity,
                             const flat_attention_config *config, float theta, uint64_t q_rope_position,
                             flat_buffer q, flat_buffer k, flat_buffer v, flat_buffer out_and_lse) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    int st;
    if ((st = check_dtype(ctx, dtype))) return st;
    if (batch == 0) return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "decode batch must be non-zero");
    if ((st = validate_decode_geometry(ctx, q_heads, kv_heads, head_dim, theta))) return st;
    if (kv_len == 0) return fail(ctx, FLAT_ERR_EMPTY_CACHE, "decode requires at least one live KV token");
    if (kv_len > kv_capacity)
        return fail(ctx, FLAT_ERR_INVALID_CACHE_LENGTH, "kv_len %llu exceeds capacity %llu", (unsigned long long)kv_len,
                    (unsigned long long)kv_capacity);
    if (!config) return fail(ctx, FLAT_ERR_NULL_POINTER, "config is null");
    if (config->causal && q_rope_position + 1 < kv_len)
        return fail(ctx, FLAT_ERR_CAUSAL_VISIBILITY_MISMATCH,
                    "causal decode query position %llu cannot see all %llu live KV tokens",
                    (unsigned long long)q_rope_position, (unsigned long long)kv_len);
    if (q_rope_position > (uint64_t)std::numeric_limits<uint32_t>::max() ||
        kv_capacity > (uint64_t)std::numeric_limits<int32_t>::max() || batch > 65535)
        return fail(ctx, FLAT_ERR_INDEX_SPACE_EXCEEDED, "decode position or capacity exceeds the index space");
    float scale;
    if ((st = resolve_scale(ctx, config, head_dim, &scale))) return st;
    const uint64_t es = dtype_size(dtype);
    const uint64_t q_elems = batch * q_heads * head_dim;
    const uint64_t kv_bytes = batch * kv_capacity * kv_heads * head_dim * es;
    const uint64_t lse_off = lse_offset_bytes(dtype, q_elems);
    if ((st = check_buffer(ctx, "Q", q, q_elems * es))) return st;
    if ((st = check_buffer(ctx, "K", k, kv_bytes))) return st;
    if ((st = check_buffer(ctx, "V", v, kv_bytes))) return st;
    if ((st = check_buffer(ctx, "O|LSE", out_and_lse, lse_off + batch * q_heads * 4))) return st;

    DecodeParams p{};
    p.q = q.ptr; p.k = k.ptr; p.v = v.ptr; p.o = out_and_lse.ptr;
    p.lse = reinterpret_cast<float *>(static_cast<char *>(out_and_lse.ptr) + lse_off);
    p.num_seqs = (int)batch; p.q_heads = (int)q_heads; p.kv_heads = (int)kv_heads; p.head_dim = (int)head_dim;
    p.group = (int)(q_heads / kv_heads);
    p.page_size = 0;
    p.status = ctx->dev_status;
    p.uniform_len = (int)kv_len;
    p.uniform_q_pos = (int64_t)q_rope_position;
    p.seq_stride_rows = (int64_t)kv_capacity;
    p.scale = scale;
    p.rope_q = 1;
    fill_inv_freq(theta, p.head_dim, p.inv_freq);
    std::vector<int32_t> offsets;
    const uint64_t scratch = plan_decode(ctx, dtype, p, nullptr, batch * kv_len, (int)kv_len, 0, &offsets);
    if ((st = ensure_workspace(ctx, kWorkspaceMeta + scratch))) return st;
    if ((st = upload_decode_plan(ctx, p, offsets))) return st;
    return run_decode(ctx, dtype, p);
}

int32_t flat_decode_paged(flat_ctx *ctx, int32_t dtype, const flat_paged_kv_table *table, uint64_t q_heads,
                          uint64_t kv_heads, uint64_t head_dim, const flat_attention_config *config, float theta,
                          uint64_t q_rope_position, flat_buffer q, flat_buffer k, flat_buffer v,
                          flat_buffer out_and_lse) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    int st;
    if ((st = check_dtype(ctx, dtype))) return st;
    if (!table) return fail(ctx, FLAT_ERR_NULL_POINTER, "page table is null");
    // src/wgpu_paged_decode.rs:306-336
    if (table->live_tokens == 0 || table->logical_pages.empty())
        return fail(ctx, FLAT_ERR_EMPTY_TABLE, "paged decode requires at least one live KV token");
    if ((st = validate_decode_geometry(ctx, q_heads, kv_heads, head_dim, theta))) return st;
    if (!config) return fail(ctx, FLAT_ERR_NULL_POINTER, "config is null");
    if (config->causal && q_rope_position + 1 < table->live_tokens)
        return fail(ctx, FLAT_ERR_CAUSAL_VISIBILITY_MISMATCH,
                    "paged causal decode query position %llu cannot see all %llu live KV tokens",
                    (unsigned long long)q_rope_position, (unsigned long long)table->live_tokens);
    const uint64_t mapped = table->logical_pages.size();
    if (mapped * table->page_size < table->live_tokens)
        return fail(ctx, FLAT_ERR_INDEX_SPACE_EXCEEDED, "page table covers fewer than %llu live tokens",
                    (unsigned long long)table->live_tokens);
    if (q_rope_position > (uint64_t)std::numeric_limits<uint32_t>::max() ||
        table->live_tokens > (uint64_t)std::numeric_limits<int32_t>::max() ||
        table->physical_pages > (uint64_t)std::numeric_limits<int32_t>::max())
        return fail(ctx, FLAT_ERR_INDEX_SPACE_EXCEEDED, "decode position or length exceeds the index space");
    std::vector<int32_t> entries(mapped);
    for (uint64_t i = 0; i < mapped; ++i) {
        if (table->logical_pages[i] >= table->physical_pages)
            return fail(ctx, FLAT_ERR_PAGE_OUT_OF_RANGE, "logical page %llu maps to physical page %llu of %llu",
                        (unsigned long long)i, (unsigned long long)table->logical_pages[i],
                        (unsigned long long)table->physical_pages);
        entries[i] = (int32_t)table->logical_pages[i];
    }
    float scale;
    if ((st = resolve_scale(ctx, config, head_dim, &scale))) return st;
    const uint64_t es = dtype_size(dtype);
    const uint64_t q_elems = q_heads * head_dim;
    const uint64_t kv_bytes = table->physical_pages * table->page_size * kv_heads * head_dim * es;
    const uint64_t lse_off = lse_offset_bytes(dtype, q_elems);
    if ((st = check_buffer(ctx, "Q", q, q_elems * es))) return st;
    if ((st = check_buffer(ctx, "K", k, kv_bytes))) return st;
    if ((st = check_buffer(ctx, "V", v, kv_bytes))) return st;
    if ((st = check_buffer(ctx, "O|LSE", out_and_lse, lse_off + q_heads * 4))) return st;
    if (mapped * sizeof(int32_t) > kSeqOffsetsAt)
        return fail(ctx, FLAT_ERR_DISPATCH_LIMIT, "single-sequence paged decode maps %llu pages, maximum is %llu",
                    (unsigned long long)mapped, (unsigned long long)(kSeqOffsetsAt / 4));
    DecodeParams p{};
    p.q = q.ptr; p.k = k.ptr; p.v = v.ptr; p.o = out_and_lse.ptr;
    p.lse = reinterpret_cast<float *>(static_cast<char *>(out_and_lse.ptr) + lse_off);
    p.num_seqs = 1; p.q_heads = (int)q_heads; p.kv_heads = (int)kv_heads; p.head_dim = (int)head_dim;
    p.group = (int)(q_heads / kv_heads);
    p.page_size = (int)table->page_size;
    p.max_pages = (int)mapped;
    p.physical_pages = (int)table->physical_pages;
    p.status = ctx->dev_status;
    p.uniform_len = (int)table->live_tokens;
    p.uniform_q_pos = (int64_t)q_rope_position;
    p.scale = scale;
    p.rope_q = 1;
    fill_inv_freq(theta, p.head_dim, p.inv_freq);
    std::vector<int32_t> offsets;
    const uint64_t scratch = plan_decode(ctx, dtype, p, nullptr, table->live_tokens, (int)table->live_tokens, 0, &offsets);
    if ((st = ensure_workspace(ctx, kWorkspaceMeta + scratch))) return st;
    FLAT_CUDA_OK(ctx, cudaMemcpyAsync(ctx->workspace, entries.data(), mapped * sizeof(int32_t), cudaMemcpyHostToDevice,
                                      ctx->stream));
    p.page_table = static_cast<const int32_t *>(ctx->workspace);
    if ((st = upload_decode_plan(ctx, p, offsets))) return st;
    return run_decode(ctx, dtype, p);
}

enum DecodeRoute { kDecodeRegular = 0, kDecodePartialF32 = 1, kDecodeStaticScratch = 2 };

static int32_t decode_paged_batched_impl(flat_ctx *ctx, int32_t dtype, uint64_t num_seqs, uint64_t q_heads,
                                         uint64_t kv_heads, uint64_t head_dim, uint64_t page_size, uint64_t physical_pages,
                                         uint64_t max_pages_per_seq, const int32_t *page_tables_dev,
                                         const int32_t *context_lens_dev, const int32_t *q_rope_positions_dev,
                                         const int32_t *host_page_tables, const int32_t *host_context_lens,
                                         const int32_t *host_q_rope_positions, const flat_attention_config *config,
                                         float theta, uint32_t kv_splits, flat_buffer q, flat_buffer k, flat_buffer v,
                                         flat_buffer out_and_lse, DecodeRoute route) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    const bool out_f32 = route == kDecodePartialF32;
    int st;
    if ((st = check_dtype(ctx, dtype))) return st;
    if (num_seqs == 0 || page_size == 0 || physical_pages == 0 || max_pages_per_seq == 0)
        return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "paged decode dimensions must all be non-zero");
    if ((st = validate_decode_geometry(ctx, q_heads, kv_heads, head_dim, theta))) return st;
    if (!page_tables_dev || !context_lens_dev || !q_rope_positions_dev || !host_context_lens)
        return fail(ctx, FLAT_ERR_NULL_POINTER, "page tables, context lengths and query positions are required");
    if (!config) return fail(ctx, FLAT_ERR_NULL_POINTER, "config is null");
    const uint64_t lim = (uint64_t)std::numeric_limits<int32_t>::max();
    uint64_t pool_rows;
    if (num_seqs > 65535 || physical_pages > lim || max_pages_per_seq > lim || page_size > lim ||
        !mul_ok(physical_pages, page_size, &pool_rows) || pool_rows > lim)
        return fail(ctx, FLAT_ERR_INDEX_SPACE_EXCEEDED, "paged decode geometry exceeds the index space");
    uint64_t total = 0;
    int max_len = 0;
    std::vector<uint8_t> used;
    if (host_page_tables) used.assign(physical_pages, 0);
    for (uint64_t s = 0; s < num_seqs; ++s) {
        const int32_t len = host_context_lens[s];
        if (len <= 0) return fail(ctx, FLAT_ERR_EMPTY_TABLE, "sequence %llu has no live KV token", (unsigned long long)s);
        const uint64_t pages = ((uint64_t)len + page_size - 1) / page_size;
        if (pages > max_pages_per_seq)
            return fail(ctx, FLAT_ERR_INDEX_SPACE_EXCEEDED, "sequence %llu needs %llu pages, table holds %llu",
                        (unsigned long long)s, (unsigned long long)pages, (unsigned long long)max_pages_per_seq);
        if (host_q_rope_positions) {
            if (host_q_rope_positions[s] < 0)
                return fail(ctx, FLAT_ERR_POSITION_OVERFLOW, "sequence %llu has a negative query position", (unsigned long long)s);
            if (config->causal && (int64_t)host_q_rope_positions[s] + 1 < (int64_t)len)
                return fail(ctx, FLAT_ERR_CAUSAL_VISIBILITY_MISMATCH,
                            "paged causal decode query position %d cannot see all %d live KV tokens (sequence %llu)",
                            host_q_rope_positions[s], len, (unsigned long long)s);
        }
        if (host_page_tables) {
            for (uint64_t i = 0; i < pages; ++i) {
                const int32_t e = host_page_tables[s * max_pages_per_seq + i];
                if (e < 0 || (uint64_t)e >= physical_pages)
                    return fail(ctx, FLAT_ERR_PAGE_OUT_OF_RANGE, "sequence %llu logical page %llu maps to physical page %d of %llu",
                                (unsigned long long)s, (unsigned long long)i, e, (unsigned long long)physical_pages);
                if (used[e])
                    return fail(ctx, FLAT_ERR_PAGE_SHARED, "physical page %d is mapped more than once (sequence %llu)", e,
                                (unsigned long long)s);
                used[e] = 1;
            }
        }
        total += (uint64_t)len;
        if (len > max_len) max_len = len;
    }
    float scale;
    if ((st = resolve_scale(ctx, config, head_dim, &scale))) return st;
    const uint64_t es = dtype_size(dtype);
    // q_heads <= 2^20 and head_dim <= 128 (validate_decode_geometry), num_seqs < 2^16, pool rows < 2^31: no product wraps
    const uint64_t rows = num_seqs * q_heads;
    const uint64_t q_elems = rows * head_dim;
    uint64_t kv_bytes;
    if (!mul_ok(pool_rows, kv_heads * head_dim * es, &kv_bytes))
        return fail(ctx, FLAT_ERR_SHAPE_OVERFLOW, "paged cache size overflows");
    const uint64_t lse_off = out_f32 ? q_elems * 4 : lse_offset_bytes(dtype, q_elems);
    if ((st = check_buffer(ctx, "Q", q, q_elems * es))) return st;
    if ((st = check_buffer(ctx, "K", k, kv_bytes))) return st;
    if ((st = check_buffer(ctx, "V", v, kv_bytes))) return st;
    if ((st = check_buffer(ctx, "O|LSE", out_and_lse, lse_off + rows * 4))) return st;

    DecodeParams p{};
    p.q = q.ptr; p.k = k.ptr; p.v = v.ptr; p.o = out_and_lse.ptr;
    p.lse = reinterpret_cast<float *>(static_cast<char *>(out_and_lse.ptr) + lse_off);
    p.num_seqs = (int)num_seqs; p.q_heads = (int)q_heads; p.kv_heads = (int)kv_heads; p.head_dim = (int)head_dim;
    p.group = (int)(q_heads / kv_heads);
    p.page_size = (int)page_size;
    p.max_pages = (int)max_pages_per_seq;
    p.physical_pages = (int)physical_pages;
    p.status = ctx->dev_status;
    p.page_table = page_tables_dev;
    p.context_lens = context_lens_dev;
    p.q_rope_positions = q_rope_positions_dev;
    p.scale = scale;
    p.rope_q = 1;
    p.out_f32 = out_f32 ? 1 : 0;
    fill_inv_freq(theta, p.head_dim, p.inv_freq);
    if (route == kDecodeStaticScratch) {
        // The partials live in the library's fixed device array; nothing here may allocate, so the balanced plan
        // (whose sequence offsets go through the context workspace) and the generic fallback kernel are not used.
        if (!decode_fast_path_ok(dtype, p.head_dim, p.group))
            return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE,
                        "the static-scratch decode needs head_dim %% %d == 0 and a query-head group of 1, 2, 4 or 8",
                        dtype == FLAT_BF16 ? 8 : 4);
        const flat_buffer bufs[] = {q, k, v, out_and_lse};
        const char *names[] = {"Q", "K", "V", "O|LSE"};
        for (int i = 0; i < 4; ++i)
            if ((reinterpret_cast<uintptr_t>(bufs[i].ptr) & 15) != 0)
                return fail(ctx, FLAT_ERR_MISALIGNED_BUFFER, "%s buffer must be 16-byte aligned", names[i]);
        const uint64_t bytes_per_split = rows * (head_dim + 1) * sizeof(float);  // >= 8, < 2^46
        const uint64_t fit = kDecodeStaticScratchBytes / bytes_per_split;
        if (kv_splits > 1 && (uint64_t)kv_splits > fit)
            return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE,
                        "split-KV partials for %u chunks need %llu bytes, the static scratch holds %llu "
                        "(num_seqs*q_heads*(head_dim+1)*4 bytes per chunk)",
                        kv_splits, (unsigned long long)(kv_splits * bytes_per_split),
                        (unsigned long long)kDecodeStaticScratchBytes);
        // automatic plan: as many chunks as fill the machine about four times, clamped to what the array holds
        // (fit == 0: a single chunk, which needs no scratch at all)
        plan_decode(ctx, dtype, p, host_context_lens, total, max_len, kv_splits, nullptr, fit ? fit : 1);
        if (p.kv_splits > 1) {
            float *scratch = nullptr;
            if ((st = decode_static_scratch(ctx, &scratch))) return st;
            p.partial_o = scratch;
            p.partial_lse = scratch + (uint64_t)p.kv_splits * rows * head_dim;
        }
        return launch_decode(ctx, dtype, p);
    }
    std::vector<int32_t> offsets;
    const uint64_t scratch = plan_decode(ctx, dtype, p, host_context_lens, total, max_len, kv_splits, &offsets);
    if ((st = ensure_workspace(ctx, kWorkspaceMeta + scratch))) return st;
    if ((st = upload_decode_plan(ctx, p, offsets))) return st;
    return run_decode(ctx, dtype, p);
}

int32_t flat_decode_paged_batched(flat_ctx *ctx, int32_t dtype, uint64_t num_seqs, uint64_t q_heads,
                                  uint64_t kv_heads, uint64_t head_dim, uint64_t page_size, uint64_t physical_pages,
                                  uint64_t max_pages_per_seq, const int32_t *page_tables_dev,
                                  const int32_t *context_lens_dev, const int32_t *q_rope_positions_dev,
                                  const int32_t *host_page_tables, const int32_t *host_context_lens,
                                  const int32_t *host_q_rope_positions, const flat_attention_config *config,
                                  float theta, uint32_t kv_splits, flat_buffer q, flat_buffer k, flat_buffer v,
                                  flat_buffer out_and_lse) {
    return decode_paged_batched_impl(ctx, dtype, num_seqs, q_heads, kv_heads, head_dim, page_size, physical_pages,
                                     max_pages_per_seq, page_tables_dev, context_lens_dev, q_rope_positions_dev,
                                     host_page_tables, host_context_lens, host_q_rope_positions, config, theta, kv_splits, q,
                                     k, v, out_and_lse, kDecodeRegular);
}

int32_t flat_decode_paged_batched_partial(flat_ctx *ctx, int32_t dtype, uint64_t num_seqs, uint64_t q_heads,
                                          uint64_t kv_heads, uint64_t head_dim, uint64_t page_size,
                                          uint64_t physical_pages, uint64_t max_pages_per_seq,
                                          const int32_t *page_tables_dev, const int32_t *context_lens_dev,
                                          const int32_t *q_rope_positions_dev, const int32_t *host_page_tables,
                                          const int32_t *host_context_lens, const flat_attention_config *config,
                                          float theta, flat_buffer q, flat_buffer k, flat_buffer v,
                                          flat_buffer partial_out_and_lse) {
    // the query position is global while this cache holds a slice of the sequence: the visibility
    // precondition is the caller's (host_q_rope_positions = null skips the per-slice check)
    return decode_paged_batched_impl(ctx, dtype, num_seqs, q_heads, kv_heads, head_dim, page_size, physical_pages,
                                     max_pages_per_seq, page_tables_dev, context_lens_dev, q_rope_positions_dev,
                                     host_page_tables, host_context_lens, nullptr, config, theta, 0, q, k, v,
                                     partial_out_and_lse, kDecodePartialF32);
}

// The batched split-KV decode for callers that must not allocate: same validation and kernels as
// flat_decode_paged_batched, partials in the fixed device array of the library image (decode.cu).
int32_t flat_decode_paged_batched_static_scratch(
    flat_ctx *ctx, int32_t dtype, uint64_t num_seqs, uint64_t q_heads, uint64_t kv_heads, uint64_t head_dim,
    uint64_t page_size, uint64_t physical_pages, uint64_t max_pages_per_seq, const int32_t *page_tables_dev,
    const int32_t *context_lens_dev, const int32_t *q_rope_positions_dev, const int32_t *host_context_lens,
    const int32_t *host_q_rope_positions, const flat_attention_config *config, float theta, uint32_t kv_splits,
    flat_buffer q, flat_buffer k, flat_buffer v, flat_buffer out_and_lse) {
    return decode_paged_batched_impl(ctx, dtype, num_seqs, q_heads, kv_heads, head_dim, page_size, physical_pages,
                                     max_pages_per_seq, page_tables_dev, context_lens_dev, q_rope_positions_dev, nullptr,
                                     host_context_lens, host_q_rope_positions, config, theta, kv_splits, q, k, v,
                                     out_and_lse, kDecodeStaticScratch);
}

int32_t flat_splitkv_merge_packed(flat_ctx *ctx, int32_t dtype, uint64_t parts, uint64_t rows, uint64_t head_dim,
                                  flat_buffer gathered, flat_buffer out_and_lse) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    int st;
    if ((st = check_dtype(ctx, dtype))) return st;
    if (parts == 0 || rows == 0 || head_dim == 0) return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "merge dimensions must be non-zero");
    if (head_dim > (uint64_t)kMaxHeadDim)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_HEAD_DIM, "head_dim %llu exceeds maximum %d", (unsigned long long)head_dim, kMaxHeadDim);
    if (parts > 65536 || rows > ((uint64_t)1 << 31))
        return fail(ctx, FLAT_ERR_INDEX_SPACE_EXCEEDED, "merge geometry exceeds the index space");
    const uint64_t part_floats = rows * (head_dim + 1);
    const uint64_t lse_off = lse_offset_bytes(dtype, rows * head_dim);
    if ((st = check_buffer(ctx, "gathered partials", gathered, parts * part_floats * 4))) return st;
    if ((st = check_buffer(ctx, "O|LSE", out_and_lse, lse_off + rows * 4))) return st;
    const float *base = static_cast<const float *>(gathered.ptr);
    return launch_splitkv_merge(ctx, dtype, (int)parts, (int64_t)rows, (int)head_dim, base, base + rows * head_dim,
                                (int64_t)part_floats, (int64_t)part_floats, out_and_lse.ptr,
                                reinterpret_cast<float *>(static_cast<char *>(out_and_lse.ptr) + lse_off));
}

int32_t flat_splitkv_merge(flat_ctx *ctx, int32_t dtype, uint64_t parts, uint64_t rows, uint64_t head_dim,
                           flat_buffer partial_o, flat_buffer partial_lse, flat_buffer out_and_lse) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    int st;
    if ((st = check_dtype(ctx, dtype))) return st;
    if (parts == 0 || rows == 0 || head_dim == 0) return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "merge dimensions must be non-zero");
    if (head_dim > (uint64_t)kMaxHeadDim)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_HEAD_DIM, "head_dim %llu exceeds maximum %d", (unsigned long long)head_dim, kMaxHeadDim);
    if (parts > 65536 || rows > ((uint64_t)1 << 31))
        return fail(ctx, FLAT_ERR_INDEX_SPACE_EXCEEDED, "merge geometry exceeds the index space");
    const uint64_t lse_off = lse_offset_bytes(dtype, rows * head_dim);
    if ((st = check_buffer(ctx, "partial O", partial_o, parts * rows * head_dim * 4))) return st;
    if ((st = check_buffer(ctx, "partial LSE", partial_lse, parts * rows * 4))) return st;
    if ((st = check_buffer(ctx, "O|LSE", out_and_lse, lse_off + rows * 4))) return st;
    return launch_splitkv_merge(ctx, dtype, (int)parts, (int64_t)rows, (int)head_dim,
                                static_cast<const float *>(partial_o.ptr), static_cast<const float *>(partial_lse.ptr),
                                (int64_t)(rows * head_dim), (int64_t)rows, out_and_lse.ptr,
                                reinterpret_cast<float *>(static_cast<char *>(out_and_lse.ptr) + lse_off));
}

// ---- chunked prefill -------------------------------------------------------------------------
int32_t flat_chunked_prefill(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                             const flat_attention_config *config, const flat_rotary_config *rotary,
                             uint64_t query_chunk_size, flat_buffer q, flat_buffer k, flat_buffer v,
                             flat_buffer out_and_lse) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    if (query_chunk_size == 0)
        return fail(ctx, FLAT_ERR_ZERO_QUERY_CHUNK_SIZE, "chunked projection prefill requires a non-zero query chunk size");
    int st;
    if ((st = check_dtype(ctx, dtype))) return st;
    Dims d;
    if ((st = validate_shape(ctx, shape, &d))) return st;
    if (shape->query_len != shape->kv_len || shape->query_position_offset != 0)
        return fail(ctx, FLAT_ERR_LENGTH_MISMATCH, "chunked prefill requires query_len == kv_len and offset 0");
    if (!rotary) return fail(ctx, FLAT_ERR_NULL_POINTER, "rotary config is null");
    if ((st = validate_rotary(ctx, rotary->theta, rotary->kv_position_offset, shape->head_dim, shape->kv_len))) return st;
    float scale;
    if ((st = resolve_scale(ctx, config, shape->head_dim, &scale))) return st;
    const uint64_t es = dtype_size(dtype);
    const uint64_t lse_off = lse_offset_bytes(dtype, d.q_elements);
    if ((st = check_buffer(ctx, "Q", q, d.q_elements * es))) return st;
    if ((st = check_buffer(ctx, "K", k, d.kv_elements * es))) return st;
    if ((st = check_buffer(ctx, "V", v, d.kv_elements * es))) return st;
    if ((st = check_buffer(ctx, "O|LSE", out_and_lse, lse_off + d.lse_elements * 4))) return st;

    // Chunks are views: the projection layout lets a chunk be addressed by a row offset and the
    // full-sequence strides, so no Q compaction or O/LSE scatter copies are needed.
    const int64_t N = (int64_t)shape->query_len, D = (int64_t)shape->head_dim;
    FwdParams base{};
    base.k = k.ptr; base.v = v.ptr;
    base.batch = (int)shape->batch; base.q_heads = (int)shape->q_heads; base.kv_heads = (int)shape->kv_heads;
    base.kv_len = (int)N; base.head_dim = (int)D; base.group = base.q_heads / base.kv_heads;
    base.q_hs = D; base.q_rs = base.q_heads * D; base.q_bs = base.q_rs * N;
    base.kv_hs = D; base.kv_rs = base.kv_heads * D; base.kv_bs = base.kv_rs * N;
    base.o_hs = base.q_hs; base.o_rs = base.q_rs; base.o_bs = base.q_bs;
    base.lse_hs = N;
    base.causal = config->causal ? 1 : 0;
    base.scale = scale;
    base.rope_q = 1; base.rope_k = 1;
    base.k_rope_off = (int64_t)rotary->kv_position_offset;
    fill_inv_freq(rotary->theta, base.head_dim, base.inv_freq);
    float *lse = reinterpret_cast<float *>(static_cast<char *>(out_and_lse.ptr) + lse_off);
    for (uint64_t start = 0; start < shape->query_len; start += query_chunk_size) {
        const uint64_t len = std::min<uint64_t>(query_chunk_size, shape->query_len - start);
        FwdParams p = base;
        p.q = static_cast<const char *>(q.ptr) + start * base.q_rs * es;
        p.o = static_cast<char *>(out_and_lse.ptr) + start * base.q_rs * es;
        p.lse = lse + start;
        p.q_len = (int)len;
        p.causal_off = (int64_t)start;
        p.q_rope_off = (int64_t)(rotary->kv_position_offset + start);
        if (dtype == FLAT_BF16 && forward_sm100_supported(p)) st = launch_forward_sm100(ctx, p);
        else st = launch_forward_simt(ctx, dtype, p);
        if (st) return st;
    }
    return FLAT_OK;
}

int32_t flat_chunked_prefill_paged(flat_ctx *ctx, flat_paged_kv_cache *cache, uint64_t q_heads, uint64_t chunk_len,
                                   const flat_attention_config *config, float theta, uint64_t position_offset,
                                   flat_buffer q_chunk, flat_buffer k_chunk, flat_buffer v_chunk,
                                   flat_buffer out_and_lse) {
    if (!ctx || !cache) return FLAT_ERR_NULL_POINTER;
    if (chunk_len == 0)
        return fail(ctx, FLAT_ERR_ZERO_QUERY_CHUNK_SIZE, "chunked projection prefill requires a non-zero query chunk size");
    const uint64_t old_len = cache->table.live_tokens;
    flat_attention_shape shape{1, q_heads, cache->kv_heads, chunk_len, old_len + chunk_len, cache->head_dim, old_len};
    int st;
    Dims d;
    if ((st = validate_shape(ctx, &shape, &d))) return st;
    if ((st = validate_rotary(ctx, theta, position_offset + old_len, cache->head_dim, chunk_len))) return st;
    float scale;
    if ((st = resolve_scale(ctx, config, cache->head_dim, &scale))) return st;
    const int dtype = cache->dtype;
    const uint64_t es = dtype_size(dtype);
    const uint64_t lse_off = lse_offset_bytes(dtype, d.q_elements);
    if ((st = check_buffer(ctx, "Q", q_chunk, d.q_elements * es))) return st;
    if ((st = check_buffer(ctx, "O|LSE", out_and_lse, lse_off + d.lse_elements * 4))) return st;
    uint64_t new_len = 0;
    if ((st = flat_paged_kv_cache_append_rotating(cache, k_chunk, v_chunk, chunk_len, theta, position_offset, &new_len)))
        return st;

    FwdParams p{};
    p.q = q_chunk.ptr; p.k = cache->k; p.v = cache->v; p.o = out_and_lse.ptr;
    p.lse = reinterpret_cast<float *>(static_cast<char *>(out_and_lse.ptr) + lse_off);
    const int64_t D = (int64_t)cache->head_dim;
    p.batch = 1; p.q_heads = (int)q_heads; p.kv_heads = (int)cache->kv_heads; p.q_len = (int)chunk_len;
    p.kv_len = (int)new_len; p.head_dim = (int)D; p.group = p.q_heads / p.kv_heads;
    p.q_hs = D; p.q_rs = p.q_heads * D; p.q_bs = p.q_rs * p.q_len;
    p.o_hs = p.q_hs; p.o_rs = p.q_rs; p.o_bs = p.q_bs;
    p.kv_hs = D; p.kv_rs = p.kv_heads * D; p.kv_bs = 0;
    p.lse_hs = p.q_len;
    p.causal = config->causal ? 1 : 0;
    p.causal_off = (int64_t)old_len;
    p.scale = scale;
    p.rope_q = 1; p.rope_k = 0;  // the cache holds pre-rotated K
    p.q_rope_off = (int64_t)(position_offset + old_len);
    fill_inv_freq(theta, p.head_dim, p.inv_freq);
    p.page_table = cache->dev_table;
    p.page_size = (int)cache->table.page_size;
    p.max_pages = (int)cache->table.physical_pages;
    p.page_row_stride = p.kv_rs;
    if (dtype == FLAT_BF16 && forward_sm100_supported(p)) {
        if (cache->k_f16) {
            // the binary16 shadow feeds the tensor core directly: no per-tile conversion in shared memory
            p.k = cache->k_f16;
            p.k_f16 = 1;
        }
        return launch_forward_sm100(ctx, p);
    }
    return launch_forward_simt(ctx, dtype, p);
}

// ---- backward --------------------------------------------------------------------------------
int32_t flat_backward_layout_for(int32_t dtype, const flat_attention_shape *shape, flat_backward_layout *out) {
    if (!out) return FLAT_ERR_NULL_POINTER;
    if (dtype != FLAT_F32 && dtype != FLAT_BF16) return FLAT_ERR_UNSUPPORTED_DTYPE;
    Dims d;
    int st = validate_shape(nullptr, shape, &d);
    if (st) return st;
    if (shape->query_len != shape->kv_len) return FLAT_ERR_LENGTH_MISMATCH;
    const uint64_t es = dtype_size(dtype);
    // f32: the reference's tight packing (src/wgpu_backward_grouped.rs:29-55).  bf16: the same
    // order with every section start rounded up to 16 bytes.
    auto align = [&](uint64_t x) { return dtype == FLAT_BF16 ? (x + 15) & ~uint64_t(15) : x; };
    out->q_elements = d.q_elements;
    out->kv_elements = d.kv_elements;
    out->lse_elements = d.lse_elements;
    uint64_t off = 0;
    out->q_offset = off; off = align(off + d.q_elements * es);
    out->k_offset = off; off = align(off + d.kv_elements * es);
    out->v_offset = off; off = align(off + d.kv_elements * es);
    out->d_out_offset = off; off = align(off + d.q_elements * es);
    out->out_offset = off; off = align(off + d.q_elements * es);
    out->lse_offset = off; off += d.lse_elements * 4;
    out->input_bytes = off;
    // gradients are f32 in both modes (tight packing; every section is a multiple of 4 bytes)
    off = 0;
    out->dq_offset = off; off = align(off + d.q_elements * 4);
    out->dk_offset = off; off = align(off + d.kv_elements * 4);
    out->dv_offset = off; off += d.kv_elements * 4;
    out->output_bytes = off;
    return FLAT_OK;
}

// validation and parameter block shared by the direct and the prepared backward entry points
static int backward_build(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape, const flat_attention_config *config,
                          flat_buffer packed_inputs, flat_buffer packed_grads, BwdParams *out) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    int st;
    if ((st = check_dtype(ctx, dtype))) return st;
    Dims d;
    if ((st = validate_shape(ctx, shape, &d))) return st;
    if (shape->query_len != shape->kv_len || shape->query_position_offset != 0)
        return fail(ctx, FLAT_ERR_LENGTH_MISMATCH, "backward requires query_len == kv_len and offset 0");
    float scale;
    if ((st = resolve_scale(ctx, config, shape->head_dim, &scale))) return st;
    flat_backward_layout L;
    if ((st = flat_backward_layout_for(dtype, shape, &L))) return st;
    if ((st = check_buffer(ctx, "Q|K|V|dO|O|LSE", packed_inputs, L.input_bytes))) return st;
    if ((st = check_buffer(ctx, "dQ|dK|dV", packed_grads, L.output_bytes))) return st;
    char *in = static_cast<char *>(packed_inputs.ptr);
    char *outp = static_cast<char *>(packed_grads.ptr);
    BwdParams p{};
    p.q = in + L.q_offset; p.k = in + L.k_offset; p.v = in + L.v_offset; p.d_out = in + L.d_out_offset;
    p.out = in + L.out_offset; p.lse = reinterpret_cast<const float *>(in + L.lse_offset);
    p.dq = outp + L.dq_offset; p.dk = outp + L.dk_offset; p.dv = outp + L.dv_offset;
    p.batch = (int)shape->batch; p.q_heads = (int)shape->q_heads; p.kv_heads = (int)shape->kv_heads;
    p.seq_len = (int)shape->query_len; p.head_dim = (int)shape->head_dim; p.group = p.q_heads / p.kv_heads;
    p.causal = config->causal ? 1 : 0;
    p.scale = scale;
    *out = p;
    return FLAT_OK;
}

static int backward_launch(flat_ctx *ctx, int dtype, const BwdParams &p) {
    if (dtype == FLAT_BF16 && backward_sm100_supported(p)) return launch_backward_sm100(ctx, p);
    return launch_backward_simt(ctx, dtype, p);
}

int32_t flat_backward_grouped(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                              const flat_attention_config *config, flat_buffer packed_inputs,
                              flat_buffer packed_grads) {
    BwdParams p{};
    int st = backward_build(ctx, dtype, shape, config, packed_inputs, packed_grads, &p);
    if (st) return st;
    return backward_launch(ctx, dtype, p);
}

// PreparedGroupedBackwardRecompute (src/wgpu_backward_grouped.rs:231-326)
struct flat_prepared_backward {
    flat_ctx *ctx;
    int dtype;
    BwdParams params;
};

int32_t flat_backward_prepare(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                              const flat_attention_config *config, flat_buffer packed_inputs, flat_buffer packed_grads,
                              flat_prepared_backward **out) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    if (!out) return fail(ctx, FLAT_ERR_NULL_POINTER, "prepared-pass output is null");
    *out = nullptr;
    BwdParams p{};
    int st = backward_build(ctx, dtype, shape, config, packed_inputs, packed_grads, &p);
    if (st) return st;
    if (dtype == FLAT_BF16 && backward_sm100_supported(p) &&
        (st = ensure_workspace(ctx, kWorkspaceMeta + backward_sm100_workspace_bytes(ctx, p))))
        return st;
    auto *prep = new (std::nothrow) flat_prepared_backward{ctx, dtype, p};
    if (!prep) return fail(ctx, FLAT_ERR_EXECUTION, "out of host memory");
    *out = prep;
    return FLAT_OK;
}

int32_t flat_backward_encode_prepared(flat_ctx *ctx, const flat_prepared_backward *prepared) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    if (!prepared) return fail(ctx, FLAT_ERR_NULL_POINTER, "prepared pass is null");
    if (prepared->ctx != ctx) return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "the pass was prepared on another context");
    return backward_launch(ctx, prepared->dtype, prepared->params);
}

void flat_prepared_backward_destroy(flat_prepared_backward *prepared) { delete prepared; }

int32_t flat_backward_mha(flat_ctx *ctx, int32_t dtype, const flat_attention_shape *shape,
                          const flat_attention_config *config, flat_buffer packed_inputs, flat_buffer packed_grads) {
    if (ctx && shape && shape->q_heads != shape->kv_heads)
        return fail(ctx, FLAT_ERR_INVALID_HEAD_GROUPING, "MHA requires q_heads == kv_heads, got %llu and %llu",
                    (unsigned long long)shape->q_heads, (unsigned long long)shape->kv_heads);
    return flat_backward_grouped(ctx, dtype, shape, config, packed_inputs, packed_grads);
}

}  // extern "C"
