// flat_attention.hpp — header-only C++17 mirror of FLAT-ATTENTION's backend structs over the C ABI.
//
// The reference is a Rust crate; where no Rust toolchain is available this header plays the part of
// its host layer: the same struct families, method names, argument meaning and error behaviour, with
// `wgpu::Buffer` replaced by DeviceBuffer (pointer + byte size) and `&mut wgpu::CommandEncoder` by the
// context's CUDA stream.  Every method forwards to one C entry point of include/flat_attention_b200.h;
// errors are thrown as flat::Error carrying the typed status and the detail string (the payload of the
// reference's error variants).  Nothing here computes anything on the CPU.
#pragma once

#include <cstdint>
#include <optional>
#include <array>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/flat_attention_b200.h"

namespace flat {

// FlatAttentionError and the per-component error enums (src/lib.rs:363-386 and Appendix of the C header).
class Error : public std::runtime_error {
  public:
    Error(int32_t status, std::string detail)
        : std::runtime_error(std::string(flat_status_str(status)) + (detail.empty() ? "" : ": " + detail)), status_(status),
          detail_(std::move(detail)) {}
    int32_t status() const { return status_; }
    const std::string &detail() const { return detail_; }

  private:
    int32_t status_;
    std::string detail_;
};

using DeviceBuffer = flat_buffer;
enum class DType : int32_t { F32 = FLAT_F32, BF16 = FLAT_BF16, F16 = FLAT_F16 };

// AttentionShape / GroupedAttentionShape / AsymmetricGroupedAttentionShape (src/lib.rs:211-245,
// src/grouped.rs:17-75, src/asymmetric_grouped.rs:26-35) in their api::v1 form (src/api.rs:24-33).
struct AttentionShape : flat_attention_shape {
    static AttentionShape mha(uint64_t batch, uint64_t heads, uint64_t seq_len, uint64_t head_dim) {
        return AttentionShape{{batch, heads, heads, seq_len, seq_len, head_dim, 0}};
    }
    static AttentionShape grouped(uint64_t batch, uint64_t q_heads, uint64_t kv_heads, uint64_t seq_len, uint64_t head_dim) {
        return AttentionShape{{batch, q_heads, kv_heads, seq_len, seq_len, head_dim, 0}};
    }
    static AttentionShape asymmetric(uint64_t batch, uint64_t q_heads, uint64_t kv_heads, uint64_t query_len, uint64_t kv_len,
                                     uint64_t head_dim, uint64_t query_position_offset) {
        return AttentionShape{{batch, q_heads, kv_heads, query_len, kv_len, head_dim, query_position_offset}};
    }
};

// FlatAttentionConfig (src/lib.rs:248-269).
struct FlatAttentionConfig {
    bool causal = false;
    std::optional<float> softmax_scale;
    flat_attention_config raw() const { return {causal ? 1 : 0, softmax_scale ? 1 : 0, softmax_scale.value_or(0.f)}; }
};

// RotaryEmbeddingConfig / AsymmetricRotaryEmbeddingConfig (src/rotary_grouped.rs:13-19, src/projection_asymmetric.rs:18-23).
struct RotaryEmbeddingConfig {
    float theta = 10000.f;
    uint64_t query_position_offset = 0, kv_position_offset = 0;
    bool rotate_k = true;  // false: K in memory is pre-rotated (encode_pre_rotated_k)
    flat_rotary_config raw() const { return {theta, rotate_k ? 1 : 0, query_position_offset, kv_position_offset}; }
};

// The device + queue pair of the reference executors (WgpuFlatAttention::new, src/wgpu_backend.rs:177-255).
class Context {
  public:
    explicit Context(int device = 0, void *cuda_stream = nullptr) {
        int32_t st = flat_ctx_create(device, cuda_stream, &ctx_);
        if (st) throw Error(st, "");
    }
    ~Context() { flat_ctx_destroy(ctx_); }
    Context(const Context &) = delete;
    Context &operator=(const Context &) = delete;
    flat_ctx *raw() const { return ctx_; }
    void check(int32_t st) const {
        if (st) throw Error(st, flat_last_error_detail(ctx_));
    }
    void synchronize() const { check(flat_synchronize(ctx_)); }
    void upload(DeviceBuffer dst, const void *host, uint64_t bytes) const { check(flat_upload(ctx_, dst, host, bytes)); }
    void download(void *host, DeviceBuffer src, uint64_t bytes) const { check(flat_download(ctx_, host, src, bytes)); }
    void reserve_workspace(uint64_t bytes) const { check(flat_ctx_reserve_workspace(ctx_, bytes)); }
    // RuntimeDeviceFingerprint / RuntimeDeviceCapabilities captured at creation (src/wgpu_backend.rs:239-316, 341-345)
    flat_device_fingerprint device_fingerprint() const {
        flat_device_fingerprint out{};
        check(flat_ctx_device_fingerprint(ctx_, &out));
        return out;
    }
    flat_device_capabilities device_capabilities() const {
        flat_device_capabilities out{};
        check(flat_ctx_device_capabilities(ctx_, &out));
        return out;
    }

  private:
    flat_ctx *ctx_ = nullptr;
};

// canonical_record / stable_fingerprint (src/runtime_telemetry.rs:49-67, 116-135)
inline std::string canonical_record(const flat_device_fingerprint &fp) {
    std::string out((size_t)flat_device_fingerprint_canonical_record(&fp, nullptr, 0), '\0');
    flat_device_fingerprint_canonical_record(&fp, out.data(), out.size() + 1);
    return out;
}
inline std::string canonical_record(const flat_device_capabilities &caps) {
    std::string out((size_t)flat_device_capabilities_canonical_record(&caps, nullptr, 0), '\0');
    flat_device_capabilities_canonical_record(&caps, out.data(), out.size() + 1);
    return out;
}
inline uint64_t stable_fingerprint(const flat_device_fingerprint &fp) { return flat_device_fingerprint_stable(&fp); }
inline uint64_t stable_fingerprint(const flat_device_capabilities &caps) { return flat_device_capabilities_stable(&caps); }

// BenchmarkManifest::canonical_json (src/benchmark_manifest.rs:140-199); throws the validation error.
inline std::string canonical_json(const flat_benchmark_manifest &m) {
    int64_t n = flat_benchmark_manifest_canonical_json(&m, nullptr, 0);
    if (n < 0) throw Error((int32_t)-n, "");
    std::string out((size_t)n, '\0');
    flat_benchmark_manifest_canonical_json(&m, out.data(), out.size() + 1);
    return out;
}

// GroupedForwardLayout / ExternalProjectionLayout (src/wgpu_forward_grouped.rs:23-42): pure, allocation-free.
inline flat_forward_layout forward_layout(DType dtype, const AttentionShape &shape) {
    flat_forward_layout out{};
    int32_t st = flat_forward_layout_for(static_cast<int32_t>(dtype), &shape, &out);
    if (st) throw Error(st, "");
    return out;
}
// ResidentDecodeLayout / PagedDecodeLayout (src/wgpu_decode.rs:437-455, src/wgpu_paged_decode.rs:268-283)
inline flat_decode_layout decode_layout(DType dtype, uint64_t batch, uint64_t q_heads, uint64_t head_dim) {
    flat_decode_layout out{};
    int32_t st = flat_decode_layout_for(static_cast<int32_t>(dtype), batch, q_heads, head_dim, &out);
    if (st) throw Error(st, flat_status_str(st));
    return out;
}
inline flat_backward_layout backward_layout(DType dtype, const AttentionShape &shape) {
    flat_backward_layout out{};
    int32_t st = flat_backward_layout_for(static_cast<int32_t>(dtype), &shape, &out);
    if (st) throw Error(st, "");
    return out;
}

// One pass of a caller-owned forward pipeline: GroupedForwardPass / ExternalProjectionPass /
// ExternalAsymmetricProjectionPass (src/wgpu_forward_grouped.rs:44-53, src/wgpu_external_asymmetric.rs:23-50).
struct ForwardPass {
    DeviceBuffer q, k, v, out_and_lse;
    AttentionShape shape;
    FlatAttentionConfig config;
    RotaryEmbeddingConfig rotary;
};

// WgpuGroupedForwardPipeline (src/wgpu_forward_grouped.rs:170-539): head-major GQA/MQA.
class CudaGroupedForwardPipeline {
  public:
    CudaGroupedForwardPipeline(const Context &ctx, DType dtype) : ctx_(ctx), dtype_(dtype) {}
    static flat_forward_layout layout(DType dtype, const AttentionShape &shape) { return forward_layout(dtype, shape); }
    flat_forward_layout encode(const ForwardPass &pass) const {
        auto cfg = pass.config.raw();
        ctx_.check(flat_forward_grouped(ctx_.raw(), static_cast<int32_t>(dtype_), &pass.shape, &cfg, pass.q, pass.k, pass.v,
                                        pass.out_and_lse));
        return forward_layout(dtype_, pass.shape);
    }
    // PreparedGroupedForward (src/wgpu_forward_grouped.rs:54-91): validated once by prepare, then only enqueued
    class Prepared {
      public:
        Prepared(const Context &ctx, flat_prepared_forward *h) : ctx_(ctx), h_(h) {}
        ~Prepared() { flat_prepared_forward_destroy(h_); }
        Prepared(const Prepared &) = delete;
        Prepared &operator=(const Prepared &) = delete;
        Prepared(Prepared &&o) noexcept : ctx_(o.ctx_), h_(o.h_) { o.h_ = nullptr; }
        const flat_prepared_forward *raw() const { return h_; }

      private:
        const Context &ctx_;
        flat_prepared_forward *h_;
    };
    Prepared prepare(const ForwardPass &pass) const {
        auto cfg = pass.config.raw();
        flat_prepared_forward *h = nullptr;
        ctx_.check(flat_forward_prepare(ctx_.raw(), static_cast<int32_t>(dtype_), FLAT_LAYOUT_HEAD_MAJOR, &pass.shape, &cfg, nullptr,
                                        pass.q, pass.k, pass.v, pass.out_and_lse, &h));
        return Prepared(ctx_, h);
    }
    void encode_prepared(const Prepared &prepared) const { ctx_.check(flat_forward_encode_prepared(ctx_.raw(), prepared.raw())); }

  private:
    const Context &ctx_;
    DType dtype_;
};

// WgpuRotaryGroupedAttention::forward_resident (src/wgpu_rotary_grouped_backend.rs:163-271).
class CudaRotaryGroupedAttention {
  public:
    CudaRotaryGroupedAttention(const Context &ctx, DType dtype) : ctx_(ctx), dtype_(dtype) {}
    flat_forward_layout forward_resident(const ForwardPass &pass) const {
        auto cfg = pass.config.raw();
        auto rot = pass.rotary.raw();
        ctx_.check(flat_forward_grouped_rope(ctx_.raw(), static_cast<int32_t>(dtype_), &pass.shape, &cfg, &rot, pass.q, pass.k,
                                             pass.v, pass.out_and_lse));
        return forward_layout(dtype_, pass.shape);
    }

  private:
    const Context &ctx_;
    DType dtype_;
};

// ExternalProjectionRotaryGroupedPipeline and ExternalAsymmetricProjectionRotaryGroupedPipeline
// (src/wgpu_external.rs:124-211, src/wgpu_external_asymmetric.rs:64-405).
class CudaExternalAsymmetricProjectionRotaryGroupedPipeline {
  public:
    CudaExternalAsymmetricProjectionRotaryGroupedPipeline(const Context &ctx, DType dtype) : ctx_(ctx), dtype_(dtype) {}
    flat_forward_layout encode(const ForwardPass &pass) const { return run(pass, true); }
    flat_forward_layout encode_pre_rotated_k(const ForwardPass &pass) const { return run(pass, false); }
    // encode_alibi / encode_pre_rotated_k_alibi (src/wgpu_external_asymmetric.rs:245-282)
    flat_forward_layout encode_alibi(const ForwardPass &pass, const std::vector<float> &slopes, uint64_t query_position_offset,
                                     uint64_t kv_position_offset) const {
        return run_alibi(pass, true, slopes, query_position_offset, kv_position_offset);
    }
    flat_forward_layout encode_pre_rotated_k_alibi(const ForwardPass &pass, const std::vector<float> &slopes,
                                                   uint64_t query_position_offset, uint64_t kv_position_offset) const {
        return run_alibi(pass, false, slopes, query_position_offset, kv_position_offset);
    }

  private:
    flat_forward_layout run_alibi(const ForwardPass &pass, bool rotate_k, const std::vector<float> &slopes, uint64_t q_off,
                                  uint64_t kv_off) const {
        auto cfg = pass.config.raw();
        auto rot = pass.rotary.raw();
        rot.rotate_k = rotate_k ? 1 : 0;
        static const float none = 0.f;  // an empty vector still reaches the length check, not the null check
        ctx_.check(flat_forward_projection_rope_asymmetric_alibi(ctx_.raw(), static_cast<int32_t>(dtype_), &pass.shape, &cfg,
                                                                 &rot, slopes.empty() ? &none : slopes.data(), slopes.size(),
                                                                 q_off, kv_off, pass.q, pass.k, pass.v, pass.out_and_lse));
        return forward_layout(dtype_, pass.shape);
    }
    flat_forward_layout run(const ForwardPass &pass, bool rotate_k) const {
        auto cfg = pass.config.raw();
        auto rot = pass.rotary.raw();
        rot.rotate_k = rotate_k ? 1 : 0;
        ctx_.check(flat_forward_projection_rope_asymmetric(ctx_.raw(), static_cast<int32_t>(dtype_), &pass.shape, &cfg, &rot,
                                                           pass.q, pass.k, pass.v, pass.out_and_lse));
        return forward_layout(dtype_, pass.shape);
    }
    const Context &ctx_;
    DType dtype_;
};

// ExternalVariableProjectionRotaryGroupedPipeline (src/wgpu_external_variable.rs:74-223).
class CudaExternalVariableProjectionRotaryGroupedPipeline {
  public:
    CudaExternalVariableProjectionRotaryGroupedPipeline(const Context &ctx, DType dtype) : ctx_(ctx), dtype_(dtype) {}
    flat_forward_layout encode(const ForwardPass &pass, const std::vector<flat_varlen_sequence> &sequences) const {
        auto cfg = pass.config.raw();
        auto rot = pass.rotary.raw();
        ctx_.check(flat_forward_projection_rope_varlen(ctx_.raw(), static_cast<int32_t>(dtype_), &pass.shape, &cfg, &rot,
                                                       sequences.data(), sequences.size(), pass.q, pass.k, pass.v,
                                                       pass.out_and_lse));
        return forward_layout(dtype_, pass.shape);
    }

  private:
    const Context &ctx_;
    DType dtype_;
};

// WgpuPreferredAttention (src/wgpu_f16_backend.rs:474-544): binary16 storage for head_dim 64 / 128, f32 otherwise.
class CudaPreferredAttention {
  public:
    explicit CudaPreferredAttention(const Context &ctx) : ctx_(ctx) {}
    static flat_io_precision io_precision_for_head_dim(uint64_t head_dim) {
        return static_cast<flat_io_precision>(flat_preferred_io_precision_for_head_dim(head_dim));
    }
    // host f32 slices in, packed host f32 [O | LSE] out; returns the precision that ran
    flat_io_precision forward(const std::vector<float> &q, const std::vector<float> &k, const std::vector<float> &v,
                              const AttentionShape &shape, const FlatAttentionConfig &config, std::vector<float> &out_and_lse) const {
        auto cfg = config.raw();
        const auto layout = forward_layout(DType::F32, shape);
        out_and_lse.resize(layout.combined_bytes / 4);
        int32_t used = FLAT_IO_F32;
        ctx_.check(flat_preferred_forward_host(ctx_.raw(), &shape, &cfg, q.data(), q.size(), k.data(), k.size(), v.data(), v.size(),
                                               out_and_lse.data(), out_and_lse.size() * 4, &used));
        return static_cast<flat_io_precision>(used);
    }

  private:
    const Context &ctx_;
};

// NumericalExecutor (src/numerical.rs:135-256).  ExactReference is CPU execution in the reference: Error(Unavailable) here.
class NumericalExecutor {
  public:
    NumericalExecutor(const Context &ctx, flat_numerical_mode mode) : ctx_(ctx), mode_(mode) {
        if (mode == FLAT_NUMERICAL_EXACT_REFERENCE) throw Error(FLAT_ERR_UNAVAILABLE, "exact-reference execution is CPU-only");
    }
    static flat_numerical_guarantees guarantees(flat_numerical_mode mode) {
        flat_numerical_guarantees g{};
        int32_t st = flat_numerical_mode_guarantees(mode, &g);
        if (st) throw Error(st, "");
        return g;
    }
    flat_numerical_mode mode() const { return mode_; }
    void forward(const std::vector<float> &q, const std::vector<float> &k, const std::vector<float> &v, const AttentionShape &shape,
                 const FlatAttentionConfig &config, std::vector<float> &out_and_lse) const {
        auto cfg = config.raw();
        const auto layout = forward_layout(DType::F32, shape);
        out_and_lse.resize(layout.combined_bytes / 4);
        ctx_.check(flat_numerical_forward_host(ctx_.raw(), mode_, &shape, &cfg, q.data(), q.size(), k.data(), k.size(), v.data(),
                                               v.size(), out_and_lse.data(), out_and_lse.size() * 4));
    }

  private:
    const Context &ctx_;
    flat_numerical_mode mode_;
};

// PagedKvTable (src/paged_kv.rs:75-188).
class PagedKvTable {
  public:
    PagedKvTable(uint64_t page_size, uint64_t physical_pages) {
        int32_t st = flat_paged_kv_table_create(page_size, physical_pages, &t_);
        if (st) throw Error(st, "");
    }
    ~PagedKvTable() { flat_paged_kv_table_destroy(t_); }
    PagedKvTable(const PagedKvTable &) = delete;
    PagedKvTable &operator=(const PagedKvTable &) = delete;
    void append(uint64_t tokens) {
        int32_t st = flat_paged_kv_table_append(t_, tokens);
        if (st) throw Error(st, "");
    }
    std::optional<flat_paged_kv_address> address(uint64_t logical_token) const {
        flat_paged_kv_address a{};
        if (flat_paged_kv_table_address(t_, logical_token, &a)) return std::nullopt;
        return a;
    }
    flat_paged_kv_telemetry telemetry() const {
        flat_paged_kv_telemetry out{};
        flat_paged_kv_table_telemetry(t_, &out);
        return out;
    }
    void reset() {
        int32_t st = flat_paged_kv_table_reset(t_);
        if (st) throw Error(st, "");
    }
    uint64_t len() const { return flat_paged_kv_table_len(t_); }
    bool is_empty() const { return len() == 0; }
    uint64_t generation() const { return flat_paged_kv_table_generation(t_); }
    const flat_paged_kv_table *raw() const { return t_; }

  private:
    flat_paged_kv_table *t_ = nullptr;
};

// WgpuPagedKvCache (src/wgpu_paged_kv_cache.rs:76-279).
class CudaPagedKvCache {
  public:
    CudaPagedKvCache(const Context &ctx, DType dtype, uint64_t page_size, uint64_t physical_pages, uint64_t kv_heads,
                     uint64_t head_dim)
        : ctx_(ctx) {
        ctx.check(flat_paged_kv_cache_create(ctx.raw(), static_cast<int32_t>(dtype), page_size, physical_pages, kv_heads, head_dim, &c_));
    }
    ~CudaPagedKvCache() { flat_paged_kv_cache_destroy(c_); }
    CudaPagedKvCache(const CudaPagedKvCache &) = delete;
    CudaPagedKvCache &operator=(const CudaPagedKvCache &) = delete;
    uint64_t record_append(DeviceBuffer k_source, DeviceBuffer v_source, uint64_t append_len) {
        uint64_t n = 0;
        ctx_.check(flat_paged_kv_cache_append(c_, k_source, v_source, append_len, &n));
        return n;
    }
    uint64_t record_append_rotating(DeviceBuffer k_source, DeviceBuffer v_source, uint64_t append_len, float theta,
                                    uint64_t kv_position_offset) {
        uint64_t n = 0;
        ctx_.check(flat_paged_kv_cache_append_rotating(c_, k_source, v_source, append_len, theta, kv_position_offset, &n));
        return n;
    }
    // binary16 copy of K for the tensor-core chunked prefill (bf16 caches; allocates once)
    void enable_prefill_shadow() { ctx_.check(flat_paged_kv_cache_enable_prefill_shadow(c_)); }
    void reset() { ctx_.check(flat_paged_kv_cache_reset(c_)); }
    uint64_t len() const { return flat_paged_kv_cache_len(c_); }
    bool is_empty() const { return len() == 0; }
    uint64_t generation() const { return flat_paged_kv_cache_generation(c_); }
    DeviceBuffer k_buffer() const { return flat_paged_kv_cache_k_buffer(c_); }
    DeviceBuffer v_buffer() const { return flat_paged_kv_cache_v_buffer(c_); }
    const flat_paged_kv_table *table() const { return flat_paged_kv_cache_table(c_); }
    flat_paged_kv_cache *raw() const { return c_; }

  private:
    const Context &ctx_;
    flat_paged_kv_cache *c_ = nullptr;
};

// WgpuResidentKvCache (src/wgpu_kv_cache.rs:79-262).
class CudaResidentKvCache {
  public:
    CudaResidentKvCache(const Context &ctx, DType dtype, uint64_t batch, uint64_t kv_heads, uint64_t capacity, uint64_t head_dim)
        : ctx_(ctx) {
        ctx.check(flat_resident_kv_cache_create(ctx.raw(), static_cast<int32_t>(dtype), batch, kv_heads, capacity, head_dim, &c_));
    }
    ~CudaResidentKvCache() { flat_resident_kv_cache_destroy(c_); }
    CudaResidentKvCache(const CudaResidentKvCache &) = delete;
    CudaResidentKvCache &operator=(const CudaResidentKvCache &) = delete;
    uint64_t record_append(DeviceBuffer k_source, DeviceBuffer v_source, uint64_t append_len) {
        uint64_t n = 0;
        ctx_.check(flat_resident_kv_cache_append(c_, k_source, v_source, append_len, &n));
        return n;
    }
    void reset() { flat_resident_kv_cache_reset(c_); }
    uint64_t len() const { return flat_resident_kv_cache_len(c_); }
    uint64_t capacity() const { return flat_resident_kv_cache_capacity(c_); }
    uint64_t remaining_capacity() const { return capacity() - len(); }
    DeviceBuffer k_buffer() const { return flat_resident_kv_cache_k_buffer(c_); }
    DeviceBuffer v_buffer() const { return flat_resident_kv_cache_v_buffer(c_); }

  private:
    const Context &ctx_;
    flat_resident_kv_cache *c_ = nullptr;
};

// ResidentDecodePass / WgpuResidentDecodePipeline::encode_external_pre_rotated_k (src/wgpu_decode.rs:18-26,263-322).
struct ResidentDecodePass {
    DeviceBuffer q, k, v, out_and_lse;
    uint64_t batch, q_heads, kv_heads, head_dim, kv_len;
    FlatAttentionConfig config;
    float theta;
    uint64_t q_rope_position;
};
class CudaResidentDecodePipeline {
  public:
    CudaResidentDecodePipeline(const Context &ctx, DType dtype) : ctx_(ctx), dtype_(dtype) {}
    static flat_decode_layout layout(DType dtype, uint64_t batch, uint64_t q_heads, uint64_t head_dim) {
        return decode_layout(dtype, batch, q_heads, head_dim);
    }
    void encode_external_pre_rotated_k(const ResidentDecodePass &p, uint64_t kv_capacity) const {
        auto cfg = p.config.raw();
        ctx_.check(flat_decode_resident(ctx_.raw(), static_cast<int32_t>(dtype_), p.batch, p.q_heads, p.kv_heads, p.head_dim,
                                        p.kv_len, kv_capacity, &cfg, p.theta, p.q_rope_position, p.q, p.k, p.v, p.out_and_lse));
    }

  private:
    const Context &ctx_;
    DType dtype_;
};

// PagedDecodePass / WgpuPagedDecodePipeline::encode (src/wgpu_paged_decode.rs:200-219,300-436).
struct PagedDecodePass {
    DeviceBuffer q, k, v, out_and_lse;
    const flat_paged_kv_table *page_table;
    uint64_t q_heads, kv_heads, head_dim;
    FlatAttentionConfig config;
    float theta;
    uint64_t q_rope_position;
};
class CudaPagedDecodePipeline {
  public:
    CudaPagedDecodePipeline(const Context &ctx, DType dtype) : ctx_(ctx), dtype_(dtype) {}
    static flat_decode_layout layout(DType dtype, uint64_t q_heads, uint64_t head_dim) {
        return decode_layout(dtype, 1, q_heads, head_dim);
    }
    void encode(const PagedDecodePass &p) const {
        auto cfg = p.config.raw();
        ctx_.check(flat_decode_paged(ctx_.raw(), static_cast<int32_t>(dtype_), p.page_table, p.q_heads, p.kv_heads, p.head_dim,
                                     &cfg, p.theta, p.q_rope_position, p.q, p.k, p.v, p.out_and_lse));
    }

  private:
    const Context &ctx_;
    DType dtype_;
};

// WgpuChunkedProjectionPrefillPipeline (src/wgpu_chunked_prefill.rs:99-300).
class CudaChunkedProjectionPrefillPipeline {
  public:
    CudaChunkedProjectionPrefillPipeline(const Context &ctx, DType dtype) : ctx_(ctx), dtype_(dtype) {}
    void encode(const ForwardPass &pass, uint64_t query_chunk_size) const {
        auto cfg = pass.config.raw();
        auto rot = pass.rotary.raw();
        ctx_.check(flat_chunked_prefill(ctx_.raw(), static_cast<int32_t>(dtype_), &pass.shape, &cfg, &rot, query_chunk_size,
                                        pass.q, pass.k, pass.v, pass.out_and_lse));
    }

  private:
    const Context &ctx_;
    DType dtype_;
};

// GroupedBackwardRecomputePass / WgpuGroupedBackwardRecomputePipeline (src/wgpu_backward_grouped.rs:58-81,158-326).
struct BackwardPass {
    DeviceBuffer packed_inputs, packed_grads;
    AttentionShape shape;
    FlatAttentionConfig config;
};
class CudaGroupedBackwardRecomputePipeline {
  public:
    CudaGroupedBackwardRecomputePipeline(const Context &ctx, DType dtype) : ctx_(ctx), dtype_(dtype) {}
    static flat_backward_layout layout(DType dtype, const AttentionShape &shape) { return backward_layout(dtype, shape); }
    flat_backward_layout encode(const BackwardPass &pass) const {
        auto cfg = pass.config.raw();
        ctx_.check(flat_backward_grouped(ctx_.raw(), static_cast<int32_t>(dtype_), &pass.shape, &cfg, pass.packed_inputs,
                                         pass.packed_grads));
        return backward_layout(dtype_, pass.shape);
    }

  private:
    const Context &ctx_;
    DType dtype_;
};

// KV-split decode of one long sequence across the GPUs of a box (no counterpart in the reference, which is
// single-device): the peer-memory exchange object.  handle() is what a rank gives the other ranks, connect() maps
// theirs; decode() is one step (flat_splitkv_decode_peer: the rank's partial, then one kernel that stores it into every
// rank's buffer, waits for the others' flags and merges).
struct SplitKvSlicePass {
    uint64_t num_seqs, q_heads, kv_heads, head_dim, page_size, physical_pages, max_pages_per_seq;
    const int32_t *page_tables_dev, *context_lens_dev, *q_rope_positions_dev;
    const int32_t *host_page_tables, *host_context_lens;  // optional (validation; all-zero lengths = an empty slice)
    FlatAttentionConfig config;
    float theta;
    DeviceBuffer q, k, v, out_and_lse;
};
class CudaSplitKvPeerExchange {
  public:
    CudaSplitKvPeerExchange(const Context &ctx, int rank, int world, uint64_t rows, uint64_t head_dim) : ctx_(ctx) {
        ctx_.check(flat_splitkv_exchange_create(ctx_.raw(), rank, world, rows, head_dim, &raw_));
    }
    ~CudaSplitKvPeerExchange() { flat_splitkv_exchange_destroy(raw_); }
    CudaSplitKvPeerExchange(const CudaSplitKvPeerExchange &) = delete;
    CudaSplitKvPeerExchange &operator=(const CudaSplitKvPeerExchange &) = delete;
    std::array<uint8_t, 64> handle() const {
        std::array<uint8_t, 64> h{};
        ctx_.check(flat_splitkv_exchange_handle(raw_, h.data()));
        return h;
    }
    void connect(const std::vector<uint8_t> &all_handles) {
        ctx_.check(flat_splitkv_exchange_connect(raw_, all_handles.data(), all_handles.size()));
    }
    void decode(DType dtype, const SplitKvSlicePass &p) const {
        auto cfg = p.config.raw();
        ctx_.check(flat_splitkv_decode_peer(ctx_.raw(), raw_, static_cast<int32_t>(dtype), p.num_seqs, p.q_heads, p.kv_heads,
                                            p.head_dim, p.page_size, p.physical_pages, p.max_pages_per_seq, p.page_tables_dev,
                                            p.context_lens_dev, p.q_rope_positions_dev, p.host_page_tables, p.host_context_lens,
                                            &cfg, p.theta, p.q, p.k, p.v, p.out_and_lse));
    }

  private:
    const Context &ctx_;
    flat_splitkv_exchange *raw_ = nullptr;
};

}  // namespace flat
