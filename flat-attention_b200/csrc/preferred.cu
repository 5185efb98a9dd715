// Precision routing (WgpuPreferredAttention, src/wgpu_f16_backend.rs:474-544) and the numerical-mode executor
// (src/numerical.rs:17-256) above the public forward entry points.  Host f32 slices in, host f32 [O | LSE] out.
#include <cmath>

#include "common.h"

namespace flat {
namespace {

// f32 -> binary16, round to nearest even (F16::from_f32, src/f16.rs:26-82); `flag` is raised when a result is not finite
__global__ void quantize_f16_kernel(const float *__restrict__ src, __half *__restrict__ dst, uint64_t n, int *flag) {
    bool bad = false;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const __half h = __float2half_rn(src[i]);
        dst[i] = h;
        bad |= (__half_as_ushort(h) & 0x7c00u) == 0x7c00u;
    }
    if (bad) atomicOr(flag, 1);
}

// binary16 -> f32, exact (F16::to_f32, src/f16.rs:85-110)
__global__ void expand_f16_kernel(const __half *__restrict__ src, float *__restrict__ dst, uint64_t n) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        dst[i] = __half2float(src[i]);
}

unsigned blocks_for(uint64_t n, int sm_count) {
    return (unsigned)std::min<uint64_t>((n + 255) / 256, (uint64_t)sm_count * 16);
}

// validate_f32_for_quantization (src/wgpu_f16_backend.rs:588-610): exact length, then the first non-finite value
int validate_slice(flat_ctx *ctx, const char *name, const float *data, uint64_t actual, uint64_t expected) {
    if (!data) return fail(ctx, FLAT_ERR_NULL_POINTER, "%s is null", name);
    if (actual != expected)
        return fail(ctx, FLAT_ERR_LENGTH_MISMATCH, "tensor %s contains %llu elements, expected %llu", name,
                    (unsigned long long)actual, (unsigned long long)expected);
    for (uint64_t i = 0; i < actual; ++i)
        if (!std::isfinite(data[i]))
            return fail(ctx, FLAT_ERR_NON_FINITE_INPUT, "tensor %s contains a non-finite value at index %llu", name,
                        (unsigned long long)i);
    return FLAT_OK;
}

int require_mha(flat_ctx *ctx, const flat_attention_shape *shape) {
    if (!shape) return fail(ctx, FLAT_ERR_NULL_POINTER, "shape is null");
    if (shape->q_heads != shape->kv_heads)
        return fail(ctx, FLAT_ERR_INVALID_HEAD_GROUPING, "MHA requires q_heads == kv_heads, got %llu and %llu",
                    (unsigned long long)shape->q_heads, (unsigned long long)shape->kv_heads);
    if (shape->query_len != shape->kv_len || shape->query_position_offset != 0)
        return fail(ctx, FLAT_ERR_LENGTH_MISMATCH, "equal-length forward requires query_len == kv_len and offset 0");
    return FLAT_OK;
}

}  // namespace
}  // namespace flat

using namespace flat;

extern "C" {

int32_t flat_preferred_io_precision_for_head_dim(uint64_t head_dim) {
    return (head_dim == 64 || head_dim == 128) ? FLAT_IO_PACKED_F16 : FLAT_IO_F32;
}

int32_t flat_preferred_forward_host(flat_ctx *ctx, const flat_attention_shape *shape, const flat_attention_config *config,
                                    const float *q, uint64_t q_elements, const float *k, uint64_t k_elements, const float *v,
                                    uint64_t v_elements, float *out_and_lse, uint64_t out_bytes, int32_t *used_precision) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    int st;
    if ((st = require_mha(ctx, shape))) return st;
    if (used_precision) *used_precision = FLAT_IO_F32;
    auto f32_route = [&]() {
        return flat_forward_host(ctx, FLAT_F32, FLAT_LAYOUT_HEAD_MAJOR, shape, config, nullptr, q, q_elements, k, k_elements, v,
                                 v_elements, 1, out_and_lse, out_bytes);
    };
    if (flat_preferred_io_precision_for_head_dim(shape->head_dim) == FLAT_IO_F32) return f32_route();

    flat_forward_layout l16, l32;
    if ((st = flat_forward_layout_for(FLAT_F16, shape, &l16)) || (st = flat_forward_layout_for(FLAT_F32, shape, &l32)))
        return fail(ctx, st, "%s", flat_status_str(st));
    const uint64_t n = l16.q_elements;
    if ((st = validate_slice(ctx, "Q", q, q_elements, n))) return st;
    if ((st = validate_slice(ctx, "K", k, k_elements, n))) return st;
    if ((st = validate_slice(ctx, "V", v, v_elements, n))) return st;
    if (!out_and_lse) return fail(ctx, FLAT_ERR_NULL_POINTER, "output is null");
    if (out_bytes < l32.combined_bytes)
        return fail(ctx, FLAT_ERR_BUFFER_TOO_SMALL, "O|LSE buffer has %llu bytes, requires %llu", (unsigned long long)out_bytes,
                    (unsigned long long)l32.combined_bytes);

    // staging: [flag | f32 scratch (one tensor, later the expanded O) | Q16 | K16 | V16 | O16|LSE]
    auto up = [](uint64_t x) { return (x + 255) & ~uint64_t(255); };
    const uint64_t f32_bytes = up(n * 4), h_bytes = up(n * 2), o_bytes = up(l16.combined_bytes);
    const uint64_t need = 256 + f32_bytes + 3 * h_bytes + o_bytes;
    if ((st = ensure_host_stage(ctx, need))) return st;
    char *base = static_cast<char *>(ctx->host_stage);
    int *flag = reinterpret_cast<int *>(base);
    float *wide = reinterpret_cast<float *>(base + 256);
    __half *h16[3] = {reinterpret_cast<__half *>(base + 256 + f32_bytes), reinterpret_cast<__half *>(base + 256 + f32_bytes + h_bytes),
                      reinterpret_cast<__half *>(base + 256 + f32_bytes + 2 * h_bytes)};
    char *o16 = base + 256 + f32_bytes + 3 * h_bytes;
    FLAT_CUDA_OK(ctx, cudaMemsetAsync(flag, 0, sizeof(int), ctx->stream));
    const float *src[3] = {q, k, v};
    for (int t = 0; t < 3; ++t) {
        FLAT_CUDA_OK(ctx, cudaMemcpyAsync(wide, src[t], n * 4, cudaMemcpyHostToDevice, ctx->stream));
        quantize_f16_kernel<<<blocks_for(n, ctx->sm_count), 256, 0, ctx->stream>>>(wide, h16[t], n, flag);
        ctx->launches += 1;
    }
    int overflowed = 0;
    FLAT_CUDA_OK(ctx, cudaMemcpyAsync(&overflowed, flag, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    FLAT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    if (overflowed) return f32_route();  // a value left the binary16 range: the call runs in f32 (src/wgpu_f16_backend.rs:521-528)

    const flat_buffer bq{h16[0], n * 2}, bk{h16[1], n * 2}, bv{h16[2], n * 2}, bo{o16, l16.combined_bytes};
    if ((st = flat_forward_mha(ctx, FLAT_F16, shape, config, bq, bk, bv, bo))) return st;
    expand_f16_kernel<<<blocks_for(n, ctx->sm_count), 256, 0, ctx->stream>>>(reinterpret_cast<const __half *>(o16), wide, n);
    ctx->launches += 1;
    FLAT_CUDA_OK(ctx, cudaMemcpyAsync(out_and_lse, wide, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    FLAT_CUDA_OK(ctx, cudaMemcpyAsync(reinterpret_cast<char *>(out_and_lse) + l32.lse_byte_offset, o16 + l16.lse_byte_offset,
                                      l16.lse_elements * 4, cudaMemcpyDeviceToHost, ctx->stream));
    FLAT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    FLAT_CUDA_OK(ctx, cudaGetLastError());
    if (used_precision) *used_precision = FLAT_IO_PACKED_F16;
    return FLAT_OK;
}

int32_t flat_numerical_mode_guarantees(int32_t mode, flat_numerical_guarantees *out) {
    if (!out) return FLAT_ERR_NULL_POINTER;
    switch (mode) {  // src/numerical.rs:70-96
        case FLAT_NUMERICAL_EXACT_REFERENCE:
            *out = {FLAT_ACC_SERIAL_FP32, FLAT_RED_SERIAL_REFERENCE, 0, 1, 0};
            return FLAT_OK;
        case FLAT_NUMERICAL_FAST_PORTABLE:
            *out = {FLAT_ACC_CAPABILITY_OPTIMIZED_FP32, FLAT_RED_CAPABILITY_OPTIMIZED, 0, 0, 1};
            return FLAT_OK;
        case FLAT_NUMERICAL_DETERMINISTIC_PORTABLE:
            *out = {FLAT_ACC_FIXED_TREE_FP32, FLAT_RED_FIXED_WORKGROUP_TREE, 0, 1, 0};
            return FLAT_OK;
    }
    return FLAT_ERR_UNSUPPORTED_SHAPE;
}

int32_t flat_numerical_forward_host(flat_ctx *ctx, int32_t mode, const flat_attention_shape *shape,
                                    const flat_attention_config *config, const float *q, uint64_t q_elements, const float *k,
                                    uint64_t k_elements, const float *v, uint64_t v_elements, float *out_and_lse,
                                    uint64_t out_bytes) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    if (mode == FLAT_NUMERICAL_EXACT_REFERENCE)
        return fail(ctx, FLAT_ERR_UNAVAILABLE, "exact-reference execution is CPU-only and is not part of this library");
    if (mode != FLAT_NUMERICAL_FAST_PORTABLE && mode != FLAT_NUMERICAL_DETERMINISTIC_PORTABLE)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "unknown numerical mode %d", mode);
    int st;
    if ((st = require_mha(ctx, shape))) return st;
    // both portable modes run the f32-arithmetic kernel: its shuffle tree and key order are fixed, so it already meets
    // the deterministic mode's guarantee
    return flat_forward_host(ctx, FLAT_F32, FLAT_LAYOUT_HEAD_MAJOR, shape, config, nullptr, q, q_elements, k, k_elements, v,
                             v_elements, 1, out_and_lse, out_bytes);
}

}  // extern "C"
