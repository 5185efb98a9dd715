// KV-cache append: copies new K/V rows to their final cache rows, through the page table for the
// paged cache, optionally rotating K on the way (the cache holds pre-rotated K, so decode and
// chunked prefill never rotate K again: src/wgpu_paged_kv_cache.rs:200-205,
// docs/m15-prerotated-k-decode.md).  One launch moves K and V; only the appended rows are
// touched, the live prefix is never moved (src/wgpu_paged_kv_cache.rs:206-279).
#include "common.h"

namespace flat {
namespace {

struct InvFreq {
    float f[kMaxHeadDim / 2];
};

template <typename T> __device__ __forceinline__ float ld(const T *p);
template <> __device__ __forceinline__ float ld<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st(T *p, float x);
template <> __device__ __forceinline__ void st<float>(float *p, float x) { *p = x; }
template <> __device__ __forceinline__ void st<__nv_bfloat16>(__nv_bfloat16 *p, float x) { *p = __float2bfloat16_rn(x); }

__device__ __forceinline__ __half f32_to_f16_sat(float x) {
    uint16_t h;
    asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(h) : "f"(x));
    return __ushort_as_half(h);
}

// bf16 -> binary16 of a whole K buffer (the shadow of a cache that already holds tokens when it is switched on)
__global__ void __launch_bounds__(256) shadow_fill_kernel(const __nv_bfloat16 *__restrict__ k, __half *__restrict__ shadow, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        shadow[i] = f32_to_f16_sat(__bfloat162float(k[i]));
}

// One thread moves one (row, pair of elements) of K and of V.  Threads of a warp cover consecutive
// pairs of a row, so loads and stores are coalesced; rows are independent.
// k_shadow (bf16 caches only, optional): a binary16 copy of the stored K, written alongside (see
// flat_paged_kv_cache_enable_prefill_shadow); the value is the bf16 number that went into the cache, converted
// exactly inside the binary16 range and saturated beyond it.
template <typename T>
__global__ void __launch_bounds__(256) append_rows_kernel(const T *__restrict__ k_src, const T *__restrict__ v_src,
                                                          T *__restrict__ k_dst, T *__restrict__ v_dst,
                                                          __half *__restrict__ k_shadow, int64_t rows,
                                                          int row_elems, int head_dim,
                                                          const int32_t *__restrict__ page_table, int page_size,
                                                          int64_t first_logical, int64_t dst_row0, int rotate,
                                                          int64_t pos0, InvFreq inv_freq) {
    const int pairs = (row_elems + 1) / 2;
    const int64_t total = rows * pairs;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / pairs;
        const int e = (int)(i % pairs) * 2;
        int64_t dst_row;
        if (page_table) {
            const int64_t t = first_logical + r;
            dst_row = (int64_t)page_table[t / page_size] * page_size + t % page_size;
        } else {
            dst_row = dst_row0 + r;
        }
        const T *ks = k_src + r * row_elems + e;
        const T *vs = v_src + r * row_elems + e;
        T *kd = k_dst + dst_row * row_elems + e;
        T *vd = v_dst + dst_row * row_elems + e;
        const bool has_odd = e + 1 < row_elems;
        float ke = ld<T>(ks), ko = has_odd ? ld<T>(ks + 1) : 0.f;
        if (rotate) {
            const int pair = (e % head_dim) >> 1;
            float angle = __fmul_rn((float)(pos0 + r), inv_freq.f[pair]);
            float s, c;
            sincosf(angle, &s, &c);
            float re = ke * c - ko * s;
            float ro = ke * s + ko * c;
            ke = re;
            ko = ro;
        }
        st<T>(kd, ke);
        if (has_odd) st<T>(kd + 1, ko);
        if (k_shadow) {
            __half *sd = k_shadow + dst_row * row_elems + e;
            sd[0] = f32_to_f16_sat(ld<T>(kd));
            if (has_odd) sd[1] = f32_to_f16_sat(ld<T>(kd + 1));
        }
        vd[0] = vs[0];
        if (has_odd) vd[1] = vs[1];
    }
}

}  // namespace

int launch_shadow_fill(flat_ctx *ctx, const void *k, void *shadow, int64_t elements) {
    const int blocks = (int)std::min<int64_t>((elements + 255) / 256, (int64_t)ctx->sm_count * 16);
    shadow_fill_kernel<<<std::max(blocks, 1), 256, 0, ctx->stream>>>(static_cast<const __nv_bfloat16 *>(k),
                                                                     static_cast<__half *>(shadow), elements);
    ctx->launches += 1;
    FLAT_CUDA_OK(ctx, cudaGetLastError());
    return FLAT_OK;
}

int launch_append_rows(flat_ctx *ctx, int dtype, const void *k_src, const void *v_src, void *k_dst, void *v_dst, void *k_shadow,
                       int64_t rows, int row_elems, int head_dim, const int32_t *page_table, int page_size,
                       int64_t first_logical, int64_t dst_row0, int rotate, int64_t pos0, const float *inv_freq) {
    InvFreq f{};
    if (rotate)
        for (int i = 0; i < head_dim / 2; ++i) f.f[i] = inv_freq[i];
    const int64_t total = rows * ((row_elems + 1) / 2);
    int blocks = (int)((total + 255) / 256);
    const int max_blocks = ctx->sm_count * 8;
    if (blocks > max_blocks) blocks = max_blocks;
    if (blocks < 1) blocks = 1;
    if (dtype == FLAT_BF16)
        append_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, ctx->stream>>>(
            (const __nv_bfloat16 *)k_src, (const __nv_bfloat16 *)v_src, (__nv_bfloat16 *)k_dst, (__nv_bfloat16 *)v_dst,
            (__half *)k_shadow, rows, row_elems, head_dim, page_table, page_size, first_logical, dst_row0, rotate, pos0, f);
    else
        append_rows_kernel<float><<<blocks, 256, 0, ctx->stream>>>((const float *)k_src, (const float *)v_src,
                                                                   (float *)k_dst, (float *)v_dst, nullptr, rows, row_elems,
                                                                   head_dim, page_table, page_size, first_logical,
                                                                   dst_row0, rotate, pos0, f);
    ctx->launches += 1;
    FLAT_CUDA_OK(ctx, cudaGetLastError());
    return FLAT_OK;
}

}  // namespace flat
