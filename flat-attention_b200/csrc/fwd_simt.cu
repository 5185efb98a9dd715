// Generic SIMT forward: f32 arithmetic, f32 or bf16 storage, every layout and mode of the
// forward contract (head-major / projection strides, rectangular shapes, three position domains,
// optional RoPE on Q and/or K, padded variable-length batches, K/V read through a page table).
// It is the f32 parity kernel and the catch-all for shapes the tcgen05 kernel does not take.
//
// Mapping: one CTA = 32 consecutive query rows of one (batch, q_head); 4 threads share a row, each
// owning every 4th float4 chunk of the head dimension.  K/V tiles of 32 keys are staged (and, when
// asked, rotated) in shared memory; the softmax is online per tile, so no N x N matrix exists.
#include "common.h"

namespace flat {
namespace {

constexpr int kRows = 32;     // query rows per CTA
constexpr int kKeys = 32;     // keys per shared-memory tile
constexpr int kThreads = 128;

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// Rotation of one interleaved pair at an absolute position (src/rotary_grouped.rs:36-50): the
// frequency comes from the host table, the angle is one f32 multiply as in the oracle.
__device__ __forceinline__ void rotate_pair(float &e, float &o, int64_t position, float inv_freq) {
    float angle = __fmul_rn((float)position, inv_freq);
    float s, c;
    sincosf(angle, &s, &c);
    float re = e * c - o * s;
    float ro = e * s + o * c;
    e = re;
    o = ro;
}

template <typename T>
__device__ __forceinline__ const T *kv_row_ptr(const FwdParams &p, const T *base, int batch, int kv_head,
                                               int64_t pos) {
    if (p.page_table) {
        int64_t page = p.page_table[(int64_t)batch * p.max_pages + pos / p.page_size];
        int64_t row = page * p.page_size + pos % p.page_size;
        return base + row * p.page_row_stride + (int64_t)kv_head * p.kv_hs;
    }
    return base + (int64_t)batch * p.kv_bs + (int64_t)kv_head * p.kv_hs + pos * p.kv_rs;
}

// DPT = floats of the (padded) head dimension owned by one thread; padded D = 4*DPT.
template <typename T, int DPT>
__global__ void __launch_bounds__(kThreads) fwd_simt_kernel(const __grid_constant__ FwdParams p) {
    constexpr int DP = 4 * DPT;       // padded head dim
    constexpr int CH = DPT / 4;       // float4 chunks per thread
    extern __shared__ float smem[];
    float *ks = smem;                 // [kKeys][DP]
    float *vs = smem + kKeys * DP;    // [kKeys][DP]

    const int tid = threadIdx.x;
    const int sub = tid & 3;
    const int row_in_tile = tid >> 2;
    const int batch = blockIdx.z;
    const int q_head = blockIdx.y;
    const int kv_head = q_head / p.group;
    const int row = blockIdx.x * kRows + row_in_tile;
    const int D = p.head_dim;

    int active_q = p.q_len, active_kv = p.kv_len;
    int64_t causal_off = p.causal_off, q_rope_off = p.q_rope_off;
    if (p.varlen) {
        flat_varlen_sequence m = p.varlen[batch];
        active_q = m.active_query_len;
        active_kv = m.active_kv_len;
        causal_off = m.causal_query_offset;
        q_rope_off = m.query_rope_offset;
    }
    const bool in_range = row < p.q_len;
    const bool valid = row < active_q;

    // this row's visible key count: keys 0..limit-1
    int64_t limit = active_kv;
    if (p.causal) limit = min((int64_t)active_kv, causal_off + row + 1);
    // the CTA streams keys up to the limit of its last valid row
    int64_t cta_limit = active_kv;
    if (p.causal) {
        int last = min(blockIdx.x * kRows + kRows, active_q) - 1;
        cta_limit = last < 0 ? 0 : min((int64_t)active_kv, causal_off + last + 1);
    }
    if (blockIdx.x * kRows >= active_q) cta_limit = 0;

    float q[DPT], o[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) q[i] = 0.f, o[i] = 0.f;
    if (valid) {
        const T *qp = (const T *)p.q + (int64_t)batch * p.q_bs + (int64_t)q_head * p.q_hs + (int64_t)row * p.q_rs;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            int d0 = (sub + 4 * c) * 4;
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (d0 + e < D) q[c * 4 + e] = to_f32<T>(qp[d0 + e]);
            if (p.rope_q) {
                if (d0 < D) rotate_pair(q[c * 4], q[c * 4 + 1], q_rope_off + row, p.inv_freq[d0 / 2]);
                if (d0 + 2 < D) rotate_pair(q[c * 4 + 2], q[c * 4 + 3], q_rope_off + row, p.inv_freq[d0 / 2 + 1]);
            }
        }
    }

    float m = -INFINITY, l = 0.f;
    const T *kbase = (const T *)p.k, *vbase = (const T *)p.v;
    // ALiBi: the position difference is formed in integers and rounded to f32 once, like the f64 difference of
    // src/attention_bias.rs:93-94
    const float slope = p.alibi_slopes ? p.alibi_slopes[q_head] : 0.f;
    const int64_t bias_delta0 = p.alibi_kv_off - p.alibi_q_off - row;

    for (int64_t k0 = 0; k0 < cta_limit; k0 += kKeys) {
        __syncthreads();
        // stage K and V: pairs of floats so RoPE can rotate in flight
        for (int idx = tid; idx < kKeys * (DP / 2); idx += kThreads) {
            int key = idx / (DP / 2), pair = idx % (DP / 2);
            int d = 2 * pair;
            int64_t pos = k0 + key;
            float ke = 0.f, ko = 0.f, ve = 0.f, vo = 0.f;
            if (pos < cta_limit && d < D) {
                const T *kr = kv_row_ptr<T>(p, kbase, batch, kv_head, pos);
                const T *vr = kv_row_ptr<T>(p, vbase, batch, kv_head, pos);
                ke = to_f32<T>(kr[d]);
                ve = to_f32<T>(vr[d]);
                if (d + 1 < D) {
                    ko = to_f32<T>(kr[d + 1]);
                    vo = to_f32<T>(vr[d + 1]);
                }
                if (p.rope_k) rotate_pair(ke, ko, p.k_rope_off + pos, p.inv_freq[pair]);
            }
            ks[key * DP + d] = ke;
            ks[key * DP + d + 1] = ko;
            vs[key * DP + d] = ve;
            vs[key * DP + d + 1] = vo;
        }
        __syncthreads();

        float s[kKeys];
        float tile_max = -INFINITY;
#pragma unroll
        for (int j = 0; j < kKeys; ++j) {
            float acc = 0.f;
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                float4 kk = *reinterpret_cast<const float4 *>(&ks[j * DP + (sub + 4 * c) * 4]);
                acc = fmaf(q[c * 4 + 0], kk.x, acc);
                acc = fmaf(q[c * 4 + 1], kk.y, acc);
                acc = fmaf(q[c * 4 + 2], kk.z, acc);
                acc = fmaf(q[c * 4 + 3], kk.w, acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            float sc = acc * p.scale;
            if (p.alibi_slopes) sc = __fadd_rn(sc, __fmul_rn(slope, (float)(bias_delta0 + k0 + j)));
            if (!(valid && (k0 + j) < limit)) sc = -INFINITY;
            s[j] = sc;
            tile_max = fmaxf(tile_max, sc);
        }
        if (tile_max != -INFINITY) {
            float m_new = fmaxf(m, tile_max);
            float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
            l *= alpha;
#pragma unroll
            for (int i = 0; i < DPT; ++i) o[i] *= alpha;
#pragma unroll
            for (int j = 0; j < kKeys; ++j) {
                float pj = (s[j] == -INFINITY) ? 0.f : expf(s[j] - m_new);
                l += pj;
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    float4 vv = *reinterpret_cast<const float4 *>(&vs[j * DP + (sub + 4 * c) * 4]);
                    o[c * 4 + 0] = fmaf(pj, vv.x, o[c * 4 + 0]);
                    o[c * 4 + 1] = fmaf(pj, vv.y, o[c * 4 + 1]);
                    o[c * 4 + 2] = fmaf(pj, vv.z, o[c * 4 + 2]);
                    o[c * 4 + 3] = fmaf(pj, vv.w, o[c * 4 + 3]);
                }
            }
            m = m_new;
        }
    }

    if (!in_range) return;
    T *op = (T *)p.o + (int64_t)batch * p.o_bs + (int64_t)q_head * p.o_hs + (int64_t)row * p.o_rs;
    float *lp = p.lse + ((int64_t)batch * p.q_heads + q_head) * p.lse_hs + row;
    if (!valid) {
        // padded query row: O = 0, LSE = -inf (src/asymmetric_grouped.rs:103-104)
#pragma unroll
        for (int c = 0; c < CH; ++c)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int d = (sub + 4 * c) * 4 + e;
                if (d < D) op[d] = from_f32<T>(0.f);
            }
        if (sub == 0) *lp = -INFINITY;
        return;
    }
    float inv = 1.0f / l;
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            int d = (sub + 4 * c) * 4 + e;
            if (d < D) op[d] = from_f32<T>(o[c * 4 + e] * inv);
        }
    if (sub == 0) *lp = m + logf(l);
}

template <typename T, int DPT>
int launch(flat_ctx *ctx, const FwdParams &p) {
    dim3 grid((p.q_len + kRows - 1) / kRows, p.q_heads, p.batch);
    size_t smem = 2 * kKeys * 4 * DPT * sizeof(float);
    fwd_simt_kernel<T, DPT><<<grid, kThreads, smem, ctx->stream>>>(p);
    ctx->launches += 1;
    FLAT_CUDA_OK(ctx, cudaGetLastError());
    return FLAT_OK;
}

template <typename T>
int dispatch(flat_ctx *ctx, const FwdParams &p) {
    if (p.head_dim <= 16) return launch<T, 4>(ctx, p);
    if (p.head_dim <= 32) return launch<T, 8>(ctx, p);
    if (p.head_dim <= 64) return launch<T, 16>(ctx, p);
    return launch<T, 32>(ctx, p);
}

}  // namespace

void forward_simt_geometry(const FwdParams &p, uint32_t *query_rows, uint32_t *kv_rows, uint32_t grid[3]) {
    *query_rows = kRows;
    *kv_rows = kKeys;
    grid[0] = (uint32_t)((p.q_len + kRows - 1) / kRows);
    grid[1] = (uint32_t)p.q_heads;
    grid[2] = (uint32_t)p.batch;
}

int launch_forward_simt(flat_ctx *ctx, int dtype, const FwdParams &p) {
    if (p.q_heads > 65535 || p.batch > 65535)
        return fail(ctx, FLAT_ERR_DISPATCH_LIMIT, "grid dimension %d exceeds 65535", p.q_heads > 65535 ? p.q_heads : p.batch);
    if (dtype == FLAT_F16) return dispatch<__half>(ctx, p);
    return dtype == FLAT_BF16 ? dispatch<__nv_bfloat16>(ctx, p) : dispatch<float>(ctx, p);
}

}  // namespace flat
