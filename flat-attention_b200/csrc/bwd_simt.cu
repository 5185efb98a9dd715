// Generic SIMT backward (LSE recompute): f32 arithmetic, f32 or bf16 inputs, f32 gradients, any head_dim <= 128.
// It is the f32 parity kernel for dQ/dK/dV and the catch-all for shapes the tcgen05 backward does
// not take.  Math per visible (query, key) pair, as in src/backward_grouped.rs:56-88:
//   delta = dO.O,  P = exp(S*scale - LSE),  dP = dO.V,  dS = P*(dP - delta),
//   dQ += dS*scale*K,  dK[kv_head] += dS*scale*Q,  dV[kv_head] += P*dO.
// Race-free by construction like the reference shaders: one CTA row owns one output row.  dQ rows
// loop over keys; dK/dV rows loop over the query heads of their group and over query rows, so the
// GQA reduction needs no atomics and the result is bitwise repeatable.
#include "common.h"

namespace flat {
namespace {

constexpr int kRows = 32;
constexpr int kTile = 32;
constexpr int kThreads = 128;

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    return x;
}

// delta[b, h, row] = sum_d dO * O   (one warp per row)
template <typename T>
__global__ void __launch_bounds__(128) delta_kernel(const T *__restrict__ d_out, const T *__restrict__ out,
                                                    float *__restrict__ delta, int64_t rows, int head_dim) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    float acc = 0.f;
    for (int d = lane; d < head_dim; d += 32)
        acc = fmaf(to_f32<T>(d_out[row * head_dim + d]), to_f32<T>(out[row * head_dim + d]), acc);
#pragma unroll
    for (int w = 16; w >= 1; w >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, w);
    if (lane == 0) delta[row] = acc;
}

template <typename T, int DPT>
__device__ __forceinline__ void load_row(const T *src, int sub, int D, float *dst) {
#pragma unroll
    for (int c = 0; c < DPT / 4; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            int d = (sub + 4 * c) * 4 + e;
            dst[c * 4 + e] = d < D ? to_f32<T>(src[d]) : 0.f;
        }
}

template <typename T, int DPT>
__device__ __forceinline__ void stage_tile(const T *base, int64_t first, int64_t limit, int D, float *dst) {
    constexpr int DP = 4 * DPT;
    for (int idx = threadIdx.x; idx < kTile * DP; idx += kThreads) {
        int r = idx / DP, d = idx % DP;
        float x = 0.f;
        if (first + r < limit && d < D) x = to_f32<T>(base[(first + r) * D + d]);
        dst[idx] = x;
    }
}

template <int DPT>
__device__ __forceinline__ float dot_smem(const float *a, const float *row, int sub) {
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < DPT / 4; ++c) {
        float4 x = *reinterpret_cast<const float4 *>(&row[(sub + 4 * c) * 4]);
        acc = fmaf(a[c * 4 + 0], x.x, acc);
        acc = fmaf(a[c * 4 + 1], x.y, acc);
        acc = fmaf(a[c * 4 + 2], x.z, acc);
        acc = fmaf(a[c * 4 + 3], x.w, acc);
    }
    return quad_sum(acc);
}

template <int DPT>
__device__ __forceinline__ void axpy_smem(float w, const float *row, int sub, float *acc) {
#pragma unroll
    for (int c = 0; c < DPT / 4; ++c) {
        float4 x = *reinterpret_cast<const float4 *>(&row[(sub + 4 * c) * 4]);
        acc[c * 4 + 0] = fmaf(w, x.x, acc[c * 4 + 0]);
        acc[c * 4 + 1] = fmaf(w, x.y, acc[c * 4 + 1]);
        acc[c * 4 + 2] = fmaf(w, x.z, acc[c * 4 + 2]);
        acc[c * 4 + 3] = fmaf(w, x.w, acc[c * 4 + 3]);
    }
}

template <typename T, int DPT>
__device__ __forceinline__ void store_row(T *dst, int sub, int D, const float *src) {
#pragma unroll
    for (int c = 0; c < DPT / 4; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            int d = (sub + 4 * c) * 4 + e;
            if (d < D) dst[d] = from_f32<T>(src[c * 4 + e]);
        }
}

// dQ: CTA = 32 query rows of one (batch, q_head); keys streamed through shared memory.
template <typename T, int DPT>
__global__ void __launch_bounds__(kThreads) bwd_dq_kernel(const __grid_constant__ BwdParams p,
                                                          const float *__restrict__ delta) {
    constexpr int DP = 4 * DPT;
    extern __shared__ float smem[];
    float *ks = smem, *vs = smem + kTile * DP;
    const int sub = threadIdx.x & 3, r = threadIdx.x >> 2;
    const int b = blockIdx.z, qh = blockIdx.y, kvh = qh / p.group;
    const int N = p.seq_len, D = p.head_dim;
    const int row = blockIdx.x * kRows + r;
    const bool valid = row < N;
    const int64_t q_base = ((int64_t)b * p.q_heads + qh) * N;
    const int64_t kv_base = ((int64_t)b * p.kv_heads + kvh) * N * (int64_t)D;

    float q[DPT], go[DPT], dq[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) q[i] = go[i] = dq[i] = 0.f;
    float lse = 0.f, dl = 0.f;
    if (valid) {
        load_row<T, DPT>((const T *)p.q + (q_base + row) * D, sub, D, q);
        load_row<T, DPT>((const T *)p.d_out + (q_base + row) * D, sub, D, go);
        lse = p.lse[q_base + row];
        dl = delta[q_base + row];
    }
    const int64_t limit = valid ? (p.causal ? row + 1 : N) : 0;
    const int64_t cta_limit = p.causal ? min((int64_t)N, (int64_t)blockIdx.x * kRows + kRows) : N;

    for (int64_t k0 = 0; k0 < cta_limit; k0 += kTile) {
        __syncthreads();
        stage_tile<T, DPT>((const T *)p.k + kv_base, k0, cta_limit, D, ks);
        stage_tile<T, DPT>((const T *)p.v + kv_base, k0, cta_limit, D, vs);
        __syncthreads();
#pragma unroll 4
        for (int j = 0; j < kTile; ++j) {
            float s = dot_smem<DPT>(q, &ks[j * DP], sub) * p.scale;
            float dp = dot_smem<DPT>(go, &vs[j * DP], sub);
            float prob = (k0 + j < limit) ? expf(s - lse) : 0.f;
            float d_dot = prob * (dp - dl) * p.scale;
            axpy_smem<DPT>(d_dot, &ks[j * DP], sub, dq);
        }
    }
    if (valid) store_row<float, DPT>((float *)p.dq + (q_base + row) * D, sub, D, dq);
}

// dK/dV: CTA = 32 key rows of one (batch, kv_head); the group's query heads and their query rows
// are streamed through shared memory in ascending order (q_head, then row).
template <typename T, int DPT>
__global__ void __launch_bounds__(kThreads) bwd_dkv_kernel(const __grid_constant__ BwdParams p,
                                                           const float *__restrict__ delta) {
    constexpr int DP = 4 * DPT;
    extern __shared__ float smem[];
    float *qs = smem, *gs = smem + kTile * DP;
    float *lse_s = smem + 2 * kTile * DP, *delta_s = lse_s + kTile;
    const int sub = threadIdx.x & 3, r = threadIdx.x >> 2;
    const int b = blockIdx.z, kvh = blockIdx.y;
    const int N = p.seq_len, D = p.head_dim;
    const int row = blockIdx.x * kRows + r;
    const bool valid = row < N;
    const int64_t kv_base = ((int64_t)b * p.kv_heads + kvh) * N;

    float k[DPT], v[DPT], dk[DPT], dv[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) k[i] = v[i] = dk[i] = dv[i] = 0.f;
    if (valid) {
        load_row<T, DPT>((const T *)p.k + (kv_base + row) * D, sub, D, k);
        load_row<T, DPT>((const T *)p.v + (kv_base + row) * D, sub, D, v);
    }
    // causal: query rows >= this key row; the CTA starts at its first key row
    const int64_t q_first = p.causal ? (int64_t)blockIdx.x * kRows : 0;

    for (int g = 0; g < p.group; ++g) {
        const int qh = kvh * p.group + g;
        const int64_t q_base = ((int64_t)b * p.q_heads + qh) * N;
        for (int64_t q0 = q_first; q0 < N; q0 += kTile) {
            __syncthreads();
            stage_tile<T, DPT>((const T *)p.q + q_base * D, q0, N, D, qs);
            stage_tile<T, DPT>((const T *)p.d_out + q_base * D, q0, N, D, gs);
            if (threadIdx.x < kTile) {
                int64_t qr = q0 + threadIdx.x;
                lse_s[threadIdx.x] = qr < N ? p.lse[q_base + qr] : 0.f;
                delta_s[threadIdx.x] = qr < N ? delta[q_base + qr] : 0.f;
            }
            __syncthreads();
#pragma unroll 4
            for (int j = 0; j < kTile; ++j) {
                const int64_t qr = q0 + j;
                float s = dot_smem<DPT>(k, &qs[j * DP], sub) * p.scale;
                float dp = dot_smem<DPT>(v, &gs[j * DP], sub);
                bool vis = valid && qr < N && (!p.causal || row <= qr);
                float prob = vis ? expf(s - lse_s[j]) : 0.f;
                float d_dot = prob * (dp - delta_s[j]) * p.scale;
                axpy_smem<DPT>(d_dot, &qs[j * DP], sub, dk);
                axpy_smem<DPT>(prob, &gs[j * DP], sub, dv);
            }
        }
    }
    if (valid) {
        store_row<float, DPT>((float *)p.dk + (kv_base + row) * D, sub, D, dk);
        store_row<float, DPT>((float *)p.dv + (kv_base + row) * D, sub, D, dv);
    }
}

template <typename T, int DPT>
int launch(flat_ctx *ctx, const BwdParams &p) {
    const int64_t rows = (int64_t)p.batch * p.q_heads * p.seq_len;
    int st = ensure_workspace(ctx, kWorkspaceMeta + rows * sizeof(float));
    if (st) return st;
    float *delta = reinterpret_cast<float *>(scratch_ptr(ctx));
    delta_kernel<T><<<(unsigned)((rows + 3) / 4), 128, 0, ctx->stream>>>((const T *)p.d_out, (const T *)p.out, delta,
                                                                         rows, p.head_dim);
    const int tiles = (p.seq_len + kRows - 1) / kRows;
    size_t smem_dq = 2 * kTile * 4 * DPT * sizeof(float);
    size_t smem_dkv = smem_dq + 2 * kTile * sizeof(float);
    bwd_dq_kernel<T, DPT><<<dim3(tiles, p.q_heads, p.batch), kThreads, smem_dq, ctx->stream>>>(p, delta);
    bwd_dkv_kernel<T, DPT><<<dim3(tiles, p.kv_heads, p.batch), kThreads, smem_dkv, ctx->stream>>>(p, delta);
    ctx->launches += 3;
    FLAT_CUDA_OK(ctx, cudaGetLastError());
    return FLAT_OK;
}

template <typename T>
int dispatch(flat_ctx *ctx, const BwdParams &p) {
    if (p.head_dim <= 16) return launch<T, 4>(ctx, p);
    if (p.head_dim <= 32) return launch<T, 8>(ctx, p);
    if (p.head_dim <= 64) return launch<T, 16>(ctx, p);
    return launch<T, 32>(ctx, p);
}

}  // namespace

int launch_backward_simt(flat_ctx *ctx, int dtype, const BwdParams &p) {
    if (p.q_heads > 65535 || p.batch > 65535)
        return fail(ctx, FLAT_ERR_DISPATCH_LIMIT, "grid dimension %d exceeds 65535", p.q_heads > 65535 ? p.q_heads : p.batch);
    return dtype == FLAT_BF16 ? dispatch<__nv_bfloat16>(ctx, p) : dispatch<float>(ctx, p);
}

}  // namespace flat
