// q_len = 1 decode over a paged or resident (contiguous) KV cache, and the split-KV merge.
//
// HBM-bound: every K/V byte is read exactly once.  One CTA owns (sequence, KV chunk) and streams
// whole cache rows: warp w serves KV head w, so the CTA's warps together read the contiguous
// kv_heads*head_dim row of every token (pages of 16 tokens are 32 KiB contiguous runs at Hkv=8,
// D=128, bf16).  Inside a warp a row slice of head_dim elements is covered by 16-byte loads, two
// (bf16) or one (f32) token per warp load; the query heads of the KV head's group all consume the
// loaded registers, so GQA never re-reads K/V.  Each half-warp keeps its own online-softmax state
// over its tokens and the states are merged with warp shuffles; chunks of one sequence are merged
// by a second small kernel through their (O, LSE) partials.
//
// Semantics follow shaders/flat_decode_paged.wgsl:129-220 and shaders/flat_decode_resident.wgsl:
// Q is rotated in-kernel at q_rope_position, K is pre-rotated, V is raw, no causal mask (the host
// enforces that the query sees the whole live prefix), physical row = table[t / page_size] *
// page_size + t % page_size.
#include <cmath>

#include "common.h"

namespace flat {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int kUnroll = 4;  // token groups in flight per warp

template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int kPerLane = 4;
    __device__ static void unpack(const uint4 &r, float *f) {
        f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y);
        f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
    }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int kPerLane = 8;
    __device__ static void unpack(const uint4 &r, float *f) {
        // bf16 -> f32 is a 16-bit shift
        f[0] = __uint_as_float(r.x << 16); f[1] = __uint_as_float(r.x & 0xffff0000u);
        f[2] = __uint_as_float(r.y << 16); f[3] = __uint_as_float(r.y & 0xffff0000u);
        f[4] = __uint_as_float(r.z << 16); f[5] = __uint_as_float(r.z & 0xffff0000u);
        f[6] = __uint_as_float(r.w << 16); f[7] = __uint_as_float(r.w & 0xffff0000u);
    }
};

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

// LPR = lanes covering one head_dim slice (power of two), G = query heads per KV head.
template <typename T, int LPR, int G>
__global__ void __launch_bounds__(256) decode_kernel(const __grid_constant__ DecodeParams p) {
    constexpr int EPL = Elem<T>::kPerLane;
    constexpr int TPW = 32 / LPR;  // tokens per warp load
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int kv_head = blockIdx.y * (blockDim.x >> 5) + warp;
    const int seq = blockIdx.z;
    const int split = blockIdx.x;
    if (kv_head >= p.kv_heads) return;

    const int ctx_len = p.context_lens ? p.context_lens[seq] : p.uniform_len;
    int begin = 0, end = ctx_len;
    if (p.kv_splits > 1) {
        begin = split * p.chunk_tokens;
        end = min(ctx_len, begin + p.chunk_tokens);
        if (begin >= end) return;  // the merge skips chunks past the context
    }

    const int D = p.head_dim;
    const int lane_in_row = lane % LPR;
    const int tok_lane = lane / LPR;
    const int d0 = lane_in_row * EPL;
    const bool lane_active = d0 < D;

    // this lane's slice of the group's query rows, rotated at the sequence's query position
    float q[G][EPL];
    const int64_t q_pos = p.q_rope_positions ? (int64_t)p.q_rope_positions[seq] : p.uniform_q_pos;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const T *qp = (const T *)p.q + ((int64_t)seq * p.q_heads + kv_head * G + g) * D + d0;
#pragma unroll
        for (int e = 0; e < EPL; ++e) q[g][e] = 0.f;
        if (lane_active) {
            uint4 raw = *reinterpret_cast<const uint4 *>(qp);
            Elem<T>::unpack(raw, q[g]);
            if (p.rope_q) {
#pragma unroll
                for (int e = 0; e < EPL; e += 2) {
                    float angle = __fmul_rn((float)q_pos, p.inv_freq[(d0 + e) >> 1]);
                    float s, c;
                    sincosf(angle, &s, &c);
                    float re = q[g][e] * c - q[g][e + 1] * s;
                    float ro = q[g][e] * s + q[g][e + 1] * c;
                    q[g][e] = re;
                    q[g][e + 1] = ro;
                }
            }
        }
        // fold the softmax scale and log2(e) into Q once: scores come out in the exp2 domain
#pragma unroll
        for (int e = 0; e < EPL; ++e) q[g][e] *= p.scale * kLog2e;
    }

    float m[G], l[G], o[G][EPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) o[g][e] = 0.f;
    }

    const char *kbase = (const char *)p.k;
    const char *vbase = (const char *)p.v;
    const int64_t row_elems = (int64_t)p.kv_heads * D;
    const int64_t head_off = (int64_t)kv_head * D + d0;
    const int32_t *table = p.page_table ? p.page_table + (int64_t)seq * p.max_pages : nullptr;

    for (int t0 = begin; t0 < end; t0 += TPW * kUnroll) {
        uint4 kraw[kUnroll], vraw[kUnroll];
        bool ok[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            int t = t0 + u * TPW + tok_lane;
            ok[u] = t < end;
            kraw[u] = make_uint4(0, 0, 0, 0);
            vraw[u] = make_uint4(0, 0, 0, 0);
            int64_t row = 0;
            if (ok[u]) {
                if (table) {
                    const int page = table[t / p.page_size];
                    // an entry outside the pool is never dereferenced: the token is masked and the call is flagged
                    if ((unsigned)page >= (unsigned)p.physical_pages) {
                        ok[u] = false;
                        if (p.status) {
                            p.status->code = FLAT_ERR_PAGE_OUT_OF_RANGE;
                            p.status->where = seq;
                        }
                    }
                    row = (int64_t)page * p.page_size + t % p.page_size;
                } else {
                    row = (int64_t)seq * p.seq_stride_rows + t;
                }
            }
            if (ok[u] && lane_active) {
                int64_t off = (row * row_elems + head_off) * (int64_t)sizeof(T);
                kraw[u] = ldg_stream(kbase + off);
                vraw[u] = ldg_stream(vbase + off);
            }
        }
        float s[kUnroll][G];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            float kf[EPL];
            Elem<T>::unpack(kraw[u], kf);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float acc = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc = fmaf(q[g][e], kf[e], acc);
#pragma unroll
                for (int w = LPR / 2; w >= 1; w >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, w);
                s[u][g] = ok[u] ? acc : -INFINITY;
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float mx = m[g];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) mx = fmaxf(mx, s[u][g]);
            if (mx == -INFINITY) continue;
            float alpha = exp2f(m[g] - mx);  // m = -inf gives 0
            m[g] = mx;
            l[g] *= alpha;
#pragma unroll
            for (int e = 0; e < EPL; ++e) o[g][e] *= alpha;
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) s[u][g] = exp2f(s[u][g] - mx);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            float vf[EPL];
            Elem<T>::unpack(vraw[u], vf);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float pj = (m[g] == -INFINITY) ? 0.f : s[u][g];
                l[g] += pj;
#pragma unroll
                for (int e = 0; e < EPL; ++e) o[g][e] = fmaf(pj, vf[e], o[g][e]);
            }
        }
    }

    // merge the token-lane states of the warp (warp-shuffle LSE merge)
#pragma unroll
    for (int w = LPR; w < 32; w <<= 1) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float m2 = __shfl_xor_sync(0xffffffffu, m[g], w);
            float l2 = __shfl_xor_sync(0xffffffffu, l[g], w);
            float mx = fmaxf(m[g], m2);
            float a1 = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mx);
            float a2 = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mx);
            l[g] = l[g] * a1 + l2 * a2;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                float o2 = __shfl_xor_sync(0xffffffffu, o[g][e], w);
                o[g][e] = o[g][e] * a1 + o2 * a2;
            }
            m[g] = mx;
        }
    }

    if (tok_lane != 0 || !lane_active) return;
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int q_head = kv_head * G + g;
        // l == 0 only when every token of the range was masked (flagged page-table entries): O = 0, LSE = -inf
        const float inv = l[g] > 0.f ? 1.0f / l[g] : 0.f;
        const float lse = l[g] > 0.f ? (m[g] + log2f(l[g])) * kLn2 : -INFINITY;
        const int64_t out_row = (int64_t)seq * p.q_heads + q_head;
        if (p.kv_splits > 1) {
            float *po = p.partial_o + ((int64_t)split * p.num_seqs * p.q_heads + out_row) * D + d0;
#pragma unroll
            for (int e = 0; e < EPL; e += 4)
                *reinterpret_cast<float4 *>(po + e) =
                    make_float4(o[g][e] * inv, o[g][e + 1] * inv, o[g][e + 2] * inv, o[g][e + 3] * inv);
            if (lane_in_row == 0) p.partial_lse[(int64_t)split * p.num_seqs * p.q_heads + out_row] = lse;
        } else {
            T *op = (T *)p.o + out_row * D + d0;
            if constexpr (sizeof(T) == 4) {
                *reinterpret_cast<float4 *>(op) =
                    make_float4(o[g][0] * inv, o[g][1] * inv, o[g][2] * inv, o[g][3] * inv);
            } else {
                __nv_bfloat162 h[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(o[g][2 * e] * inv, o[g][2 * e + 1] * inv);
                *reinterpret_cast<uint4 *>(op) = *reinterpret_cast<uint4 *>(h);
            }
            if (lane_in_row == 0) p.lse[out_row] = lse;
        }
    }
}

// Merge of split-KV partials: one CTA of 128 threads per (sequence, q_head) row.
//   LSE = log(sum_i exp(LSE_i)),  O = sum_i exp(LSE_i - LSE) O_i
// Phase 1: the threads reduce max and sum of the parts' LSE; phase 2: thread d accumulates column d
// over the parts with the weights staged in shared memory (coalesced rows, several loads in flight).
// Fixed-chunk mode: only ceil(ctx/chunk) parts of a row are live.  Balanced mode: one slot per CTA that
// touched the sequence; a single slot was already written as the final result.
constexpr int kMergeDims = 128;    // threads along the head dimension (kMaxHeadDim)
constexpr int kMergeGroupsWide = 4;  // thread groups of the wide variant; group g takes the parts g, g + 4, ... of a batch
constexpr int kMergeWideFrom = 17;   // rows with this many parts or more are merged by the wide variant
constexpr int kMergeBatch = 512;   // weights staged per pass

// Merge of the split-KV partials of one row: LSE = log sum exp(LSE_i), O = sum exp(LSE_i - LSE) O_i.  GROUPS = 1: 128
// threads, the parts are added in order (a batch of many short sequences: few parts per row, thousands of rows).
// GROUPS = 4: a long context cut into short spans gives a row hundreds of parts and a batch only a few rows, so the
// parts are spread over four thread groups (the loop is a chain of L2 round trips otherwise) and the groups' sums are
// added in group order.  Either way eight independent loads are in flight per thread and the result is a fixed
// function of the inputs and of the part count.
template <typename T, int GROUPS>
__global__ void __launch_bounds__(kMergeDims * GROUPS) merge_kernel(int parts, int64_t rows, int head_dim,
                                                              const float *__restrict__ partial_o,
                                                              const float *__restrict__ partial_lse, T *__restrict__ o,
                                                              float *__restrict__ lse, const int32_t *context_lens,
                                                              int uniform_len, int chunk_tokens, int rows_per_seq,
                                                              const int32_t *seq_offsets, int span_tokens, int64_t stride_o,
                                                              int64_t stride_lse) {
    constexpr int kMergeGroups = GROUPS, kMergeThreads = kMergeDims * GROUPS;
    __shared__ float w_s[kMergeBatch];
    __shared__ float red[kMergeThreads / 32];
    __shared__ float acc_s[kMergeGroups][kMergeDims];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int dim = tid % kMergeDims, group = tid / kMergeDims;
    const int64_t row = blockIdx.x;
    int live = parts;
    if (seq_offsets) {
        const int seq = (int)(row / rows_per_seq);
        live = (seq_offsets[seq + 1] - 1) / span_tokens - seq_offsets[seq] / span_tokens + 1;
        if (live <= 1) return;
    } else if (chunk_tokens > 0) {
        int len = context_lens ? context_lens[row / rows_per_seq] : uniform_len;
        live = min(parts, (len + chunk_tokens - 1) / chunk_tokens);
    }
    auto block_reduce = [&](float x, bool is_max) {
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
            const float y = __shfl_xor_sync(0xffffffffu, x, s);
            x = is_max ? fmaxf(x, y) : x + y;
        }
        __syncthreads();
        if (lane == 0) red[warp] = x;
        __syncthreads();
        float r = red[0];
        for (int i = 1; i < kMergeThreads / 32; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
        return r;
    };
    float mx = -INFINITY;
    for (int i = tid; i < live; i += kMergeThreads) mx = fmaxf(mx, partial_lse[(int64_t)i * stride_lse + row]);
    mx = block_reduce(mx, true);
    float sum = 0.f;
    for (int i = tid; i < live; i += kMergeThreads) sum += expf(partial_lse[(int64_t)i * stride_lse + row] - mx);
    sum = block_reduce(sum, false);
    const float total = mx + logf(sum);
    float acc = 0.f;
    for (int base = 0; base < live; base += kMergeBatch) {
        const int n = min(kMergeBatch, live - base);
        __syncthreads();
        for (int i = tid; i < n; i += kMergeThreads) w_s[i] = expf(partial_lse[(int64_t)(base + i) * stride_lse + row] - total);
        __syncthreads();
        if (dim < head_dim) {
            const float *src = partial_o + (int64_t)base * stride_o + row * head_dim + dim;
            int i = group;
            for (; i + 7 * kMergeGroups < n; i += 8 * kMergeGroups) {
                float a[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) a[u] = src[(int64_t)(i + u * kMergeGroups) * stride_o];
#pragma unroll
                for (int u = 0; u < 8; ++u) acc = fmaf(w_s[i + u * kMergeGroups], a[u], acc);
            }
            for (; i < n; i += kMergeGroups) acc = fmaf(w_s[i], src[(int64_t)i * stride_o], acc);
        }
    }
    acc_s[group][dim] = acc;
    __syncthreads();
    if (group == 0 && dim < head_dim) {
        float r = acc_s[0][dim];
#pragma unroll
        for (int g = 1; g < kMergeGroups; ++g) r += acc_s[g][dim];
        if constexpr (sizeof(T) == 4) o[row * head_dim + dim] = r;
        else o[row * head_dim + dim] = __float2bfloat16_rn(r);
    }
    if (tid == 0) lse[row] = total;
}

template <typename T>
int merge_chunks(flat_ctx *ctx, const DecodeParams &p) {
    if (p.kv_splits <= 1) return FLAT_OK;
    int64_t rows = (int64_t)p.num_seqs * p.q_heads;
    int blocks = (int)rows;
    if (p.kv_splits >= kMergeWideFrom)
        merge_kernel<T, kMergeGroupsWide><<<blocks, kMergeDims * kMergeGroupsWide, 0, ctx->stream>>>(
            p.kv_splits, rows, p.head_dim, p.partial_o, p.partial_lse, (T *)p.o, p.lse, p.context_lens, p.uniform_len,
            p.chunk_tokens, p.q_heads, p.balanced ? p.seq_offsets : nullptr, p.span_tokens, rows * p.head_dim, rows);
    else
        merge_kernel<T, 1><<<blocks, kMergeDims, 0, ctx->stream>>>(
            p.kv_splits, rows, p.head_dim, p.partial_o, p.partial_lse, (T *)p.o, p.lse, p.context_lens, p.uniform_len,
            p.chunk_tokens, p.q_heads, p.balanced ? p.seq_offsets : nullptr, p.span_tokens, rows * p.head_dim, rows);
    ctx->launches += 1;
    FLAT_CUDA_OK(ctx, cudaGetLastError());
    return FLAT_OK;
}

template <typename T, int LPR, int G>
int launch_lg(flat_ctx *ctx, const DecodeParams &p) {
    int warps = p.kv_heads < 8 ? p.kv_heads : 8;
    dim3 grid(p.kv_splits, (p.kv_heads + warps - 1) / warps, p.num_seqs);
    {
        KernelTimer timer(ctx);
        decode_kernel<T, LPR, G><<<grid, warps * 32, 0, ctx->stream>>>(p);
    }
    ctx->launches += 1;
    FLAT_CUDA_OK(ctx, cudaGetLastError());
    return merge_chunks<T>(ctx, p);
}

template <typename T, int LPR>
int launch_l(flat_ctx *ctx, const DecodeParams &p) {
    switch (p.group) {
        case 1: return launch_lg<T, LPR, 1>(ctx, p);
        case 2: return launch_lg<T, LPR, 2>(ctx, p);
        case 4: return launch_lg<T, LPR, 4>(ctx, p);
        case 8: return launch_lg<T, LPR, 8>(ctx, p);
    }
    return FLAT_ERR_UNSUPPORTED_SHAPE;
}

template <typename T>
int launch_t(flat_ctx *ctx, const DecodeParams &p) {
    int lanes = (p.head_dim + Elem<T>::kPerLane - 1) / Elem<T>::kPerLane;
    if (lanes <= 1) return launch_l<T, 1>(ctx, p);
    if (lanes <= 2) return launch_l<T, 2>(ctx, p);
    if (lanes <= 4) return launch_l<T, 4>(ctx, p);
    if (lanes <= 8) return launch_l<T, 8>(ctx, p);
    if (lanes <= 16) return launch_l<T, 16>(ctx, p);
    return launch_l<T, 32>(ctx, p);
}

}  // namespace

uint64_t decode_workspace_bytes(const DecodeParams &p) {
    if (p.kv_splits <= 1) return 0;
    uint64_t rows = (uint64_t)p.num_seqs * p.q_heads;
    return (uint64_t)p.kv_splits * rows * (p.head_dim + 1) * sizeof(float);
}

// The streaming kernel needs head_dim to be a whole number of 16-byte lanes and a power-of-two
// group of at most 8; other shapes are served by the generic forward kernel (q_len = 1).
bool decode_fast_path_ok(int dtype, int head_dim, int group) {
    int epl = dtype == FLAT_BF16 ? 8 : 4;
    return head_dim % epl == 0 && (group == 1 || group == 2 || group == 4 || group == 8);
}

int launch_decode(flat_ctx *ctx, int dtype, const DecodeParams &p) {
    if (p.num_seqs > 65535) return fail(ctx, FLAT_ERR_DISPATCH_LIMIT, "decode batch %d exceeds 65535", p.num_seqs);
    if (decode_mma_supported(dtype, p)) {
        launch_decode_mma(ctx, p);
        ctx->launches += 1;
        FLAT_CUDA_OK(ctx, cudaGetLastError());
        return p.out_f32 ? merge_chunks<float>(ctx, p) : merge_chunks<__nv_bfloat16>(ctx, p);
    }
    if (p.out_f32 && dtype != FLAT_F32)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "f32 partial output needs the tensor-core decode shape (head_dim 64/128, group <= 8, pages of 16)");
    int st = dtype == FLAT_BF16 ? launch_t<__nv_bfloat16>(ctx, p) : launch_t<float>(ctx, p);
    return st;
}

int launch_splitkv_merge(flat_ctx *ctx, int dtype, int parts, int64_t rows, int head_dim, const float *partial_o,
                         const float *partial_lse, int64_t part_stride_o, int64_t part_stride_lse, void *o, float *lse) {
    int blocks = (int)rows;
    auto launch = [&](auto kernel, int threads, auto *out) {
        kernel<<<blocks, threads, 0, ctx->stream>>>(parts, rows, head_dim, partial_o, partial_lse, out, lse, nullptr, 0, 0, 1, nullptr,
                                                   0, part_stride_o, part_stride_lse);
    };
    const bool wide = parts >= kMergeWideFrom;
    if (dtype == FLAT_BF16) {
        if (wide) launch(merge_kernel<__nv_bfloat16, kMergeGroupsWide>, kMergeDims * kMergeGroupsWide, (__nv_bfloat16 *)o);
        else launch(merge_kernel<__nv_bfloat16, 1>, kMergeDims, (__nv_bfloat16 *)o);
    } else {
        if (wide) launch(merge_kernel<float, kMergeGroupsWide>, kMergeDims * kMergeGroupsWide, (float *)o);
        else launch(merge_kernel<float, 1>, kMergeDims, (float *)o);
    }
    ctx->launches += 1;
    FLAT_CUDA_OK(ctx, cudaGetLastError());
    return FLAT_OK;
}

}  // namespace flat

// ---- fixed scratch for callers that must not allocate ------------------------------------------
// Some hosts of this library cannot call cudaMalloc at the moment they need a decode step:
// latency-critical serving loops where an allocation would synchronise the device, plug-ins living under a
// framework allocator that forbids side allocations, or processes whose memory budget was fixed at start-up.
// The split-KV decode needs scratch for its per-chunk (O, LSE) partials; the regular entry point takes it
// from the context workspace, which may grow.  flat_decode_paged_batched_static_scratch keeps the partials
// in this fixed array, which is part of the library image, so the call itself allocates nothing.
namespace flat {
namespace {

static __device__ __align__(256) float g_decode_static_scratch[kDecodeStaticScratchBytes / sizeof(float)];

constexpr int kMaxDevices = 64;
float *g_static_scratch_ptr[kMaxDevices] = {};

}  // namespace

// The array's name is only a host-side stand-in; the device address has to be asked for, once per
// device, with that device current.
int decode_static_scratch(flat_ctx *ctx, float **out) {
    if (ctx->device < 0 || ctx->device >= kMaxDevices)
        return fail(ctx, FLAT_ERR_UNAVAILABLE, "device index %d is outside the supported range", ctx->device);
    if (!g_static_scratch_ptr[ctx->device]) {
        int current = -1;
        FLAT_CUDA_OK(ctx, cudaGetDevice(&current));
        if (current != ctx->device) FLAT_CUDA_OK(ctx, cudaSetDevice(ctx->device));
        float *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_decode_static_scratch);
        if (current != ctx->device && current >= 0) cudaSetDevice(current);
        if (e != cudaSuccess || !ptr)
            return fail(ctx, FLAT_ERR_EXECUTION, "cudaGetSymbolAddress(static decode scratch): %s", cudaGetErrorString(e));
        g_static_scratch_ptr[ctx->device] = ptr;
    }
    *out = g_static_scratch_ptr[ctx->device];
    return FLAT_OK;
}

}  // namespace flat
