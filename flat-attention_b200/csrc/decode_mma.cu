// bf16 q_len = 1 decode with the score and value products on the warp-level tensor cores.
//
// The streaming SIMT decode kernel issues ~120 warp instructions per (token, KV head) and is
// issue-bound at a third of HBM bandwidth.  Here one warp still owns one KV head of one
// (sequence, KV chunk) and still reads every K/V byte once with 16-byte loads, but the loaded
// registers are used directly as mma.sync.m16n8k16 fragments, about 8 instructions per token:
//
//   S^T[16 tokens x 8 heads] = K[16 tokens x D] * Q^T[D x 8 heads]
//       A = K: thread (g = lane/4, c = lane%4) loads 16 bytes (8 dims) of tokens g and g+8 per
//       32-dim chunk; a dot product does not care in which order dims are summed, so the 8
//       contiguous dims are assigned to the fragment's k-slots of two k-steps and Q^T uses the same
//       assignment.  Q^T (B operand) is built once: rotated at the query position in f32, scaled by
//       scale*log2(e), split into bf16 hi + lo so the rotation does not lose precision.
//   O^T[D x 8 heads] += V^T[D x 16 tokens] * P^T[16 tokens x 8 heads]
//       A = V^T: thread loads 16 dims of tokens 2c, 2c+1, 2c+8, 2c+9 and pairs the same dim of two
//       tokens with byte permutes; which dim lands in which output row is bookkeeping only.
//       B = P^T: the packed S^T accumulators transposed with movmatrix.
//
// Heads of the group sit on the n = 8 axis (group <= 8).  Softmax state (running max, partial sums)
// is per head; the max is made warp-consistent with three shuffles per tile, the sums are reduced
// once at the end.  Chunks of one sequence are merged by the same merge kernel as the SIMT path.
#include "common.h"

namespace flat {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One warp: KV head `kv_head` of sequence `seq`, tokens [begin, end) (begin a multiple of 16).
// to_partial: write the normalised (O, LSE) of this range to partial slot `slot`, else the final result.
template <int D>
__device__ __forceinline__ void decode_range(const DecodeParams &p, int seq, int kv_head, int begin, int end, int slot,
                                             bool to_partial) {
    constexpr int kChunks = D / 32;   // 32-dim chunks of the QK product
    constexpr int kVecs = D / 64;     // 16-byte vectors per token of this thread's V slice (D/8 dims)
    constexpr int kPv = D / 16;       // PV mma per tile
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int split = slot;
    const int G = p.group;

    // Q^T fragments: head g of the group, dims 32j + 8c .. +7, rotated, scaled, split hi/lo.
    // The rotation angle depends on (position, pair) only, so the warp evaluates each of the D/2 pairs once
    // (lane l takes pairs l and l + 32; at long-context positions sincosf runs its slow argument reduction)
    // and the fragments fetch their (cos, sin) with shuffles: pair 16j + 4c + e sits in lane
    // 16 (j mod 2) + 4c + e, slot j / 2.
    uint32_t qhi[kChunks][4], qlo[kChunks][4];
    {
        const int64_t q_pos = p.q_rope_positions ? (int64_t)p.q_rope_positions[seq] : p.uniform_q_pos;
        const float fold = p.scale * kLog2e;
        constexpr int kSlots = D / 64;
        float cs_c[kSlots], cs_s[kSlots];
#pragma unroll
        for (int sl = 0; sl < kSlots; ++sl) {
            cs_c[sl] = 1.f;
            cs_s[sl] = 0.f;
            if (p.rope_q) sincosf(__fmul_rn((float)q_pos, p.inv_freq[lane + 32 * sl]), &cs_s[sl], &cs_c[sl]);
        }
#pragma unroll
        for (int j = 0; j < kChunks; ++j) {
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (g < G)
                raw = *reinterpret_cast<const uint4 *>((const __nv_bfloat16 *)p.q +
                                                       ((int64_t)seq * p.q_heads + kv_head * G + g) * D + 32 * j + 8 * c);
            const uint32_t rr[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int src = 16 * (j & 1) + 4 * c + e;
                const float co = __shfl_sync(0xffffffffu, cs_c[j >> 1], src), s = __shfl_sync(0xffffffffu, cs_s[j >> 1], src);
                float x = __uint_as_float(rr[e] << 16), y = __uint_as_float(rr[e] & 0xffff0000u);
                const float rx = x * co - y * s, ry = x * s + y * co;  // (cos, sin) = (1, 0) without RoPE: exact
                x = rx * fold;
                y = ry * fold;
                const __nv_bfloat162 hi = __floats2bfloat162_rn(x, y);
                const float2 hf = __bfloat1622float2(hi);
                qhi[j][e] = *reinterpret_cast<const uint32_t *>(&hi);
                qlo[j][e] = pack_bf16(x - hf.x, y - hf.y);
            }
        }
    }

    float acc[kPv][4];
#pragma unroll
    for (int i = 0; i < kPv; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // heads 2c and 2c+1

    const char *kbase = (const char *)p.k;
    const char *vbase = (const char *)p.v;
    const int64_t row_bytes = (int64_t)p.kv_heads * D * 2;
    const int64_t head_bytes = (int64_t)kv_head * D * 2;
    const int32_t *table = p.page_table ? p.page_table + (int64_t)seq * p.max_pages : nullptr;

    for (int t0 = begin; t0 < end; t0 += 16) {
        int64_t row0;
        if (table) {
            const int page = table[t0 / p.page_size];
            // an entry outside the pool is never dereferenced: the tile is skipped and the call is flagged
            if ((unsigned)page >= (unsigned)p.physical_pages) {
                if (lane == 0 && p.status) {
                    p.status->code = FLAT_ERR_PAGE_OUT_OF_RANGE;
                    p.status->where = seq;
                }
                continue;
            }
            row0 = (int64_t)page * p.page_size + t0 % p.page_size;
        } else {
            row0 = (int64_t)seq * p.seq_stride_rows + t0;
        }
        const char *ktile = kbase + row0 * row_bytes + head_bytes;
        const char *vtile = vbase + row0 * row_bytes + head_bytes;

        // ---- loads: K rows g, g+8 (8 dims per 32-dim chunk); V rows 2c, 2c+1, 2c+8, 2c+9 (D/8 dims)
        uint4 ka[kChunks], kb[kChunks], vv[4][kVecs];
        const bool ok_a = t0 + g < end, ok_b = t0 + g + 8 < end;
#pragma unroll
        for (int j = 0; j < kChunks; ++j) {
            ka[j] = ok_a ? ldg_stream(ktile + (int64_t)g * row_bytes + (32 * j + 8 * c) * 2) : make_uint4(0, 0, 0, 0);
            kb[j] = ok_b ? ldg_stream(ktile + (int64_t)(g + 8) * row_bytes + (32 * j + 8 * c) * 2) : make_uint4(0, 0, 0, 0);
        }
        const int vt[4] = {2 * c, 2 * c + 1, 2 * c + 8, 2 * c + 9};
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const bool ok = t0 + vt[x] < end;
#pragma unroll
            for (int u = 0; u < kVecs; ++u)
                vv[x][u] = ok ? ldg_stream(vtile + (int64_t)vt[x] * row_bytes + ((D / 8) * g + 8 * u) * 2)
                              : make_uint4(0, 0, 0, 0);
        }

        // ---- S^T = K Q^T (hi + lo)
        float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < kChunks; ++j) {
            mma_bf16(s, ka[j].x, kb[j].x, ka[j].y, kb[j].y, qhi[j][0], qhi[j][1]);
            mma_bf16(s, ka[j].z, kb[j].z, ka[j].w, kb[j].w, qhi[j][2], qhi[j][3]);
            mma_bf16(s, ka[j].x, kb[j].x, ka[j].y, kb[j].y, qlo[j][0], qlo[j][1]);
            mma_bf16(s, ka[j].z, kb[j].z, ka[j].w, kb[j].w, qlo[j][2], qlo[j][3]);
        }
        if (!ok_a) s[0] = s[1] = -INFINITY;
        if (!ok_b) s[2] = s[3] = -INFINITY;

        // ---- online softmax per head (columns 2c, 2c+1); tokens live on g: reduce over lanes 4, 8, 16
        float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
        for (int w = 4; w < 32; w <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, w));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, w));
        }
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);  // finite: every tile has a live token g = 0
        const float a0 = ex2f(m0 - n0), a1 = ex2f(m1 - n1);    // m = -inf gives 0
        m0 = n0;
        m1 = n1;
        s[0] = ex2f(s[0] - n0);
        s[2] = ex2f(s[2] - n0);
        s[1] = ex2f(s[1] - n1);
        s[3] = ex2f(s[3] - n1);
        l0 = l0 * a0 + s[0] + s[2];
        l1 = l1 * a1 + s[1] + s[3];
        if (__any_sync(0xffffffffu, a0 != 1.0f || a1 != 1.0f)) {
#pragma unroll
            for (int i = 0; i < kPv; ++i) {
                acc[i][0] *= a0;
                acc[i][2] *= a0;
                acc[i][1] *= a1;
                acc[i][3] *= a1;
            }
        }
        const uint32_t b0 = movmatrix_trans(pack_bf16(s[0], s[1]));  // {P[2c][g], P[2c+1][g]}
        const uint32_t b1 = movmatrix_trans(pack_bf16(s[2], s[3]));  // {P[2c+8][g], P[2c+9][g]}

        // ---- O^T += V^T P^T: mma i covers dims (D/8)*g + 2i (row g) and + 2i + 1 (row g + 8)
#pragma unroll
        for (int u = 0; u < kVecs; ++u) {
            const uint32_t r0[4] = {vv[0][u].x, vv[0][u].y, vv[0][u].z, vv[0][u].w};
            const uint32_t r1[4] = {vv[1][u].x, vv[1][u].y, vv[1][u].z, vv[1][u].w};
            const uint32_t r2[4] = {vv[2][u].x, vv[2][u].y, vv[2][u].z, vv[2][u].w};
            const uint32_t r3[4] = {vv[3][u].x, vv[3][u].y, vv[3][u].z, vv[3][u].w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
                mma_bf16(acc[u * 4 + e], __byte_perm(r0[e], r1[e], 0x5410), __byte_perm(r0[e], r1[e], 0x7632),
                         __byte_perm(r2[e], r3[e], 0x5410), __byte_perm(r2[e], r3[e], 0x7632), b0, b1);
        }
    }

#pragma unroll
    for (int w = 4; w < 32; w <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, w);
        l1 += __shfl_xor_sync(0xffffffffu, l1, w);
    }

    // thread (g, c) holds heads 2c, 2c+1 and dims (D/8)*g .. +D/8-1 (acc[i][0], acc[i][2] interleaved)
    constexpr int kDims = D / 8;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int head_in_group = 2 * c + hh;
        if (head_in_group >= G) continue;
        const float m = hh ? m1 : m0, l = hh ? l1 : l0;
        // l == 0 only when every tile of the range was skipped (flagged page-table entries): O = 0, LSE = -inf
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        const float lse = l > 0.f ? (m + log2f(l)) * kLn2 : -INFINITY;
        const int64_t out_row = (int64_t)seq * p.q_heads + kv_head * G + head_in_group;
        float vals[kDims];
#pragma unroll
        for (int i = 0; i < kPv; ++i) {
            vals[2 * i] = acc[i][hh] * inv;
            vals[2 * i + 1] = acc[i][2 + hh] * inv;
        }
        if (to_partial) {
            float *po = p.partial_o + ((int64_t)split * p.num_seqs * p.q_heads + out_row) * D + kDims * g;
#pragma unroll
            for (int e = 0; e < kDims; e += 4)
                *reinterpret_cast<float4 *>(po + e) = make_float4(vals[e], vals[e + 1], vals[e + 2], vals[e + 3]);
            if (g == 0) p.partial_lse[(int64_t)split * p.num_seqs * p.q_heads + out_row] = lse;
        } else if (p.out_f32) {
            float *po = (float *)p.o + out_row * D + kDims * g;
#pragma unroll
            for (int e = 0; e < kDims; e += 4)
                *reinterpret_cast<float4 *>(po + e) = make_float4(vals[e], vals[e + 1], vals[e + 2], vals[e + 3]);
            if (g == 0) p.lse[out_row] = lse;
        } else {
            __nv_bfloat16 *op = (__nv_bfloat16 *)p.o + out_row * D + kDims * g;
#pragma unroll
            for (int e = 0; e < kDims; e += 8) {
                uint4 pk;
                pk.x = pack_bf16(vals[e], vals[e + 1]);
                pk.y = pack_bf16(vals[e + 2], vals[e + 3]);
                pk.z = pack_bf16(vals[e + 4], vals[e + 5]);
                pk.w = pack_bf16(vals[e + 6], vals[e + 7]);
                *reinterpret_cast<uint4 *>(op + e) = pk;
            }
            if (g == 0) p.lse[out_row] = lse;
        }
    }
}

template <int D>
__global__ void __launch_bounds__(256, 2) decode_mma_kernel(const __grid_constant__ DecodeParams p) {
    const int warp = threadIdx.x >> 5;
    const int kv_head = blockIdx.y * (blockDim.x >> 5) + warp;
    if (kv_head >= p.kv_heads) return;
    if (!p.balanced) {
        const int seq = blockIdx.z;
        const int split = blockIdx.x;
        const int ctx_len = p.context_lens ? p.context_lens[seq] : p.uniform_len;
        int begin = 0, end = ctx_len;
        if (p.kv_splits > 1) {
            begin = split * p.chunk_tokens;
            end = min(ctx_len, begin + p.chunk_tokens);
            if (begin >= end) return;
        }
        decode_range<D>(p, seq, kv_head, begin, end, split, p.kv_splits > 1);
        return;
    }
    // balanced: this CTA streams [cta*span, (cta+1)*span) of the concatenated (16-padded) sequences
    const int cta = blockIdx.x;
    const int total = p.seq_offsets[p.num_seqs];
    int pos = cta * p.span_tokens;
    const int span_end = min(total, pos + p.span_tokens);
    if (pos >= span_end) return;
    int seq = 0;
    while (seq + 1 < p.num_seqs && p.seq_offsets[seq + 1] <= pos) ++seq;
    while (pos < span_end) {
        const int off = p.seq_offsets[seq], next = p.seq_offsets[seq + 1];
        const int seg_end = min(span_end, next);
        const int ctx_len = p.context_lens ? p.context_lens[seq] : p.uniform_len;
        const int first_cta = off / p.span_tokens, last_cta = (next - 1) / p.span_tokens;
        decode_range<D>(p, seq, kv_head, pos - off, min(ctx_len, seg_end - off), cta - first_cta, last_cta > first_cta);
        pos = seg_end;
        ++seq;
    }
}

}  // namespace

bool decode_mma_supported(int dtype, const DecodeParams &p) {
    if (dtype != FLAT_BF16) return false;
    if (p.head_dim != 64 && p.head_dim != 128) return false;
    if (p.group > 8) return false;
    if (p.page_size != 0 && p.page_size % 16 != 0) return false;  // a 16-token tile must stay inside one page
    if (p.kv_splits > 1 && p.chunk_tokens % 16 != 0) return false;
    return true;
}

int launch_decode_mma(flat_ctx *ctx, const DecodeParams &p) {
    const int warps = p.kv_heads < 8 ? p.kv_heads : 8;
    dim3 grid(p.kv_splits, (p.kv_heads + warps - 1) / warps, p.num_seqs);
    if (p.balanced) grid = dim3(p.num_ctas, (p.kv_heads + warps - 1) / warps, 1);
    KernelTimer timer(ctx);
    if (p.head_dim == 128) decode_mma_kernel<128><<<grid, warps * 32, 0, ctx->stream>>>(p);
    else decode_mma_kernel<64><<<grid, warps * 32, 0, ctx->stream>>>(p);
    return FLAT_OK;
}

}  // namespace flat
