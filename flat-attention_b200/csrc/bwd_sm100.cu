// tcgen05 backward (LSE recompute) for bf16, head_dim 64 or 128, head-major, equal length, any
// seq_len (rows past it are zero-filled by TMA, their LSE / delta slots are zero).  Math per visible (query q, key k) pair (src/backward_grouped.rs:56-88):
//   P = exp(S*scale - LSE),  dP = dO.V,  dS = P*(dP - delta),  delta = dO.O
//   dV[kv_head] += P^T dO,  dK[kv_head] += scale * dS^T Q,  dQ += scale * dS K
// Two deterministic kernels, no atomics, results bitwise repeatable like the reference:
//
//  * KV-stationary (dK, dV): one CTA owns 128 keys of one (batch, kv_head); K and V stay in shared
//    memory, (Q_i, dO_i) tiles of every query head of the group stream through a TMA ring.  Per
//    tile: S^T = K Q_i^T and dP^T = V dO_i^T (SS MMAs into TMEM, keys on TMEM lanes), the eight
//    elementwise warps turn them into bf16 P^T and dS^T in place (a thread owns a key row and half of
//    the query columns; LSE and delta are per-column values read from shared memory), then
//    dV += P^T dO_i and dK += dS^T Q_i (A operand from TMEM) accumulate in TMEM over all tiles and
//    all heads of the group: the GQA reduction never leaves the SM.
//    The elementwise work is split in two phases (P^T, then dS^T) that overlap the MMAs.
//  * Q-stationary (dQ): one CTA owns 128 queries of one (batch, q_head); (K_j, V_j) stream;
//    S = Q K_j^T (Q as TMEM A operand), dP = dO V_j^T, dS in TMEM columns of its own, dQ += dS K_j
//    in TMEM; the next tile's products are issued while the elementwise warps work.
//
// The score recompute is done twice (7 GEMM units instead of 5); in exchange nothing is accumulated
// through global memory.  A prologue kernel writes delta and -LSE*log2(e) to context scratch.
//
// When the context's backward scratch budget allows it (flat_ctx_set_backward_scratch_budget), the recompute is
// spent once only: the KV-stationary kernel also writes every bf16 dS^T tile it forms to scratch (SPILL; one 32 KiB
// bulk store per streamed tile, issued by an otherwise idle thread), and dQ comes from a third kernel that only
// streams those tiles and the K tiles through the tensor core, dQ_i = sum_j dS_ij K_j (5 GEMM units executed, no
// elementwise work, HBM-bound).  The scratch holds one tile per visible (key tile, query tile) pair: O(N^2) bytes,
// which is why a budget decides.
// Gradients are written in f32: the accumulators are f32, and a bf16 rounding of a gradient above 4
// (ulp 2^-5) would by itself use up the 2e-2 absolute error bound.
#include <cuda.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "common.h"
#include "sm100_host.cuh"
#include "sm100_ptx.cuh"

namespace flat {
namespace {

using namespace sm100;

constexpr int kTile = 128;
constexpr int kThreads = 384;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr float kLog2e = 1.4426950408889634f;

// Debug timeline (compiled in with -DFLAT_TRACE), same layout as in the forward kernel.
#ifdef FLAT_TRACE
#define TRACE(role, it, slot)                                                                          \
    do {                                                                                               \
        if (p.trace && blockIdx.x == 0 && (it) < 64) p.trace[((role) * 64 + (it)) * 8 + (slot)] = clock64(); \
    } while (0)
#else
#define TRACE(role, it, slot) do { } while (0)
#endif

struct BwdKernelParams {
    CUtensorMap map_q, map_k, map_v, map_do;
    const float *neg_lse2;  // -LSE * log2(e), [B, Hq, N]
    const float *delta;     // dO . O, [B, Hq, N]
    void *out0, *out1;      // f32 outputs.  KV-stationary kernel: dV, dK; dQ kernels: dQ, null
    uint8_t *ds_spill;      // SPILL: bf16 dS^T tiles, 32 KiB each, tile (key tile j, query tile i) of (batch, q head) at
                            // ((batch * q_heads + head) * tiles_per_head + (causal ? i (i + 1) / 2 + j : i * n_tiles + j))
    int batch, q_heads, kv_heads, seq_len, group, n_tiles;
    int seq_pad;            // seq_len rounded up to whole tiles: row stride of neg_lse2 / delta
    int causal;
    float scale, scale_log2;
    uint32_t idesc_k, idesc_mn, idesc_dq;
    DeviceStatus *status;
    long long *trace;
};

template <int D> struct BCfg {
    static constexpr int kBoxes = D / 64;
    static constexpr int kBoxBytes = kTile * 128;
    static constexpr int kTileBytes = kBoxes * kBoxBytes;
    static constexpr int kStageBytes = 2 * kTileBytes + 1024;  // two tiles + 128 f32 lse + 128 f32 delta
    static constexpr int kStages = D == 128 ? 2 : 4;
    static constexpr int kBars = 2 * kStages + 12;  // enough for either kernel's barrier set
#ifdef FLAT_TRACE
    static constexpr int kTraceBytes = 32 * 8 * 4;
#else
    static constexpr int kTraceBytes = 0;
#endif
    static constexpr int kDsBytes = 2 * kBoxBytes;  // SPILL: the dS^T tile (128 keys x 128 queries, bf16) staged for its bulk store
    // the dynamic shared array is declared 1024-byte aligned (the 128-byte swizzle needs it): no slack is added
    static constexpr int kSmemBytes = 2 * kTileBytes + kStages * kStageBytes + kDsBytes + kBars * 8 + 16 + kTraceBytes;
    static_assert(kSmemBytes <= 232448, "shared memory of one CTA");
};

__device__ __forceinline__ long long ds_tile_index(const BwdKernelParams &p, int b, int head, int j, int i) {
    const long long per_head = p.causal ? (long long)p.n_tiles * (p.n_tiles + 1) / 2 : (long long)p.n_tiles * p.n_tiles;
    return ((long long)b * p.q_heads + head) * per_head + (p.causal ? (long long)i * (i + 1) / 2 + j : (long long)i * p.n_tiles + j);
}

__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void bulk_copy_s2g(void *dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void timeout(const BwdKernelParams &p, int where) {
    if (p.status) {
        p.status->code = FLAT_ERR_DEVICE_WAIT_TIMEOUT;
        p.status->where = where;
    }
}

// KV-stationary kernel: stationary (K, V), streamed (Q_i, dO_i), outputs dV (out0) and dK (out1).
// Per streamed tile the work is split so that the tensor pipe and the elementwise warps overlap:
//   S^T = K Q_i^T                      -> phase 1: P^T = exp2(S^T c - lse) as bf16 over S^T (P stays in registers)
//   dP^T = V dO_i^T (runs under phase 1)
//   dV += P^T dO_i, S^T of tile i + 1  -> phase 2: dS^T = P^T (dP^T - delta) as bf16 over dP^T
//   dK += dS^T Q_i, dP^T of tile i + 1
template <int D, bool SPILL>
__global__ void __launch_bounds__(kThreads, 1) bwd_sm100_kernel(const __grid_constant__ BwdKernelParams p) {
    using C = BCfg<D>;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *st0 = smem;                    // K tile
    uint8_t *st1 = smem + C::kTileBytes;    // V tile
    uint8_t *ring = smem + 2 * C::kTileBytes;
    uint8_t *ds_s = ring + C::kStages * C::kStageBytes;  // SPILL: dS^T tile, two 64-query boxes of 128 key rows x 128 B, swizzled
    uint64_t *bars = reinterpret_cast<uint64_t *>(ds_s + C::kDsBytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + C::kBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
#ifdef FLAT_TRACE
    volatile uint32_t *tr_s = reinterpret_cast<volatile uint32_t *>(tmem_slot + 4);
#define TRS(it, slot) do { if ((it) < 32) tr_s[(it) * 8 + (slot)] = (uint32_t)clock(); } while (0)
#else
#define TRS(it, slot) do { } while (0)
#endif

    const uint32_t bar0 = smem_u32(bars);
    const uint32_t st_full = bar0;
    auto rg_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto rg_empty = [&](int s) { return bar0 + 8u * (1 + C::kStages + s); };
    const uint32_t x_full = bar0 + 8u * (1 + 2 * C::kStages);     // S^T in TMEM
    const uint32_t y_full = bar0 + 8u * (2 + 2 * C::kStages);     // dP^T in TMEM
    const uint32_t p_ready = bar0 + 8u * (3 + 2 * C::kStages);    // bf16 P^T written
    const uint32_t ds_ready = bar0 + 8u * (4 + 2 * C::kStages);   // bf16 dS^T written
    const uint32_t acc_final = bar0 + 8u * (5 + 2 * C::kStages);
    const uint32_t ds_staged = bar0 + 8u * (6 + 2 * C::kStages);  // SPILL: the dS^T tile is complete in shared memory
    const uint32_t ds_free = bar0 + 8u * (7 + 2 * C::kStages);    // SPILL: ... and its bulk store has read it

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // block -> (key tile, kv head, batch); early key tiles see the most queries and go first
    const int heads = p.kv_heads;
    const int lin = blockIdx.x;
    const int tile_rank = lin / (heads * p.batch);
    const int bh = lin % (heads * p.batch);
    const int b = bh / heads, h = bh % heads;
    const int t_own = tile_rank;
    const int first = p.causal ? t_own : 0;
    const int per_head = p.n_tiles - first;
    const int n_iter = per_head * p.group;

    if (threadIdx.x == 0) {
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;  // a misplaced shared window would break the swizzle: refuse to run
        if (*abort_flag) timeout(p, 90);
        mbar_init(st_full, 1);
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(rg_full(s), 1);
            mbar_init(rg_empty(s), 1);
        }
        mbar_init(x_full, 1);
        mbar_init(y_full, 1);
        mbar_init(p_ready, 8);
        mbar_init(ds_ready, 8);
        mbar_init(acc_final, 1);
        mbar_init(ds_staged, 8);
        mbar_init(ds_free, 1);
        mbar_fence_init();
        fence_proxy_async();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    constexpr uint32_t kColX = 0, kColY = 128, kColA0 = 256, kColA1 = 256 + D;

    if (warp >= 8) {
        // 72 x 128 + 216 x 256 registers: exactly the CTA's launch allocation of 168 x 384
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        if (warp == kProducerWarp && lane == 0) {
            // ================= TMA producer =================
            mbar_expect_tx(st_full, 2 * C::kTileBytes);
            for (int kb = 0; kb < C::kBoxes; ++kb) {
                tma_load_4d(smem_u32(st0 + kb * C::kBoxBytes), &p.map_k, kb * 64, t_own * kTile, h, b, st_full);
                tma_load_4d(smem_u32(st1 + kb * C::kBoxBytes), &p.map_v, kb * 64, t_own * kTile, h, b, st_full);
            }
            for (int it = 0; it < n_iter; ++it) {
                const int s = it % C::kStages;
                const uint32_t phase = (it / C::kStages) & 1;
                if (!mbar_wait(rg_empty(s), phase ^ 1, abort_flag)) {
                    timeout(p, 100 + s);
                    break;
                }
                const int t = first + it % per_head;
                const int hs = h * p.group + it / per_head;  // query head of the streamed tensors
                uint8_t *stage = ring + s * C::kStageBytes;
                mbar_expect_tx(rg_full(s), C::kStageBytes);
                for (int kb = 0; kb < C::kBoxes; ++kb) {
                    tma_load_4d(smem_u32(stage + kb * C::kBoxBytes), &p.map_q, kb * 64, t * kTile, hs, b, rg_full(s));
                    tma_load_4d(smem_u32(stage + C::kTileBytes + kb * C::kBoxBytes), &p.map_do, kb * 64, t * kTile, hs, b,
                                rg_full(s));
                }
                // per-query LSE and delta of the streamed query tile
                const long long row0 = ((long long)b * p.q_heads + hs) * p.seq_pad + (long long)t * kTile;
                bulk_copy_g2s(smem_u32(stage + 2 * C::kTileBytes), p.neg_lse2 + row0, 512, rg_full(s));
                bulk_copy_g2s(smem_u32(stage + 2 * C::kTileBytes + 512), p.delta + row0, 512, rg_full(s));
            }
        } else if (warp == kMmaWarp && lane == 0) {
            // ================= MMA issuer =================
            bool ok = true;
            auto wait = [&](uint32_t bar, uint32_t parity, int where) {
                if (!ok) return;
                if (!mbar_wait(bar, parity, abort_flag)) {
                    timeout(p, where);
                    ok = false;
                }
            };
            // scores = stationary * streamed^T: both operands K-major tiles in shared memory
            auto issue_xy = [&](uint32_t col, const uint8_t *a_tile, const uint8_t *b_tile) {
                const uint64_t a_desc = make_smem_desc(smem_u32(a_tile), 0, 1024);
                const uint64_t b_desc = make_smem_desc(smem_u32(b_tile), 0, 1024);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    mma_ss_off(tmem_base + col, a_desc, b_desc, (kk >> 2) * (C::kBoxBytes >> 4) + (kk & 3) * 2, p.idesc_k, kk > 0);
            };
            // acc (+)= A[tmem, 128 x 128 bf16 in two 32-column halves] * B[smem tile as MN-major, 128 x D]
            auto issue_acc = [&](uint32_t col_acc, uint32_t col_a, const uint8_t *b_tile, bool accumulate) {
                const uint64_t b_desc = make_smem_desc(smem_u32(b_tile), C::kBoxBytes, 1024);
#pragma unroll
                for (int kk = 0; kk < kTile / 16; ++kk) {
                    const uint32_t a_col = col_a + (kk < 4 ? kk * 8 : 64 + (kk - 4) * 8);
                    mma_ts_off(tmem_base + col_acc, tmem_base + a_col, b_desc, kk * (16 * 128 >> 4), p.idesc_mn,
                               (accumulate || kk > 0));
                }
            };
            wait(st_full, 0, 200);
            wait(rg_full(0), 0, 210);
            if (ok) {
                tc_fence_after();
                issue_xy(kColX, st0, ring);                  // S^T(0) = K Q_0^T
                tc_commit(x_full);
                issue_xy(kColY, st1, ring + C::kTileBytes);  // dP^T(0) = V dO_0^T
                tc_commit(y_full);
            }
            for (int it = 0; ok && it < n_iter; ++it) {
                const int s = it % C::kStages;
                const uint8_t *stage = ring + s * C::kStageBytes;
                const uint8_t *stage_n = ring + ((it + 1) % C::kStages) * C::kStageBytes;
                const bool more = it + 1 < n_iter;
                if (it < 16) TRS(it, 0);
                wait(p_ready, it & 1, 220);
                if (!ok) break;
                if (it < 16) TRS(it, 1);
                tc_fence_after();
                issue_acc(kColA0, kColX, stage + C::kTileBytes, it > 0);  // dV += P^T dO
                if (more) {
                    wait(rg_full((it + 1) % C::kStages), ((it + 1) / C::kStages) & 1, 230);
                    if (!ok) break;
                    tc_fence_after();
                    issue_xy(kColX, st0, stage_n);                        // S^T of the next tile over P^T
                    tc_commit(x_full);
                }
                if (it < 16) TRS(it, 2);
                wait(ds_ready, it & 1, 240);
                if (!ok) break;
                if (it < 16) TRS(it, 3);
                tc_fence_after();
                issue_acc(kColA1, kColY, stage, it > 0);                  // dK += dS^T Q
                tc_commit(rg_empty(s));
                if (more) {
                    issue_xy(kColY, st1, stage_n + C::kTileBytes);        // dP^T of the next tile over dS^T
                    tc_commit(y_full);
                }
                if (it < 16) TRS(it, 4);
            }
            if (ok) tc_commit(acc_final);
        } else if (SPILL && warp == kMmaWarp + 1 && lane == 0) {
            // ================= dS^T spill =================
            // One bulk store of the staged 32 KiB tile per streamed tile; the elementwise warps may refill the staging
            // space once the store has read it.  The latency of the stores is spent here, not in the warps that compute.
            for (int it = 0; it < n_iter; ++it) {
                if (!mbar_wait(ds_staged, it & 1, abort_flag)) {
                    timeout(p, 400);
                    break;
                }
                const int t = first + it % per_head;
                const int hs = h * p.group + it / per_head;
                bulk_copy_s2g(p.ds_spill + ds_tile_index(p, b, hs, t_own, t) * C::kDsBytes, smem_u32(ds_s), C::kDsBytes);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                mbar_arrive(ds_free);
            }
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // the tiles are in memory before the CTA retires
        }
    } else {
        // ================= elementwise warps + epilogue =================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int half = warp >> 2;                  // which 64 query columns of the 128
        const int lane_base = (warp & 3) * 32;
        const int row_local = lane_base + lane;      // TMEM lane = key
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_base) << 16);
        const uint32_t t_x = t_lane + kColX + half * 64, t_y = t_lane + kColY + half * 64;
        bool ok = true;
        for (int it = 0; ok && it < n_iter; ++it) {
            const int s = it % C::kStages;
            const uint8_t *stage = ring + s * C::kStageBytes;
            if (!mbar_wait(rg_full(s), (it / C::kStages) & 1, abort_flag)) {  // LSE / delta of this stage
                timeout(p, 300);
                ok = false;
                break;
            }
            const float *lse_s = reinterpret_cast<const float *>(stage + 2 * C::kTileBytes) + half * 64;
            const float *delta_s = lse_s + 128;
            const int t = first + it % per_head;
            const bool diag = p.causal && t == t_own;
            // ---- phase 1: P^T ----
            if (!mbar_wait(x_full, it & 1, abort_flag)) {
                timeout(p, 310);
                ok = false;
                break;
            }
            tc_fence_after();
            if (warp == 0 && lane == 0 && it < 16) TRS(it, 5);
            uint32_t x[64];  // scores, then P in f32 (kept for phase 2)
            tmem_ld32(t_x, x);
            tmem_ld32(t_x + 32, x + 32);
            tc_wait_ld();
            if (warp == 0 && lane == 0 && it < 16) TRS(16 + it, 0);
            {
                const float c = p.scale_log2;
                uint32_t pp[32];
                if (!diag) {
                    // three passes over the registers: the 64 independent exp2 keep the special-function unit full
#pragma unroll
                    for (int i = 0; i < 64; i += 2) {
                        const float2 nl = *reinterpret_cast<const float2 *>(lse_s + i);
                        x[i] = __float_as_uint(fmaf(__uint_as_float(x[i]), c, nl.x));
                        x[i + 1] = __float_as_uint(fmaf(__uint_as_float(x[i + 1]), c, nl.y));
                    }
#pragma unroll
                    for (int i = 0; i < 64; ++i) x[i] = __float_as_uint(ex2(__uint_as_float(x[i])));
#pragma unroll
                    for (int i = 0; i < 64; i += 2) {
                        const __nv_bfloat162 pb = __floats2bfloat162_rn(__uint_as_float(x[i]), __uint_as_float(x[i + 1]));
                        pp[i >> 1] = *reinterpret_cast<const uint32_t *>(&pb);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 64; i += 2) {
                        const float2 nl = *reinterpret_cast<const float2 *>(lse_s + i);
                        float p0 = ex2(fmaf(__uint_as_float(x[i]), c, nl.x));
                        float p1 = ex2(fmaf(__uint_as_float(x[i + 1]), c, nl.y));
                        // visible iff key <= query: row = key, column = query
                        const int c0 = half * 64 + i;
                        if (row_local > c0) p0 = 0.f;
                        if (row_local > c0 + 1) p1 = 0.f;
                        x[i] = __float_as_uint(p0);
                        x[i + 1] = __float_as_uint(p1);
                        const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
                        pp[i >> 1] = *reinterpret_cast<const uint32_t *>(&pb);
                    }
                }
                if (warp == 0 && lane == 0 && it < 16) TRS(16 + it, 1);
                tmem_st32(t_x, pp);  // bf16 P^T in the first 32 columns of this warp group's 64-column range
                tc_wait_st();
                if (warp == 0 && lane == 0 && it < 16) TRS(16 + it, 2);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready);
            if (warp == 0 && lane == 0 && it < 16) TRS(it, 6);
            // ---- phase 2: dS^T ----
            if (!mbar_wait(y_full, it & 1, abort_flag)) {
                timeout(p, 315);
                ok = false;
                break;
            }
            tc_fence_after();
            if (warp == 0 && lane == 0 && it < 16) TRS(16 + it, 3);
            {
                uint32_t y[64], ds[32];
                tmem_ld32(t_y, y);
                tmem_ld32(t_y + 32, y + 32);
                tc_wait_ld();
                if (warp == 0 && lane == 0 && it < 16) TRS(16 + it, 4);
#pragma unroll
                for (int i = 0; i < 64; i += 2) {
                    const float2 dl = *reinterpret_cast<const float2 *>(delta_s + i);
                    const float e0 = __uint_as_float(y[i]) - dl.x, e1 = __uint_as_float(y[i + 1]) - dl.y;
                    const __nv_bfloat162 dsb = __floats2bfloat162_rn(__uint_as_float(x[i]) * e0, __uint_as_float(x[i + 1]) * e1);
                    ds[i >> 1] = *reinterpret_cast<const uint32_t *>(&dsb);
                }
                if (warp == 0 && lane == 0 && it < 16) TRS(16 + it, 5);
                if constexpr (SPILL) {
                    // a zero-filled key row past seq_len must reach the dQ kernel as zeros (it scores 0, which against a
                    // very negative LSE could give a huge P)
                    if (t_own * kTile + row_local >= p.seq_len) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) ds[i] = 0u;
                    }
                }
                tmem_st32(t_y, ds);  // bf16 dS^T over dP^T
                if constexpr (SPILL) {
                    // ... and into the staging tile of the spill: row = key, this warp group's 64 queries = 128 bytes of box
                    // `half`, 16-byte chunks swizzled by the row (the layout the dQ kernel's MMAs read it back in)
                    if (!mbar_wait(ds_free, (it & 1) ^ 1, abort_flag)) {  // the previous tile's store has read the space
                        timeout(p, 317);
                        ok = false;
                        break;
                    }
                    uint8_t *row_s = ds_s + half * C::kBoxBytes + row_local * 128;
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch)
                        *reinterpret_cast<uint4 *>(row_s + ((ch ^ (row_local & 7)) << 4)) =
                            make_uint4(ds[ch * 4], ds[ch * 4 + 1], ds[ch * 4 + 2], ds[ch * 4 + 3]);
                    fence_proxy_async();  // generic-proxy writes -> visible to the bulk store's async proxy
                }
                tc_wait_st();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(ds_ready);
            if (SPILL && lane == 0) mbar_arrive(ds_staged);
            if (warp == 0 && lane == 0 && it < 16) TRS(it, 7);
        }
        if (ok && !mbar_wait(acc_final, 0, abort_flag)) {
            timeout(p, 320);
            ok = false;
        }
        if (ok) {
            tc_fence_after();
            // each warp group writes half of the head dimension of the accumulator rows
            const long long out_row = ((long long)b * heads + h) * p.seq_len + (long long)t_own * kTile + row_local;
            const bool store = t_own * kTile + row_local < p.seq_len;  // keys past seq_len were zero-filled, not real
            constexpr int kColsPerHalf = D / 2;
#pragma unroll
            for (int a = 0; a < 2; ++a) {
                const float mul = a == 0 ? 1.0f : p.scale;  // dV unscaled; dK carries the softmax scale
                float *op = reinterpret_cast<float *>(a == 0 ? p.out0 : p.out1) + out_row * D + half * kColsPerHalf;
                const uint32_t t_acc = t_lane + (a == 0 ? kColA0 : kColA1) + half * kColsPerHalf;
#pragma unroll
                for (int c = 0; c < kColsPerHalf / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(t_acc + c * 32, r);
                    tc_wait_ld();
                    float4 *dst = reinterpret_cast<float4 *>(op + c * 32);
                    if (!store) continue;
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4)
                        dst[q4] = make_float4(__uint_as_float(r[q4 * 4]) * mul, __uint_as_float(r[q4 * 4 + 1]) * mul,
                                              __uint_as_float(r[q4 * 4 + 2]) * mul, __uint_as_float(r[q4 * 4 + 3]) * mul);
                }
            }
        }
    }

    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before the CTA exits
    }
    tc_fence_before();
    __syncthreads();
#ifdef FLAT_TRACE
    if (p.trace && blockIdx.x == 0)
        for (int i = threadIdx.x; i < 32 * 8; i += kThreads) p.trace[1 * 64 * 8 + i] = tr_s[i];
#endif
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}
#undef TRS

// Q-stationary dQ kernel, pipelined.  One CTA owns 128 queries of one (batch, q_head); (K_j, V_j) tiles stream
// through a three-stage TMA ring.  Q is copied once from shared memory into TMEM and is the A operand of every
// S MMA; dO stays in shared memory.  The bf16 dS tile has TMEM columns of its own, so the score buffers are
// free again as soon as the elementwise warps have loaded them into registers, and the tensor pipe computes the
// next tile's scores while those warps work on the current one:
//   S = Q K_j^T (TS MMA), dP = dO V_j^T (SS MMA)  ->  dS = exp2(S c - lse) * (dP - delta) as bf16
//   ->  dQ += dS K_j (TS MMA).
// TMEM columns: Q [0, 64), S [64, 192), dP [192, 320), dS [320, 384), dQ [384, 384 + D).
template <int D> struct DqCfg {
    static constexpr int kBoxes = D / 64;
    static constexpr int kBoxBytes = kTile * 128;
    static constexpr int kTileBytes = kBoxes * kBoxBytes;
    static constexpr int kStageBytes = 2 * kTileBytes;  // K tile + V tile
    static constexpr int kStages = 3;
    static constexpr int kBars = 2 * kStages + 7;
#ifdef FLAT_TRACE
    static constexpr int kTraceBytes = 32 * 8 * 4;
#else
    static constexpr int kTraceBytes = 0;
#endif
    static constexpr int kSmemBytes = kTileBytes + kStages * kStageBytes + kBars * 8 + 16 + kTraceBytes + 1024;
};

template <int D>
__global__ void __launch_bounds__(kThreads, 1) bwd_dq_sm100_kernel(const __grid_constant__ BwdKernelParams p) {
    using C = DqCfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *do_s = smem;                   // dO tile
    uint8_t *ring = smem + C::kTileBytes;   // the Q tile passes through the last stage's space on its way to TMEM
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring + C::kStages * C::kStageBytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + C::kBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
#ifdef FLAT_TRACE
    volatile uint32_t *tr_s = reinterpret_cast<volatile uint32_t *>(tmem_slot + 4);
#define TRS(it, slot) do { if ((it) < 32) tr_s[(it) * 8 + (slot)] = (uint32_t)clock(); } while (0)
#else
#define TRS(it, slot) do { } while (0)
#endif
    auto stage_ptr = [&](int s) { return ring + s * C::kStageBytes; };
    uint8_t *q_s = stage_ptr(C::kStages - 1);

    const uint32_t bar0 = smem_u32(bars);
    const uint32_t st_full = bar0;
    auto rg_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto rg_empty = [&](int s) { return bar0 + 8u * (1 + C::kStages + s); };
    const uint32_t xy_full = bar0 + 8u * (1 + 2 * C::kStages);   // S and dP of a tile are in TMEM
    const uint32_t xy_taken = bar0 + 8u * (2 + 2 * C::kStages);  // ... and have been loaded into registers
    const uint32_t ds_full = bar0 + 8u * (3 + 2 * C::kStages);   // bf16 dS written
    const uint32_t ds_free = bar0 + 8u * (4 + 2 * C::kStages);   // ... and consumed by the dQ MMAs
    const uint32_t acc_final = bar0 + 8u * (5 + 2 * C::kStages);
    const uint32_t a_ready = bar0 + 8u * (6 + 2 * C::kStages);   // Q is in TMEM

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // block -> (query tile, head, batch); late query tiles see the most keys and go first
    const int lin = blockIdx.x;
    const int tile_rank = lin / (p.q_heads * p.batch);
    const int bh = lin % (p.q_heads * p.batch);
    const int b = bh / p.q_heads, h = bh % p.q_heads;
    const int t_own = p.causal ? p.n_tiles - 1 - tile_rank : tile_rank;
    const int n_iter = p.causal ? t_own + 1 : p.n_tiles;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(st_full, 1);
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(rg_full(s), 1);
            mbar_init(rg_empty(s), 1);
        }
        mbar_init(xy_full, 1);
        mbar_init(xy_taken, 8);
        mbar_init(ds_full, 8);
        mbar_init(ds_free, 1);
        mbar_init(acc_final, 1);
        mbar_init(a_ready, 8);
        mbar_fence_init();
        fence_proxy_async();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    constexpr uint32_t kColQ = 0, kColX = 64, kColY = 192, kColDS = 320, kColAcc = 384;

    if (warp >= 8) {
        // 72 x 128 + 216 x 256 registers: exactly the CTA's launch allocation of 168 x 384
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        if (warp == kProducerWarp && lane == 0) {
            // ================= TMA producer =================
            mbar_expect_tx(st_full, 2 * C::kTileBytes);
            for (int kb = 0; kb < C::kBoxes; ++kb) {
                tma_load_4d(smem_u32(q_s + kb * C::kBoxBytes), &p.map_q, kb * 64, t_own * kTile, h, b, st_full);
                tma_load_4d(smem_u32(do_s + kb * C::kBoxBytes), &p.map_do, kb * 64, t_own * kTile, h, b, st_full);
            }
            const int hs = h / p.group;
            for (int it = 0; it < n_iter; ++it) {
                const int s = it % C::kStages;
                const uint32_t phase = (it / C::kStages) & 1;
                if (!mbar_wait(rg_empty(s), phase ^ 1, abort_flag)) {
                    timeout(p, 100 + s);
                    break;
                }
                if (it == C::kStages - 1 && !mbar_wait(a_ready, 0, abort_flag)) {  // the Q tile has left this space
                    timeout(p, 110);
                    break;
                }
                uint8_t *stage = stage_ptr(s);
                mbar_expect_tx(rg_full(s), C::kStageBytes);
                for (int kb = 0; kb < C::kBoxes; ++kb) {
                    tma_load_4d(smem_u32(stage + kb * C::kBoxBytes), &p.map_k, kb * 64, it * kTile, hs, b, rg_full(s));
                    tma_load_4d(smem_u32(stage + C::kTileBytes + kb * C::kBoxBytes), &p.map_v, kb * 64, it * kTile, hs, b,
                                rg_full(s));
                }
            }
        } else if (warp == kMmaWarp && lane == 0) {
            // ================= MMA issuer =================
            bool ok = true;
            auto wait = [&](uint32_t bar, uint32_t parity, int where) {
                if (!ok) return;
                if (!mbar_wait(bar, parity, abort_flag)) {
                    timeout(p, where);
                    ok = false;
                }
            };
            const uint64_t do_desc = make_smem_desc(smem_u32(do_s), 0, 1024);
            auto issue_xy = [&](const uint8_t *stage) {
                const uint64_t bk = make_smem_desc(smem_u32(stage), 0, 1024);
                const uint64_t bv = make_smem_desc(smem_u32(stage + C::kTileBytes), 0, 1024);
                // the two products alternate, so that consecutive MMAs never wait on the same accumulator
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off16 = (kk >> 2) * (C::kBoxBytes >> 4) + (kk & 3) * 2;
                    mma_ts_off(tmem_base + kColX, tmem_base + kColQ + kk * 8, bk, off16, p.idesc_k, kk > 0);  // S = Q K^T
                    mma_ss_off(tmem_base + kColY, do_desc, bv, off16, p.idesc_k, kk > 0);                      // dP = dO V^T
                }
            };
            // dQ (+)= dS[tmem, 128 x 128 bf16] * K[smem tile as MN-major B, 128 x D]
            auto issue_acc = [&](const uint8_t *stage, bool accumulate) {
                const uint64_t bk = make_smem_desc(smem_u32(stage), C::kBoxBytes, 1024);
#pragma unroll
                for (int kk = 0; kk < kTile / 16; ++kk)
                    mma_ts_off(tmem_base + kColAcc, tmem_base + kColDS + kk * 8, bk, kk * (16 * 128 >> 4), p.idesc_mn,
                               (accumulate || kk > 0));
            };
            wait(a_ready, 0, 200);
            wait(rg_full(0), 0, 210);
            if (ok) {
                tc_fence_after();
                issue_xy(stage_ptr(0));
                tc_commit(xy_full);
            }
            for (int it = 0; ok && it < n_iter; ++it) {
                const int s = it % C::kStages;
                TRS(it, 0);
                if (it + 1 < n_iter) {
                    // the next tile's scores, as soon as the current ones sit in the elementwise warps' registers
                    const int sn = (it + 1) % C::kStages;
                    wait(xy_taken, it & 1, 220);
                    wait(rg_full(sn), ((it + 1) / C::kStages) & 1, 230);
                    if (!ok) break;
                    TRS(it, 1);
                    tc_fence_after();
                    issue_xy(stage_ptr(sn));
                    tc_commit(xy_full);
                    TRS(it, 2);
                }
                wait(ds_full, it & 1, 240);
                if (!ok) break;
                TRS(it, 3);
                tc_fence_after();
                issue_acc(stage_ptr(s), it > 0);
                tc_commit(ds_free);
                tc_commit(rg_empty(s));
                TRS(it, 4);
            }
            if (ok) tc_commit(acc_final);
        }
    } else {
        // ================= elementwise warps + epilogue =================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int half = warp >> 2;                  // which 64 of the tile's 128 key columns
        const int lane_base = (warp & 3) * 32;
        const int row_local = lane_base + lane;      // TMEM lane = query
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_base) << 16);
        bool ok = true;

        // Q rows from the swizzled TMA tile into TMEM: lane = row, 32-bit column c holds elements 2c, 2c + 1 (the
        // layout of an A operand); warp group `half` copies the 64-element box `half`
        if (!mbar_wait(st_full, 0, abort_flag)) {
            timeout(p, 290);
            ok = false;
        }
        if (ok && half < C::kBoxes) {
            uint32_t v[32];
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(q_s + half * C::kBoxBytes + row_local * 128 +
                                                                   ((ch ^ (row_local & 7)) << 4));
                v[ch * 4] = raw.x; v[ch * 4 + 1] = raw.y; v[ch * 4 + 2] = raw.z; v[ch * 4 + 3] = raw.w;
            }
            tmem_st32(t_lane + kColQ + half * 32, v);
            tc_wait_st();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_ready);

        uint64_t c2, nl2, dl2;
        {
            const long long row = ((long long)b * p.q_heads + h) * p.seq_pad + (long long)t_own * kTile + row_local;
            const float my_neg_lse2 = p.neg_lse2[row], my_delta = p.delta[row];  // zero in the padding
            asm("mov.b64 %0, {%1, %1};" : "=l"(c2) : "f"(p.scale_log2));
            asm("mov.b64 %0, {%1, %1};" : "=l"(nl2) : "f"(my_neg_lse2));
            asm("mov.b64 %0, {%1, %1};" : "=l"(dl2) : "f"(my_delta));
        }
        const uint32_t t_x = t_lane + kColX + half * 64, t_y = t_lane + kColY + half * 64;
        for (int it = 0; ok && it < n_iter; ++it) {
            if (!mbar_wait(xy_full, it & 1, abort_flag)) {
                timeout(p, 310);
                ok = false;
                break;
            }
            tc_fence_after();
            if (warp == 0 && lane == 0) TRACE(0, it, 0);
            const bool diag = p.causal && it == t_own;
            const int live_keys = p.seq_len - it * kTile;  // < 128 only in the last key tile of a ragged sequence
            const bool edge = diag || live_keys < kTile;
            uint32_t x[64], y[64];
            tmem_ld32(t_x, x);
            tmem_ld32(t_x + 32, x + 32);
            tmem_ld32(t_y, y);
            tmem_ld32(t_y + 32, y + 32);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(xy_taken);  // the score buffers may be overwritten
            if (warp == 0 && lane == 0) TRACE(0, it, 1);
            uint32_t ds[32];
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                uint64_t s2, t2, y2, d2;
                asm("mov.b64 %0, {%1, %2};" : "=l"(s2) : "r"(x[i]), "r"(x[i + 1]));
                asm("mov.b64 %0, {%1, %2};" : "=l"(y2) : "r"(y[i]), "r"(y[i + 1]));
                asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(t2) : "l"(s2), "l"(c2), "l"(nl2));
                asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d2) : "l"(y2), "l"(dl2));
                float t0, t1, e0, e1;
                asm("mov.b64 {%0, %1}, %2;" : "=f"(t0), "=f"(t1) : "l"(t2));
                asm("mov.b64 {%0, %1}, %2;" : "=f"(e0), "=f"(e1) : "l"(d2));
                float p0 = ex2(t0), p1 = ex2(t1);
                if (edge) {
                    // visible iff key <= query (diagonal tile: row = query, column = key) and the key exists: keys past
                    // seq_len are zero rows, whose score 0 could still give a huge P against a very negative LSE
                    const int c0 = half * 64 + i;
                    const int last = diag ? min(row_local, live_keys - 1) : live_keys - 1;
                    if (c0 > last) p0 = 0.f;
                    if (c0 + 1 > last) p1 = 0.f;
                }
                const __nv_bfloat162 dsb = __floats2bfloat162_rn(p0 * e0, p1 * e1);
                ds[i >> 1] = *reinterpret_cast<const uint32_t *>(&dsb);
            }
            if (warp == 0 && lane == 0) TRACE(0, it, 2);
            if (it > 0 && !mbar_wait(ds_free, (it - 1) & 1, abort_flag)) {  // the dQ MMAs of the previous tile read dS
                timeout(p, 315);
                ok = false;
                break;
            }
            tc_fence_after();
            tmem_st32(t_lane + kColDS + half * 32, ds);  // this group's 64 keys = 32 columns
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(ds_full);
            if (warp == 0 && lane == 0) TRACE(0, it, 3);
        }
        if (ok && !mbar_wait(acc_final, 0, abort_flag)) {
            timeout(p, 320);
            ok = false;
        }
        if (ok) {
            tc_fence_after();
            // each warp group writes half of the head dimension of the accumulator rows
            const long long out_row = ((long long)b * p.q_heads + h) * p.seq_len + (long long)t_own * kTile + row_local;
            constexpr int kColsPerHalf = D / 2;
            float *op = reinterpret_cast<float *>(p.out0) + out_row * D + half * kColsPerHalf;
            const uint32_t t_acc = t_lane + kColAcc + half * kColsPerHalf;
            const bool store = t_own * kTile + row_local < p.seq_len;  // queries past seq_len were zero-filled, not real
#pragma unroll
            for (int c = 0; c < kColsPerHalf / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(t_acc + c * 32, r);
                tc_wait_ld();
                float4 *dst = reinterpret_cast<float4 *>(op + c * 32);
                if (!store) continue;
#pragma unroll
                for (int q4 = 0; q4 < 8; ++q4)
                    dst[q4] = make_float4(__uint_as_float(r[q4 * 4]) * p.scale, __uint_as_float(r[q4 * 4 + 1]) * p.scale,
                                          __uint_as_float(r[q4 * 4 + 2]) * p.scale, __uint_as_float(r[q4 * 4 + 3]) * p.scale);
            }
        }
    }

    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before the CTA exits
    }
    tc_fence_before();
    __syncthreads();
#ifdef FLAT_TRACE
    if (p.trace && blockIdx.x == 0)
        for (int i = threadIdx.x; i < 32 * 8; i += kThreads) p.trace[2 * 64 * 8 + i] = tr_s[i];
#endif
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}
#undef TRS

// dQ from spilled dS^T tiles: one CTA owns 128 queries of one (batch, q_head) and streams, per visible key tile j, the
// 32 KiB dS^T tile (one contiguous bulk copy: the tile sits in scratch in the swizzled layout it was staged in) and
// the K_j tile; dQ += dS_ij K_j is eight SS MMAs (A = the dS^T tile read M-major, B = K_j read N-major).  No
// elementwise work; the kernel is bound by the stream of dS^T tiles from HBM.  Warps 0-3 epilogue, 4 producer, 5 MMA.
template <int D> struct DqSpillCfg {
    static constexpr int kBoxes = D / 64;
    static constexpr int kBoxBytes = kTile * 128;
    static constexpr int kTileBytes = kBoxes * kBoxBytes;
    static constexpr int kDsBytes = 2 * kBoxBytes;
    static constexpr int kStageBytes = kDsBytes + kTileBytes;
    static constexpr int kStages = 3;
    static constexpr int kBars = 2 * kStages + 1;
    static constexpr int kThreadsDq = 192;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBars * 8 + 16;
};

template <int D>
__global__ void __launch_bounds__(DqSpillCfg<D>::kThreadsDq, 1) bwd_dq_spill_kernel(const __grid_constant__ BwdKernelParams p) {
    using C = DqSpillCfg<D>;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + C::kStages * C::kStageBytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + C::kBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto rg_full = [&](int s) { return bar0 + 8u * s; };
    auto rg_empty = [&](int s) { return bar0 + 8u * (C::kStages + s); };
    const uint32_t acc_final = bar0 + 8u * (2 * C::kStages);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // block -> (query tile, head, batch); late query tiles see the most keys and go first
    const int lin = blockIdx.x;
    const int tile_rank = lin / (p.q_heads * p.batch);
    const int bh = lin % (p.q_heads * p.batch);
    const int b = bh / p.q_heads, h = bh % p.q_heads;
    const int t_own = p.causal ? p.n_tiles - 1 - tile_rank : tile_rank;
    const int n_iter = p.causal ? t_own + 1 : p.n_tiles;
    constexpr uint32_t kTmemCols = D;  // 64 or 128: a power of two >= 32

    if (threadIdx.x == 0) {
        *abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;
        if (*abort_flag) timeout(p, 91);
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(rg_full(s), 1);
            mbar_init(rg_empty(s), 1);
        }
        mbar_init(acc_final, 1);
        mbar_fence_init();
        fence_proxy_async();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 4 && lane == 0 && !*abort_flag) {
        // ================= producer =================
        const int kvh = h / p.group;
        for (int it = 0; it < n_iter; ++it) {
            const int s = it % C::kStages;
            if (!mbar_wait(rg_empty(s), ((it / C::kStages) & 1) ^ 1, abort_flag)) {
                timeout(p, 100 + s);
                break;
            }
            uint8_t *stage = smem + s * C::kStageBytes;
            mbar_expect_tx(rg_full(s), C::kStageBytes);
            bulk_copy_g2s(smem_u32(stage), p.ds_spill + ds_tile_index(p, b, h, it, t_own) * C::kDsBytes, C::kDsBytes, rg_full(s));
            for (int kb = 0; kb < C::kBoxes; ++kb)
                tma_load_4d(smem_u32(stage + C::kDsBytes + kb * C::kBoxBytes), &p.map_k, kb * 64, it * kTile, kvh, b, rg_full(s));
        }
    } else if (warp == 5 && lane == 0 && !*abort_flag) {
        // ================= MMA issuer =================
        bool ok = true;
        for (int it = 0; ok && it < n_iter; ++it) {
            const int s = it % C::kStages;
            if (!mbar_wait(rg_full(s), (it / C::kStages) & 1, abort_flag)) {
                timeout(p, 210);
                ok = false;
                break;
            }
            tc_fence_after();
            const uint8_t *stage = smem + s * C::kStageBytes;
            const uint64_t a_desc = make_smem_desc(smem_u32(stage), C::kBoxBytes, 1024);                // dS^T, M-major
            const uint64_t b_desc = make_smem_desc(smem_u32(stage + C::kDsBytes), C::kBoxBytes, 1024);  // K_j, N-major
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)
                mma_ss_off(tmem_base, a_desc, b_desc, kk * (16 * 128 >> 4), p.idesc_dq, (it > 0 || kk > 0));
            tc_commit(rg_empty(s));
        }
        if (ok) tc_commit(acc_final);
    } else if (warp < 4) {
        // ================= epilogue =================
        const int row_local = warp * 32 + lane;  // TMEM lane = query row
        if (mbar_wait(acc_final, 0, abort_flag)) {
            tc_fence_after();
            const long long out_row = ((long long)b * p.q_heads + h) * p.seq_len + (long long)t_own * kTile + row_local;
            float *op = reinterpret_cast<float *>(p.out0) + out_row * D;
            const bool store = t_own * kTile + row_local < p.seq_len;
            const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(t_acc + c * 32, r);
                tc_wait_ld();
                if (!store) continue;
                float4 *dst = reinterpret_cast<float4 *>(op + c * 32);
#pragma unroll
                for (int q4 = 0; q4 < 8; ++q4)
                    dst[q4] = make_float4(__uint_as_float(r[q4 * 4]) * p.scale, __uint_as_float(r[q4 * 4 + 1]) * p.scale,
                                          __uint_as_float(r[q4 * 4 + 2]) * p.scale, __uint_as_float(r[q4 * 4 + 3]) * p.scale);
            }
        } else {
            timeout(p, 320);
        }
    }

    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// delta = dO . O and -LSE*log2(e).  A thread takes 8 elements (16 bytes) of a row of each tensor, head_dim / 8
// neighbouring lanes share a row, so a warp covers 256 / head_dim rows with full-width loads.
__global__ void __launch_bounds__(256) bwd_prep_kernel(const __nv_bfloat16 *__restrict__ d_out,
                                                       const __nv_bfloat16 *__restrict__ out, const float *__restrict__ lse,
                                                       float *__restrict__ delta, float *__restrict__ neg_lse2, int64_t rows,
                                                       int head_dim, int seq_len, int seq_pad) {
    const int lanes_per_row = head_dim / 8;  // 8 or 16
    const int rows_per_block = 256 / lanes_per_row;
    const int sub = threadIdx.x % lanes_per_row;
    const int64_t row = (int64_t)blockIdx.x * rows_per_block + threadIdx.x / lanes_per_row;
    float acc = 0.f;
    if (row < rows) {
        const uint4 a = __ldg(reinterpret_cast<const uint4 *>(d_out + row * head_dim) + sub);
        const uint4 o = __ldg(reinterpret_cast<const uint4 *>(out + row * head_dim) + sub);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            acc = fmaf(__uint_as_float(aw[e] << 16), __uint_as_float(ow[e] << 16), acc);
            acc = fmaf(__uint_as_float(aw[e] & 0xffff0000u), __uint_as_float(ow[e] & 0xffff0000u), acc);
        }
    }
    for (int w = lanes_per_row / 2; w >= 1; w >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, w);
    if (sub == 0 && row < rows) {
        const int64_t dst = row / seq_len * seq_pad + row % seq_len;  // rows of a (batch, head) padded to whole tiles
        delta[dst] = acc;
        neg_lse2[dst] = -lse[row] * kLog2e;
    }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

bool backward_sm100_supported(const BwdParams &p) {
    if (p.head_dim != 64 && p.head_dim != 128) return false;
    const void *ptrs[] = {p.q, p.k, p.v, p.d_out, p.out, p.dq, p.dk, p.dv};
    for (const void *x : ptrs)
        if (!aligned16(x)) return false;
    return true;
}

namespace {
// bytes of the dS^T spill: one 32 KiB tile per visible (key tile, query tile) pair of every (batch, q head)
uint64_t spill_bytes(const BwdParams &p) {
    const uint64_t n = ((uint64_t)p.seq_len + kTile - 1) / kTile;
    const uint64_t per_head = p.causal ? n * (n + 1) / 2 : n * n;
    return (uint64_t)p.batch * p.q_heads * per_head * (2 * kTile * 128);
}
uint64_t small_scratch_bytes(const BwdParams &p) {
    const uint64_t seq_pad = ((uint64_t)p.seq_len + kTile - 1) / kTile * kTile;
    return (2 * (uint64_t)p.batch * p.q_heads * seq_pad * sizeof(float) + 1023) & ~uint64_t(1023);
}
bool use_spill(const flat_ctx *ctx, const BwdParams &p) { return spill_bytes(p) <= ctx->backward_scratch_budget; }
}  // namespace

uint64_t backward_sm100_workspace_bytes(const flat_ctx *ctx, const BwdParams &p) {
    return small_scratch_bytes(p) + (use_spill(ctx, p) ? spill_bytes(p) : 0);
}

int launch_backward_sm100(flat_ctx *ctx, const BwdParams &p) {
    int st = ensure_workspace(ctx, kWorkspaceMeta + backward_sm100_workspace_bytes(ctx, p));
    if (st) return st;
    const int D = p.head_dim, N = p.seq_len;
    const bool spill = use_spill(ctx, p);
    const int64_t rows = (int64_t)p.batch * p.q_heads * N;
    const int seq_pad = (N + kTile - 1) / kTile * kTile;
    const int64_t rows_pad = (int64_t)p.batch * p.q_heads * seq_pad;
    float *delta = reinterpret_cast<float *>(scratch_ptr(ctx));
    float *neg_lse2 = delta + rows_pad;
    // the slots of rows past seq_len must hold finite values: with zeros the zero-filled Q / dO rows contribute nothing
    if (seq_pad != N) FLAT_CUDA_OK(ctx, cudaMemsetAsync(delta, 0, 2 * rows_pad * sizeof(float), ctx->stream));
    const int prep_rows_per_block = 256 / (D / 8);
    bwd_prep_kernel<<<(unsigned)((rows + prep_rows_per_block - 1) / prep_rows_per_block), 256, 0, ctx->stream>>>(
        static_cast<const __nv_bfloat16 *>(p.d_out), static_cast<const __nv_bfloat16 *>(p.out), p.lse, delta, neg_lse2, rows, D,
        N, seq_pad);
    ctx->launches += 1;

    BwdKernelParams kp{};
    const int64_t rs = D, hs = (int64_t)N * D;
    if ((st = make_map(ctx, &kp.map_q, false, p.q, D, N, p.q_heads, p.batch, rs, hs, hs * p.q_heads, kTile))) return st;
    if ((st = make_map(ctx, &kp.map_do, false, p.d_out, D, N, p.q_heads, p.batch, rs, hs, hs * p.q_heads, kTile))) return st;
    if ((st = make_map(ctx, &kp.map_k, false, p.k, D, N, p.kv_heads, p.batch, rs, hs, hs * p.kv_heads, kTile))) return st;
    if ((st = make_map(ctx, &kp.map_v, false, p.v, D, N, p.kv_heads, p.batch, rs, hs, hs * p.kv_heads, kTile))) return st;
    kp.neg_lse2 = neg_lse2;
    kp.delta = delta;
    kp.batch = p.batch; kp.q_heads = p.q_heads; kp.kv_heads = p.kv_heads; kp.seq_len = N; kp.group = p.group;
    kp.n_tiles = seq_pad / kTile;
    kp.seq_pad = seq_pad;
    kp.causal = p.causal;
    kp.scale = p.scale;
    kp.scale_log2 = p.scale * kLog2e;
    kp.idesc_k = make_idesc(kFmtBF16, kFmtBF16, 0, 0, 128, 128);
    kp.idesc_mn = make_idesc(kFmtBF16, kFmtBF16, 0, 1, 128, (uint32_t)D);
    kp.idesc_dq = make_idesc(kFmtBF16, kFmtBF16, 1, 1, 128, (uint32_t)D);
    kp.ds_spill = spill ? reinterpret_cast<uint8_t *>(scratch_ptr(ctx)) + small_scratch_bytes(p) : nullptr;
    kp.status = ctx->dev_status;
    kp.trace = nullptr;
#ifdef FLAT_TRACE
    if (const char *tp = getenv("FLAT_TRACE_PTR")) kp.trace = reinterpret_cast<long long *>(strtoull(tp, nullptr, 0));
#endif

    auto run = [&](auto kernel, int smem_bytes, long long grid, int threads = kThreads) -> int {
        FLAT_CUDA_OK(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        KernelTimer timer(ctx);
        kernel<<<(unsigned)grid, threads, smem_bytes, ctx->stream>>>(kp);
        return FLAT_OK;
    };
    const long long grid_kv = (long long)kp.n_tiles * p.kv_heads * p.batch;
    const long long grid_q = (long long)kp.n_tiles * p.q_heads * p.batch;
    kp.out0 = p.dv;
    kp.out1 = p.dk;
    if (spill) {
        if (D == 128) st = run(bwd_sm100_kernel<128, true>, BCfg<128>::kSmemBytes, grid_kv);
        else st = run(bwd_sm100_kernel<64, true>, BCfg<64>::kSmemBytes, grid_kv);
    } else if (D == 128) st = run(bwd_sm100_kernel<128, false>, BCfg<128>::kSmemBytes, grid_kv);
    else st = run(bwd_sm100_kernel<64, false>, BCfg<64>::kSmemBytes, grid_kv);
    if (st) return st;
    kp.out0 = p.dq;
    kp.out1 = nullptr;
    if (spill) {
        if (D == 128) st = run(bwd_dq_spill_kernel<128>, DqSpillCfg<128>::kSmemBytes, grid_q, DqSpillCfg<128>::kThreadsDq);
        else st = run(bwd_dq_spill_kernel<64>, DqSpillCfg<64>::kSmemBytes, grid_q, DqSpillCfg<64>::kThreadsDq);
    } else if (D == 128) st = run(bwd_dq_sm100_kernel<128>, DqCfg<128>::kSmemBytes, grid_q);
    else st = run(bwd_dq_sm100_kernel<64>, DqCfg<64>::kSmemBytes, grid_q);
    if (st) return st;
    ctx->launches += 2;
    FLAT_CUDA_OK(ctx, cudaGetLastError());
    return FLAT_OK;
}

}  // namespace flat
