// tcgen05 forward: causal / non-causal online-softmax attention for bf16 storage, head_dim 64 or
// 128, GQA by head mapping, RoPE, rectangular shapes, K/V contiguous or read through a page table.
//
// One CTA owns 256 consecutive query rows of one (batch, q_head) as two 128-row tiles that
// ping-pong on the tensor core.  Warp roles (384 threads):
//   warps 0-3  softmax of Q tile 0 : thread t owns query row t (TMEM lane t), no shuffles
//   warps 4-7  softmax of Q tile 1
//   warp  8    TMA producer        : Q tiles once, then K_j, V_j through an mbarrier ring
//   warp  9    MMA issuer          : one thread issues every tcgen05.mma and tcgen05.commit
//   warps 10-11 K converters       : bf16 -> fp16 of each K tile in place (only when Q is rotated against bf16 K)
// Per KV tile j and Q tile w:  S_w = Q_w K_j^T (SS MMA, f32 in TMEM)  ->  softmax warps read S_w
// from TMEM, track the running max (rescaling O_w in TMEM only when the max grows by more than
// 2^8), write P_w = exp2(S_w*c - m) as bf16 over S_w  ->  O_w += P_w V_j (A operand from TMEM).
// The N x N matrix never leaves TMEM.  Tensor-core order S0 S1 | PV0 S0' PV1 S1' | ... keeps the
// pipe busy with one tile's MMAs while the other tile is in softmax.
//
// RoPE: Q is rotated inside this kernel.  The raw bf16 Q tile lands in shared memory by TMA, the
// softmax thread that owns a row rotates it in place with a (cos, sin) table of the call's
// positions and hands the tile to the MMA warp; rotated operands are stored as fp16, which keeps
// their rounding eight times smaller than bf16 would (the 2e-3 LSE tolerance needs that).  K is
// rotated once per call by a small prologue kernel into fp16 scratch (every K tile is read by
// many CTAs, so rotating it in-kernel would repeat the work 32 times).  When the cache already
// holds rotated bf16 K (rotate_k = 0) only Q is rotated; tcgen05.mma kind::f16 takes A and B of
// one format only, so each bf16 K tile is then converted to fp16 in place in shared memory by two
// otherwise idle warps (CONVK; exact for |k| in the normal fp16 range, saturating beyond 65504)
// before the MMA warp may use it.
// Semantics: Appendix of the forward contract (src/projection_asymmetric.rs:97-238): key k is
// visible to local row q iff !causal || k <= query_position_offset + q; LSE = max + ln(sum).
#include <cuda.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "common.h"
#include "sm100_host.cuh"
#include "sm100_ptx.cuh"

namespace flat {
namespace {

using namespace sm100;

constexpr int kTileRows = 128;
constexpr int kThreads = 384;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;  // log2 domain

// Debug timeline (compiled in with -DFLAT_TRACE): clock64 stamps of CTA FLAT_TRACE_BLOCK (default 0), written to the buffer whose
// address is given in the environment variable FLAT_TRACE_PTR.  Layout [role 0..2][iteration 0..63][slot 0..7].
#ifndef FLAT_TRACE_ITEM
#define FLAT_TRACE_ITEM 0  // the item of the CTA whose KV loop is stamped
#endif
#ifdef FLAT_TRACE
#ifndef FLAT_TRACE_BLOCK
#define FLAT_TRACE_BLOCK 0
#endif
#define TRACE(role, it, slot)                                                                          \
    do {                                                                                               \
        if (p.trace && trace_item && blockIdx.x == FLAT_TRACE_BLOCK && (it) < 64) p.trace[((role) * 64 + (it)) * 8 + (slot)] = clock64(); \
    } while (0)
#define TRACEB(k, role, slot)                                                                                \
    do {                                                                                                     \
        if (p.trace && blockIdx.x == FLAT_TRACE_BLOCK && (k) >= 0 && (k) < 4)                                 \
            p.trace[((role) * 64 + 56 + (k)) * 8 + (slot)] = clock64();                                      \
    } while (0)
// Stamps of the softmax loop are kept in registers and written one iteration later, so that no global store is
// outstanding when the thread signals the MMA warp.
#define TRACE_LOCAL long long tr_[5] = {0, 0, 0, 0, 0}
#define TRACE_STAMP(slot) tr_[slot] = clock64()
#define TRACE_FLUSH(role, it)                                                                                  \
    do {                                                                                                       \
        if (p.trace && trace_item && blockIdx.x == FLAT_TRACE_BLOCK && (it) >= 0 && (it) < 64)                               \
            for (int s_ = 0; s_ < 5; ++s_) p.trace[((role) * 64 + (it)) * 8 + s_] = tr_[s_];                   \
    } while (0)
#else
#define TRACE(role, it, slot) do { } while (0)
#define TRACE_LOCAL do { } while (0)
#define TRACE_STAMP(slot) do { } while (0)
#define TRACE_FLUSH(role, it) do { } while (0)
#define TRACEB(k, role, slot) do { } while (0)
#endif

// Division of a non-negative int by a divisor fixed for the launch, as a multiply-high and a shift (the work-item
// arithmetic below runs on the critical path of every item boundary, where an emulated 32-bit division costs about a
// hundred cycles).  mul = ceil(2^(31 + ceil(log2 d)) / d), shr = ceil(log2 d) - 1; exact for 0 <= n < 2^31.
struct FastDiv {
    uint32_t mul, shr, one;  // one: the divisor is 1 (the quotient is n itself)
};
inline FastDiv make_fastdiv(int d) {
    FastDiv f{0, 0, d == 1 ? 1u : 0u};
    if (d > 1) {
        int l = 0;
        while ((1ll << l) < d) ++l;  // ceil(log2 d)
        const int p = 31 + l;
        f.mul = (uint32_t)(((1ull << p) + (unsigned long long)d - 1) / (unsigned long long)d);
        f.shr = (uint32_t)(p - 32);
    }
    return f;
}
__device__ __forceinline__ int fast_div(int n, const FastDiv &f) {
    return f.one ? n : (int)(__umulhi((uint32_t)n, f.mul) >> f.shr);
}

struct KernelParams {
    CUtensorMap map_q, map_k, map_v;
    CUtensorMap map_o;  // O as (d, row, head, batch) with boxes of 64 columns x 32 rows: the epilogue's bulk stores, one per warp
    int o_tma;          // the epilogue stores O tiles through shared memory with bulk copies (not for padded batches)
    void *o;
    float *lse;
    int64_t o_bs, o_hs, o_rs, lse_hs;
    int o_align32;  // every O row starts on a 32-byte boundary: 256-bit stores may be used
    int batch, q_heads, kv_heads, q_len, kv_len, group;
    FastDiv div_bh, div_heads, div_group;  // by batch * q_heads, by q_heads, by group
    int causal;
    long long causal_off;
    float scale_log2;
    uint32_t idesc_qk, idesc_pv;
    const int32_t *page_table;
    int page_size, max_pages, physical_pages;
    int q_blocks;
    long long total_items;  // q_blocks * batch * q_heads work items; with a split last round, its parts counted one by one
    // Work distribution: whole rounds in which every CTA takes one item, then one round for the `rem_items` items that
    // are left.  When those are few, each is cut along KV into `split` parts that run on different CTAs (a part
    // writes its unnormalised O, running max and sum to part_o / part_ml; a merge kernel finishes the rows), so the
    // last round keeps every SM busy instead of a fraction of them.  Item indices from split_first on name parts:
    // index split_first + v is part v / rem_items of item split_first + v % rem_items.
    int split_first, rem_items, split;  // split_first: first item index of the split round (INT_MAX when nothing is split)
    float *part_o;    // [rem_items * split][256 rows][D] f32, unnormalised
    float2 *part_ml;  // [rem_items * split][256 rows] (running max in the log2 domain, running sum)
    DeviceStatus *status;
    const flat_varlen_sequence *varlen;  // per batch element: active lengths, causal and RoPE offsets; null = uniform
    long long rope_table_base;           // varlen: position of the table's first row (the smallest query_rope_offset)
    const float2 *rope_q_table;  // (cos, sin) of row r, pair j at [r * D/2 + j]; null = Q is used as loaded
    float2 rope_step[kMaxHeadDim / 2];  // (cos, sin)(rows_per_step * inv_freq[j]): advances a row's rotation
    const float *alibi_slopes;  // ALIBI kernels: one slope per query head (device)
    int alibi_delta;            // ALIBI kernels: bias position of key 0 minus bias position of query row 0
    float alibi_inv_scale;      // ALIBI kernels: 1 / softmax scale
    long long *trace;
};

// CONVK: K tiles are bf16 in memory and are converted to fp16 in shared memory (Q is rotated to fp16).
template <int D, bool CONVK> struct Cfg {
    static constexpr int kBoxes = D / 64;                  // 64-element (128-byte) column boxes per row
    static constexpr int kBoxBytes = kTileRows * 128;      // 128 rows x 128 B
    static constexpr int kTileBytes = kBoxes * kBoxBytes;  // one Q / K / V tile
    static constexpr int kStages = D == 128 ? 4 : 8;  // K/V ring entries
    static constexpr int kOutStageBytes = kTileRows * 128;  // one box of the O tile: 128 rows x 64 columns of 16 bits
    static constexpr int kBars = 2 + 3 * kStages + 10;
    static constexpr int kSmemBytes = (2 + kStages) * kTileBytes + 2 * kOutStageBytes + kBars * 8 + 16 + 32 + 1024;
    static_assert(kSmemBytes <= 232448, "shared memory of one CTA");
};

__device__ __forceinline__ void record_timeout(const KernelParams &p, int where) {
    if (p.status) {
        p.status->code = FLAT_ERR_DEVICE_WAIT_TIMEOUT;
        p.status->where = where;
    }
}

// One unit of work: 256 consecutive query rows of one (batch, q_head), over all visible KV tiles or, for a split
// item of the last round, over one contiguous part of them.
struct WorkItem {
    int b, h, kvh, r0;
    int n_tiles[2];  // KV tiles each of the two Q tiles visits in this item (0 = nothing to do for that tile)
    int j0;          // first KV tile of the item (0 unless it is a part of a split item)
    int part_slot;   // split items: index of this part's partial record; -1 = the item writes the final result
    int q_len, kv_len;     // this batch element's live rows (the call's lengths unless it is a variable-length batch)
    long long causal_off;  // key k is visible to local row q iff k <= causal_off + q
    int table_row0;        // row of the (cos, sin) table that belongs to local query row 0
};

// What a CTA needs to know about the part of a split item it runs in the last round; decoded once per CTA into
// shared memory (the roles that walk the items then read five words instead of redoing the arithmetic).
struct SplitRecord {
    int lin;        // the item the part belongs to
    int j0;         // first KV tile of the part
    int n_tiles[2]; // KV tiles of the part per Q tile
    int part_slot;  // index of its partial record
};

__device__ __forceinline__ WorkItem make_item_whole(const KernelParams &p, int lin) {
    // item index -> (query block, batch, head); late (long) query blocks first
    WorkItem it;
    const int total_bh = p.batch * p.q_heads;
    const int q_lin = fast_div(lin, p.div_bh);
    const int qb = p.q_blocks - 1 - q_lin;
    const int bh = lin - q_lin * total_bh;
    it.b = fast_div(bh, p.div_heads);
    it.h = bh - it.b * p.q_heads;
    it.kvh = fast_div(it.h, p.div_group);
    it.r0 = qb * 2 * kTileRows;
    it.q_len = p.q_len;
    it.kv_len = p.kv_len;
    it.causal_off = p.causal_off;
    it.table_row0 = 0;
    it.j0 = 0;
    it.part_slot = -1;
    if (p.varlen) {  // padded batch: src/wgpu_external_variable.rs:21-33
        const flat_varlen_sequence m = p.varlen[it.b];
        it.q_len = (int)m.active_query_len;
        it.kv_len = (int)m.active_kv_len;
        it.causal_off = m.causal_query_offset;
        it.table_row0 = (int)((long long)m.query_rope_offset - p.rope_table_base);
    }
#pragma unroll
    for (int w = 0; w < 2; ++w) {
        const int first = it.r0 + w * kTileRows;
        long long visible = it.kv_len;
        if (p.causal) {
            const long long last_row = min(first + kTileRows - 1, it.q_len - 1);
            visible = min((long long)it.kv_len, it.causal_off + last_row + 1);
        }
        it.n_tiles[w] = first < it.q_len ? (int)((visible + kTileRows - 1) / kTileRows) : 0;
    }
    return it;
}

// Item indices from split_first on name parts of the last round's items: index split_first + v is part v / rem_items of
// item split_first + v % rem_items, and covers KV tiles [part * n / split, (part + 1) * n / split) of the item's n.
__device__ __forceinline__ SplitRecord decode_part(const KernelParams &p, int idx) {
    SplitRecord r;
    const int v = idx - p.split_first;
    const int part = v / p.rem_items;
    r.lin = p.split_first + v % p.rem_items;
    const WorkItem it = make_item_whole(p, r.lin);
    const int n = max(it.n_tiles[0], it.n_tiles[1]);
    const int lo = part * n / p.split, hi = (part + 1) * n / p.split;
    r.j0 = lo;
    r.n_tiles[0] = max(0, min(it.n_tiles[0], hi) - lo);
    r.n_tiles[1] = max(0, min(it.n_tiles[1], hi) - lo);
    r.part_slot = (r.lin - p.split_first) * p.split + part;
    return r;
}

// SPLIT: the launch cuts the items of its last round into KV parts (a template flag, so that launches without a split
// carry none of its bookkeeping); `rec` is the CTA's decoded part in shared memory.
template <bool SPLIT>
__device__ __forceinline__ WorkItem make_item(const KernelParams &p, int lin, const volatile SplitRecord *rec) {
    if (SPLIT && lin >= p.split_first) {
        WorkItem it = make_item_whole(p, rec->lin);
        it.j0 = rec->j0;
        it.n_tiles[0] = rec->n_tiles[0];
        it.n_tiles[1] = rec->n_tiles[1];
        it.part_slot = rec->part_slot;
        return it;
    }
    return make_item_whole(p, lin);
}

// The k-th item of this CTA, or -1.  Items are sorted longest first; CTAs take them in rounds of gridDim.x,
// odd rounds in reverse CTA order, so that every CTA gets nearly the same number of KV tiles.
__device__ __forceinline__ int item_index(const KernelParams &p, int k) {
    const int g = (int)gridDim.x;
    const long long idx = (long long)k * g + ((k & 1) ? g - 1 - (int)blockIdx.x : (int)blockIdx.x);
    return idx < p.total_items ? (int)idx : -1;
}

// ALIBI: the softmax warps add slope[q_head] * (key position - query position) to every scaled score
// (src/attention_bias.rs:82-95) before the running maximum is taken.
// F16IO: Q, K, V and O are IEEE binary16 instead of bf16 (P is then written as binary16 too, since one MMA takes A and B
// of one format); accumulation, softmax and LSE stay f32.
template <int D, bool CONVK, bool ALIBI, bool F16IO, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1) fwd_sm100_kernel(const __grid_constant__ KernelParams p) {
    using C = Cfg<D, CONVK>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *q_s = smem;
    uint8_t *kv_s = smem + 2 * C::kTileBytes;
    uint8_t *o_stage = kv_s + C::kStages * C::kTileBytes;  // per slot: staging of one 64-column box of the O tile
    uint64_t *bars = reinterpret_cast<uint64_t *>(o_stage + 2 * C::kOutStageBytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + C::kBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    volatile SplitRecord *split_rec = reinterpret_cast<volatile SplitRecord *>(tmem_slot + 2);

    const uint32_t bar0 = smem_u32(bars);
    auto q_full = [&](int w) { return bar0 + 8u * w; };
    auto kv_full = [&](int s) { return bar0 + 8u * (2 + s); };
    auto kv_empty = [&](int s) { return bar0 + 8u * (2 + C::kStages + s); };
    auto s_full = [&](int w) { return bar0 + 8u * (2 + 2 * C::kStages + w); };
    auto p_full = [&](int w) { return bar0 + 8u * (4 + 2 * C::kStages + w); };
    auto o_final = [&](int w) { return bar0 + 8u * (6 + 2 * C::kStages + w); };
    auto q_ready = [&](int w) { return bar0 + 8u * (8 + 2 * C::kStages + w); };
    auto q_empty = [&](int w) { return bar0 + 8u * (10 + 2 * C::kStages + w); };
    auto k_ready = [&](int s) { return bar0 + 8u * (12 + 2 * C::kStages + s); };  // K tile converted (CONVK)

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (warp == kProducerWarp && lane == 0) {
        *abort_flag = 0;
        for (int w = 0; w < 2; ++w) {
            mbar_init(q_full(w), 1);
            mbar_init(s_full(w), 1);
            mbar_init(p_full(w), 4);
            mbar_init(o_final(w), 1);
            mbar_init(q_ready(w), 4);
            mbar_init(q_empty(w), 1);
        }
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(kv_full(s), 1);
            mbar_init(kv_empty(s), 1);
            mbar_init(k_ready(s), 2);  // one arrival per converter warp
        }
        mbar_fence_init();
        fence_proxy_async();
        tma_prefetch_desc(&p.map_q);
        tma_prefetch_desc(&p.map_k);
        tma_prefetch_desc(&p.map_v);
        tma_prefetch_desc(&p.map_o);
        if constexpr (SPLIT) {
            // the part this CTA runs in the last round, if any: decoded once, read by every role
            const int g = (int)gridDim.x, k_last = p.split_first / g;
            const long long idx = (long long)k_last * g + ((k_last & 1) ? g - 1 - (int)blockIdx.x : (int)blockIdx.x);
            if (idx < p.total_items) {
                const SplitRecord r = decode_part(p, (int)idx);
                split_rec->lin = r.lin;
                split_rec->j0 = r.j0;
                split_rec->n_tiles[0] = r.n_tiles[0];
                split_rec->n_tiles[1] = r.n_tiles[1];
                split_rec->part_slot = r.part_slot;
            }
        }
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t col_s[2] = {0u, 128u};
    const uint32_t col_o[2] = {256u, 256u + D};

    // Register rebalancing: a softmax thread holds a whole 128-column score row in registers.  The pool that
    // setmaxnreg.inc draws from is what the CTA was launched with (168 registers x 384 threads), not the whole
    // register file: 56 x 128 + 224 x 256 uses exactly that, and a larger request would block for ever.
    static_assert(56 * 128 + 224 * 256 <= 168 * kThreads, "setmaxnreg split exceeds the CTA's register allocation");
    if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == kProducerWarp) {
        // ================= TMA producer =================
        // The whole warp walks the loop (waits are uniform); lane 0 issues the contiguous loads, and with a page
        // table lane i fetches the id of page i of the tile and issues that page's boxes, so that the page-table
        // reads of a tile are one parallel access instead of a chain of dependent loads in one thread.
        {
            bool ok = true;
            uint32_t ring = 0;             // K/V ring entries requested so far
            uint32_t q_loads[2] = {0, 0};  // Q tiles requested so far, per slot
            for (int k = 0; ok; ++k) {
                const int lin = item_index(p, k);
                if (lin < 0) break;
                const WorkItem it = make_item<SPLIT>(p, lin, split_rec);
                const int n_max = max(it.n_tiles[0], it.n_tiles[1]);
                for (int w = 0; w < 2 && ok; ++w) {
                    if (it.n_tiles[w] == 0) continue;
                    // the slot is free once every S MMA of its previous tile has completed
                    if (q_loads[w] > 0 && !mbar_wait(q_empty(w), (q_loads[w] - 1) & 1, abort_flag)) {
                        if (lane == 0) record_timeout(p, 110 + w);
                        ok = false;
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    ++q_loads[w];
                    if (lane == 0) {
                        mbar_expect_tx(q_full(w), C::kTileBytes);
                        for (int kb = 0; kb < C::kBoxes; ++kb)
                            tma_load_4d(smem_u32(q_s + w * C::kTileBytes + kb * C::kBoxBytes), &p.map_q, kb * 64,
                                        it.r0 + w * kTileRows, it.h, it.b, q_full(w));
                    }
                }
                int page = 0;  // this lane's page of the current KV tile (paged mode), fetched with the K entry
                for (int i = 0; ok && i < 2 * n_max; ++i, ++ring) {
                    const int s = ring % C::kStages;
                    const uint32_t phase = (ring / C::kStages) & 1;
                    if (!mbar_wait(kv_empty(s), phase ^ 1, abort_flag)) {
                        if (lane == 0) record_timeout(p, 100 + s);
                        ok = false;
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    const int j = i >> 1;
                    const CUtensorMap *map = (i & 1) ? &p.map_v : &p.map_k;
                    const uint32_t dst = smem_u32(kv_s + s * C::kTileBytes);
                    if (lane == 0) mbar_expect_tx(kv_full(s), C::kTileBytes);
                    if (p.page_table) {
                        const int pages_per_tile = kTileRows / p.page_size;
                        if ((i & 1) == 0 && lane < pages_per_tile) {
                            const int tok = (it.j0 + j) * kTileRows + lane * p.page_size;
                            page = tok < p.kv_len ? p.page_table[(long long)it.b * p.max_pages + tok / p.page_size]
                                                  : p.physical_pages;  // out of range: zero fill
                        }
                        __syncwarp();  // the expect_tx above precedes every load of the entry
                        if (lane < pages_per_tile) {
                            for (int kb = 0; kb < C::kBoxes; ++kb)
                                tma_load_4d(dst + kb * C::kBoxBytes + lane * p.page_size * 128, map, kb * 64, 0, it.kvh, page,
                                            kv_full(s));
                        }
                    } else if (lane == 0) {
                        for (int kb = 0; kb < C::kBoxes; ++kb)
                            tma_load_4d(dst + kb * C::kBoxBytes, map, kb * 64, (it.j0 + j) * kTileRows, it.kvh, it.b, kv_full(s));
                    }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ================= MMA issuer =================
        if (lane == 0) {
            bool ok = true;
            auto wait = [&](uint32_t bar, uint32_t parity, int where) {
                if (!ok) return;
                if (!mbar_wait(bar, parity, abort_flag)) {
                    record_timeout(p, where);
                    ok = false;
                }
            };
            // The issue loops are unrolled (a rolled loop's dependent instructions cost 100+ cycles per MMA on this
            // single thread, more than the tensor pipe needs), and each descriptor is the tile's base descriptor plus
            // a compile-time constant, which keeps the thread inside its small register budget.
            auto issue_s = [&](int w, int stage) {
                const uint64_t b_desc = make_smem_desc(smem_u32(kv_s + stage * C::kTileBytes), 0, 1024);
                const uint64_t a_desc = make_smem_desc(smem_u32(q_s + w * C::kTileBytes), 0, 1024);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off16 = (kk >> 2) * (C::kBoxBytes >> 4) + (kk & 3) * 2;  // byte offset / 16
                    mma_ss_off(tmem_base + col_s[w], a_desc, b_desc, off16, p.idesc_qk, kk > 0);
                }
            };
            auto issue_pv = [&](int w, int stage, int j) {
                const uint64_t b_desc = make_smem_desc(smem_u32(kv_s + stage * C::kTileBytes), C::kBoxBytes, 1024);
#pragma unroll
                for (int kk = 0; kk < kTileRows / 16; ++kk)
                    mma_ts_off(tmem_base + col_o[w], tmem_base + col_s[w] + kk * 8, b_desc, kk * (16 * 128 >> 4), p.idesc_pv,
                               (j > 0 || kk > 0));
            };
            uint32_t ring0 = 0;           // ring entry of K_0 of the current item
            uint32_t q_uses[2] = {0, 0};  // Q tiles consumed so far, per slot
            uint32_t p_waits[2] = {0, 0}; // P hand-overs consumed so far, per slot
            auto stage_of = [&](uint32_t i) { return (int)((ring0 + i) % C::kStages); };
            auto phase_of = [&](uint32_t i) { return (uint32_t)(((ring0 + i) / C::kStages) & 1); };

            for (int k = 0; ok; ++k) {
                const int lin = item_index(p, k);
                if (lin < 0) break;
                const WorkItem it = make_item<SPLIT>(p, lin, split_rec);
                const int n_max = max(it.n_tiles[0], it.n_tiles[1]);
                const bool trace_item = k == FLAT_TRACE_ITEM;
                (void)trace_item;
                TRACEB(k, 2, 0);
                // prologue: S_w(0) as soon as the slot's Q tile is ready (the other slot may still be finishing the
                // previous item)
                bool k0_ready = false;
                for (int w = 0; w < 2 && ok; ++w) {
                    if (it.n_tiles[w] == 0) continue;
                    wait(p.rope_q_table ? q_ready(w) : q_full(w), q_uses[w] & 1, 200 + w);
                    ++q_uses[w];
                    TRACEB(k, 2, 1 + w);
                    if (!k0_ready) {
                        wait(CONVK ? k_ready(stage_of(0)) : kv_full(stage_of(0)), phase_of(0), 210);
                        k0_ready = true;
                    }
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(w, stage_of(0));
                    tc_commit(s_full(w));
                    if (it.n_tiles[w] == 1) tc_commit(q_empty(w));  // the slot's last S of this item
                }
                if (ok) {
                    tc_commit(kv_empty(stage_of(0)));
                    TRACEB(k, 2, 3);
                }
                for (int j = 0; ok && j < n_max; ++j) {
                    const uint32_t iv = 2 * j + 1, ik = 2 * j + 2;
                    wait(kv_full(stage_of(iv)), phase_of(iv), 220);
                    bool k_next = false;
                    for (int w = 0; w < 2 && ok; ++w) {
                        if (j >= it.n_tiles[w]) continue;
                        wait(p_full(w), p_waits[w] & 1, 230 + w);
                        if (!ok) break;
                        ++p_waits[w];
                        TRACE(2, j, w * 4 + 0);
                        tc_fence_after();
                        issue_pv(w, stage_of(iv), j);
                        TRACE(2, j, w * 4 + 1);
                        if (w == 1 || j >= it.n_tiles[1]) tc_commit(kv_empty(stage_of(iv)));  // last reader of V_j
                        if (j + 1 < it.n_tiles[w]) {
                            if (!k_next) {
                                wait(CONVK ? k_ready(stage_of(ik)) : kv_full(stage_of(ik)), phase_of(ik), 240);
                                if (!ok) break;
                                tc_fence_after();
                                k_next = true;
                            }
                            issue_s(w, stage_of(ik));
                            tc_commit(s_full(w));
                            if (j + 2 == it.n_tiles[w]) tc_commit(q_empty(w));  // the slot's last S of this item
                            TRACE(2, j, w * 4 + 2);
                            if (w == 1 || j + 1 >= it.n_tiles[1]) tc_commit(kv_empty(stage_of(ik)));  // last reader of K_{j+1}
                        } else {
                            tc_commit(o_final(w));
                        }
                    }
                }
                ring0 += 2 * n_max;
            }
        }
    } else if (CONVK) {
        // ================= K converters (warps 10, 11) =================
        // Each K tile of the ring is rewritten in place from bf16 to fp16 (the values are bf16 numbers, so the
        // conversion is exact inside the normal fp16 range and saturates beyond it); warp 10 takes rows 0-63,
        // warp 11 rows 64-127.  K tiles sit at the even ring entries.
        const int cw = warp - (kMmaWarp + 1);
        bool ok = true;
        uint32_t ring = 0;
        for (int k = 0; ok; ++k) {
            const int lin = item_index(p, k);
            if (lin < 0) break;
            const WorkItem it = make_item<SPLIT>(p, lin, split_rec);
            const int n_max = max(it.n_tiles[0], it.n_tiles[1]);
            for (int j = 0; ok && j < n_max; ++j, ring += 2) {
                const int s = ring % C::kStages;
                if (!mbar_wait(kv_full(s), (ring / C::kStages) & 1, abort_flag)) {
                    record_timeout(p, 400 + s);
                    ok = false;
                    break;
                }
                uint8_t *tile = kv_s + s * C::kTileBytes;
                // a warp covers 64 rows x (D / 8) 16-byte chunks; consecutive lanes take consecutive chunks of a row
                constexpr int kChunks = 64 * (D / 8);
#pragma unroll 4
                for (int c = lane; c < kChunks; c += 32) {
                    const int row = 64 * cw + c / (D / 8), ch = c % (D / 8);
                    uint4 *ptr = reinterpret_cast<uint4 *>(tile + (ch >> 3) * C::kBoxBytes + row * 128 + ((ch & 7) << 4));
                    uint4 v = *ptr;
                    uint32_t in[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float lo = __uint_as_float(in[e] << 16), hi = __uint_as_float(in[e] & 0xffff0000u);
                        asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(in[e]) : "f"(hi), "f"(lo));
                    }
                    *ptr = make_uint4(in[0], in[1], in[2], in[3]);
                }
                fence_proxy_async();  // generic-proxy writes -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(k_ready(s));
            }
        }
    }
    } else {
        // ================= softmax + epilogue =================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        const int w = warp >> 2;
        const int lane_base = (warp & 3) * 32;
        const int row_in_tile = lane_base + lane;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_base) << 16);
        const uint32_t t_s = t_lane + col_s[w];
        const uint32_t t_o = t_lane + col_o[w];
        bool ok = true;
        uint32_t done = 0;     // finished items of this slot (its tile was inside q_len)
        uint32_t s_waits = 0;  // score tiles of this slot consumed so far
        bool store_pending = false;  // (lane 0) a bulk store of this warp's staging rows has not been waited for

        // Iteration k runs the KV loop of item k, then rotates the Q tile of item k + 1 (its TMA was issued as soon as
        // the slot's last S MMA had completed), then stores item k: the next item's first S MMA runs during the
        // epilogue.  k = -1 only rotates the first tile.
        for (int k = -1; ok; ++k) {
            // (item indices are recomputed where they are needed rather than kept in registers across the KV loop)
            const bool trace_item = k == FLAT_TRACE_ITEM;
            (void)trace_item;
            float m = -INFINITY, l = 0.f;
            bool run = false;
            if (k >= 0) {
                const WorkItem it = make_item<SPLIT>(p, item_index(p, k), split_rec);
                run = it.n_tiles[w] > 0;
                const int n = it.n_tiles[w];
                int lim = it.kv_len - 1;  // last visible key of this row
                int lim_first = lim;     // ... and of the tile's first row: tiles below it need no mask at all
                if (p.causal) {
                    const int first = it.r0 + w * kTileRows;
                    lim = (int)min((long long)lim, it.causal_off + first + row_in_tile);
                    lim_first = (int)min((long long)lim_first, it.causal_off + first);
                }
                // keys are counted from the item's first KV tile below (a part of a split item starts at tile j0)
                lim -= it.j0 * kTileRows;
                lim_first -= it.j0 * kTileRows;
                // ALiBi is added to the raw score as (slope / scale) * position difference, so that the scaling of the
                // softmax passes covers it.  Positions stay below 2^24 in magnitude (checked on the host): the float
                // position arithmetic is exact.
                float slope_rel = 0.f, bias_pos0 = 0.f;
                if constexpr (ALIBI) {
                    slope_rel = __ldg(p.alibi_slopes + it.h) * p.alibi_inv_scale;
                    bias_pos0 = (float)(p.alibi_delta + it.j0 * kTileRows - (it.r0 + w * kTileRows + row_in_tile));
                }

                // Online softmax, log2 domain, one thread per row; the whole 128-column score row sits in
                // registers.  O in TMEM is rescaled only when the running max grew by more than 2^8.
                TRACE_LOCAL;
                for (int j = 0; ok && j < n; ++j) {
                    if (!mbar_wait(s_full(w), s_waits & 1, abort_flag)) {
                        record_timeout(p, 300 + w);
                        ok = false;
                        break;
                    }
                    ++s_waits;
                    tc_fence_after();
                    if ((warp & 3) == 0 && lane == 0) {
                        TRACE_FLUSH(w, j - 1);
                        TRACE_STAMP(0);
                    }
                    const int key0 = j * kTileRows;
                    const bool tile_masked = key0 + kTileRows - 1 > lim_first;  // uniform over the Q tile
                    const int vis = min(kTileRows, lim - key0 + 1);             // visible columns of this row
                    const float c_log2 = p.scale_log2;
                    uint32_t r[128];  // four loads in flight, one wait
#pragma unroll
                    for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, r + c * 32);
                    tc_wait_ld();
                    if ((warp & 3) == 0 && lane == 0) TRACE_STAMP(1);
                    // ALiBi: the bias of column i is (slope / c) * i on top of a part that is the same for the whole tile
                    // row (bias_base).  It is never added to the scores in a pass of its own: the exponent pass below
                    // folds it into the addend of its FMA (a running pair that advances by two columns per step), and
                    // the maximum is taken per 32-column chunk of raw scores plus the chunk's largest bias, which bounds
                    // the true maximum from above by at most 31 columns' worth of slope (any reference point at or above
                    // the maximum serves the online softmax: P only gets smaller, O and the row sum with it).
                    float bias_base = 0.f;
                    if constexpr (ALIBI) bias_base = slope_rel * (bias_pos0 + (float)key0);
                    if (tile_masked) {
#pragma unroll
                        for (int i = 0; i < 128; ++i)
                            if (i >= vis) r[i] = 0xff800000u;  // -inf: exp2 gives exactly 0
                    }
                    float mx = -INFINITY, mx1 = -INFINITY;  // two chains for instruction-level parallelism
                    if constexpr (ALIBI) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            float a = -INFINITY, b = -INFINITY;
#pragma unroll
                            for (int i = 32 * c; i < 32 * c + 32; i += 4) {
                                asm("max.f32 %0, %0, %1, %2;" : "+f"(a) : "f"(__uint_as_float(r[i])), "f"(__uint_as_float(r[i + 1])));
                                asm("max.f32 %0, %0, %1, %2;" : "+f"(b) : "f"(__uint_as_float(r[i + 2])), "f"(__uint_as_float(r[i + 3])));
                            }
                            // the chunk's largest bias sits at its last column for a positive slope, at its first otherwise
                            const float edge = slope_rel >= 0.f ? (float)(32 * c + 31) : (float)(32 * c);
                            mx = fmaxf(mx, fmaf(slope_rel, edge, fmaxf(a, b)));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 128; i += 4) {
                            asm("max.f32 %0, %0, %1, %2;" : "+f"(mx) : "f"(__uint_as_float(r[i])), "f"(__uint_as_float(r[i + 1])));
                            asm("max.f32 %0, %0, %1, %2;" : "+f"(mx1) : "f"(__uint_as_float(r[i + 2])), "f"(__uint_as_float(r[i + 3])));
                        }
                    }
                    const float m_cand = fmaxf(m, (fmaxf(mx, mx1) + bias_base) * c_log2);
                    const bool grow = (m_cand - m) > kRescaleThreshold;
                    float alpha = 1.0f;
                    if (grow) {
                        alpha = ex2(m - m_cand);
                        m = m_cand;
                    }
                    if (j > 0 && __any_sync(0xffffffffu, grow)) {
                        uint32_t o[32];
#pragma unroll
                        for (int c = 0; c < D / 32; ++c) {
                            tmem_ld32(t_o + c * 32, o);
                            tc_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                            tmem_st32(t_o + c * 32, o);
                        }
                    }
                    l *= alpha;
                    if ((warp & 3) == 0 && lane == 0) TRACE_STAMP(2);
                    // P = exp2(S*c - m) as bf16, written over S; two scores per packed f32x2 FMA
                    uint64_t c2, nm2, sum2 = 0, sum3 = 0;
                    // m is still -inf only while every key this row has met was masked (the first tile of a split
                    // part may lie wholly behind the row's diagonal): all its scores are -inf and P must come out 0
                    const float neg_m0 = m == -INFINITY ? 0.f : fmaf(bias_base, c_log2, -m);
                    asm("mov.b64 %0, {%1, %1};" : "=l"(nm2) : "f"(neg_m0));
                    asm("mov.b64 %0, {%1, %1};" : "=l"(c2) : "f"(c_log2));
                    [[maybe_unused]] uint64_t step2 = 0;  // ALiBi: the addend's advance per pair of columns
                    [[maybe_unused]] float cs = 0.f;
                    if constexpr (ALIBI) {
                        cs = slope_rel * c_log2;
                        asm("mov.b64 %0, {%1, %1};" : "=l"(step2) : "f"(2.f * cs));
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t pk[16];
                        if constexpr (ALIBI) {
                            // the addend of the chunk's first pair, exact; the running sum then covers 16 steps only
                            const float a0 = fmaf(cs, (float)(32 * c), neg_m0), a1 = fmaf(cs, (float)(32 * c + 1), neg_m0);
                            asm("mov.b64 %0, {%1, %2};" : "=l"(nm2) : "f"(a0), "f"(a1));
                        }
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            uint64_t s2, t2, p2;
                            asm("mov.b64 %0, {%1, %2};" : "=l"(s2) : "r"(r[c * 32 + i]), "r"(r[c * 32 + i + 1]));
                            asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(t2) : "l"(s2), "l"(c2), "l"(nm2));
                            if constexpr (ALIBI) asm("add.rn.f32x2 %0, %0, %1;" : "+l"(nm2) : "l"(step2));
                            float t0, t1;
                            asm("mov.b64 {%0, %1}, %2;" : "=f"(t0), "=f"(t1) : "l"(t2));
                            const float p0 = ex2(t0), p1 = ex2(t1);
                            asm("mov.b64 %0, {%1, %2};" : "=l"(p2) : "f"(p0), "f"(p1));
                            if (i & 2) asm("add.rn.f32x2 %0, %0, %1;" : "+l"(sum3) : "l"(p2));
                            else asm("add.rn.f32x2 %0, %0, %1;" : "+l"(sum2) : "l"(p2));
                            if constexpr (F16IO) {
                                __half2 h2 = __floats2half2_rn(p0, p1);
                                pk[i >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                            } else {
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                                pk[i >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                            }
                        }
                        tmem_st16(t_s + c * 16, pk);
                    }
                    {
                        float s0, s1, s2f, s3;
                        asm("mov.b64 {%0, %1}, %2;" : "=f"(s0), "=f"(s1) : "l"(sum2));
                        asm("mov.b64 {%0, %1}, %2;" : "=f"(s2f), "=f"(s3) : "l"(sum3));
                        l += (s0 + s1) + (s2f + s3);
                    }
                    if ((warp & 3) == 0 && lane == 0) TRACE_STAMP(3);
                    tc_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(p_full(w));
                    if ((warp & 3) == 0 && lane == 0) TRACE_STAMP(4);
                }
                if ((warp & 3) == 0 && lane == 0) TRACE_FLUSH(w, n - 1);
            }

            if ((warp & 3) == 0 && lane == 0) TRACEB(k, w, 0);
            const int next_lin = item_index(p, k + 1);
            if (p.rope_q_table && next_lin >= 0 && ok) {
                const WorkItem nx = make_item<SPLIT>(p, next_lin, split_rec);
                if (nx.n_tiles[w] > 0) {
                    // Rotate the Q tile in place (bf16 in, fp16 out).  A warp rotates its 32 rows; lane l
                    // takes the 16-byte chunk (l mod CH) of row (step * RPS + l / CH), so that the (cos, sin) table is
                    // read in contiguous row segments.
                    constexpr int CH = D / 8;     // 16-byte chunks (8 elements, 4 pairs) per row
                    constexpr int RPS = 32 / CH;  // rows per step of one warp
                    const int ch = lane % CH;
                    const int first_row = nx.r0 + w * kTileRows;
                    // (cos, sin) of the lane's first row come from the table; each further step advances the angle by
                    // RPS positions with the rotation (cos, sin)(RPS * inv_freq), which keeps the table traffic at two
                    // 16-byte loads per thread.  The recurrence error (a few 1e-7 over CH steps) is far below the
                    // rounding of the fp16 result.
                    float cc[4], ss[4], cstep[4], sstep[4];
                    {
                        const int rr = nx.table_row0 + min(first_row + lane_base + lane / CH, nx.q_len - 1);
                        const float4 *tp = reinterpret_cast<const float4 *>(p.rope_q_table + (long long)rr * (D / 2)) + 2 * ch;
                        const float4 cs0 = __ldg(tp), cs1 = __ldg(tp + 1);  // (c, s, c, s) x 2
                        cc[0] = cs0.x; ss[0] = cs0.y; cc[1] = cs0.z; ss[1] = cs0.w;
                        cc[2] = cs1.x; ss[2] = cs1.y; cc[3] = cs1.z; ss[3] = cs1.w;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 stp = p.rope_step[ch * 4 + e];
                            cstep[e] = stp.x;
                            sstep[e] = stp.y;
                        }
                    }
                    // rotations before this one: the finished items plus the current one
                    if (!mbar_wait(q_full(w), (done + (run ? 1u : 0u)) & 1, abort_flag)) {
                        record_timeout(p, 290 + w);
                        ok = false;
                    }
                    if ((warp & 3) == 0 && lane == 0) TRACEB(k, w, 1);
                    if (ok) {
                        uint8_t *tile = q_s + w * C::kTileBytes;
                        // all of the thread's chunks are fetched before any is written back: the loads are then in
                        // flight together instead of each waiting behind the previous step's store
                        uint4 raw[CH];
#pragma unroll
                        for (int st = 0; st < CH; ++st) {
                            const int rt = lane_base + st * RPS + lane / CH;  // row in tile
                            raw[st] = *reinterpret_cast<const uint4 *>(tile + (ch >> 3) * C::kBoxBytes + rt * 128 + (((ch & 7) ^ (rt & 7)) << 4));
                        }
#pragma unroll
                        for (int st = 0; st < CH; ++st) {
                            const int rt = lane_base + st * RPS + lane / CH;  // row in tile
                            const int off = (ch >> 3) * C::kBoxBytes + rt * 128 + (((ch & 7) ^ (rt & 7)) << 4);
                            if (st > 0) {
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float c1 = cc[e] * cstep[e] - ss[e] * sstep[e];
                                    ss[e] = ss[e] * cstep[e] + cc[e] * sstep[e];
                                    cc[e] = c1;
                                }
                            }
                            if (first_row + rt >= nx.q_len) continue;  // rows past q_len are not used
                            const uint32_t in[4] = {raw[st].x, raw[st].y, raw[st].z, raw[st].w};
                            uint32_t hi[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float x, y;
                                if constexpr (F16IO) {
                                    const float2 xy = __half22float2(*reinterpret_cast<const __half2 *>(&in[e]));
                                    x = xy.x;
                                    y = xy.y;
                                } else {
                                    x = __uint_as_float(in[e] << 16);
                                    y = __uint_as_float(in[e] & 0xffff0000u);
                                }
                                const float rx = x * cc[e] - y * ss[e], ry = x * ss[e] + y * cc[e];
                                const __half2 h2 = __floats2half2_rn(rx, ry);
                                hi[e] = *reinterpret_cast<const uint32_t *>(&h2);
                            }
                            *reinterpret_cast<uint4 *>(tile + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        }
                    }
                    fence_proxy_async();  // generic-proxy writes -> visible to the tensor core's async proxy
                    __syncwarp();
                    if (lane == 0) mbar_arrive(q_ready(w));
                    if ((warp & 3) == 0 && lane == 0) TRACEB(k, w, 2);
                }
            }

            if (run && ok) {
                if (!mbar_wait(o_final(w), done & 1, abort_flag)) {
                    record_timeout(p, 310 + w);
                    ok = false;
                }
                ++done;
            }
            if ((warp & 3) == 0 && lane == 0) TRACEB(k, w, 3);
            if (run && ok) {
                tc_fence_after();
                const WorkItem it = make_item<SPLIT>(p, item_index(p, k), split_rec);
                const int row = it.r0 + w * kTileRows + row_in_tile, b = it.b, h = it.h;
                if (SPLIT && it.part_slot >= 0) {
                    // a part of a split item: unnormalised O, running max and sum go to the partial record
                    const long long prow = (long long)it.part_slot * (2 * kTileRows) + w * kTileRows + row_in_tile;
                    float4 *po = reinterpret_cast<float4 *>(p.part_o + prow * D);
                    uint32_t r[32];
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        tmem_ld32(t_o + c * 32, r);
                        tc_wait_ld();
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4)
                            po[c * 8 + q4] = make_float4(__uint_as_float(r[q4 * 4]), __uint_as_float(r[q4 * 4 + 1]),
                                                         __uint_as_float(r[q4 * 4 + 2]), __uint_as_float(r[q4 * 4 + 3]));
                    }
                    p.part_ml[prow] = make_float2(m, l);
                    tc_fence_before();
                } else if (p.o_tma) {
                    // O leaves through shared memory: every thread writes its row's 128 bytes of a 64-column box in the
                    // swizzled box layout and each warp sends its 32 rows with one bulk store (whole lines), instead of
                    // 32-byte stores 256 bytes apart per thread
                    const float inv = 1.0f / l;
                    uint8_t *stg = o_stage + w * C::kOutStageBytes;
                    uint32_t ro[D];  // the whole row of O: all loads in flight, one wait
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) tmem_ld32(t_o + c * 32, ro + c * 32);
                    tc_wait_ld();
#pragma unroll
                    for (int hf = 0; hf < D / 64; ++hf) {
                        const uint32_t *r = ro + hf * 64;
                        uint32_t pk[32];
#pragma unroll
                        for (int i = 0; i < 64; i += 2) {
                            if constexpr (F16IO) {
                                __half2 h2 = __floats2half2_rn(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                                pk[i >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                            } else {
                                __nv_bfloat162 h2 =
                                    __floats2bfloat162_rn(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                                pk[i >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                            }
                        }
                        // A warp stages and sends its own 32 rows, so the four warps of the slot never wait for one
                        // another here.  The staging rows are reused by the next box: the lane that sent the previous one
                        // waits for that bulk store's read only now, after the next box has been fetched and converted
                        // (or an item later), when it is long done.
                        if (lane == 0 && store_pending) {
                            bulk_wait_group_read0();
                            store_pending = false;
                        }
                        __syncwarp();
#pragma unroll
                        for (int ch = 0; ch < 8; ++ch)
                            *reinterpret_cast<uint4 *>(stg + row_in_tile * 128 + ((ch ^ (row_in_tile & 7)) << 4)) =
                                make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
                        fence_proxy_async();  // generic-proxy writes -> visible to the bulk copy's async proxy
                        __syncwarp();
                        // (rows past q_len are clipped by the tensor map; a box that starts past it is not sent at all)
                        if (lane == 0 && it.r0 + w * kTileRows + lane_base < it.q_len) {
                            tma_store_4d(&p.map_o, hf * 64, it.r0 + w * kTileRows + lane_base, h, b, smem_u32(stg + lane_base * 128));
                            bulk_commit_group();
                            store_pending = true;
                        }
                    }
                    if (row < it.q_len) p.lse[((long long)b * p.q_heads + h) * p.lse_hs + row] = (m + log2f(l)) * kLn2;
                    tc_fence_before();
                } else {
                const float inv = 1.0f / l;
                const bool store = row < it.q_len;
                __nv_bfloat16 *op = reinterpret_cast<__nv_bfloat16 *>(p.o) + (long long)b * p.o_bs + (long long)h * p.o_hs +
                                    (long long)row * p.o_rs;
                uint32_t r[32];
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    tmem_ld32(t_o + c * 32, r);
                    tc_wait_ld();
                    if (store) {
                        uint32_t pk[16];
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            if constexpr (F16IO) {
                                __half2 h2 = __floats2half2_rn(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                                pk[i >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                            } else {
                                __nv_bfloat162 h2 =
                                    __floats2bfloat162_rn(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                                pk[i >> 1] = *reinterpret_cast<uint32_t *>(&h2);
                            }
                        }
                        if (p.o_align32) {
                            // 32-byte stores: a lane fills whole 32-byte sectors of its row
#pragma unroll
                            for (int q8 = 0; q8 < 2; ++q8)
                                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(op + c * 32 + q8 * 16),
                                             "r"(pk[q8 * 8]), "r"(pk[q8 * 8 + 1]), "r"(pk[q8 * 8 + 2]), "r"(pk[q8 * 8 + 3]),
                                             "r"(pk[q8 * 8 + 4]), "r"(pk[q8 * 8 + 5]), "r"(pk[q8 * 8 + 6]), "r"(pk[q8 * 8 + 7])
                                             : "memory");
                        } else {
                            uint4 *dst = reinterpret_cast<uint4 *>(op + c * 32);
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4)
                                dst[q4] = make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]);
                        }
                    }
                }
                if (store) p.lse[((long long)b * p.q_heads + h) * p.lse_hs + row] = (m + log2f(l)) * kLn2;
                // the O columns are overwritten by the next item's first PV MMA, which is issued only after this
                // thread's next hand-over of P: program order keeps the reads above ahead of it
                tc_fence_before();
                }
            } else if (SPLIT && k >= 0 && ok) {
                // a part in which this Q tile has no KV tile at all still owns a partial record: an empty one
                const WorkItem it = make_item<SPLIT>(p, item_index(p, k), split_rec);
                if (it.part_slot >= 0)
                    p.part_ml[(long long)it.part_slot * (2 * kTileRows) + w * kTileRows + row_in_tile] = make_float2(-INFINITY, 0.f);
            }
            if ((warp & 3) == 0 && lane == 0) TRACEB(k, w, 4);
            if (next_lin < 0) break;
        }
        if (store_pending) bulk_wait_group_read0();  // the staging space must outlive the last store's read
    }

    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before the CTA exits
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// (cos, sin) of every (row, pair) of a call: angle = f32(pos_off + row) * inv_freq[pair], the same
// f32 product the oracle forms (src/rotary_grouped.rs:44-48); sincosf is within 2 ulp of libm.
struct InvFreq {
    float f[kMaxHeadDim / 2];
};

__global__ void __launch_bounds__(256) rope_table_kernel(float2 *__restrict__ table, int rows, int half_dim,
                                                         int64_t pos_off, InvFreq inv_freq) {
    const int64_t total = (int64_t)rows * half_dim;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int pair = (int)(i % half_dim);
        const int64_t row = i / half_dim;
        const float angle = __fmul_rn((float)(pos_off + row), inv_freq.f[pair]);
        float s, c;
        sincosf(angle, &s, &c);
        table[i] = make_float2(c, s);
    }
}

__global__ void __launch_bounds__(256) fill_u32_kernel(uint32_t *__restrict__ dst, uint32_t value, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) dst[i] = value;
}

// Finishes the rows of the split items of the last round: for each row the parts' unnormalised O_i, running maxima
// m_i (log2 domain) and sums l_i combine to  M = max m_i,  L = sum 2^(m_i - M) l_i,  O = sum 2^(m_i - M) O_i / L,
// LSE = (M + log2 L) ln 2.  Eight CTAs per item (32 rows each), one warp per row, a lane owns D / 32 consecutive
// columns; the kernel is a chain of dependent global loads per row, so rows are spread wide rather than looped over.
constexpr int kMergeCtasPerItem = 8;
template <int D, bool F16IO>
__global__ void __launch_bounds__(256) fwd_split_merge_kernel(const __grid_constant__ KernelParams p, int first_lin) {
    constexpr int kCols = D / 32;
    constexpr int kRowsPerCta = 2 * kTileRows / kMergeCtasPerItem;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int item = blockIdx.x / kMergeCtasPerItem;
    const int lin = first_lin + item;
    const int total_bh = p.batch * p.q_heads;
    const int qb = p.q_blocks - 1 - lin / total_bh, bh = lin % total_bh;
    const int b = bh / p.q_heads, h = bh % p.q_heads;
    const int r0 = qb * 2 * kTileRows;
#pragma unroll
    for (int q = 0; q < kRowsPerCta / 8; ++q) {
        const int rr = (blockIdx.x % kMergeCtasPerItem) * kRowsPerCta + q * 8 + warp;
        const int row = r0 + rr;
        if (row >= p.q_len) continue;
        const long long prow0 = ((long long)item * p.split) * (2 * kTileRows) + rr;
        float mx = -INFINITY;
        for (int i = 0; i < p.split; ++i) mx = fmaxf(mx, p.part_ml[prow0 + (long long)i * (2 * kTileRows)].x);
        float acc[kCols], sum = 0.f;
#pragma unroll
        for (int c = 0; c < kCols; ++c) acc[c] = 0.f;
        for (int i = 0; i < p.split; ++i) {
            const long long prow = prow0 + (long long)i * (2 * kTileRows);
            const float2 ml = p.part_ml[prow];
            if (ml.y == 0.f) continue;  // an empty part
            const float wgt = ex2(ml.x - mx);
            sum = fmaf(wgt, ml.y, sum);
            const float *src = p.part_o + prow * D + lane * kCols;
#pragma unroll
            for (int c = 0; c < kCols; ++c) acc[c] = fmaf(wgt, src[c], acc[c]);
        }
        const float inv = 1.0f / sum;
        uint16_t *op = reinterpret_cast<uint16_t *>(p.o) + (long long)b * p.o_bs + (long long)h * p.o_hs + (long long)row * p.o_rs +
                       lane * kCols;
#pragma unroll
        for (int c = 0; c < kCols; c += 2) {
            uint32_t packed;
            if constexpr (F16IO) {
                const __half2 h2 = __floats2half2_rn(acc[c] * inv, acc[c + 1] * inv);
                packed = *reinterpret_cast<const uint32_t *>(&h2);
            } else {
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[c] * inv, acc[c + 1] * inv);
                packed = *reinterpret_cast<const uint32_t *>(&h2);
            }
            *reinterpret_cast<uint32_t *>(op + c) = packed;
        }
        if (lane == 0) p.lse[((long long)b * p.q_heads + h) * p.lse_hs + row] = (mx + log2f(sum)) * kLn2;
    }
}

// K rotation prologue: x (bf16, strided) -> y (fp16, compact [B, H, N, D]) with interleaved pairs
// (src/rotary_grouped.rs:36-50).  One thread moves 8 elements (16 bytes).
template <bool F16IN>
__global__ void __launch_bounds__(256) rotate_to_f16_kernel(const uint16_t *__restrict__ x, __half *__restrict__ y,
                                                            const float2 *__restrict__ table, int heads, int rows,
                                                            int head_dim, int64_t bs, int64_t hs, int64_t rs,
                                                            int64_t total_vec) {
    const int vec_per_row = head_dim / 8;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += (int64_t)gridDim.x * blockDim.x) {
        const int v = (int)(i % vec_per_row);
        const int64_t rowi = i / vec_per_row;
        const int n = (int)(rowi % rows);
        const int64_t bh = rowi / rows;
        const int hh = (int)(bh % heads);
        const int64_t bb = bh / heads;
        const uint4 raw = *reinterpret_cast<const uint4 *>(x + bb * bs + hh * hs + (int64_t)n * rs + v * 8);
        const float4 *tab = reinterpret_cast<const float4 *>(table + (int64_t)n * (head_dim / 2) + v * 4);
        const float4 cs0 = __ldg(tab), cs1 = __ldg(tab + 1);
        const float cc[4] = {cs0.x, cs0.z, cs1.x, cs1.z}, ss[4] = {cs0.y, cs0.w, cs1.y, cs1.w};
        const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t out[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float fx, fy;
            if constexpr (F16IN) {
                const float2 xy = __half22float2(*reinterpret_cast<const __half2 *>(&in[e]));
                fx = xy.x;
                fy = xy.y;
            } else {
                fx = __uint_as_float(in[e] << 16);
                fy = __uint_as_float(in[e] & 0xffff0000u);
            }
            const __half2 h2 = __floats2half2_rn(fx * cc[e] - fy * ss[e], fx * ss[e] + fy * cc[e]);
            out[e] = *reinterpret_cast<const uint32_t *>(&h2);
        }
        *reinterpret_cast<uint4 *>(y + rowi * head_dim + v * 8) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// (cos, sin) table of `rows` positions starting at pos_off, from the context's cache or computed now on its stream.
int rope_table(flat_ctx *ctx, const InvFreq &f, int half_dim, int rows, int64_t pos_off, const float2 **out) {
    flat_ctx::RopeTable *slot = nullptr;
    for (auto &t : ctx->rope_tables) {
        if (t.rows >= rows && t.half_dim == half_dim && t.pos_off == pos_off &&
            std::memcmp(t.inv_freq, f.f, sizeof(float) * half_dim) == 0) {
            t.last_use = ++ctx->rope_clock;
            *out = static_cast<const float2 *>(t.dev);
            return FLAT_OK;
        }
        if (!slot || t.last_use < slot->last_use) slot = &t;
    }
    const uint64_t bytes = (uint64_t)rows * half_dim * sizeof(float2);
    if (slot->bytes < bytes) {
        slot->rows = 0;
        if (slot->dev) FLAT_CUDA_OK(ctx, cudaFree(slot->dev));  // waits for kernels that still read it
        slot->dev = nullptr;
        slot->bytes = 0;
        FLAT_CUDA_OK(ctx, cudaMalloc(&slot->dev, bytes));
        slot->bytes = bytes;
    }
    const int64_t n = (int64_t)rows * half_dim;
    rope_table_kernel<<<(int)std::min<int64_t>((n + 255) / 256, 4096), 256, 0, ctx->stream>>>(
        static_cast<float2 *>(slot->dev), rows, half_dim, pos_off, f);
    ctx->launches += 1;
    std::memcpy(slot->inv_freq, f.f, sizeof(float) * half_dim);
    slot->half_dim = half_dim;
    slot->rows = rows;
    slot->pos_off = pos_off;
    slot->last_use = ++ctx->rope_clock;
    *out = static_cast<const float2 *>(slot->dev);
    return FLAT_OK;
}

}  // namespace

bool forward_sm100_supported(const FwdParams &p) {
    if (p.head_dim != 64 && p.head_dim != 128) return false;
    if (p.varlen) {
        // padded variable-length batch: one (cos, sin) table spans every sequence's query positions
        if (p.page_table || !p.rope_q) return false;
        const int64_t rows = p.varlen_rope_max - p.varlen_rope_min + p.q_len;
        if (rows * (p.head_dim / 2) * (int64_t)sizeof(float2) > (64ll << 20)) return false;
    }
    if (p.q_len < 32 || p.kv_len < 32) return false;  // tiny shapes: the generic kernel is the better fit
    if (!aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v) || !aligned16(p.o)) return false;
    const int64_t strides[] = {p.q_bs, p.q_hs, p.q_rs, p.kv_bs, p.kv_hs, p.kv_rs, p.o_bs, p.o_hs, p.o_rs};
    for (int64_t s : strides)
        if (s % 8 != 0) return false;
    if (p.page_table) {
        if (p.rope_k) return false;  // the paged cache holds rotated K
        if (p.batch != 1) return false;
        const int ps = p.page_size;
        if (!(ps == 8 || ps == 16 || ps == 32 || ps == 64 || ps == 128)) return false;
    }
    if (p.rope_k && !p.rope_q) return false;
    if (p.f16_io && p.alibi_slopes) return false;  // no binary16 instantiation of the ALiBi kernel
    if (p.alibi_slopes) {
        // the kernel forms bias positions in f32: they must stay exact
        if (p.varlen || p.page_table) return false;
        const int64_t delta = p.alibi_kv_off - p.alibi_q_off;
        if ((delta < 0 ? -delta : delta) + std::max(p.q_len, p.kv_len) >= (1 << 24)) return false;
        // the bias enters as slope / scale: keep that quotient far from overflow
        if (!(p.alibi_max_abs_slope / p.scale < 1.0e30f)) return false;
    }
    return true;
}

namespace {

// Work distribution of one launch (see KernelParams): the grid, the whole rounds, what is left for the last round and
// into how many KV parts each of those items is cut.
constexpr int kMinPartTiles = 16;
struct SplitPlan {
    unsigned grid;
    int full_rounds, rem_items, split;
    long long total_items;
};

SplitPlan plan_split(int sm_count, const FwdParams &p) {
    SplitPlan pl{};
    const int q_blocks = (p.q_len + 2 * kTileRows - 1) / (2 * kTileRows);
    pl.total_items = (long long)q_blocks * p.batch * p.q_heads;
    const long long g = std::min<long long>(pl.total_items, sm_count);
    pl.grid = (unsigned)g;
    pl.full_rounds = (int)(pl.total_items / g);
    pl.rem_items = (int)(pl.total_items % g);
    pl.split = 1;
    if (p.varlen) return pl;  // per-sequence lengths: the parts' tile counts are not known here
    // fewer items than SMs: the only round is the incomplete one
    if (pl.total_items < sm_count) {
        pl.full_rounds = 0;
        pl.rem_items = (int)pl.total_items;
    }
    if (pl.rem_items == 0) return pl;
    int split = std::min(sm_count / pl.rem_items, 8);
    // a part costs a Q load, a rotation, an epilogue of its own and a share of the merge launch (about 10 us together):
    // it should keep at least kMinPartTiles KV tiles.  The last round holds the shortest items, the shortest of all is
    // the first query block
    long long visible = p.kv_len;
    if (p.causal) visible = std::min<long long>(p.kv_len, p.causal_off + std::min(p.q_len, 2 * kTileRows));
    const int n_min = (int)((visible + kTileRows - 1) / kTileRows);
    split = std::min(split, n_min / kMinPartTiles);
    if (split < 2) return pl;
    pl.split = split;
    if (pl.full_rounds == 0) pl.grid = (unsigned)(pl.rem_items * split);
    return pl;
}

uint64_t split_scratch_bytes(const SplitPlan &pl, int head_dim) {
    if (pl.split <= 1) return 0;
    return (uint64_t)pl.rem_items * pl.split * (2 * kTileRows) * (head_dim + 2) * sizeof(float);
}

}  // namespace

// scratch: rotated fp16 K (rope_k) and the partial records of split items; the (cos, sin) tables live in the context's
// table cache
uint64_t forward_sm100_workspace_bytes(const flat_ctx *ctx, const FwdParams &p) {
    uint64_t bytes = 0;
    if (p.rope_k) bytes += ((uint64_t)p.batch * p.kv_heads * p.kv_len * p.head_dim * 2 + 255) & ~uint64_t(255);
    bytes += (split_scratch_bytes(plan_split(ctx->sm_count, p), p.head_dim) + 255) & ~uint64_t(255);
    return bytes;
}

void forward_sm100_geometry(const flat_ctx *ctx, const FwdParams &p, uint32_t *query_rows, uint32_t *kv_rows, uint32_t grid[3],
                            uint32_t *dispatches) {
    *query_rows = 2 * kTileRows;  // one work item: two 128-row Q tiles of one (batch, q_head)
    *kv_rows = kTileRows;
    const SplitPlan pl = plan_split(ctx->sm_count, p);
    grid[0] = pl.grid;  // persistent: one CTA per SM
    grid[1] = grid[2] = 1;
    // the attention kernel, the K rotation pass when K arrives raw, the LSE fill of a padded variable-length batch and
    // the merge of the last round's split items
    *dispatches = 1 + (p.rope_k ? 1 : 0) + (p.varlen ? 1 : 0) + (pl.split > 1 ? 1 : 0);
}

int launch_forward_sm100(flat_ctx *ctx, const FwdParams &p) {
    int st = ensure_workspace(ctx, kWorkspaceMeta + forward_sm100_workspace_bytes(ctx, p));
    if (st) return st;
    const int D = p.head_dim;
    const SplitPlan plan = plan_split(ctx->sm_count, p);
    const void *k_ptr = p.k;
    int64_t k_rs = p.kv_rs, k_hs = p.kv_hs, k_bs = p.kv_bs;
    bool k_f16 = false;
    const bool io16 = p.f16_io != 0;                    // binary16 storage: every operand is fp16 from the start
    const bool k_shadow = p.k_f16 != 0;                 // K arrives as binary16 although V and Q are bf16 (paged cache shadow)
    const bool convk = p.rope_q && !p.rope_k && !io16 && !k_shadow;  // Q rotated against rotated bf16 K: K tiles become fp16 in smem
    const bool q_f16 = p.rope_q || io16;
    char *scratch = scratch_ptr(ctx);
    const float2 *q_table = nullptr;
    if (p.rope_q) {
        InvFreq f;
        std::memcpy(f.f, p.inv_freq, sizeof f.f);
        __half *rk = reinterpret_cast<__half *>(scratch);
        if (p.varlen) {
            const int rows = (int)(p.varlen_rope_max - p.varlen_rope_min) + p.q_len;
            if ((st = rope_table(ctx, f, D / 2, rows, p.varlen_rope_min, &q_table))) return st;
        } else if ((st = rope_table(ctx, f, D / 2, p.q_len, p.q_rope_off, &q_table))) {
            return st;
        }
        if (p.rope_k) {
            const float2 *kt = nullptr;
            if ((st = rope_table(ctx, f, D / 2, p.kv_len, p.k_rope_off, &kt))) return st;
            const int64_t kvecs = (int64_t)p.batch * p.kv_heads * p.kv_len * (D / 8);
            const int blocks = (int)std::min<int64_t>((kvecs + 255) / 256, (int64_t)ctx->sm_count * 16);
            if (p.f16_io)
                rotate_to_f16_kernel<true><<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<const uint16_t *>(p.k), rk, kt, p.kv_heads,
                                                                            p.kv_len, D, p.kv_bs, p.kv_hs, p.kv_rs, kvecs);
            else
                rotate_to_f16_kernel<false><<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<const uint16_t *>(p.k), rk, kt, p.kv_heads,
                                                                             p.kv_len, D, p.kv_bs, p.kv_hs, p.kv_rs, kvecs);
            ctx->launches += 1;
            k_ptr = rk;
            k_rs = D; k_hs = (int64_t)p.kv_len * D; k_bs = k_hs * p.kv_heads;
            k_f16 = true;
        }
    }

    KernelParams kp{};
    // Q always arrives as the caller's bf16 tensor; rotation (if any) happens in shared memory
    if ((st = make_map(ctx, &kp.map_q, io16, p.q, D, p.q_len, p.q_heads, p.batch, p.q_rs, p.q_hs, p.q_bs, kTileRows))) return st;
    if (p.page_table) {
        // physical layout [pages, page_size, kv_heads*D]: dims (d, token in page, head, page)
        const int64_t row = p.page_row_stride;
        if ((st = make_map(ctx, &kp.map_k, io16 || k_shadow, p.k, D, p.page_size, p.kv_heads, p.max_pages, row, p.kv_hs,
                           row * p.page_size, p.page_size))) return st;
        if ((st = make_map(ctx, &kp.map_v, io16, p.v, D, p.page_size, p.kv_heads, p.max_pages, row, p.kv_hs,
                           row * p.page_size, p.page_size))) return st;
    } else {
        if ((st = make_map(ctx, &kp.map_k, k_f16 || io16, k_ptr, D, p.kv_len, p.kv_heads, p.batch, k_rs, k_hs, k_bs, kTileRows))) return st;
        if ((st = make_map(ctx, &kp.map_v, io16, p.v, D, p.kv_len, p.kv_heads, p.batch, p.kv_rs, p.kv_hs, p.kv_bs, kTileRows))) return st;
    }
    // the epilogue's bulk stores clip at the call's q_len, not at a sequence's active length: padded batches keep the
    // per-thread stores
    kp.o_tma = p.varlen ? 0 : 1;
    if (kp.o_tma && (st = make_map(ctx, &kp.map_o, io16, p.o, D, p.q_len, p.q_heads, p.batch, p.o_rs, p.o_hs, p.o_bs, 32)))
        return st;
    kp.o = p.o;
    kp.lse = p.lse;
    kp.o_bs = p.o_bs; kp.o_hs = p.o_hs; kp.o_rs = p.o_rs; kp.lse_hs = p.lse_hs;
    kp.o_align32 = (reinterpret_cast<uintptr_t>(p.o) % 32 == 0 && p.o_bs % 16 == 0 && p.o_hs % 16 == 0 && p.o_rs % 16 == 0) ? 1 : 0;
    kp.batch = p.batch; kp.q_heads = p.q_heads; kp.kv_heads = p.kv_heads; kp.q_len = p.q_len; kp.kv_len = p.kv_len;
    kp.group = p.group;
    kp.div_bh = make_fastdiv(p.batch * p.q_heads);
    kp.div_heads = make_fastdiv(p.q_heads);
    kp.div_group = make_fastdiv(p.group);
    kp.causal = p.causal;
    kp.causal_off = p.causal_off;
    kp.scale_log2 = p.scale * kLog2e;
    kp.idesc_qk = make_idesc(q_f16 ? kFmtF16 : kFmtBF16, (k_f16 || convk || io16 || k_shadow) ? kFmtF16 : kFmtBF16, 0, 0, 128, 128);
    kp.idesc_pv = io16 ? make_idesc(kFmtF16, kFmtF16, 0, 1, 128, (uint32_t)D) : make_idesc(kFmtBF16, kFmtBF16, 0, 1, 128, (uint32_t)D);
    kp.page_table = p.page_table;
    kp.page_size = p.page_size;
    kp.max_pages = p.max_pages;
    kp.physical_pages = p.max_pages;
    kp.q_blocks = (p.q_len + 2 * kTileRows - 1) / (2 * kTileRows);
    kp.status = ctx->dev_status;
    kp.rope_q_table = q_table;
    kp.varlen = p.varlen;
    kp.rope_table_base = p.varlen ? p.varlen_rope_min : 0;
    if (p.varlen) {
        // padded query rows: O = 0, LSE = -inf (src/asymmetric_grouped.rs:103-104); the kernel writes only live rows.
        // The projection layout of this entry point makes O one contiguous block.
        const int64_t o_elems = (int64_t)p.batch * p.q_len * p.q_heads * D, lse_elems = (int64_t)p.batch * p.q_heads * p.q_len;
        FLAT_CUDA_OK(ctx, cudaMemsetAsync(p.o, 0, o_elems * 2, ctx->stream));
        fill_u32_kernel<<<(unsigned)std::min<int64_t>((lse_elems + 255) / 256, 4096), 256, 0, ctx->stream>>>(
            reinterpret_cast<uint32_t *>(p.lse), 0xff800000u, lse_elems);
        ctx->launches += 1;
    }
    if (q_table) {
        const double rows_per_step = 32.0 / (D / 8);
        for (int j = 0; j < D / 2; ++j) {
            const double a = rows_per_step * (double)p.inv_freq[j];
            kp.rope_step[j] = make_float2((float)std::cos(a), (float)std::sin(a));
        }
    }
    kp.trace = nullptr;
#ifdef FLAT_TRACE
    if (const char *tp = getenv("FLAT_TRACE_PTR")) kp.trace = reinterpret_cast<long long *>(strtoull(tp, nullptr, 0));
#endif

    // Persistent launch: one CTA per SM walks its share of the (query block, batch, head) items.
    kp.total_items = plan.total_items;
    if (kp.total_items > 2147483647LL - 8 * (long long)ctx->sm_count)
        return fail(ctx, FLAT_ERR_DISPATCH_LIMIT, "forward grid of %lld blocks is too large", kp.total_items);
    const unsigned grid = plan.grid;
    kp.split_first = 2147483647;
    kp.rem_items = plan.rem_items;
    kp.split = plan.split;
    if (plan.split > 1) {
        // the parts of the last round's items are dealt like items of their own
        kp.split_first = plan.full_rounds * (int)grid;
        kp.total_items = (long long)kp.split_first + (long long)plan.rem_items * plan.split;
        // partial records sit behind the rotated K in the scratch
        char *at = scratch + (p.rope_k ? (((uint64_t)p.batch * p.kv_heads * p.kv_len * D * 2 + 255) & ~uint64_t(255)) : 0);
        kp.part_o = reinterpret_cast<float *>(at);
        kp.part_ml = reinterpret_cast<float2 *>(at + (uint64_t)plan.rem_items * plan.split * (2 * kTileRows) * D * sizeof(float));
    }
    auto run = [&](auto kernel, int smem_bytes) -> int {
        FLAT_CUDA_OK(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        KernelTimer timer(ctx);
        kernel<<<grid, kThreads, smem_bytes, ctx->stream>>>(kp);
        if (plan.split > 1) {
            const int first_lin = plan.full_rounds * (int)grid;
            if (D == 128) {
                if (io16) fwd_split_merge_kernel<128, true><<<plan.rem_items * kMergeCtasPerItem, 256, 0, ctx->stream>>>(kp, first_lin);
                else fwd_split_merge_kernel<128, false><<<plan.rem_items * kMergeCtasPerItem, 256, 0, ctx->stream>>>(kp, first_lin);
            } else {
                if (io16) fwd_split_merge_kernel<64, true><<<plan.rem_items * kMergeCtasPerItem, 256, 0, ctx->stream>>>(kp, first_lin);
                else fwd_split_merge_kernel<64, false><<<plan.rem_items * kMergeCtasPerItem, 256, 0, ctx->stream>>>(kp, first_lin);
            }
            ctx->launches += 1;
        }
        return FLAT_OK;
    };
    kp.alibi_slopes = p.alibi_slopes;
    kp.alibi_delta = (int)(p.alibi_kv_off - p.alibi_q_off);
    kp.alibi_inv_scale = 1.0f / p.scale;
    // <head_dim, CONVK, ALIBI, F16IO, SPLIT>
    auto pick = [&](auto d_tag, auto convk_tag, auto alibi_tag, auto f16_tag) -> int {
        constexpr int kD = decltype(d_tag)::value;
        constexpr bool kConv = decltype(convk_tag)::value, kAlibi = decltype(alibi_tag)::value, kF16 = decltype(f16_tag)::value;
        if (plan.split > 1) return run(fwd_sm100_kernel<kD, kConv, kAlibi, kF16, true>, Cfg<kD, kConv>::kSmemBytes);
        return run(fwd_sm100_kernel<kD, kConv, kAlibi, kF16, false>, Cfg<kD, kConv>::kSmemBytes);
    };
    using T = std::true_type;
    using F = std::false_type;
    using D128 = std::integral_constant<int, 128>;
    using D64 = std::integral_constant<int, 64>;
    if (io16) {
        st = D == 128 ? pick(D128{}, F{}, F{}, T{}) : pick(D64{}, F{}, F{}, T{});
    } else if (p.alibi_slopes) {
        if (D == 128) st = convk ? pick(D128{}, T{}, T{}, F{}) : pick(D128{}, F{}, T{}, F{});
        else st = convk ? pick(D64{}, T{}, T{}, F{}) : pick(D64{}, F{}, T{}, F{});
    } else if (D == 128) st = convk ? pick(D128{}, T{}, F{}, F{}) : pick(D128{}, F{}, F{}, F{});
    else st = convk ? pick(D64{}, T{}, F{}, F{}) : pick(D64{}, F{}, F{}, F{});
    if (st) return st;
    ctx->launches += 1;
    FLAT_CUDA_OK(ctx, cudaGetLastError());
    return FLAT_OK;
}

}  // namespace flat
