// KV-split decode, exchange and merge in one launch over NVLink peer stores.
//
// Each rank (one process per GPU) owns one device allocation that the other ranks of the box map into their address
// space (CUDA IPC).  A decode step writes the rank's normalised f32 partial [O | LSE] into its staging block; one
// kernel then stores that block into every rank's receive buffer with plain 16-byte peer stores, raises a flag there,
// waits (bounded) until every rank's flag has arrived in its own buffer and merges the blocks:
//   LSE = log sum_r exp(LSE_r),   O = sum_r exp(LSE_r - LSE) O_r.
// The blocks are small (33 KB per rank for 64 query heads of 128 dims), so the step is bound by latency: this route
// replaces "all-gather kernel, then merge kernel" by one kernel whose stores cross NVLink once.  No TMA, no multicast
// and no collective library is involved; every wait gives up after about a second, records
// FLAT_ERR_DEVICE_WAIT_TIMEOUT in the context's device status word and lets the kernel end.
//
// Protocol state lives on the device, so a captured CUDA graph of the step can be replayed: `counter` is the number
// of finished steps, a step's epoch is counter + 1 and its parity selects one of two receive buffers.  A rank can be
// at most one step ahead of another one (it cannot pass a step's wait before every rank has started that step, and a
// rank starts a step only after its previous one has ended), so two buffers are enough.  The reference is
// single-device (src/wgpu_backend.rs:208-217) and has no counterpart.
#include <cstring>

#include "common.h"

namespace flat {
namespace {

constexpr int kMaxWorld = 16;
constexpr int kXchgThreads = 256;
constexpr long long kXchgWaitCycles = 2000000000ll;  // about one second

struct XchgLayout {
    uint64_t block_bytes;  // one rank's partial, rounded up to 16 bytes
    uint64_t staging_off, data_off, flags_off, counter_off, total;
};

XchgLayout xchg_layout(int world, uint64_t rows, uint64_t head_dim) {
    XchgLayout l{};
    l.block_bytes = (rows * (head_dim + 1) * 4 + 15) / 16 * 16;
    l.staging_off = 0;
    l.data_off = l.block_bytes;                                          // [2 parities][world] blocks
    l.flags_off = l.data_off + 2 * (uint64_t)world * l.block_bytes;      // [2 parities][kMaxWorld] epochs
    l.counter_off = l.flags_off + 2 * kMaxWorld * sizeof(uint32_t);      // finished steps, then the CTA ticket
    l.total = l.counter_off + 2 * sizeof(uint32_t);
    return l;
}

struct XchgParams {
    char *local;              // this rank's allocation
    char *peers[kMaxWorld];   // every rank's allocation as mapped here (own entry = local)
    int rank, world;
    int rows, head_dim;
    uint64_t block_bytes, data_off, flags_off, counter_off;
    void *o;      // merged O in the call's dtype
    float *lse;   // merged LSE
    DeviceStatus *status;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// grid = world CTAs.  CTA d stores this rank's block into rank d's receive buffer and raises this rank's flag
// there; then every CTA waits for all flags of this rank's own buffer and merges its share of the rows.
template <typename T>
__global__ void __launch_bounds__(kXchgThreads) peer_exchange_merge_kernel(const XchgParams p) {
    __shared__ int give_up;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t *counter = reinterpret_cast<uint32_t *>(p.local + p.counter_off);
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(counter) + 1u;
    const uint32_t parity = epoch & 1u;
    if (tid == 0) give_up = 0;

    // ---- push: staging block -> destination rank's buffer, slot (parity, this rank)
    const int dst = blockIdx.x;
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(p.local);  // staging sits at offset 0
        uint4 *out = reinterpret_cast<uint4 *>(p.peers[dst] + p.data_off + ((uint64_t)parity * p.world + p.rank) * p.block_bytes);
        const int n16 = (int)(p.block_bytes / 16);
        for (int i = tid; i < n16; i += kXchgThreads) out[i] = src[i];
        __threadfence_system();  // the block is visible system-wide before the flag is
        __syncthreads();
        if (tid == 0) {
            uint32_t *flag = reinterpret_cast<uint32_t *>(p.peers[dst] + p.flags_off) + parity * kMaxWorld + p.rank;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
        }
    }

    // ---- wait for every rank's block of this step (thread r watches rank r's flag)
    if (tid < p.world) {
        const uint32_t *flag = reinterpret_cast<const uint32_t *>(p.local + p.flags_off) + parity * kMaxWorld + tid;
        const long long start = clock64();
        while (ld_acquire_sys(flag) != epoch) {
            if (clock64() - start > kXchgWaitCycles) {
                give_up = 1;
                if (p.status) {
                    p.status->code = FLAT_ERR_DEVICE_WAIT_TIMEOUT;
                    p.status->where = 500 + tid;
                }
                break;
            }
            __nanosleep(40);
        }
    }
    __syncthreads();

    // ---- merge: rows are dealt to the CTAs, a warp takes a row.  Lane r holds rank r's LSE; maximum and sum go
    // through the same butterfly as the merge kernel of the all-gather route, and the weighted sum runs over the
    // ranks in order, so that both routes give the same bits.
    if (!give_up) {
        const char *data = p.local + p.data_off + (uint64_t)parity * p.world * p.block_bytes;
        const int D = p.head_dim;
        for (int row = blockIdx.x * (kXchgThreads / 32) + warp; row < p.rows; row += gridDim.x * (kXchgThreads / 32)) {
            const float mine = lane < p.world
                                   ? __ldcg(reinterpret_cast<const float *>(data + lane * p.block_bytes) + (size_t)p.rows * D + row)
                                   : -INFINITY;
            float mx = mine;
#pragma unroll
            for (int sft = 16; sft >= 1; sft >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sft));
            float sum = lane < p.world ? expf(mine - mx) : 0.f;
#pragma unroll
            for (int sft = 16; sft >= 1; sft >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, sft);
            const float total = mx + logf(sum);
            const float w_mine = lane < p.world ? expf(mine - total) : 0.f;
            // (at most 16 ranks: the merge kernel of the all-gather route adds so few parts in order)
            float acc[kMaxHeadDim / 32];
#pragma unroll
            for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.f;
            for (int r = 0; r < p.world; ++r) {
                const float w = __shfl_sync(0xffffffffu, w_mine, r);
                const float *blk = reinterpret_cast<const float *>(data + r * p.block_bytes) + (size_t)row * D;
#pragma unroll
                for (int i = 0; i < kMaxHeadDim / 32; ++i)
                    if (lane + 32 * i < D) acc[i] = fmaf(w, __ldcg(blk + lane + 32 * i), acc[i]);
            }
#pragma unroll
            for (int i = 0; i < kMaxHeadDim / 32; ++i) {
                const int d = lane + 32 * i;
                if (d >= D) continue;
                if constexpr (sizeof(T) == 4) reinterpret_cast<float *>(p.o)[(size_t)row * D + d] = acc[i];
                else reinterpret_cast<__nv_bfloat16 *>(p.o)[(size_t)row * D + d] = __float2bfloat16_rn(acc[i]);
            }
            if (lane == 0) p.lse[row] = total;
        }
    }

    // ---- the last CTA to get here closes the step
    __syncthreads();
    if (tid == 0) {
        uint32_t *ticket = counter + 1;
        __threadfence();
        if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
            *ticket = 0u;
            *reinterpret_cast<volatile uint32_t *>(counter) = epoch;
            __threadfence();
        }
    }
}

__global__ void fill_u32_xchg_kernel(uint32_t *dst, uint32_t value, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = value;
}

}  // namespace
}  // namespace flat

using namespace flat;

struct flat_splitkv_exchange {
    flat_ctx *ctx = nullptr;
    int rank = 0, world = 0;
    uint64_t rows = 0, head_dim = 0;
    XchgLayout layout{};
    char *local = nullptr;
    char *peers[kMaxWorld] = {};
    bool connected = false;
    cudaIpcMemHandle_t handle{};
};

extern "C" {

int32_t flat_splitkv_exchange_create(flat_ctx *ctx, int32_t rank, int32_t world_size, uint64_t rows, uint64_t head_dim,
                                     flat_splitkv_exchange **out) {
    if (!ctx || !out) return FLAT_ERR_NULL_POINTER;
    *out = nullptr;
    if (world_size <= 0 || world_size > kMaxWorld || rank < 0 || rank >= world_size)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "rank %d of %d ranks: the peer exchange serves 1 to %d ranks", rank, world_size,
                    kMaxWorld);
    if (rows == 0 || head_dim == 0) return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "exchange dimensions must be non-zero");
    if (head_dim > (uint64_t)kMaxHeadDim)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_HEAD_DIM, "head_dim %llu exceeds maximum %d", (unsigned long long)head_dim, kMaxHeadDim);
    if (rows > ((uint64_t)1 << 24)) return fail(ctx, FLAT_ERR_INDEX_SPACE_EXCEEDED, "exchange geometry exceeds the index space");
    auto *x = new flat_splitkv_exchange();
    x->ctx = ctx;
    x->rank = rank;
    x->world = world_size;
    x->rows = rows;
    x->head_dim = head_dim;
    x->layout = xchg_layout(world_size, rows, head_dim);
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&x->local), x->layout.total);
    if (e == cudaSuccess) e = cudaMemset(x->local, 0, x->layout.total);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&x->handle, x->local);
    if (e != cudaSuccess) {
        if (x->local) cudaFree(x->local);
        delete x;
        cudaGetLastError();
        return fail(ctx, FLAT_ERR_EXECUTION, "peer exchange buffer: %s", cudaGetErrorString(e));
    }
    x->peers[rank] = x->local;
    x->connected = world_size == 1;
    *out = x;
    return FLAT_OK;
}

int32_t flat_splitkv_exchange_handle(const flat_splitkv_exchange *x, uint8_t out[64]) {
    if (!x || !out) return FLAT_ERR_NULL_POINTER;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the IPC handle is exchanged as 64 bytes");
    std::memcpy(out, &x->handle, 64);
    return FLAT_OK;
}

int32_t flat_splitkv_exchange_connect(flat_splitkv_exchange *x, const uint8_t *handles, uint64_t handle_bytes) {
    if (!x) return FLAT_ERR_NULL_POINTER;
    flat_ctx *ctx = x->ctx;
    if (!handles) return fail(ctx, FLAT_ERR_NULL_POINTER, "peer handles are null");
    if (handle_bytes < (uint64_t)x->world * 64)
        return fail(ctx, FLAT_ERR_BUFFER_TOO_SMALL, "peer handles have %llu bytes, requires %llu", (unsigned long long)handle_bytes,
                    (unsigned long long)((uint64_t)x->world * 64));
    if (x->world == 1) return FLAT_OK;  // nothing to map
    if (x->connected) return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "the exchange is already connected");
    for (int r = 0; r < x->world; ++r) {
        if (r == x->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles + (uint64_t)r * 64, 64);
        if (std::memcmp(&h, &x->handle, 64) == 0) {
            // this process's own buffer named for another rank (a single-process harness): IPC cannot open a handle in
            // the process that made it, and need not
            x->peers[r] = x->local;
            continue;
        }
        void *ptr = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            for (int q = 0; q < r; ++q)
                if (q != x->rank && x->peers[q]) {
                    if (x->peers[q] != x->local) cudaIpcCloseMemHandle(x->peers[q]);
                    x->peers[q] = nullptr;
                }
            return fail(ctx, FLAT_ERR_UNAVAILABLE, "rank %d's exchange buffer cannot be mapped: %s", r, cudaGetErrorString(e));
        }
        x->peers[r] = static_cast<char *>(ptr);
    }
    x->connected = true;
    return FLAT_OK;
}

void flat_splitkv_exchange_destroy(flat_splitkv_exchange *x) {
    if (!x) return;
    cudaStreamSynchronize(x->ctx->stream);
    for (int r = 0; r < x->world; ++r)
        if (r != x->rank && x->peers[r] && x->peers[r] != x->local) cudaIpcCloseMemHandle(x->peers[r]);
    if (x->local) cudaFree(x->local);
    delete x;
}

int32_t flat_splitkv_decode_peer(flat_ctx *ctx, flat_splitkv_exchange *x, int32_t dtype, uint64_t num_seqs, uint64_t q_heads,
                                 uint64_t kv_heads, uint64_t head_dim, uint64_t page_size, uint64_t physical_pages,
                                 uint64_t max_pages_per_seq, const int32_t *page_tables_dev, const int32_t *context_lens_dev,
                                 const int32_t *q_rope_positions_dev, const int32_t *host_page_tables,
                                 const int32_t *host_context_lens, const flat_attention_config *config, float theta,
                                 flat_buffer q, flat_buffer k, flat_buffer v, flat_buffer out_and_lse) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    if (!x) return fail(ctx, FLAT_ERR_NULL_POINTER, "peer exchange is null");
    if (x->ctx != ctx) return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "the exchange belongs to another context");
    if (!x->connected) return fail(ctx, FLAT_ERR_UNAVAILABLE, "the exchange is not connected to its peers");
    if (dtype != FLAT_BF16 && dtype != FLAT_F32) return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "unknown dtype %d", dtype);
    if (num_seqs == 0 || q_heads == 0 || head_dim == 0)
        return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "paged decode dimensions must all be non-zero");
    if (q_heads > ((uint64_t)1 << 20) || num_seqs > 65535)
        return fail(ctx, FLAT_ERR_DISPATCH_LIMIT, "decode geometry exceeds the dispatch limits");
    const uint64_t rows = num_seqs * q_heads;
    if (rows != x->rows || head_dim != x->head_dim)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "the exchange was created for %llu rows of %llu dims, the call has %llu of %llu",
                    (unsigned long long)x->rows, (unsigned long long)x->head_dim, (unsigned long long)rows,
                    (unsigned long long)head_dim);
    const uint64_t lse_off = dtype == FLAT_BF16 ? (rows * head_dim * 2 + 3) / 4 * 4 : rows * head_dim * 4;
    if (!out_and_lse.ptr) return fail(ctx, FLAT_ERR_NULL_POINTER, "O|LSE buffer is null");
    if (out_and_lse.bytes < lse_off + rows * 4)
        return fail(ctx, FLAT_ERR_BUFFER_TOO_SMALL, "O|LSE has %llu bytes, requires %llu", (unsigned long long)out_and_lse.bytes,
                    (unsigned long long)(lse_off + rows * 4));
    const uint64_t block_floats = rows * (head_dim + 1);
    float *staging = reinterpret_cast<float *>(x->local + x->layout.staging_off);
    bool empty = host_context_lens != nullptr;
    for (uint64_t s = 0; empty && s < num_seqs; ++s) empty = host_context_lens[s] == 0;
    if (empty) {
        // this rank holds no token of any sequence: it contributes weight zero (O = 0, LSE = -inf)
        FLAT_CUDA_OK(ctx, cudaMemsetAsync(staging, 0, rows * head_dim * 4, ctx->stream));
        fill_u32_xchg_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, ctx->stream>>>(
            reinterpret_cast<uint32_t *>(staging + rows * head_dim), 0xff800000u, (int)rows);
        ctx->launches += 1;
        FLAT_CUDA_OK(ctx, cudaGetLastError());
    } else {
        const int st = flat_decode_paged_batched_partial(ctx, dtype, num_seqs, q_heads, kv_heads, head_dim, page_size,
                                                         physical_pages, max_pages_per_seq, page_tables_dev, context_lens_dev,
                                                         q_rope_positions_dev, host_page_tables, host_context_lens, config, theta,
                                                         q, k, v, flat_buffer{staging, block_floats * 4});
        if (st) return st;
    }
    XchgParams p{};
    p.local = x->local;
    for (int r = 0; r < x->world; ++r) p.peers[r] = x->peers[r];
    p.rank = x->rank;
    p.world = x->world;
    p.rows = (int)rows;
    p.head_dim = (int)head_dim;
    p.block_bytes = x->layout.block_bytes;
    p.data_off = x->layout.data_off;
    p.flags_off = x->layout.flags_off;
    p.counter_off = x->layout.counter_off;
    p.o = out_and_lse.ptr;
    p.lse = reinterpret_cast<float *>(static_cast<char *>(out_and_lse.ptr) + lse_off);
    p.status = ctx->dev_status;
    if (dtype == FLAT_BF16)
        peer_exchange_merge_kernel<__nv_bfloat16><<<x->world, kXchgThreads, 0, ctx->stream>>>(p);
    else
        peer_exchange_merge_kernel<float><<<x->world, kXchgThreads, 0, ctx->stream>>>(p);
    ctx->launches += 1;
    FLAT_CUDA_OK(ctx, cudaGetLastError());
    return FLAT_OK;
}

}  // extern "C"
