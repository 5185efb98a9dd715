// The one exchange of the attention path: single-sequence long-context decode split along KV across the GPUs of
// a box.  Every rank decodes its slice of the cache into a normalised f32 partial [O | LSE], the partials are
// all-gathered with NCCL over NVLink and every rank merges them locally (LSE = log sum exp(LSE_i),
// O = sum exp(LSE_i - LSE) O_i).  The reference is single-device (src/wgpu_backend.rs:208-217) and has no
// counterpart.
//
// NCCL is not linked: a host that owns an ncclComm_t has the library in its process already (PyTorch loads its
// bundled copy), and the communicator must be used with exactly that copy, so the two entry points needed are
// looked up in the loaded libnccl.so.2 at the first call.  Hosts without NCCL can still load this library; the
// exchange entry points then return FLAT_ERR_UNAVAILABLE.
#include <dlfcn.h>

#include "common.h"

namespace flat {
namespace {

using NcclAllGatherFn = int (*)(const void *, void *, size_t, int, void *, cudaStream_t);
using NcclErrorStringFn = const char *(*)(int);
constexpr int kNcclFloat32 = 7;  // ncclFloat32 of nccl.h

struct NcclApi {
    NcclAllGatherFn all_gather = nullptr;
    NcclErrorStringFn error_string = nullptr;
    const char *why = nullptr;
};

const NcclApi &nccl_api() {
    static const NcclApi api = [] {
        NcclApi a;
        // the copy the process already uses, else whatever the loader finds
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            a.why = "libnccl.so.2 is not loaded and cannot be found";
            return a;
        }
        a.all_gather = reinterpret_cast<NcclAllGatherFn>(dlsym(h, "ncclAllGather"));
        a.error_string = reinterpret_cast<NcclErrorStringFn>(dlsym(h, "ncclGetErrorString"));
        if (!a.all_gather) a.why = "ncclAllGather is missing from libnccl.so.2";
        return a;
    }();
    return api;
}

__global__ void fill_u32_small_kernel(uint32_t *dst, uint32_t value, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = value;
}

}  // namespace
}  // namespace flat

using namespace flat;

extern "C" {

int32_t flat_splitkv_merge_nccl(flat_ctx *ctx, void *nccl_comm, int32_t rank, int32_t world_size, int32_t dtype,
                                uint64_t rows, uint64_t head_dim, flat_buffer gathered, flat_buffer out_and_lse) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    if (!nccl_comm) return fail(ctx, FLAT_ERR_NULL_POINTER, "NCCL communicator is null");
    if (world_size <= 0 || rank < 0 || rank >= world_size)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "rank %d is outside a communicator of %d ranks", rank, world_size);
    if (rows == 0 || head_dim == 0) return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "merge dimensions must be non-zero");
    if (head_dim > (uint64_t)kMaxHeadDim)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_HEAD_DIM, "head_dim %llu exceeds maximum %d", (unsigned long long)head_dim, kMaxHeadDim);
    if (rows > ((uint64_t)1 << 31)) return fail(ctx, FLAT_ERR_INDEX_SPACE_EXCEEDED, "merge geometry exceeds the index space");
    const uint64_t block_floats = rows * (head_dim + 1);
    if (!gathered.ptr) return fail(ctx, FLAT_ERR_NULL_POINTER, "gather buffer is null");
    if (gathered.bytes < (uint64_t)world_size * block_floats * 4)
        return fail(ctx, FLAT_ERR_BUFFER_TOO_SMALL, "gather buffer has %llu bytes, requires %llu", (unsigned long long)gathered.bytes,
                    (unsigned long long)((uint64_t)world_size * block_floats * 4));
    const NcclApi &api = nccl_api();
    if (!api.all_gather) return fail(ctx, FLAT_ERR_UNAVAILABLE, "NCCL is unavailable: %s", api.why);
    // in place: this rank's block already sits in its slot of the gather buffer
    float *base = static_cast<float *>(gathered.ptr);
    const int rc = api.all_gather(base + (uint64_t)rank * block_floats, base, block_floats, kNcclFloat32, nccl_comm, ctx->stream);
    if (rc != 0)
        return fail(ctx, FLAT_ERR_EXECUTION, "ncclAllGather failed: %s", api.error_string ? api.error_string(rc) : "unknown error");
    return flat_splitkv_merge_packed(ctx, dtype, (uint64_t)world_size, rows, head_dim, gathered, out_and_lse);
}

int32_t flat_splitkv_decode_nccl(flat_ctx *ctx, void *nccl_comm, int32_t rank, int32_t world_size, int32_t dtype,
                                 uint64_t num_seqs, uint64_t q_heads, uint64_t kv_heads, uint64_t head_dim, uint64_t page_size,
                                 uint64_t physical_pages, uint64_t max_pages_per_seq, const int32_t *page_tables_dev,
                                 const int32_t *context_lens_dev, const int32_t *q_rope_positions_dev,
                                 const int32_t *host_page_tables, const int32_t *host_context_lens,
                                 const flat_attention_config *config, float theta, flat_buffer q, flat_buffer k, flat_buffer v,
                                 flat_buffer gathered, flat_buffer out_and_lse) {
    if (!ctx) return FLAT_ERR_NULL_POINTER;
    if (world_size <= 0 || rank < 0 || rank >= world_size)
        return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "rank %d is outside a communicator of %d ranks", rank, world_size);
    if (num_seqs == 0 || q_heads == 0 || head_dim == 0)
        return fail(ctx, FLAT_ERR_ZERO_DIMENSION, "paged decode dimensions must all be non-zero");
    if (q_heads > ((uint64_t)1 << 20) || num_seqs > 65535 || head_dim > (uint64_t)kMaxHeadDim)
        return fail(ctx, FLAT_ERR_DISPATCH_LIMIT, "decode geometry exceeds the dispatch limits");
    const uint64_t rows = num_seqs * q_heads, block_floats = rows * (head_dim + 1);
    if (!gathered.ptr) return fail(ctx, FLAT_ERR_NULL_POINTER, "gather buffer is null");
    if (gathered.bytes < (uint64_t)world_size * block_floats * 4)
        return fail(ctx, FLAT_ERR_BUFFER_TOO_SMALL, "gather buffer has %llu bytes, requires %llu", (unsigned long long)gathered.bytes,
                    (unsigned long long)((uint64_t)world_size * block_floats * 4));
    float *mine = static_cast<float *>(gathered.ptr) + (uint64_t)rank * block_floats;
    bool empty = host_context_lens != nullptr;
    for (uint64_t s = 0; empty && s < num_seqs; ++s) empty = host_context_lens[s] == 0;
    if (empty) {
        // this rank holds no token of any sequence: it contributes weight zero (O = 0, LSE = -inf)
        FLAT_CUDA_OK(ctx, cudaMemsetAsync(mine, 0, rows * head_dim * 4, ctx->stream));
        fill_u32_small_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, ctx->stream>>>(
            reinterpret_cast<uint32_t *>(mine + rows * head_dim), 0xff800000u, (int)rows);
        ctx->launches += 1;
        FLAT_CUDA_OK(ctx, cudaGetLastError());
    } else {
        const int st = flat_decode_paged_batched_partial(ctx, dtype, num_seqs, q_heads, kv_heads, head_dim, page_size,
                                                         physical_pages, max_pages_per_seq, page_tables_dev, context_lens_dev,
                                                         q_rope_positions_dev, host_page_tables, host_context_lens, config, theta,
                                                         q, k, v, flat_buffer{mine, block_floats * 4});
        if (st) return st;
    }
    return flat_splitkv_merge_nccl(ctx, nccl_comm, rank, world_size, dtype, rows, head_dim, gathered, out_and_lse);
}

}  // extern "C"
