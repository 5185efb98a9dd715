// Device-side finiteness scan of uploaded inputs: validate_input (src/lib.rs:428-447) rejects a tensor at
// its first non-finite element.  The host-slice entry points upload Q, K and V chunk by chunk; each chunk is
// scanned on the device as soon as it has landed (one more read at HBM speed instead of a scalar host loop
// over hundreds of MB), and the first offending index per tensor is read back once, before the call returns.
#include "common.h"

namespace flat {
namespace {

__device__ __forceinline__ bool bad32(uint32_t w) { return (w & 0x7f800000u) == 0x7f800000u; }
__device__ __forceinline__ bool bad16(uint32_t h, uint32_t mask) { return (h & mask) == mask; }

// 16-byte loads; `first` of a segment holds the smallest absolute element index found so far.
__global__ void __launch_bounds__(256) finite_scan_kernel(FiniteScan scan) {
    const int seg_i = blockIdx.y;
    const FiniteScan::Segment seg = scan.seg[seg_i];
    if (!seg.data || seg.elements == 0) return;
    const int per_vec = scan.elem_size == 4 ? 4 : 8;
    // elements in front of the first 16-byte boundary (a chunk of an odd-sized tensor need not start on one)
    const uint64_t lead = min(seg.elements, (uint64_t)(((16 - (reinterpret_cast<uintptr_t>(seg.data) & 15)) & 15) / scan.elem_size));
    const uint64_t vecs = (seg.elements - lead) / per_vec;
    const uint32_t mask16 = scan.mask16;
    unsigned long long found = ~0ull;
    const uint4 *v = reinterpret_cast<const uint4 *>(static_cast<const char *>(seg.data) + lead * scan.elem_size);
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint4 r = v[i];
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
        int hit = -1;
        if (scan.elem_size == 4) {
#pragma unroll
            for (int e = 3; e >= 0; --e)
                if (bad32(w[e])) hit = e;
        } else {
#pragma unroll
            for (int e = 3; e >= 0; --e) {
                if (bad16(w[e] >> 16, mask16)) hit = 2 * e + 1;
                if (bad16(w[e] & 0xffffu, mask16)) hit = 2 * e;
            }
        }
        if (hit >= 0) {
            found = seg.base_index + lead + i * per_vec + hit;
            break;  // later vectors of this thread have larger indices
        }
    }
    // what does not fill a vector at either end (at most 7 elements each), by the first thread
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        auto bad_at = [&](uint64_t e) {
            return scan.elem_size == 4 ? bad32(static_cast<const uint32_t *>(seg.data)[e])
                                       : bad16(static_cast<const uint16_t *>(seg.data)[e], mask16);
        };
        for (uint64_t e = 0; e < lead; ++e)
            if (bad_at(e)) {
                found = min(found, (unsigned long long)(seg.base_index + e));
                break;
            }
        for (uint64_t e = lead + vecs * per_vec; e < seg.elements; ++e)
            if (bad_at(e)) {
                found = min(found, (unsigned long long)(seg.base_index + e));
                break;
            }
    }
    if (found != ~0ull) atomicMin(scan.first + seg.slot, found);
}

}  // namespace

int launch_finite_scan(flat_ctx *ctx, const FiniteScan &scan, cudaStream_t stream) {
    uint64_t most = 0;
    for (const auto &s : scan.seg) most = std::max<uint64_t>(most, s.elements);
    if (most == 0) return FLAT_OK;
    const uint64_t vecs = most / (scan.elem_size == 4 ? 4 : 8) + 1;
    const unsigned blocks = (unsigned)std::min<uint64_t>((vecs + 255) / 256, (uint64_t)ctx->sm_count * 8);
    finite_scan_kernel<<<dim3(blocks, 3), 256, 0, stream>>>(scan);
    ctx->launches += 1;
    FLAT_CUDA_OK(ctx, cudaGetLastError());
    return FLAT_OK;
}

}  // namespace flat
