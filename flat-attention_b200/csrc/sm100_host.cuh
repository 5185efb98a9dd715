// Host-side helpers shared by the tensor-core kernels: TMA tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "common.h"

namespace flat {
namespace sm100 {

using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return reinterpret_cast<EncodeFn>(sym);
    }();
    return fn;
}

// 4-D map over (d, row, head, batch) with a (64, box_rows, 1, 1) box and 128-byte swizzle.
inline int make_map(flat_ctx *ctx, CUtensorMap *map, bool f16, const void *base, uint64_t head_dim, uint64_t rows,
             uint64_t heads, uint64_t batch, int64_t rs, int64_t hs, int64_t bs, uint32_t box_rows) {
    EncodeFn fn = encode_fn();
    if (!fn) return fail(ctx, FLAT_ERR_UNAVAILABLE, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[4] = {head_dim, rows, heads, batch};
    cuuint64_t strides[3] = {(cuuint64_t)rs * 2, (cuuint64_t)hs * 2, (cuuint64_t)bs * 2};
    for (int i = 0; i < 3; ++i)
        if (strides[i] == 0) strides[i] = 16;  // extent-1 dimensions still need a legal stride
    cuuint32_t box[4] = {64, box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                    const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, FLAT_ERR_EXECUTION, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return FLAT_OK;
}


}  // namespace sm100
}  // namespace flat
