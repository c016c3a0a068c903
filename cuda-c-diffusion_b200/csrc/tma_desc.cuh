// Host helper: encode a 2-D tiled tensor map (TMA descriptor) over a dense row-major fp32 matrix.  The driver
// entry point is resolved through the runtime, so the library does not link libcuda directly.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

typedef CUresult (*TensorMapEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline TensorMapEncodeTiledFn tensor_map_encoder()
{
    static TensorMapEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess
            && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<TensorMapEncodeTiledFn>(p);
        else
            (void)cudaGetLastError();
    }
    return fn;
}

// Matrix [rows, cols] of fp32 at `base` (16-byte aligned, cols a multiple of 4); boxes of [box_rows, box_cols]
// (each at most 256, box_cols a multiple of 4) land in shared memory densely, row-major, unswizzled.
static inline bool make_tensor_map_2d(CUtensorMap* map, const float* base, uint64_t rows, uint64_t cols,
    uint32_t box_rows, uint32_t box_cols, int l2_promotion = 0)
{
    TensorMapEncodeTiledFn enc = tensor_map_encoder();
    if (!enc || box_rows == 0 || box_rows > 256 || box_cols == 0 || box_cols > 256 || (box_cols & 3u) != 0
        || (cols & 3u) != 0 || (reinterpret_cast<uintptr_t>(base) & 15u) != 0 || rows > 0x7fffffffull)
        return false;
    cuuint64_t gdim[2] = { cols, rows };
    cuuint64_t gstride[1] = { cols * sizeof(float) };
    cuuint32_t box[2] = { box_cols, box_rows };
    cuuint32_t estride[2] = { 1, 1 };
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), gdim, gstride, box, estride,
        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
        l2_promotion == 3 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : l2_promotion == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
            : l2_promotion == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace b200
