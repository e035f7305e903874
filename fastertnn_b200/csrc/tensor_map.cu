// Tensor maps (the descriptors the copy engine reads) are encoded by driver functions; the
// library does not link the driver, it asks the runtime for the entry points on first use.
#include <cuda.h>

#include "internal.h"

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
}

// Two-dimensional tiled map: `dim0` elements per row (contiguous), `dim1` rows `stride1_bytes`
// apart; a copy moves a box of box0 x box1 elements, zero-filled past the edges, written to shared
// memory plainly (swizzle_bytes 0) or in the 32 / 64 / 128-byte swizzle pattern (box0 bytes = that span).
// elem_bytes: 1 (bytes) or 4 (fp32).  `map` points at 128 bytes, 64-byte aligned.
int tnns_tensor_map_2d(void* map, int elem_bytes, const void* base, unsigned long long dim0, unsigned long long dim1,
                       unsigned long long stride1_bytes, unsigned box0, unsigned box1, int swizzle_bytes) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        TNNS_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || !fn) return tnns_fail(TNNS_ERR_UNSUPPORTED, "the driver offers no cuTensorMapEncodeTiled");
        encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    if (elem_bytes != 1 && elem_bytes != 4) return tnns_fail(TNNS_ERR_INVALID, "tensor map element size %d", elem_bytes);
    const cuuint64_t dims[2] = {dim0, dim1};
    const cuuint64_t strides[1] = {stride1_bytes};
    const cuuint32_t box[2] = {box0, box1};
    const cuuint32_t estr[2] = {1, 1};
    if (swizzle_bytes != 0 && swizzle_bytes != 32 && swizzle_bytes != 64 && swizzle_bytes != 128)
        return tnns_fail(TNNS_ERR_INVALID, "tensor map swizzle of %d bytes", swizzle_bytes);
    const CUtensorMapSwizzle swz = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                   : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
    const CUresult r = encode(reinterpret_cast<CUtensorMap*>(map), elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                              2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return tnns_fail(TNNS_ERR_CUDA, "cuTensorMapEncodeTiled failed with driver error %d", (int)r);
    return TNNS_OK;
}
