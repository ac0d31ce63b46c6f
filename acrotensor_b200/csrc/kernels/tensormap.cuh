// Host side of tiled bulk copies: encoding a tensor map (CUtensorMap) for a row-major fp64 matrix.
// The driver's encoder is looked up through the runtime (cudaGetDriverEntryPoint), so the library
// does not link against the driver library.
#ifndef ACRO_B200_KERNELS_TENSORMAP_CUH
#define ACRO_B200_KERNELS_TENSORMAP_CUH

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace acro_b200_detail
{

// A map over `rows` rows of `cols` doubles (row-major, contiguous, base 16-byte aligned, cols even) whose copies move
// boxes of box_cols x box_rows doubles and lay them out in shared memory with the 64-byte swizzle (box_cols = 8: rows
// of 64 bytes, the 16-byte unit of a row exchanged with the unit numbered (row / 2) % 4).  Returns false when the
// encoder is unavailable or refuses the arguments.
inline bool encode_matrix_map(CUtensorMap *map, const double *base, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows)
{
    typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn encode = [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) != cudaSuccess || found != cudaDriverEntryPointSuccess) fn = nullptr;
        return reinterpret_cast<encode_fn>(fn);
    }();
    if (encode == nullptr) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * sizeof(double)};       // bytes between rows
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 2, const_cast<double *>(base), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}

#endif
