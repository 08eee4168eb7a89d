// Host-side encoder for TMA tensor maps.  The driver entry point is resolved
// through the runtime (cudaGetDriverEntryPoint), so the library does not link
// libcuda.  Tensor maps are passed to kernels by value (__grid_constant__), so
// no device memory is allocated for them.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace nob200 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn();  // nullptr when the driver does not offer it

// Rank-3 row-major view [d2][d1][d0] with byte strides (stride1 for d1, stride2
// for d2; d0 is contiguous), box (b0,b1,b2), 128-byte swizzle unless `swizzle`
// says otherwise, zero fill outside the tensor.  Returns 0 or a negative status.
int make_tensor_map_3d(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t d0, uint64_t d1,
                       uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                       uint32_t b2, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B);

}  // namespace nob200
