// Tiled TMA descriptors: host-side encoding through the driver entry point (no link against libcuda),
// device-side 2-D tile load into shared memory that signals an mbarrier with its byte count.
#pragma once

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace weft {

// A 2-D row-major array of `rows` x `inner` elements with `row_pitch` bytes between rows (a multiple of 16,
// base 16-byte aligned); the copied box is box_inner x box_rows elements, rows packed in shared memory,
// optionally with the 128-byte swizzle (16-byte chunk c of row r stored at chunk c ^ (r & 7); box rows of
// exactly 128 bytes, destination 1024-byte aligned).  Elements outside the array read as zero and still
// count toward the barrier's bytes.
inline cudaError_t encode_tile_map(CUtensorMap *map, CUtensorMapDataType type, const void *base, unsigned long long inner,
                                   unsigned long long rows, unsigned long long row_pitch, unsigned box_inner, unsigned box_rows,
                                   bool swizzle128 = false) {
    static PFN_cuTensorMapEncodeTiled_v12000 encode = [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query) != cudaSuccess || query != cudaDriverEntryPointSuccess) fn = nullptr;
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }();
    if (!encode) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {row_pitch};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    const CUresult r = encode(map, type, 2, const_cast<void *>(base), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// x (innermost, in elements) times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar)) : "memory");
}

}  // namespace weft
