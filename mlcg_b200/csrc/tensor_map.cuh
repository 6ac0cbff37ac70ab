// Tensor maps for the copy engine (TMA) and the shared -> global tensor stores the tensor-core kernels use to write
// their 128-row output tiles: the tile is staged in shared memory as 32-column boxes in the 128-byte swizzle, one thread
// hands the boxes to the copy engine, and the CTA goes on while they drain.
#pragma once
#include <cuda.h>

#include <cstring>

#include "tc_common.cuh"

namespace mlcgb {

// cuTensorMapEncodeTiled through the runtime's driver entry point (the library does not link libcuda)
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                      const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline TensorMapEncodeFn tensor_map_encoder() {
    static TensorMapEncodeFn fn = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) != cudaSuccess || res != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return (TensorMapEncodeFn)ptr;
    }();
    return fn;
}

// Map of a row-major fp32 matrix M[rows][cols] for boxes of 32 columns x 128 rows in the 128-byte swizzle.
// Needs rows >= 128, cols a multiple of 4 and a 16-byte aligned base (the copy engine's rules); false otherwise.
inline bool make_rows_map(CUtensorMap *map, float *base, int64_t rows, int64_t cols) {
    memset(map, 0, sizeof(*map));
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc || rows < tc::kRows || cols < 4 || (cols & 3) != 0 || (uintptr_t)base % 16 != 0) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * sizeof(float)};
    const cuuint32_t box[2] = {32, (cuuint32_t)tc::kRows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Staging tile as four boxes of [128 rows][128 bytes]: address of 16-byte chunk `chunk` (0..7) of row `row` in box `box`
__device__ __forceinline__ float4 *box_chunk(uint8_t *stage, int box, int row, int chunk) {
    return reinterpret_cast<float4 *>(stage + box * 16384 + row * 128 + ((chunk ^ (row & 7)) << 4));
}

// One box to rows [y, y+128), columns [x, x+32) of the mapped matrix; x must be a multiple of 4 (16 bytes).  Rows and
// columns past the end of the matrix are clipped by the copy engine.
__device__ __forceinline__ void tensor_store_box(const CUtensorMap *map, int x, int y, const uint8_t *src_box) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x),
                 "r"(y), "r"(tc::smem_u32(src_box))
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest `Pending` groups of this thread have finished reading shared memory
template <int Pending>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(Pending) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

}  // namespace mlcgb
