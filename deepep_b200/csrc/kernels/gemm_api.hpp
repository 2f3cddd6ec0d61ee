// Launch interface of the tcgen05 GEMM family (no torch types).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace ep {
namespace gemm {

struct GemmParams {
    int M, N, K;                 // C[M, N] = A[M, K] * B[g][N, K]^T
    int num_groups;              // 1 = plain GEMM
    const int* group_end;        // device [num_groups]: group g owns rows [align(group_end[g-1], group_alignment), group_end[g]);
                                 // null = one group with rows [0, M)
    int group_alignment;
    int zero_gap;                // 1: rows of a tile beyond its group's end are written as zeros (needs group_alignment % 128 == 0)
    // Groups along K (bf16 only): C[g][M, N] = A[:, k range of g] * B[:, k range of g]^T with the k range of group g =
    // [align(group_end[g-1], group_alignment), group_end[g]) -- the weight gradients of all experts in one launch, the
    // rows of an expert being the contraction dimension. A is [M, K], B is [N, K] (one matrix), columns of a range
    // beyond its end up to the next multiple of 64 must be zero. A group without rows gives zeros.
    int k_grouped;
    int64_t c_group_stride;      // elements between C[g] and C[g + 1]
    __nv_bfloat16* C;
    int64_t ldc;                 // elements between rows of C
    // e4m3 inputs: fp32 block scales (ignored for bf16)
    const float* sfa;            // A scales, element (row, kblock) at sfa[row * sfa_row_stride + kblock * sfa_k_stride]
    int64_t sfa_row_stride, sfa_k_stride;
    const float* sfb;            // [num_groups][N / 128][K / 128]
    int scales_pow2;             // every scale is an exact power of two: the block-scaled tensor-core instruction may apply them
    int* error;                  // device int, set to a StatusCode when a pipeline wait runs out
    uint64_t timeout_ns;
};

bool make_kmajor_map(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                     uint32_t box_rows);

// A: [M, K] with row pitch `a_row_stride_bytes`; B: [num_groups * N, K] with row pitch `b_row_stride_bytes`;
// both bf16 (fp8 = false) or e4m3.
cudaError_t launch_gemm(const GemmParams& p, const void* a, int64_t a_row_stride_bytes, const void* b, int64_t b_row_stride_bytes,
                        bool fp8, int num_sms, cudaStream_t stream);

}  // namespace gemm
}  // namespace ep
