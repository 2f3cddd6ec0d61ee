// Launch interface of the fused tensor-parallel operators (no torch types).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "../common/layout.hpp"

namespace ep {
namespace gemm {

struct AgGemmParams {
    CommCtx c;
    int rows_per_rank;            // Ml: rows of every rank's shard (multiple of 128)
    int N, K;
    const uint8_t* a_local;       // [Ml, K] bf16, this rank's shard
    int64_t a_stride_bytes;
    __nv_bfloat16* C;             // [R * Ml, N]
    int64_t ldc;
    uint64_t off_gather;          // this call's half of the gather buffer inside every heap: [R][Ml][K] bf16
    uint32_t epoch;
    int num_comm_ctas;            // CTAs that push the shard instead of computing
    int* error;
};
constexpr int kTpMaxVRanks = 4;   // virtual ranks one launch may carry (single-GPU emulation); production passes 1
// `gather_base[v]` = rank v's own heap + off_gather (the TMA map of the gathered rows reads local memory only)
cudaError_t launch_ag_gemm(const AgGemmParams* params, const void* const* b, const void* const* gather_base, int num_vranks,
                           int ctas_per_rank, cudaStream_t stream);

struct GemmRsParams {
    CommCtx c;
    int rows_per_rank;            // Ml: output rows of every rank (multiple of 128); A has R * Ml rows
    int N, K;                     // K = this rank's slice of the reduction dimension
    __nv_bfloat16* out;           // [Ml, N]
    int64_t ldo;
    uint64_t off_partial[2];      // per half: [R sources][Ml][N] bf16
    uint64_t off_flags[2];        // per half: [R sources][tiles] arrival counters (zero at set-up, only grow)
    uint32_t epoch;
    int flag_target;              // arrivals a tile flag must have reached for this call
    int fuse_own;                 // 1: the epilogue of the rank's own rows adds the peers' partial tiles and writes the result;
                                  // 0: own rows go to the local partial slot and a reduction pass follows the GEMM
    int* error;
};
cudaError_t launch_gemm_rs(const GemmRsParams* params, const void* const* a, const int64_t* a_stride_bytes, const void* const* b,
                           int num_vranks, int ctas_per_rank, cudaStream_t stream);

}  // namespace gemm
}  // namespace ep
