// Routing layout of one rank: tokens per destination rank (a token counts once per rank),
// (token, expert) pairs per expert, and the token x rank membership matrix.
//
// Parity: csrc/kernels/legacy/layout.cu:10-122 (get_dispatch_layout) of the reference,
// which splits experts and ranks over separate SM groups; here every block histograms its
// own slice of tokens in shared memory and merges with one atomic per non-zero bin.
#include "api.hpp"
#include "../common/device_utils.cuh"

namespace ep {

namespace {

__global__ void __launch_bounds__(256) layout_kernel(const void* __restrict__ topk_idx, bool idx32, int num_tokens, int num_topk, int num_ranks,
                                                     int num_experts, int* num_tokens_per_rank, int* num_tokens_per_expert,
                                                     bool* is_token_in_rank) {
    extern __shared__ int s_hist[];   // [num_experts + num_ranks]
    int* s_expert = s_hist;
    int* s_rank = s_hist + num_experts;
    for (int i = threadIdx.x; i < num_experts + num_ranks; i += blockDim.x) s_hist[i] = 0;
    __syncthreads();
    const int experts_per_rank = num_experts / num_ranks;
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < num_tokens; t += gridDim.x * blockDim.x) {
        uint32_t mask = 0;
        for (int k = 0; k < num_topk; ++k) {
            const int e = load_topk_idx(topk_idx, idx32, static_cast<int64_t>(t) * num_topk + k, num_experts);
            if (e >= 0) {
                atomicAdd(s_expert + e, 1);
                mask |= 1u << (e / experts_per_rank);
            }
        }
        for (int r = 0; r < num_ranks; ++r) {
            const bool in = (mask >> r) & 1u;
            is_token_in_rank[static_cast<int64_t>(t) * num_ranks + r] = in;
            if (in) atomicAdd(s_rank + r, 1);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < num_experts; i += blockDim.x)
        if (s_expert[i] != 0) atomicAdd(num_tokens_per_expert + i, s_expert[i]);
    for (int i = threadIdx.x; i < num_ranks; i += blockDim.x)
        if (s_rank[i] != 0) atomicAdd(num_tokens_per_rank + i, s_rank[i]);
}

}  // namespace

cudaError_t launch_dispatch_layout(const void* topk_idx, bool idx32, int num_tokens, int num_topk, int num_ranks, int num_experts,
                                   int* num_tokens_per_rank, int* num_tokens_per_expert, bool* is_token_in_rank,
                                   cudaStream_t stream) {
    cudaError_t err = cudaMemsetAsync(num_tokens_per_rank, 0, sizeof(int) * num_ranks, stream);
    if (err != cudaSuccess) return err;
    err = cudaMemsetAsync(num_tokens_per_expert, 0, sizeof(int) * num_experts, stream);
    if (err != cudaSuccess) return err;
    if (num_tokens == 0) return cudaSuccess;
    int blocks = (num_tokens + 255) / 256;
    if (blocks > 148) blocks = 148;
    layout_kernel<<<blocks, 256, (num_experts + num_ranks) * sizeof(int), stream>>>(
        topk_idx, idx32, num_tokens, num_topk, num_ranks, num_experts, num_tokens_per_rank, num_tokens_per_expert, is_token_in_rank);
    return cudaGetLastError();
}

}  // namespace ep
