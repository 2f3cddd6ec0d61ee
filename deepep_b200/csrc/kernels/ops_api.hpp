// Launch interface of the small MoE operators (no torch types).
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

namespace ep {
namespace ops {

// top-k experts per token (ties: lowest id) and softmax weights over the selected logits
cudaError_t router_topk(const float* logits, int num_tokens, int num_experts, int num_topk, int64_t* topk_idx, float* topk_weights,
                        cudaStream_t stream);
// bf16 [rows, hidden] -> e4m3 [rows, hidden] + fp32 scales (element (row, block) at scales[row * row_stride + block * col_stride])
cudaError_t quant_1x128(const void* x, int64_t x_stride_bytes, int rows, int hidden, bool pow2, void* out, float* scales,
                        int64_t sf_row_stride, int64_t sf_col_stride, cudaStream_t stream);
cudaError_t dequant_1x128(const void* q, const float* scales, int64_t sf_row_stride, int64_t sf_col_stride, int rows, int hidden, void* out,
                          cudaStream_t stream);
// x [rows, 2 * inter] bf16 (gate | up) -> out [rows, inter]: silu(gate) * up * row_weight; bf16, or e4m3 + 1x128 scales with `quant`.
// `num_valid_rows` (device, optional) limits the work to the first rows. `pow2`: scales rounded up to powers of two.
cudaError_t swiglu(const void* x, int rows, int inter, const float* row_weight, const int* num_valid_rows, void* out, bool quant,
                   float* scales, int64_t sf_row_stride, int64_t sf_col_stride, bool pow2, cudaStream_t stream);
// dx [rows, 2 * inter] from dout [rows, inter]; optional by-products of the same pass: act_out [rows, inter] bf16 =
// silu(gate) * up * row_weight and dweight [rows] fp32 = sum_i dout_i * silu(gate_i) * up_i (gradient of the row weight)
cudaError_t swiglu_backward(const void* x, const void* dout, int rows, int inter, const float* row_weight, void* dx, void* act_out,
                            float* dweight, cudaStream_t stream);
cudaError_t transpose_bf16(const void* in, int64_t in_stride, int rows, int cols, void* out, int64_t out_stride, cudaStream_t stream);

}  // namespace ops
}  // namespace ep
