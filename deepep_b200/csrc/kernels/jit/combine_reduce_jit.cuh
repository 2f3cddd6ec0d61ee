// Combine reduction with the hidden size and the lane count as compile-time constants, meant to be
// instantiated by the run-time compiler. out[t] = sum over the lanes flagged in `lane_mask[t]` of
// region[lane][t] (fp32, ascending lane), rounded to bf16 once.
// Parity: deep_ep/include/deep_ep/impls/combine_reduce_epilogue.cuh:12-143 of the reference, which is
// likewise instantiated per shape by its JIT.
#pragma once

#include <cuda_bf16.h>
#include <cstdint>

namespace ep {
namespace jit {

struct CombineReduceParams {
    const uint8_t* region;      // [lanes][num_max_tokens][hidden] bf16
    const uint32_t* lane_mask;  // [tokens]
    uint8_t* out;               // [tokens][hidden] bf16
    int num_tokens;
    int num_max_tokens;
};

template <int kHidden, int kLanes>
__device__ __forceinline__ void combine_reduce(const CombineReduceParams& p) {
    static_assert(kHidden % 8 == 0, "rows are moved in 16-byte vectors");
    constexpr int kVecs = kHidden / 8;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int num_warps = (gridDim.x * blockDim.x) >> 5;
    for (int t = warp; t < p.num_tokens; t += num_warps) {
        const uint32_t mask = p.lane_mask[t];
        for (int v = lane; v < kVecs; v += 32) {
            int4 raw[kLanes];
#pragma unroll
            for (int l = 0; l < kLanes; ++l) {
                raw[l] = make_int4(0, 0, 0, 0);
                if ((mask >> l) & 1u)
                    raw[l] = *reinterpret_cast<const int4*>(p.region + ((static_cast<uint64_t>(l) * p.num_max_tokens + t) * kHidden + v * 8) * 2);
            }
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int l = 0; l < kLanes; ++l) {
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[l]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(h2[i]);
                    acc[2 * i] += f.x;
                    acc[2 * i + 1] += f.y;
                }
            }
            int4 out;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
            for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            *reinterpret_cast<int4*>(p.out + (static_cast<uint64_t>(t) * kHidden + v * 8) * 2) = out;
        }
    }
}

}  // namespace jit
}  // namespace ep
