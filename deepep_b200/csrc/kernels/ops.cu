// Small memory-bound operators of the MoE layer (sm_100a): router top-k + softmax, SwiGLU (with an
// optional fused 1x128 e4m3 cast for the second expert GEMM), 1x128 block quantisation and
// dequantisation, and a 2-D bf16 transpose for weight-gradient GEMMs.
// All of them stream each byte once (16-byte accesses, no shared-memory staging except the
// transpose) and are bound by HBM bandwidth.
//
// The reference has none of these as kernels; its test helpers (deep_ep/utils/math.py:30-56) are
// the arithmetic these follow.
#include "ops_api.hpp"
#include "../common/device_utils.cuh"

namespace ep {
namespace ops {

namespace {

// ---------------------------------------------------------------- router: top-k over experts, softmax over the selection
// one warp per token; the warp keeps the row in registers (experts <= 2048 -> 64 values per lane)
template <int kPerLane>
__global__ void __launch_bounds__(256) router_topk_kernel(const float* __restrict__ logits, int num_tokens, int num_experts, int num_topk,
                                                          int64_t* __restrict__ topk_idx, float* __restrict__ topk_weights) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = lane_id();
    if (warp >= num_tokens) return;
    const float* row = logits + static_cast<int64_t>(warp) * num_experts;
    float v[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        const int e = i * 32 + lane;
        v[i] = e < num_experts ? row[e] : -INFINITY;
    }
    float sel_val = 0.f;
    int sel_idx = -1;
    float vmax = -INFINITY;
    for (int k = 0; k < num_topk; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const int e = i * 32 + lane;
            if (v[i] > best) { best = v[i]; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }   // ties: lowest expert id
        }
        if (k == 0) vmax = best;
        if ((best_e & 31) == lane) {
#pragma unroll
            for (int i = 0; i < kPerLane; ++i)
                if (i == (best_e >> 5)) v[i] = -INFINITY;
        }
        if (lane == k) { sel_val = best; sel_idx = best_e; }
    }
    float ex = (lane < num_topk) ? __expf(sel_val - vmax) : 0.f;
    float sum = ex;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane < num_topk) {
        topk_idx[static_cast<int64_t>(warp) * num_topk + lane] = sel_idx;
        topk_weights[static_cast<int64_t>(warp) * num_topk + lane] = ex / sum;
    }
}

// ---------------------------------------------------------------- 1x128 quantisation
// thread = 8 channels, 16 threads = one scale group; rows * (hidden / 8) threads in total
__global__ void __launch_bounds__(256) quant_kernel(const uint8_t* __restrict__ x, int64_t x_stride_bytes, int rows, int hidden, int pow2,
                                                    uint8_t* __restrict__ out, float* __restrict__ scales, int64_t sf_row_stride,
                                                    int64_t sf_col_stride) {
    const int vec_per_row = hidden / 8;
    const int64_t total = static_cast<int64_t>(rows) * vec_per_row;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * blockDim.x; base < total; base += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t i = base + threadIdx.x;
        const bool active = i < total;
        const int row = active ? static_cast<int>(i / vec_per_row) : 0, ch = active ? static_cast<int>(i % vec_per_row) * 8 : 0;
        int4 raw = make_int4(0, 0, 0, 0);
        if (active) raw = ld_nc_int4(x + row * x_stride_bytes + ch * 2);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 t = __bfloat1622float2(h2[j]);
            f[2 * j] = t.x;
            f[2 * j + 1] = t.y;
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
        amax = warp_reduce_max_width(amax, 16);   // hidden % 128 == 0: a 16-lane group never straddles rows
        float scale, inv;
        fp8_scale_from_amax(amax, pow2 != 0, scale, inv);
        uint2 packed;
        packed.x = pack4_e4m3(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
        packed.y = pack4_e4m3(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
        if (active) {
            *reinterpret_cast<uint2*>(out + static_cast<int64_t>(row) * hidden + ch) = packed;
            if ((threadIdx.x & 15) == 0) scales[row * sf_row_stride + (ch >> 7) * sf_col_stride] = scale;
        }
    }
}

__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scales, int64_t sf_row_stride,
                                                      int64_t sf_col_stride, int rows, int hidden, uint8_t* __restrict__ out) {
    const int vec_per_row = hidden / 8;
    const int64_t total = static_cast<int64_t>(rows) * vec_per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(i / vec_per_row), ch = static_cast<int>(i % vec_per_row) * 8;
        const uint2 raw = *reinterpret_cast<const uint2*>(q + static_cast<int64_t>(row) * hidden + ch);
        const float s = scales[row * sf_row_stride + (ch >> 7) * sf_col_stride];
        const __nv_fp8x2_storage_t* p2 = reinterpret_cast<const __nv_fp8x2_storage_t*>(&raw);
        int4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(p2[j], __NV_E4M3);
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
            o2[j] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
        *reinterpret_cast<int4*>(out + (static_cast<int64_t>(row) * hidden + ch) * 2) = o;
    }
}

// ---------------------------------------------------------------- SwiGLU: out = silu(gate) * up (* row weight), optional fused 1x128 cast
template <bool kQuant>
__global__ void __launch_bounds__(256) swiglu_kernel(const uint8_t* __restrict__ x, int rows, int inter, const float* __restrict__ row_weight,
                                                     const int* __restrict__ num_valid_rows, uint8_t* __restrict__ out,
                                                     float* __restrict__ scales, int64_t sf_row_stride, int64_t sf_col_stride, int pow2) {
    const int vec_per_row = inter / 8;
    const int valid = num_valid_rows != nullptr ? min(*num_valid_rows, rows) : rows;
    const int64_t total = static_cast<int64_t>(valid) * vec_per_row;
    for (int64_t base = static_cast<int64_t>(blockIdx.x) * blockDim.x; base < total; base += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t i = base + threadIdx.x;
        const bool active = i < total;
        const int row = active ? static_cast<int>(i / vec_per_row) : 0, ch = active ? static_cast<int>(i % vec_per_row) * 8 : 0;
        int4 g = make_int4(0, 0, 0, 0), u = make_int4(0, 0, 0, 0);
        if (active) {
            const uint8_t* src = x + (static_cast<int64_t>(row) * 2 * inter + ch) * 2;
            g = ld_nc_int4(src);
            u = ld_nc_int4(src + static_cast<int64_t>(inter) * 2);
        }
        const float wr = (active && row_weight != nullptr) ? row_weight[row] : 1.f;
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 gv = __bfloat1622float2(g2[j]), uv = __bfloat1622float2(u2[j]);
            f[2 * j] = gv.x / (1.f + __expf(-gv.x)) * uv.x * wr;
            f[2 * j + 1] = gv.y / (1.f + __expf(-gv.y)) * uv.y * wr;
        }
        if constexpr (!kQuant) {
            if (active) {
                int4 o;
                __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
                *reinterpret_cast<int4*>(out + (static_cast<int64_t>(row) * inter + ch) * 2) = o;
            }
        } else {
            // the cast sees what a bf16 round trip would see, so fused and unfused paths agree bit for bit
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(__float2bfloat16_rn(f[j]));
            float amax = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
            amax = warp_reduce_max_width(amax, 16);
            float scale, inv;
            fp8_scale_from_amax(amax, pow2 != 0, scale, inv);
            uint2 packed;
            packed.x = pack4_e4m3(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
            packed.y = pack4_e4m3(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
            if (active) {
                *reinterpret_cast<uint2*>(out + static_cast<int64_t>(row) * inter + ch) = packed;
                if ((threadIdx.x & 15) == 0) scales[row * sf_row_stride + (ch >> 7) * sf_col_stride] = scale;
            }
        }
    }
}

// d(gate|up) from d(out): dgate = dout * up * sig * (1 + gate * (1 - sig)), dup = dout * silu(gate), both times the
// row's gate weight. One block per row (grid-strided), so that the two by-products of the MoE backward pass come out
// of the same read of (gate, up, dout): the weighted activation silu(gate) * up * w (the operand of the W2 weight
// gradient) and the gradient of the gate weight, sum_i dout_i * silu(gate_i) * up_i (a row dot product).
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ dout, int rows, int inter,
                                                         const float* __restrict__ row_weight, uint8_t* __restrict__ dx,
                                                         uint8_t* __restrict__ act_out, float* __restrict__ dweight) {
    __shared__ float s_part[8];
    const int vec_per_row = inter / 8;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float wr = row_weight != nullptr ? row_weight[row] : 1.f;
        float dot = 0.f;
        for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
            const int ch = v * 8;
            const uint8_t* src = x + (static_cast<int64_t>(row) * 2 * inter + ch) * 2;
            const int4 g = ld_nc_int4(src), u = ld_nc_int4(src + static_cast<int64_t>(inter) * 2);
            const int4 d = ld_nc_int4(dout + (static_cast<int64_t>(row) * inter + ch) * 2);
            const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
            const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
            const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&d);
            int4 og, ou, oa;
            __nv_bfloat162* og2 = reinterpret_cast<__nv_bfloat162*>(&og);
            __nv_bfloat162* ou2 = reinterpret_cast<__nv_bfloat162*>(&ou);
            __nv_bfloat162* oa2 = reinterpret_cast<__nv_bfloat162*>(&oa);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 gv = __bfloat1622float2(g2[j]), uv = __bfloat1622float2(u2[j]), dv = __bfloat1622float2(d2[j]);
                const float sx = 1.f / (1.f + __expf(-gv.x)), sy = 1.f / (1.f + __expf(-gv.y));
                const float dx_ = dv.x * wr, dy_ = dv.y * wr;
                og2[j] = __floats2bfloat162_rn(dx_ * uv.x * sx * (1.f + gv.x * (1.f - sx)), dy_ * uv.y * sy * (1.f + gv.y * (1.f - sy)));
                ou2[j] = __floats2bfloat162_rn(dx_ * gv.x * sx, dy_ * gv.y * sy);
                // the activation as the forward pass rounded it (bf16), before the weight
                const __nv_bfloat162 a = __floats2bfloat162_rn(gv.x * sx * uv.x, gv.y * sy * uv.y);
                const float2 af = __bfloat1622float2(a);
                dot = fmaf(dv.x, af.x, fmaf(dv.y, af.y, dot));
                oa2[j] = __floats2bfloat162_rn(af.x * wr, af.y * wr);
            }
            uint8_t* dst = dx + (static_cast<int64_t>(row) * 2 * inter + ch) * 2;
            *reinterpret_cast<int4*>(dst) = og;
            *reinterpret_cast<int4*>(dst + static_cast<int64_t>(inter) * 2) = ou;
            if (act_out != nullptr) *reinterpret_cast<int4*>(act_out + (static_cast<int64_t>(row) * inter + ch) * 2) = oa;
        }
        if (dweight != nullptr) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            __syncthreads();
            if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = dot;
            __syncthreads();
            if (threadIdx.x == 0) {
                float acc = 0.f;
                for (int i = 0; i < 8; ++i) acc += s_part[i];      // fixed order: the result does not depend on timing
                dweight[row] = acc;
            }
        }
    }
}

// ---------------------------------------------------------------- bf16 transpose [rows, cols] -> [cols, rows], 64 x 64 tiles
// Interior tiles of aligned tensors move 16 bytes per thread on both sides: a thread loads eight columns of two
// consecutive rows, pairs them up column by column (one 32-bit word = the same column of both rows) and stores the
// words transposed into shared memory (pitch 33 words); the write side reads four words = eight rows of one column
// and stores them as one 16-byte vector. Edge tiles and unaligned tensors take the element-wise path.
__global__ void __launch_bounds__(256) transpose_kernel(const __nv_bfloat16* __restrict__ in, int64_t in_stride, int rows, int cols,
                                                        __nv_bfloat16* __restrict__ out, int64_t out_stride, int aligned) {
    __shared__ uint32_t tile_t[64 * 33];      // [column][row pair]
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    if (aligned && r0 + 64 <= rows && c0 + 64 <= cols) {
        const int rp = threadIdx.x >> 3, cv = threadIdx.x & 7;
        const int4 a = ld_nc_int4(reinterpret_cast<const uint8_t*>(in + (r0 + 2 * rp) * in_stride + c0 + cv * 8));
        const int4 b = ld_nc_int4(reinterpret_cast<const uint8_t*>(in + (r0 + 2 * rp + 1) * in_stride + c0 + cv * 8));
        const uint32_t aw[4] = {static_cast<uint32_t>(a.x), static_cast<uint32_t>(a.y), static_cast<uint32_t>(a.z), static_cast<uint32_t>(a.w)};
        const uint32_t bw[4] = {static_cast<uint32_t>(b.x), static_cast<uint32_t>(b.y), static_cast<uint32_t>(b.z), static_cast<uint32_t>(b.w)};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // columns 2j and 2j + 1 of this thread's eight: low halves of both rows, then high halves
            tile_t[(cv * 8 + 2 * j) * 33 + rp] = __byte_perm(aw[j], bw[j], 0x5410);
            tile_t[(cv * 8 + 2 * j + 1) * 33 + rp] = __byte_perm(aw[j], bw[j], 0x7632);
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int i = threadIdx.x + u * 256;
            const int c = i >> 3, rv = i & 7;
            int4 v;
            v.x = static_cast<int>(tile_t[c * 33 + 4 * rv]);
            v.y = static_cast<int>(tile_t[c * 33 + 4 * rv + 1]);
            v.z = static_cast<int>(tile_t[c * 33 + 4 * rv + 2]);
            v.w = static_cast<int>(tile_t[c * 33 + 4 * rv + 3]);
            st_na_int4(reinterpret_cast<uint8_t*>(out + (c0 + c) * out_stride + r0 + rv * 8), v);
        }
        return;
    }
    __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(tile_t);     // [64][66]
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int r = i / 64, c = i % 64;
        tile[r * 66 + c] = (r0 + r < rows && c0 + c < cols) ? in[(r0 + r) * in_stride + c0 + c] : __float2bfloat16(0.f);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        const int c = i / 64, r = i % 64;
        if (c0 + c < cols && r0 + r < rows) out[(c0 + c) * out_stride + r0 + r] = tile[r * 66 + c];
    }
}

int grid_for(int64_t threads_needed) {
    int64_t blocks = (threads_needed + 255) / 256;
    const int64_t cap = 148 * 16;
    return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

cudaError_t router_topk(const float* logits, int num_tokens, int num_experts, int num_topk, int64_t* topk_idx, float* topk_weights,
                        cudaStream_t stream) {
    if (num_tokens == 0) return cudaSuccess;
    if (num_experts > 2048 || num_topk > 32 || num_topk > num_experts) return cudaErrorInvalidValue;
    const int blocks = (num_tokens * 32 + 255) / 256;
    const int per_lane = (num_experts + 31) / 32;
    if (per_lane <= 2) router_topk_kernel<2><<<blocks, 256, 0, stream>>>(logits, num_tokens, num_experts, num_topk, topk_idx, topk_weights);
    else if (per_lane <= 8) router_topk_kernel<8><<<blocks, 256, 0, stream>>>(logits, num_tokens, num_experts, num_topk, topk_idx, topk_weights);
    else if (per_lane <= 16) router_topk_kernel<16><<<blocks, 256, 0, stream>>>(logits, num_tokens, num_experts, num_topk, topk_idx, topk_weights);
    else router_topk_kernel<64><<<blocks, 256, 0, stream>>>(logits, num_tokens, num_experts, num_topk, topk_idx, topk_weights);
    return cudaGetLastError();
}

cudaError_t quant_1x128(const void* x, int64_t x_stride_bytes, int rows, int hidden, bool pow2, void* out, float* scales,
                        int64_t sf_row_stride, int64_t sf_col_stride, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    if (hidden % 128 != 0) return cudaErrorInvalidValue;
    quant_kernel<<<grid_for(static_cast<int64_t>(rows) * hidden / 8), 256, 0, stream>>>(
        static_cast<const uint8_t*>(x), x_stride_bytes, rows, hidden, pow2, static_cast<uint8_t*>(out), scales, sf_row_stride, sf_col_stride);
    return cudaGetLastError();
}

cudaError_t dequant_1x128(const void* q, const float* scales, int64_t sf_row_stride, int64_t sf_col_stride, int rows, int hidden, void* out,
                          cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    if (hidden % 128 != 0) return cudaErrorInvalidValue;
    dequant_kernel<<<grid_for(static_cast<int64_t>(rows) * hidden / 8), 256, 0, stream>>>(
        static_cast<const uint8_t*>(q), scales, sf_row_stride, sf_col_stride, rows, hidden, static_cast<uint8_t*>(out));
    return cudaGetLastError();
}

cudaError_t swiglu(const void* x, int rows, int inter, const float* row_weight, const int* num_valid_rows, void* out, bool quant,
                   float* scales, int64_t sf_row_stride, int64_t sf_col_stride, bool pow2, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    if (inter % 8 != 0 || (quant && inter % 128 != 0)) return cudaErrorInvalidValue;
    const int grid = grid_for(static_cast<int64_t>(rows) * inter / 8);
    if (quant)
        swiglu_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(x), rows, inter, row_weight, num_valid_rows,
                                                      static_cast<uint8_t*>(out), scales, sf_row_stride, sf_col_stride, pow2 ? 1 : 0);
    else
        swiglu_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(x), rows, inter, row_weight, num_valid_rows,
                                                       static_cast<uint8_t*>(out), nullptr, 0, 0, 0);
    return cudaGetLastError();
}

cudaError_t swiglu_backward(const void* x, const void* dout, int rows, int inter, const float* row_weight, void* dx, void* act_out,
                            float* dweight, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    if (inter % 8 != 0) return cudaErrorInvalidValue;
    swiglu_bwd_kernel<<<min(rows, 148 * 8), 256, 0, stream>>>(
        static_cast<const uint8_t*>(x), static_cast<const uint8_t*>(dout), rows, inter, row_weight, static_cast<uint8_t*>(dx),
        static_cast<uint8_t*>(act_out), dweight);
    return cudaGetLastError();
}

cudaError_t transpose_bf16(const void* in, int64_t in_stride, int rows, int cols, void* out, int64_t out_stride, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return cudaSuccess;
    dim3 grid((cols + 63) / 64, (rows + 63) / 64);
    const int aligned = in_stride % 8 == 0 && out_stride % 8 == 0 && reinterpret_cast<uintptr_t>(in) % 16 == 0 &&
                        reinterpret_cast<uintptr_t>(out) % 16 == 0;
    transpose_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(in), in_stride, rows, cols,
                                               static_cast<__nv_bfloat16*>(out), out_stride, aligned);
    return cudaGetLastError();
}

}  // namespace ops
}  // namespace ep
