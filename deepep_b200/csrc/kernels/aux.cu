// Auxiliary primitives (sm_100a): the flag wait / signal kernel behind AGRS sessions and the PP
// slot rings (payload on the copy engines, this 1-block kernel for ordering), the slot reduction
// of the reduce-scatter primitive, and the Engram gather that pulls table rows from peer memory
// with plain (non-multicast) bulk loads.
//
// Parity: csrc/kernels/backend/cuda_driver.cu:12-52 (stream batch mem-ops) and
// deep_ep/include/deep_ep/impls/{engram_fetch,pp_send_recv}.cuh of the reference.
#include "aux_api.hpp"
#include "../common/device_utils.cuh"

namespace ep {
namespace aux {

namespace {

struct FlagOps {
    int num_ops;
    FlagOp op[kMaxVRanks];
};

__global__ void __launch_bounds__(32) flag_kernel(const __grid_constant__ FlagOps ops) {
    const FlagOp& o = ops.op[blockIdx.x];
    const WaitCtx w = make_wait_ctx(o.c);
    const int lane = lane_id();
    if (o.signal_first) {
        fence_acq_rel_sys();
        if (lane < o.num_signal) st_release_sys_u64(o.signal_ptrs[lane], o.signal_value);
    }
    if (lane < o.num_wait) {
        const uint64_t* ptr = o.wait_ptrs[lane];
        bounded_wait(w, o.status_code, lane, static_cast<uint32_t>(o.wait_value), [&]() { return ld_acquire_sys_u64(ptr) >= o.wait_value; });
    }
    __syncwarp();
    if (!o.signal_first) {
        fence_acq_rel_sys();
        if (lane < o.num_signal) st_release_sys_u64(o.signal_ptrs[lane], o.signal_value);
    }
}

template <bool kBf16>
__global__ void __launch_bounds__(256) reduce_slots_kernel(const uint8_t* __restrict__ slots, int64_t slot_stride, int num_slots,
                                                           uint8_t* __restrict__ out, int64_t num_vec) {
    for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < num_vec; v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        if constexpr (kBf16) {
            float acc[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.f;
            for (int s = 0; s < num_slots; ++s) {
                const int4 raw = ld_nc_int4(slots + s * slot_stride + v * 16);
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(h2[i]);
                    acc[2 * i] += f.x;
                    acc[2 * i + 1] += f.y;
                }
            }
            int4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            *reinterpret_cast<int4*>(out + v * 16) = o;
        } else {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < num_slots; ++s) {
                const int4 raw = ld_nc_int4(slots + s * slot_stride + v * 16);
                acc.x += __int_as_float(raw.x);
                acc.y += __int_as_float(raw.y);
                acc.z += __int_as_float(raw.z);
                acc.w += __int_as_float(raw.w);
            }
            *reinterpret_cast<float4*>(out + v * 16) = acc;
        }
    }
}

__global__ void __launch_bounds__(1024, 1) engram_kernel(const __grid_constant__ Multi<EngramParams> m) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int vr = blockIdx.x / m.blocks_per_rank;
    const int bid = blockIdx.x % m.blocks_per_rank, nb = m.blocks_per_rank;
    const EngramParams& p = m.r[vr];
    const CommCtx& c = p.c;
    const WaitCtx w = make_wait_ctx(c);
    const int lane = lane_id(), warp = warp_id(), num_warps = blockDim.x >> 5;
    const int stage = align_up(p.row_bytes, 128) + 16;
    uint8_t* buf = smem + static_cast<size_t>(warp) * stage;
    uint64_t* bar = reinterpret_cast<uint64_t*>(buf + align_up(p.row_bytes, 128));
    if (lane == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    __syncwarp();
    uint32_t parity = 0;
    for (int i = bid * num_warps + warp; i < p.num_indices; i += nb * num_warps) {
        const int e = p.indices[i];
        const int owner = e / p.entries_per_rank, row = e % p.entries_per_rank;
        const bool valid = e >= 0 && owner < c.num_ranks;
        bulk_wait_read_all();
        __syncwarp();
        if (valid && p.table_on_host) {
            // host segment: sixteen bytes per lane and load, eight loads in flight, straight to the output
            const uint8_t* src = p.table[owner] + static_cast<uint64_t>(row) * p.row_bytes;
            uint8_t* dst = p.out + static_cast<uint64_t>(i) * p.row_bytes;
            const int vecs = p.row_bytes / 16;
            for (int v = lane; v < vecs; v += 256) {
                int4 raw[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (v + 32 * j < vecs) raw[j] = ld_nc_int4(src + (v + 32 * j) * 16);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (v + 32 * j < vecs) *reinterpret_cast<int4*>(dst + (v + 32 * j) * 16) = raw[j];
            }
            if (p.sf_table != nullptr) {
                const int token = i / p.entries_per_token, slot = i % p.entries_per_token;
                for (int k = lane; k < p.sf_packs; k += 32)
                    p.out_sf[token * p.out_sf_token_stride + (slot * p.sf_packs + k) * p.out_sf_pack_stride] =
                        p.sf_table[static_cast<int64_t>(e) * p.sf_packs + k];
            }
        } else if (valid) {
            if (lane == 0) {
                mbar_arrive_expect_tx(bar, p.row_bytes);
                bulk_g2s(buf, p.table[owner] + static_cast<uint64_t>(row) * p.row_bytes, p.row_bytes, bar);
            }
            if (p.sf_table != nullptr) {
                const int token = i / p.entries_per_token, slot = i % p.entries_per_token;
                for (int k = lane; k < p.sf_packs; k += 32)
                    p.out_sf[token * p.out_sf_token_stride + (slot * p.sf_packs + k) * p.out_sf_pack_stride] =
                        p.sf_table[static_cast<int64_t>(e) * p.sf_packs + k];
            }
            const bool landed = mbar_wait(w, bar, parity, kStatusTmaLoad, i);
            parity ^= 1;
            if (!__all_sync(0xffffffffu, landed)) break;
            if (lane == 0) {
                bulk_s2g(p.out + static_cast<uint64_t>(i) * p.row_bytes, buf, p.row_bytes);
                bulk_commit();
            }
        }
    }
    bulk_wait_all();
}

}  // namespace

cudaError_t launch_flag_op(const FlagOp* ops, int num_ops, cudaStream_t stream) {
    if (num_ops < 1 || num_ops > kMaxVRanks) return cudaErrorInvalidValue;
    FlagOps all;
    all.num_ops = num_ops;
    for (int i = 0; i < num_ops; ++i) all.op[i] = ops[i];
    void* args[] = {&all};
    // cooperative: with several virtual ranks the blocks wait on one another
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(flag_kernel), dim3(num_ops), dim3(32), args, 0, stream);
}

cudaError_t launch_reduce_slots(const void* slots, int64_t slot_stride_bytes, int num_slots, void* out, int64_t num_elems, bool is_bf16,
                                cudaStream_t stream) {
    const int64_t bytes = num_elems * (is_bf16 ? 2 : 4);
    if (bytes % 16 != 0 || slot_stride_bytes % 16 != 0) return cudaErrorInvalidValue;
    if (bytes == 0) return cudaSuccess;
    const int64_t num_vec = bytes / 16;
    int blocks = static_cast<int>((num_vec + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (is_bf16)
        reduce_slots_kernel<true><<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(slots), slot_stride_bytes, num_slots, static_cast<uint8_t*>(out), num_vec);
    else
        reduce_slots_kernel<false><<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(slots), slot_stride_bytes, num_slots, static_cast<uint8_t*>(out), num_vec);
    return cudaGetLastError();
}

cudaError_t launch_engram_gather(const EngramParams* params, int num_vranks, int num_sms, int smem_optin, cudaStream_t stream) {
    Multi<EngramParams> m;
    m.num_vranks = num_vranks;
    m.blocks_per_rank = num_sms;
    for (int v = 0; v < num_vranks; ++v) m.r[v] = params[v];
    const int stage = align_up(params[0].row_bytes, 128) + 16;
    int warps = smem_optin / stage;
    if (warps > 32) warps = 32;
    if (warps < 1 || params[0].row_bytes % 16 != 0) return cudaErrorInvalidValue;
    const int smem_bytes = warps * stage;
    cudaError_t err = cudaFuncSetAttribute(engram_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (err != cudaSuccess) return err;
    engram_kernel<<<num_vranks * num_sms, warps * 32, smem_bytes, stream>>>(m);
    return cudaGetLastError();
}

}  // namespace aux
}  // namespace ep
