// Cross-rank GPU barrier over NVLink: every rank stores its epoch into a word of each
// peer's control area and waits (bounded) until all of its own words carry the epoch.
// Words are epoch-tagged and never cleared, so back-to-back barriers need no reset.
//
// Parity: deep_ep/include/deep_ep/impls/barrier.cuh:16-40 and the NVLink half of
// common/comm.cuh:88-129 in the reference (which flips a phase counter with red.add).
#include "api.hpp"
#include "../common/device_utils.cuh"

namespace ep {

__global__ void __launch_bounds__(32, 1) barrier_kernel(const __grid_constant__ Multi<BarrierParams> m) {
    const BarrierParams& p = m.r[blockIdx.x / m.blocks_per_rank];
    const CommCtx& c = p.c;
    const WaitCtx w = make_wait_ctx(c);
    const int lane = lane_id();
    // Make everything this rank wrote before the barrier visible to the peers first.
    fence_acq_rel_sys();
    if (lane < c.num_ranks) {
        uint64_t* remote = reinterpret_cast<uint64_t*>(c.heap[lane]) + kCtlBarrier + c.rank;
        st_release_sys_u64(remote, pack_epoch(p.epoch, 0));
        const uint64_t* mine = reinterpret_cast<const uint64_t*>(c.heap[c.rank]) + kCtlBarrier + lane;
        bounded_wait(w, kStatusBarrierPeer, lane, p.epoch, [&]() { return epoch_reached(ld_acquire_sys_u64(mine), p.epoch); });
    }
    __syncwarp();
}

cudaError_t launch_barrier(const Multi<BarrierParams>& m, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(m.num_vranks * m.blocks_per_rank);
    cfg.blockDim = dim3(32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, barrier_kernel, m);
}

}  // namespace ep
