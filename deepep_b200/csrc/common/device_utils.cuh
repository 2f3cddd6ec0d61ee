// Device-side primitives shared by every kernel of the library (sm_100a only).
//
// Everything that waits is bounded: a wait returns `false` after `timeout_ns`
// (or as soon as another waiter of the same kernel has given up), the caller
// records a status word that the host reads, and the kernel runs to its end.
// Nothing here traps, asserts or spins without a limit.
//
// Parity: plays the role of deep_ep/include/deep_ep/common/{ptx,comm}.cuh in
// the reference (inline PTX wrappers, timeout_while, gpu_barrier).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cstdint>

#include "layout.hpp"

namespace ep {

// ---------------------------------------------------------------- misc
__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ int warp_id() { return threadIdx.x >> 5; }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t lanemask_lt() {
    uint32_t m;
    asm volatile("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// ---------------------------------------------------------------- scoped loads / stores
__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t ld_relaxed_sys_u64(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t ld_acquire_gpu_u64(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u64(uint64_t* p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u64(uint64_t* p, uint64_t v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_gpu_u64(uint64_t* p, uint64_t v) {
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys_u64(uint64_t* p, uint64_t v) {
    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_gpu_s32(int* p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu_s32(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

__device__ __forceinline__ int atom_add_acq_rel_gpu_s32(int* p, int v) {
    int old;
    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}

__device__ __forceinline__ uint64_t atom_add_acq_rel_gpu_u64(uint64_t* p, uint64_t v) {
    uint64_t old;
    asm volatile("atom.add.acq_rel.gpu.global.u64 %0, [%1], %2;" : "=l"(old) : "l"(p), "l"(v) : "memory");
    return old;
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may start while its predecessor in the
// stream still runs: its blocks become resident once every block of the predecessor has called
// launch_dependents() (or exited). dependency_wait() then blocks until the predecessor has completed and its
// memory operations are visible. Both are no-ops in a kernel launched without the attribute.
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Routing entry i of a top-k index tensor that holds int64 or int32 values; anything outside [0, limit) is -1.
__device__ __forceinline__ int load_topk_idx(const void* base, bool idx32, int64_t i, int limit) {
    if (idx32) {
        const int v = reinterpret_cast<const int*>(base)[i];
        return (v >= 0 && v < limit) ? v : -1;
    }
    const int64_t v = reinterpret_cast<const int64_t*>(base)[i];
    return (v >= 0 && v < limit) ? static_cast<int>(v) : -1;
}

// 16-byte streaming accesses (read-once data: keep it out of L1).
__device__ __forceinline__ int4 ld_nc_int4(const void* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_nc_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_na_int4(void* p, const int4& v) {
    asm volatile("st.global.L1::no_allocate.v4.s32 [%0], {%1,%2,%3,%4};"
                 ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---------------------------------------------------------------- status / bounded waits
struct WaitCtx {
    uint64_t deadline_ns;   // absolute %globaltimer value after which waits give up
    uint64_t* poison;       // device word, non-zero once any wait of this rank has given up
    uint64_t* host_status;  // mapped host words: [0] = first failure record (0 = healthy)
    int rank;
};

__device__ __forceinline__ WaitCtx make_wait_ctx(const CommCtx& c) {
    WaitCtx w;
    w.deadline_ns = globaltimer_ns() + c.timeout_ns;
    w.poison = c.local_ws + kWsPoison;
    w.host_status = c.host_status;
    w.rank = c.rank;
    return w;
}

// Records the first failure of this rank: code | waiting rank | awaited peer | tag.
static __device__ __noinline__ void report_timeout(const WaitCtx& w, int code, int peer, uint32_t tag) {
    const uint64_t rec = (static_cast<uint64_t>(code & 0xff) << 56) | (static_cast<uint64_t>(w.rank & 0xfff) << 44) |
                         (static_cast<uint64_t>(peer & 0xfff) << 32) | tag;
    atomicCAS(reinterpret_cast<unsigned long long*>(w.host_status), 0ull, static_cast<unsigned long long>(rec));
    atomicExch(reinterpret_cast<unsigned long long*>(w.poison), 1ull);
    __threadfence_system();
}

// Spins until pred() holds. Returns false on timeout (after recording it) or
// when the rank is already poisoned by an earlier failed wait.
template <typename Pred>
__device__ __forceinline__ bool bounded_wait(const WaitCtx& w, int code, int peer, uint32_t tag, Pred pred) {
    if (pred()) return true;
    uint32_t spins = 0;
    while (true) {
        if (pred()) return true;
        if ((++spins & 63u) == 0) {
            if (*reinterpret_cast<volatile uint64_t*>(w.poison) != 0) return false;
            if (globaltimer_ns() > w.deadline_ns) {
                report_timeout(w, code, peer, tag);
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(const WaitCtx& w, uint64_t* bar, uint32_t parity, int code, uint32_t tag) {
    return bounded_wait(w, code, -1, tag, [&]() { return mbar_try_wait(bar, parity); });
}

// ---------------------------------------------------------------- bulk async copies (1-D TMA, never multicast)
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Source smem of all committed groups has been read (buffers may be reused).
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// All but the N most recent committed groups have completed, their writes included.
template <int N>
__device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
// All committed groups have completed, their writes included.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Orders generic-proxy writes to shared memory before later async-proxy reads of it.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// ---------------------------------------------------------------- grid-wide barrier among the blocks of one rank
// `counter` only ever grows; the host passes the value it had before the launch
// and the n-th barrier of the launch waits for base + n * num_blocks.
// The kernel must be launched cooperatively so that all blocks are resident.
__device__ __forceinline__ bool grid_barrier(const WaitCtx& w, uint64_t* counter, uint64_t target, uint32_t tag) {
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) {
        red_add_release_gpu_u64(counter, 1);
        ok = bounded_wait(w, kStatusGridBarrier, -1, tag, [&]() { return ld_acquire_gpu_u64(counter) >= target; });
    }
    __syncthreads();
    return ok;
}

// ---------------------------------------------------------------- epoch-tagged words
// A control word carries (epoch << 32 | value): a reader that sees the epoch it
// expects also sees the value, so no separate flag or fence is needed and the
// words never have to be cleared.
__device__ __forceinline__ uint64_t pack_epoch(uint32_t epoch, uint32_t value) {
    return (static_cast<uint64_t>(epoch) << 32) | value;
}
__device__ __forceinline__ bool epoch_matches(uint64_t word, uint32_t epoch) { return static_cast<uint32_t>(word >> 32) == epoch; }
__device__ __forceinline__ bool epoch_reached(uint64_t word, uint32_t epoch) { return static_cast<uint32_t>(word >> 32) >= epoch; }

// ---------------------------------------------------------------- warp reductions
__device__ __forceinline__ float warp_reduce_max_width(float v, int width) {
    for (int o = width >> 1; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_reduce_sum(int v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------- FP8 (e4m3, 1x128 block scales)
constexpr float kFP8Max = 448.0f;
constexpr float kFP8AmaxFloor = 1e-4f;

// Scale such that x / scale fits e4m3; `inv` is what the payload is multiplied with.
__device__ __forceinline__ void fp8_scale_from_amax(float amax, bool round_pow2, float& scale, float& inv) {
    amax = fmaxf(amax, kFP8AmaxFloor);
    if (round_pow2) {
        // scale = 2^ceil(log2(amax / 448)), exactly representable as UE8M0
        const float raw = amax / kFP8Max;
        int e;
        const float m = frexpf(raw, &e);  // raw = m * 2^e, m in [0.5, 1)
        const int ce = (m == 0.5f) ? e - 1 : e;
        scale = ldexpf(1.0f, ce);
        inv = ldexpf(1.0f, -ce);
    } else {
        // one correctly rounded reciprocal and two multiplications (the PyTorch restatement in
        // utils/math.py does exactly the same, so kernel and reference agree bit for bit)
        scale = amax * (1.0f / kFP8Max);
        inv = kFP8Max * __frcp_rn(amax);
    }
}

// max |x| over the eight bf16 values of a 16-byte vector, computed with packed bf16 min/max (exact)
__device__ __forceinline__ float amax_bf16x8(const int4& raw) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    __nv_bfloat162 m = __hmax2(__habs2(h2[0]), __habs2(h2[1]));
    m = __hmax2(m, __hmax2(__habs2(h2[2]), __habs2(h2[3])));
    const float2 f = __bfloat1622float2(m);
    return fmaxf(f.x, f.y);
}

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

}  // namespace ep
