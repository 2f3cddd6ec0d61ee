// tcgen05 / TMEM GEMM core for sm_100a, written for fusion with the collectives of this library.
//
//   C[M, N] (bf16) = A[M, K] * B[g][N, K]^T        A, B K-major (row-major with K innermost)
//
// One persistent CTA per SM, warp-specialised:
//   warp 0        TMA producer: cp.async.bulk.tensor 2-D tiles (128B swizzle) of A (BM x BK) and
//                 B (BN x BK) into a ring of shared-memory stages; never multicast
//   warp 1        MMA issuer: one elected lane issues tcgen05.mma (M=128, N=BN, K=16 for bf16 /
//                 K=32 for e4m3) with the accumulator in tensor memory, tcgen05.commit releases the
//                 stage and, after the last k-block, hands the accumulator to the epilogue
//   warps 2..5    epilogue: tcgen05.ld (32 lanes x 32 columns per instruction), convert, store.
// Two accumulators (2 x BN columns of TMEM) let the epilogue of tile i overlap the main loop of
// tile i+1. With FP8 inputs every 128-wide k-block gets its own accumulator pass and the epilogue
// warps apply the 1x128 (A) and 128x128 (B) scales in fp32 registers (software block scaling).
//
// Fusion hooks (see gemm_sm100.cu):
//   * grouped: rows are segmented by `group_end` (device array, the expanded layout of dispatch);
//     group g multiplies with weight matrix g;
//   * a_ready: before loading the A rows of row-chunk c the producer waits (bounded) for a flag
//     that the all-gather part of the same kernel sets when the chunk has landed locally;
//   * the epilogue can store the tile into a peer's memory and raise a per-tile flag
//     (reduce-scatter), or apply SwiGLU to interleaved gate/up columns.
//
// Every wait is bounded; a wait that runs out sets `*error`, all roles leave their loops, tensor
// memory is released and the kernel returns.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "../common/device_utils.cuh"

namespace ep {
namespace gemm {

constexpr int BM = 128;
constexpr int kNumEpilogueWarps = 4;
constexpr int kNumThreads = (2 + kNumEpilogueWarps) * 32;

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]
template <bool kFp8>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if constexpr (kFp8) {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    }
}
// the mbarrier is signalled when all tcgen05.mma issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 16 consecutive 32-bit columns of this thread's tensor-memory lane (lane = 32 * (warp % 4) + lane id)
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= (A[smem] * 2^(sfa - 127)) * (B[smem] * 2^(sfb - 127)): e4m3 operands with one UE8M0 scale factor per row
// (column) and 32 elements of K, read from tensor memory by the tensor core itself. The scale factors of the 128 rows of
// A occupy four 32-bit columns: in every lane quarter, lane r holds in column j the factors of row r + 32 j, one byte
// per 32-wide slice of a 128-wide k-block (the byte is picked by the id fields of the instruction descriptor); those of
// 256 columns of B occupy eight columns in the same arrangement.
__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate,
                                        uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n" ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}
// the CTA-pair form: M = 256 (128 rows per CTA), the scale factors of a CTA's own rows of A and of all columns of B are
// read from that CTA's tensor memory at the same addresses
__device__ __forceinline__ void umma_mx_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate,
                                             uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n" ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}
// Instruction descriptor of the block-scaled kind: A / B e4m3 K-major, scale factors UE8M0, D fp32 (implied).
// `sf_id` = which byte of a scale-factor column (which 32-wide slice of the 128-wide k-block) both operands use.
__host__ __device__ constexpr uint32_t make_idesc_mx(int m, int n, uint32_t sf_id) {
    uint32_t d = 0;
    d |= (sf_id & 3u) << 4;                         // B scale-factor id
    d |= static_cast<uint32_t>(n >> 3) << 17;       // N / 8
    d |= 1u << 23;                                  // scale format: E8M0
    d |= static_cast<uint32_t>(m >> 4) << 24;       // M / 16
    d |= (sf_id & 3u) << 29;                        // A scale-factor id
    return d;
}

// ---------------------------------------------------------------- CTA-pair (cta_group::2) forms
// Two CTAs of a cluster work on one 256-row tile: each holds its own 128 rows of A, half of the B tile and the
// accumulator rows of its half in tensor memory. The even CTA (the leader) issues the MMAs for both. Loads are
// plain per-CTA TMA copies (never multicast) that report to the LEADER's barrier.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of the same shared-memory object in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
    return out;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// the same without release semantics: for a signal whose payload is already complete by other means (tensor-memory
// stores behind tcgen05.wait::st). A release at cluster scope was measured at about a microsecond per arrival, which
// is a whole k-block of an e4m3 tile.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// dst in this CTA's shared memory, completion bytes reported to the barrier at `bar_cluster_addr` (the leader's)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_pair_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_pair_fp8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor of a K-major tile whose rows are exactly one 128-byte swizzle
// span (BK * element size == 128): 8-row groups are 1024 bytes apart, version 1, SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_smem_desc(const void* smem_tile) {
    const uint32_t addr = smem_u32(smem_tile);
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((addr & 0x3ffff) >> 4);          // start address, bits [0, 14)
    desc |= static_cast<uint64_t>(0) << 16;                        // leading byte offset (unused for swizzled K-major)
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;                // stride byte offset, bits [32, 46)
    desc |= static_cast<uint64_t>(1) << 46;                        // descriptor version of sm_100
    desc |= static_cast<uint64_t>(2) << 61;                        // SWIZZLE_128B
    return desc;
}

// Instruction descriptor: D fp32, A/B bf16 (kind::f16) or e4m3 (kind::f8f6f4), both K-major.
template <bool kFp8>
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    uint32_t d = 0;
    d |= 1u << 4;                                   // D format: F32
    d |= (kFp8 ? 0u : 1u) << 7;                     // A format: E4M3 (0) / BF16 (1)
    d |= (kFp8 ? 0u : 1u) << 10;                    // B format
    d |= static_cast<uint32_t>(n >> 3) << 17;       // N / 8
    d |= static_cast<uint32_t>(m >> 4) << 24;       // M / 16
    return d;
}

// ---------------------------------------------------------------- bounded mbarrier wait shared by the roles
struct PipeCtx {
    int* error;             // global, non-zero once any role has given up
    uint64_t deadline_ns;
};
__device__ __forceinline__ bool pipe_wait(const PipeCtx& pc, uint64_t* bar, uint32_t parity) {
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0) {
            if (*reinterpret_cast<volatile int*>(pc.error) != 0) return false;
            if (globaltimer_ns() > pc.deadline_ns) {
                atomicExch(pc.error, static_cast<int>(kStatusGemmPipe));
                return false;
            }
        }
    }
    return true;
}

}  // namespace gemm
}  // namespace ep
