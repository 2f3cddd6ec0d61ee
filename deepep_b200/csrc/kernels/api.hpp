// Launch interface between the host runtime and the CUDA kernels. No torch types here:
// every launcher takes plain parameter blocks and a stream, so that the kernels compile
// in seconds and can also be driven from C (ctypes) or from the run-time compiler.
//
// Parity: csrc/kernels/elastic/{barrier,dispatch,combine}.hpp and the host wrappers at the
// bottom of csrc/kernels/legacy/*.cu in the reference.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

#include "../common/layout.hpp"

namespace ep {

// Shared-memory set-up of a kernel before its launch: the dynamic shared memory it may use, and the largest
// shared-memory carve-out as the preferred one. All communication kernels ask for the same carve-out, whatever they
// use: an SM has to drain and reconfigure when consecutive kernels prefer different ones, which costs microseconds
// between the back-to-back kernels of a dispatch / combine step.
template <typename Kernel>
inline cudaError_t prepare_kernel(Kernel kernel, int dynamic_smem_bytes) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dynamic_smem_bytes);
    if (err != cudaSuccess) return err;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

// ---------------------------------------------------------------- cross-rank barrier
struct BarrierParams {
    CommCtx c;
    uint32_t epoch;
};
cudaError_t launch_barrier(const Multi<BarrierParams>& m, cudaStream_t stream);

// ---------------------------------------------------------------- high-throughput dispatch
enum QuantMode : int {
    kQuantNone = 0,        // payload rows are sent as they are (bf16, or fp8 with caller-made scales)
    kQuantE4M3 = 1,        // bf16 in, e4m3 + float 1x128 scales out (made in the kernel)
    kQuantE4M3Pow2 = 2,    // same with power-of-two scales
};

struct DispatchParams {
    CommCtx c;
    // problem
    int num_tokens;
    int num_topk;
    int num_experts;
    int num_local_experts;
    int num_max_tokens;     // per-rank upper bound, equal on all ranks
    int src_row_bytes;      // bytes of one input row
    int x_row_bytes;        // bytes of one payload row as it is sent and received
    int sf_bytes;           // bytes of scale factors per token (0 = none)
    int meta_bytes;         // bytes of the record's meta part (ht_meta_bytes)
    int rec_pitch;          // bytes between records of the receive region (multiple of 128)
    int quant_mode;
    int expert_alignment;
    int do_expand;          // expert prefix sums follow the expanded layout
    int cached;             // reuse token_slot / pair_row of an earlier dispatch, no counting
    int idx32;              // topk_idx holds int32 (else int64)
    int smem_scratch_bytes; // dynamic shared memory after the header (filled in by the launcher)
    // inputs
    const uint8_t* x;
    int64_t x_stride_bytes;
    const uint8_t* sf;          // 4-byte packs, [tokens][packs] with the strides below (in packs)
    int64_t sf_token_stride;
    int64_t sf_pack_stride;
    const void* topk_idx;       // [T, K] int64 or int32, -1 = unused lane
    const float* topk_weights;  // [T, K] or null
    // handle tensors (device, owned by the caller)
    int* token_slot;        // [T, R]  row in the destination rank's receive region, -1 = not sent
    int* pair_row;          // [T, K]  row in the destination rank's expanded (expert-major) layout
    int* psum_rank;         // [R]     inclusive prefix of received tokens per source rank
    int* psum_expert;       // [E_local + 1]
    int* num_unaligned;     // [E_local] received (token, expert) pairs per local expert
    int* recv_stats;        // [E_local] cumulative statistics or null
    int* count_matrix;      // [R, R] tokens that rank i sends to rank j (every rank sees the whole matrix), or null
    // heap
    uint64_t off_recv;      // receive region (records) of this call's parity
    uint32_t epoch;
    uint64_t grid_bar_base;
    uint64_t* host_counts;  // mapped pinned: [0] received tokens, [1] expanded rows, [2 + e] per local expert (aligned)
};

struct DispatchLaunch {
    int num_sms;            // blocks per rank
    int num_warps;          // send warps per block
    int smem_bytes;
    int scratch_bytes;      // smem_bytes minus the header
};
// Picks warps / shared memory for a dispatch of this shape. Returns false if a row (or the routing
// scratch of the ordering pass) does not fit.
bool plan_dispatch(const DispatchParams& p, int num_sms, int smem_optin, DispatchLaunch* out);
cudaError_t launch_dispatch(const Multi<DispatchParams>& m, const DispatchLaunch& l, cudaStream_t stream);

struct DispatchEpilogueParams {
    // receive side of one rank
    CommCtx c;               // for the bounded wait on the peers' completion words
    uint32_t epoch;          // of the dispatch whose records are unpacked
    int wait_done;           // 1: wait until every peer has reported its rows of `epoch` as landed
    int num_ranks;
    int num_topk;
    int num_local_experts;
    int num_max_tokens;
    int x_row_bytes;
    int sf_bytes;
    int rec_pitch;
    int do_expand;
    int copy_x;              // 0: recv_x aliases the receive region (zero copy), rows are not moved
    int expert_alignment;
    int do_zero_padding;
    int write_metadata;      // 0 for cached dispatches (metadata is reused)
    int idx32;               // recv_topk_idx holds int32 (else int64)
    const uint8_t* region;   // records
    const int* psum_rank;    // [R] inclusive; [R-1] = number of received rows
    const int* psum_expert;  // [E_local + 1]
    const int* num_unaligned;
    // outputs
    uint8_t* recv_x;          // [rows, x_row_bytes]
    uint8_t* recv_sf;         // packs of 4 bytes, or null (none, or the caller reads them in place)
    int64_t recv_sf_row_stride, recv_sf_pack_stride;   // in packs
    void* recv_topk_idx;      // [num_idx_rows, K] (non-expand) or null
    float* recv_topk_weights; // [num_idx_rows, K] or [rows] (expand) or null
    int* recv_src_metadata;   // [num_idx_rows, K + 2]
    int num_out_rows;         // capacity of recv_x in rows (expand: expanded rows)
    int num_idx_rows;         // rows of the routing outputs; rows past the received count are filled with -1 / 0
};
cudaError_t launch_dispatch_epilogue(const DispatchEpilogueParams* params, int num_vranks, int num_sms, int smem_optin,
                                     cudaStream_t stream, bool programmatic = false);

// ---------------------------------------------------------------- high-throughput combine
struct CombineEpilogueParams {
    int num_tokens;
    int num_topk;
    int num_ranks;
    int num_local_experts;
    int num_max_tokens;
    int hidden;               // bf16 elements
    int num_lanes;
    int use_rank_layout;
    int idx32;                // topk_idx holds int32 (else int64)
    int weighted;             // top-k layout only: row k is multiplied by its top-k weight (region_w) before it is added
    const uint8_t* region_x;
    const float* region_w;    // [lanes][T_max][K] or null
    const void* topk_idx;     // [T, K] the dispatch's routing
    const uint8_t* bias0;
    const uint8_t* bias1;
    uint8_t* combined_x;              // [T, hidden] bf16
    float* combined_topk_weights;     // [T, K] or null
    // Arrival-driven mode (arrivals != null): the kernel runs beside the send kernel and sums a token as soon as the
    // arrival counters of all its rows are full; every wait is bounded through `c`.
    CommCtx c;
    uint32_t epoch;
    const uint32_t* arrivals; // [R][flag_chunks] rows-landed counters of this combine's parity in this rank's heap, or null
    int flag_chunks;
    const int* dst_slot;      // [T, R] row of each of this rank's tokens in every destination's receive order (-1 = none)
    const int* count_matrix;  // [R, R] tokens rank i dispatched to rank j (arrival-driven mode)
    uint64_t* local_ws;       // private workspace (kernel timeline)
};
struct CombineParams {
    CommCtx c;
    int num_topk;
    int num_max_tokens;
    int row_bytes;            // hidden * 2 (bf16)
    int do_expand;
    int num_lanes;            // rows per token in the receive region (ranks, or top-k)
    int use_rank_layout;      // 1: lane = sending rank (pre-reduced), 0: lane = top-k slot
    int weighted;             // expanded input: rows are multiplied by their top-k weight (rank layout: in the pre-reduce)
    const uint8_t* x;         // [N or expanded rows, hidden] bf16
    int64_t x_stride_bytes;
    const float* topk_weights;   // non-expand [N, K]; expand [rows]; or null
    const int* recv_src_metadata;   // [N, K + 2]
    const int* psum_rank;     // [R] inclusive (device truth for N)
    uint64_t off_comb_x;
    uint64_t off_comb_w;
    uint32_t epoch;
    uint64_t grid_bar_base;
    // fuse_reduce != 0: every landed row is counted in the receiver's heap (one counter per sender and per
    // `kCombineFlagRows` consecutive rows of what the sender holds for that receiver); a reduce kernel launched right
    // behind this one (programmatic dependent launch, on the SMs this kernel leaves free) sums tokens as their
    // counters fill up.
    int fuse_reduce;
    int num_send_warps;       // warps of a block (one staging buffer each); filled in by the launcher
    int num_send_blocks;      // blocks of the grid
    int direct_out;           // single rank, no bias, one row per token: rows go straight to red.combined_x, no reduce
    int flag_chunks;          // counters per source rank = ceil(ranks * max tokens / kCombineFlagRows)
    uint64_t off_comb_flag;   // [2 parities][R][flag_chunks] uint32 rows-landed counters
    CombineEpilogueParams red;
};
struct CombineLaunch {
    int num_sms;
    int num_warps;            // send warps (one staging buffer each)
    int smem_bytes;
};
bool plan_combine(const CombineParams& p, int num_sms, int smem_optin, CombineLaunch* out);
cudaError_t launch_combine(const Multi<CombineParams>& m, const CombineLaunch& l, cudaStream_t stream);

// `programmatic`: launched as a programmatic dependent of the kernel before it in the stream (the send kernel).
cudaError_t launch_combine_epilogue(const CombineEpilogueParams* params, int num_vranks, int num_sms, cudaStream_t stream,
                                    bool programmatic = false);

// ---------------------------------------------------------------- layout (legacy get_dispatch_layout)
cudaError_t launch_dispatch_layout(const void* topk_idx, bool idx32, int num_tokens, int num_topk, int num_ranks, int num_experts,
                                   int* num_tokens_per_rank, int* num_tokens_per_expert, bool* is_token_in_rank,
                                   cudaStream_t stream);

// ---------------------------------------------------------------- low-latency dispatch / combine
enum LLPhase : int { kLLSend = 1, kLLRecv = 2 };

struct LLDispatchParams {
    CommCtx c;
    int num_tokens, hidden, num_topk, num_experts, num_local_experts, num_max_tokens;
    int use_fp8, round_scale, use_ue8m0;
    int phases;
    int shrink;                      // a peer that does not answer in time is masked instead of reported
    const uint8_t* x;                // [T, hidden] bf16
    const void* topk_idx;            // [T, K] int64 or int32
    int idx32;                       // topk_idx holds int32
    uint8_t* packed_recv_x;          // [EL][R * T_max][hidden] e4m3 or bf16
    uint8_t* packed_recv_sf;         // float [EL][hidden / 128][R * T_max] or int32 [EL][hidden / 512][R * T_max]
    int* packed_recv_src_info;       // [EL][R * T_max]  token | lane << 16
    int64_t* packed_recv_layout_range;   // [EL][R]  begin << 32 | count
    int* packed_recv_count;          // [EL]
    int* cumulative_stats;           // [EL] or null
    int64_t* wait_stats;             // [R] accumulated wait time per source rank (ns) or null
    uint64_t off_recv_x[2], off_recv_count[2];
};
cudaError_t launch_ll_dispatch(const Multi<LLDispatchParams>& m, int num_sms, cudaStream_t stream);

struct LLCombineParams {
    CommCtx c;
    int num_tokens, hidden, num_topk, num_experts, num_local_experts, num_max_tokens;
    int phases;
    int shrink;
    int use_logfmt;                  // rows travel in the 10-bit log format where a group of 128 channels allows it
    const uint8_t* x;                // [EL][R * T_max][hidden] bf16
    const void* topk_idx;            // [T, K] routing of the tokens this rank dispatched, int64 or int32
    int idx32;                       // topk_idx holds int32
    const float* topk_weights;       // [T, K]
    const int* src_info;             // handle
    const int64_t* layout_range;     // handle
    uint8_t* combined_x;             // [T, hidden] bf16
    int64_t* wait_stats;             // [R] or null
    uint64_t off_combine_x[2], off_combine_flag[2];
};
cudaError_t launch_ll_combine(const Multi<LLCombineParams>& m, int num_sms, int smem_optin, cudaStream_t stream);

// rank mask (shrink mode) kept in the private workspace
cudaError_t ll_update_mask(uint64_t* local_ws, int rank, int value, cudaStream_t stream);
cudaError_t ll_query_mask(uint64_t* local_ws, int* out, int num_ranks, cudaStream_t stream);

}  // namespace ep
