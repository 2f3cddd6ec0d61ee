// Launch interface of the auxiliary primitives: flag wait / signal (AGRS sessions and PP slot
// rings, whose payload moves on the copy engines), slot reduction (reduce-scatter) and the
// Engram table gather.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

#include "../common/layout.hpp"

namespace ep {
namespace aux {

// One tiny kernel: wait (bounded) until `num_wait` words are >= `wait_value` and store `signal_value`
// (release, system scope) into `num_signal` words, in the order given by `signal_first`.
struct FlagOp {
    CommCtx c;
    const uint64_t* wait_ptrs[kMaxRanks];
    int num_wait;
    uint64_t wait_value;
    uint64_t* signal_ptrs[kMaxRanks];
    int num_signal;
    uint64_t signal_value;
    int status_code;
    int signal_first;   // 1: publish, then wait (arrival rounds); 0: wait, then publish
};
cudaError_t launch_flag_op(const FlagOp* ops, int num_ops, cudaStream_t stream);

// out[i] = sum over s of slots[s][i] (fp32 accumulation in slot order); bf16 or fp32 elements
cudaError_t launch_reduce_slots(const void* slots, int64_t slot_stride_bytes, int num_slots, void* out, int64_t num_elems, bool is_bf16,
                                cudaStream_t stream);

// rows[i] = table row indices[i]: entry e lives on rank e / entries_per_rank, row e % entries_per_rank of that rank's
// heap at `off_table`; every row is `row_bytes` long (multiple of 16). Rows are read from peer memory over NVLink.
struct EngramParams {
    CommCtx c;
    const int* indices;
    int num_indices;
    int entries_per_rank;
    int row_bytes;
    const uint8_t* table[kMaxRanks];   // rank r's shard as this rank's kernels address it: heap[r] + offset, or r's host segment
    int table_on_host;                 // the shards are pinned host memory: fetched with plain loads over PCIe
    uint8_t* out;
    // optional replicated scale table (local memory): sf_packs 4-byte packs per entry
    const uint32_t* sf_table;
    int sf_packs;
    uint32_t* out_sf;
    int64_t out_sf_token_stride, out_sf_pack_stride;   // in packs; a token owns entries_per_token consecutive indices
    int entries_per_token;
};
cudaError_t launch_engram_gather(const EngramParams* params, int num_vranks, int num_sms, int smem_optin, cudaStream_t stream);

}  // namespace aux
}  // namespace ep
