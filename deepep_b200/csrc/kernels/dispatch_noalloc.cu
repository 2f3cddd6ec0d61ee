// Single-GPU token dispatch for callers that cannot allocate device memory
// (declaration and contract: dispatch_noalloc.h). This entry point has no counterpart in
// the reference library.
//
// It runs the same dispatch kernel and the same local epilogue as the regular path
// (dispatch_ht.cu) with a world of one rank. Everything those kernels need beyond the
// caller's inputs and outputs -- the control words, the receive region, the private
// workspace, the routing tables and the status words -- is carved from ONE file-scope
// device array, so no call here reaches cudaMalloc, cudaFree, cudaHostAlloc or any
// allocating library routine.
#include "dispatch_noalloc.h"

#include <mutex>

#include "api.hpp"

namespace {

using namespace ep;

constexpr size_t kMaxTokens = DEEPEP_B200_NOALLOC_MAX_TOKENS;
constexpr size_t kMaxRowBytes = DEEPEP_B200_NOALLOC_MAX_ROW_BYTES;
constexpr size_t kMaxTopkNA = DEEPEP_B200_NOALLOC_MAX_TOPK;
constexpr size_t kMaxExpertsNA = DEEPEP_B200_NOALLOC_MAX_EXPERTS;

constexpr size_t a256(size_t v) { return (v + 255) / 256 * 256; }

// carve-up of the scratch array (byte offsets, all 256-aligned)
constexpr size_t kOffHeap = 0;                                            // control words of the one-rank "heap"
constexpr size_t kOffRecv = a256(kCtlWords * 8);                          // receive region: one record per token
constexpr size_t kMetaMax = 12 * kMaxTopkNA + 16;                          // routing words of a record (no scale factors here)
constexpr size_t kPitchMax = (kMaxRowBytes + kMetaMax + 127) / 128 * 128;
constexpr size_t kOffWs = kOffRecv + a256(kMaxTokens * kPitchMax);
constexpr size_t kOffTokenSlot = kOffWs + a256(kWsBytes);
constexpr size_t kOffPairRow = kOffTokenSlot + a256(kMaxTokens * 4);
constexpr size_t kOffPsumRank = kOffPairRow + a256(kMaxTokens * kMaxTopkNA * 4);
constexpr size_t kOffUnaligned = kOffPsumRank + 256;
constexpr size_t kOffStatus = kOffUnaligned + a256(kMaxExpertsNA * 4);
constexpr size_t kScratchBytes = kOffStatus + 256;

// Held by every GPU that loads this library, from module load until the process exits.
// In host code this name is only a stand-in for the symbol: the device address comes from
// cudaGetSymbolAddress (see state_for_current_device).
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct DeviceState {
    unsigned char* scratch = nullptr;   // device address of g_noalloc_scratch on this device
    uint32_t epoch = 0;                 // control words are epoch-tagged: nothing to clear between calls
    uint64_t grid_bar_base = 0;         // the grid-barrier counter only grows; this is its value before the next launch
    int num_sms = 0, smem_optin = 0;
};

std::mutex g_mutex;
DeviceState g_state[64];

// First call on a device: resolve the device address of the scratch array (with that device
// current) and read the device limits. No allocation.
cudaError_t state_for_current_device(DeviceState** out) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    DeviceState& st = g_state[dev];
    if (st.scratch == nullptr) {
        void* ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (err != cudaSuccess) return err;
        err = cudaDeviceGetAttribute(&st.num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (err != cudaSuccess) return err;
        err = cudaDeviceGetAttribute(&st.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (err != cudaSuccess) return err;
        st.scratch = static_cast<unsigned char*>(ptr);
    }
    *out = &st;
    return cudaSuccess;
}

}  // namespace

extern "C" size_t deepep_b200_noalloc_scratch_bytes(void) { return kScratchBytes; }

extern "C" int deepep_b200_dispatch_local_noalloc(const void* x, long long x_stride_bytes, int row_bytes, const long long* topk_idx,
                                                  const float* topk_weights, int num_tokens, int num_topk, int num_experts,
                                                  int do_expand, int expert_alignment, int num_sms, void* recv_x,
                                                  int num_recv_x_rows, long long* recv_topk_idx, float* recv_topk_weights,
                                                  int* recv_src_metadata, int* psum_num_recv_per_expert, int* num_recv_tokens,
                                                  void* stream_ptr) {
    // ---- sizes beyond the fixed scratch are refused, nothing is launched
    if (num_tokens < 0 || num_tokens > static_cast<int>(kMaxTokens)) return DEEPEP_B200_NOALLOC_ERR_TOKENS;
    if (row_bytes <= 0 || row_bytes > static_cast<int>(kMaxRowBytes) || row_bytes % 16 != 0) return DEEPEP_B200_NOALLOC_ERR_ROW_BYTES;
    if (num_topk < 1 || num_topk > static_cast<int>(kMaxTopkNA)) return DEEPEP_B200_NOALLOC_ERR_TOPK;
    if (num_experts < 1 || num_experts > static_cast<int>(kMaxExpertsNA)) return DEEPEP_B200_NOALLOC_ERR_EXPERTS;
    if (x == nullptr || topk_idx == nullptr || recv_x == nullptr || recv_src_metadata == nullptr ||
        psum_num_recv_per_expert == nullptr || num_recv_tokens == nullptr || expert_alignment < 1 ||
        x_stride_bytes % 16 != 0 || reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(recv_x) % 16 != 0)
        return DEEPEP_B200_NOALLOC_ERR_ARGUMENT;
    // the output must hold the worst case: the kernels place rows by routing data and never look at the caller's sizes again
    const long long rows_needed = do_expand ? static_cast<long long>(num_tokens) * num_topk + static_cast<long long>(num_experts) * (expert_alignment - 1)
                                            : num_tokens;
    if (num_recv_x_rows < rows_needed) return DEEPEP_B200_NOALLOC_ERR_ARGUMENT;

    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState* st = nullptr;
    if (state_for_current_device(&st) != cudaSuccess) return DEEPEP_B200_NOALLOC_ERR_CUDA;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
    unsigned char* s = st->scratch;
    if (num_sms <= 0) num_sms = 8;
    if (num_sms > st->num_sms) num_sms = st->num_sms;

    Multi<DispatchParams> m;
    m.num_vranks = 1;
    m.blocks_per_rank = num_sms;
    DispatchParams& p = m.r[0];
    p.c.rank = 0;
    p.c.num_ranks = 1;
    for (int r = 0; r < kMaxRanks; ++r) p.c.heap[r] = r == 0 ? s + kOffHeap : nullptr;
    p.c.local_ws = reinterpret_cast<uint64_t*>(s + kOffWs);
    p.c.host_status = reinterpret_cast<uint64_t*>(s + kOffStatus);   // device words here: read back with ..._status()
    p.c.timeout_ns = 10ull * 1000 * 1000 * 1000;
    p.num_tokens = num_tokens;
    p.num_topk = num_topk;
    p.num_experts = num_experts;
    p.num_local_experts = num_experts;
    p.num_max_tokens = static_cast<int>(kMaxTokens);
    p.src_row_bytes = row_bytes;
    p.x_row_bytes = row_bytes;
    p.sf_bytes = 0;
    p.meta_bytes = ht_meta_bytes(0, num_topk);
    p.rec_pitch = ht_record_pitch(row_bytes, 0, num_topk);
    p.idx32 = 0;
    p.smem_scratch_bytes = 0;
    p.quant_mode = kQuantNone;
    p.expert_alignment = expert_alignment;
    p.do_expand = do_expand ? 1 : 0;
    p.cached = 0;
    p.x = static_cast<const uint8_t*>(x);
    p.x_stride_bytes = x_stride_bytes;
    p.sf = nullptr;
    p.sf_token_stride = 0;
    p.sf_pack_stride = 0;
    p.topk_idx = topk_idx;
    p.topk_weights = topk_weights;
    p.token_slot = reinterpret_cast<int*>(s + kOffTokenSlot);
    p.pair_row = reinterpret_cast<int*>(s + kOffPairRow);
    p.psum_rank = num_recv_tokens;
    p.psum_expert = psum_num_recv_per_expert;
    p.num_unaligned = reinterpret_cast<int*>(s + kOffUnaligned);
    p.recv_stats = nullptr;
    p.count_matrix = nullptr;
    p.off_recv = kOffRecv;
    // the call counter and the barrier base move only once the launch has happened: a refused launch must not
    // leave the host ahead of the device counters
    p.epoch = st->epoch + 1;
    p.grid_bar_base = st->grid_bar_base;
    p.host_counts = nullptr;

    DispatchLaunch launch;
    if (!plan_dispatch(p, num_sms, st->smem_optin, &launch)) return DEEPEP_B200_NOALLOC_ERR_ROW_BYTES;
    if (launch_dispatch(m, launch, stream) != cudaSuccess) return DEEPEP_B200_NOALLOC_ERR_CUDA;
    st->epoch = p.epoch;
    st->grid_bar_base += 2ull * num_sms;

    DispatchEpilogueParams q;
    q.c = p.c;
    q.epoch = p.epoch;
    q.wait_done = 1;
    q.idx32 = 0;
    q.rec_pitch = p.rec_pitch;
    q.num_ranks = 1;
    q.num_topk = num_topk;
    q.num_local_experts = num_experts;
    q.num_max_tokens = static_cast<int>(kMaxTokens);
    q.x_row_bytes = row_bytes;
    q.sf_bytes = 0;
    q.do_expand = p.do_expand;
    q.copy_x = 1;
    q.expert_alignment = expert_alignment;
    q.do_zero_padding = 0;
    q.write_metadata = 1;
    q.region = s + kOffRecv;
    q.psum_rank = num_recv_tokens;
    q.psum_expert = psum_num_recv_per_expert;
    q.num_unaligned = p.num_unaligned;
    q.recv_x = static_cast<uint8_t*>(recv_x);
    q.recv_sf = nullptr;
    q.recv_sf_row_stride = 0;
    q.recv_sf_pack_stride = 0;
    q.recv_topk_idx = do_expand ? nullptr : static_cast<void*>(recv_topk_idx);
    q.recv_topk_weights = recv_topk_weights;
    q.recv_src_metadata = recv_src_metadata;
    q.num_out_rows = num_recv_x_rows;
    q.num_idx_rows = num_tokens;
    if (launch_dispatch_epilogue(&q, 1, st->num_sms, st->smem_optin, stream) != cudaSuccess) return DEEPEP_B200_NOALLOC_ERR_CUDA;
    return DEEPEP_B200_NOALLOC_OK;
}

extern "C" int deepep_b200_noalloc_reset(void) {
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState* st = nullptr;
    if (state_for_current_device(&st) != cudaSuccess) return DEEPEP_B200_NOALLOC_ERR_CUDA;
    if (cudaDeviceSynchronize() != cudaSuccess) return DEEPEP_B200_NOALLOC_ERR_CUDA;
    // private workspace (barrier counter, poison word, hand-out counters) and the status word start over; the
    // control words keep their call tags, so the call counter goes on
    if (cudaMemset(st->scratch + kOffWs, 0, kWsBytes) != cudaSuccess) return DEEPEP_B200_NOALLOC_ERR_CUDA;
    if (cudaMemset(st->scratch + kOffStatus, 0, 256) != cudaSuccess) return DEEPEP_B200_NOALLOC_ERR_CUDA;
    st->grid_bar_base = 0;
    return DEEPEP_B200_NOALLOC_OK;
}

extern "C" int deepep_b200_noalloc_status(unsigned long long* record) {
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState* st = nullptr;
    if (state_for_current_device(&st) != cudaSuccess) return DEEPEP_B200_NOALLOC_ERR_CUDA;
    unsigned long long host = 0;
    if (cudaMemcpy(&host, st->scratch + kOffStatus, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess)
        return DEEPEP_B200_NOALLOC_ERR_CUDA;
    if (record != nullptr) *record = host;
    return DEEPEP_B200_NOALLOC_OK;
}
