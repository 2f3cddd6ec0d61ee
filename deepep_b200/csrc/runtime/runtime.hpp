// Host runtime of one rank: symmetric heap, private workspace, mapped status / count words,
// the communication stream, epoch bookkeeping, and the dispatch / combine / barrier drivers.
// Every driver takes a LIST of runtimes: production passes one (this process' rank); the
// single-GPU emulation passes all virtual ranks, which then run as one cooperative launch.
//
// Parity: csrc/elastic/buffer.hpp (ElasticBuffer: ctor :81-140, barrier :181-208,
// stream control :526-584, dispatch :693-1177, combine :1179-1343) and csrc/utils/event.hpp
// of the reference.
#pragma once

#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/types.h>

#include <chrono>
#include <memory>
#include <optional>
#include <vector>

#include "../common/exception.hpp"
#include "../common/layout.hpp"
#include "../kernels/api.hpp"
#include "symmetric.hpp"

namespace ep {

// ------------------------------------------------------------------------ events
struct EventHandle {
    std::shared_ptr<at::cuda::CUDAEvent> event;
    std::vector<at::Tensor> keep_alive;

    EventHandle() : event(std::make_shared<at::cuda::CUDAEvent>()) { event->record(at::cuda::getCurrentCUDAStream()); }
    explicit EventHandle(const at::cuda::CUDAStream& stream) : event(std::make_shared<at::cuda::CUDAEvent>()) { event->record(stream); }
    void current_stream_wait() const { event->block(at::cuda::getCurrentCUDAStream()); }
    void stream_wait(const at::cuda::CUDAStream& stream) const { event->block(stream); }
};

inline void stream_wait(const at::cuda::CUDAStream& waiter, const at::cuda::CUDAStream& waited) {
    at::cuda::CUDAEvent ev;
    ev.record(waited);
    ev.block(waiter);
}

// ------------------------------------------------------------------------ argument / result blocks
struct StreamControl {
    std::optional<EventHandle> previous_event;
    std::optional<EventHandle> previous_event_before_epilogue;
    bool async_with_compute_stream = false;
    bool allocate_on_comm_stream = false;
};

struct DispatchArgs {
    at::Tensor x;
    std::optional<at::Tensor> sf, topk_idx, topk_weights, cumulative_stats;
    int num_experts = 0, num_max_tokens = 0, expert_alignment = 1, num_sms = 0, quant_mode = 0;
    bool do_expand = false, do_zero_padding = false, do_cpu_sync = true, zero_copy = false, col_major_sf = false;
    // without CPU sync: rows of the outputs (0 = ranks x num_max_tokens); the routing outputs past the received
    // count are filled with -1 / 0 (csrc/legacy/buffer.hpp:571-577 and intranode.cu:536-540 of the reference)
    int num_worst_tokens = 0;
    // cached dispatch: tensors of an earlier handle
    bool cached = false;
    std::optional<at::Tensor> h_token_slot, h_pair_row, h_psum_rank, h_psum_expert, h_num_unaligned, h_recv_src_metadata;
    int h_num_recv_tokens = 0, h_num_expanded_tokens = 0;
    StreamControl sc;
};

struct DispatchResult {
    at::Tensor recv_x;
    std::optional<at::Tensor> recv_sf, recv_topk_idx, recv_topk_weights;
    at::Tensor token_slot, pair_row, psum_rank, psum_expert, num_unaligned, recv_src_metadata;
    at::Tensor count_matrix;   // [R, R] tokens rank i sent to rank j (undefined for cached dispatches)
    int num_recv_tokens = 0, num_expanded_tokens = 0, num_sms = 0;
    std::vector<int> num_recv_tokens_per_expert_list;
    std::optional<EventHandle> event;
};

struct CombineArgs {
    at::Tensor x;
    std::optional<at::Tensor> topk_weights, bias0, bias1;
    at::Tensor recv_src_metadata, topk_idx, psum_rank;
    int num_experts = 0, num_max_tokens = 0, num_sms = 0;
    bool do_expand = false, allow_multiple_reduction = true;
    bool weighted = false;     // expanded rows are multiplied by their top-k weight before they are summed
    // [T, R] row of every token in each destination's receive region (the dispatch handle has it). With it, and
    // unless an event has to be awaited between send and reduce, the reduce overlaps the sends.
    std::optional<at::Tensor> dst_slot;
    std::optional<at::Tensor> count_matrix;   // [R, R] tokens rank i dispatched to rank j (the handle has it)
    int fuse_reduce = 1;       // 1: arrival-driven reduce kernel beside the send kernel, 0: the reduce kernel after it
    StreamControl sc;
};

struct CombineResult {
    at::Tensor combined_x;
    std::optional<at::Tensor> combined_topk_weights;
    std::optional<EventHandle> event;
};

// ------------------------------------------------------------------------ runtime
class Runtime {
public:
    // `num_cpu_bytes` > 0 puts a pinned CPU segment behind the GPU segment in the heap's address range (needs the
    // virtual-memory heap, EP_HEAP_BACKEND=vmm)
    Runtime(int rank, int num_ranks, int64_t num_bytes, double gpu_timeout_secs, double cpu_timeout_secs, int64_t num_cpu_bytes = 0);
    ~Runtime();
    void destroy();

    // peer table
    std::string export_handle() const { return heap_->export_handle(); }
    void open_peers(const std::vector<std::string>& handles) { heap_->open_peers(handles); }
    void finish_export() { heap_->finish_export(); }     // after a barrier: every peer has mapped this rank's heap
    bool heap_is_vmm() const { return heap_->backend() == SymmetricHeap::Backend::kVmm; }
    static bool heap_backend_is_vmm() { return SymmetricHeap::backend_from_env() == SymmetricHeap::Backend::kVmm; }
    static void connect_local(const std::vector<std::shared_ptr<Runtime>>& runtimes);

    // status words
    uint64_t status() const { return host_words_[0]; }
    void check_status() const;           // throws EPTimeoutError when a device wait gave up
    void clear_status();                 // after the cause is gone: forget the failure and un-poison the rank

    CommCtx ctx() const;
    at::cuda::CUDAStream comm_stream() const { return comm_stream_; }
    int rank() const { return rank_; }
    int num_ranks() const { return num_ranks_; }
    int64_t num_bytes() const { return static_cast<int64_t>(heap_->num_bytes()); }
    int num_device_sms() const { return num_device_sms_; }
    int smem_optin() const { return smem_optin_; }
    SymmetricHeap& heap() { return *heap_; }
    at::Tensor heap_tensor(int64_t offset, int64_t num_bytes) const;   // uint8 view of the own heap (no ownership)
    void set_gpu_timeout(double secs) { gpu_timeout_ns_ = static_cast<uint64_t>(secs * 1e9); }

    // Optional device timing of the last dispatch / combine: events around the communication
    // kernel and around the local epilogue (what the reference reports as two separate kernels).
    // mode 1: events around each pair (kernel + epilogue; their overlap stays as in production). mode 2: also an event
    // between the two launches, which serialises them: kernel-only figures as the reference reports them.
    void enable_profiling(int mode);
    // kernels this runtime has launched so far (barrier, dispatch, combine and their epilogues)
    int64_t num_kernel_launches() const { return num_launches_; }
    // {dispatch kernel, dispatch epilogue, combine kernel, combine epilogue, dispatch pair, combine pair} in ms,
    // -1 = not measured (the first four need mode 2)
    std::vector<float> last_timings();
    // %globaltimer stamps of the last dispatch kernel, dispatch epilogue, combine send and combine reduce kernel:
    // {start, end} each, ns relative to the start of the dispatch kernel (-1 = never ran); then six phase stamps of
    // the last low-latency combine kernel (start, rows issued, flags raised, send handed over, tokens reduced, end)
    // relative to its start. Synchronises the device.
    std::vector<int64_t> last_timeline();

    // Phase timestamps (ns after kernel start) of the last dispatch kernel: totals counted, order pass done, peers'
    // totals in, first rows published, block 0 out of tokens, its stores complete, last block done.
    // Synchronises the device.
    std::vector<int64_t> last_dispatch_phases();

    // drivers
    static void barrier(const std::vector<std::shared_ptr<Runtime>>& rts, bool use_comm_stream, bool with_cpu_sync);
    static std::vector<DispatchResult> dispatch(const std::vector<std::shared_ptr<Runtime>>& rts, std::vector<DispatchArgs>& args);
    static std::vector<CombineResult> combine(const std::vector<std::shared_ptr<Runtime>>& rts, std::vector<CombineArgs>& args);

    // sizing
    static int64_t ht_buffer_size(int num_ranks, int num_max_tokens, int hidden, int num_topk) {
        return static_cast<int64_t>(ht_layout(num_ranks, num_max_tokens, hidden, num_topk).end);
    }

    // epoch counters are public to the sibling subsystems (low latency, AGRS, PP) that share the heap
    uint32_t barrier_epoch = 0, dispatch_epoch = 0, combine_epoch = 0;
    uint64_t grid_bar_base = 0;
    // fused tensor-parallel operators
    uint32_t tp_ag_epoch = 0, tp_rs_epoch = 0;
    int64_t tp_rs_config = 0;   // (rows_per_rank, N, flag offsets) of the first GEMM->RS call: arrival counters depend on it
    uint64_t* host_words() const { return host_words_; }
    uint64_t* host_words_dev() const { return host_words_dev_; }
    uint64_t* local_ws() const { return local_ws_; }
    double cpu_timeout_secs() const { return cpu_timeout_secs_; }

    static constexpr int kHostStatusWords = 8;    // [0] failure record
    static constexpr int kHostCountWords = 2 + kMaxLocalExperts;

private:
    int rank_, num_ranks_;
    std::unique_ptr<SymmetricHeap> heap_;
    uint64_t* local_ws_ = nullptr;
    uint64_t* host_words_ = nullptr;       // mapped pinned: status words then count words
    uint64_t* host_words_dev_ = nullptr;
    uint64_t gpu_timeout_ns_;
    double cpu_timeout_secs_;
    at::cuda::CUDAStream comm_stream_;
    int num_device_sms_ = 0, smem_optin_ = 0;
    bool destroyed_ = false;
    int profiling_ = 0;
    bool use_pdl_ = true;
    bool prof_split_[2] = {false, false};
    int64_t num_launches_ = 0;
    cudaEvent_t prof_events_[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    bool prof_valid_[2] = {false, false};
    void prof_record(int idx, cudaStream_t stream) {
        if (profiling_ != 0) cudaEventRecord(prof_events_[idx], stream);
    }
};

}  // namespace ep
