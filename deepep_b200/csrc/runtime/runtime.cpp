// Implementation of the per-rank host runtime (see runtime.hpp).
#include "runtime.hpp"

#include <ATen/ops/empty.h>
#include <ATen/ops/empty_strided.h>
#include <ATen/ops/from_blob.h>
#include <c10/cuda/CUDACachingAllocator.h>

#include <sstream>
#include <thread>

namespace ep {

namespace {

const char* status_name(int code) {
    switch (code) {
        case kStatusGridBarrier: return "grid barrier";
        case kStatusBarrierPeer: return "cross-rank barrier";
        case kStatusDispatchCounts: return "dispatch count exchange";
        case kStatusDispatchDone: return "dispatch completion";
        case kStatusCombineDone: return "combine completion";
        case kStatusTmaLoad: return "bulk load";
        case kStatusLLRecv: return "low-latency dispatch receive";
        case kStatusLLCombine: return "low-latency combine receive";
        case kStatusEntry: return "cached dispatch entry";
        case kStatusPP: return "pipeline send/recv";
        case kStatusAgrs: return "all-gather arrival";
        case kStatusGemmPipe: return "GEMM pipeline";
        case kStatusTileFlag: return "fused GEMM tile flag";
        default: return "unknown";
    }
}

bool env_flag(const char* name) {
    const char* v = std::getenv(name);
    return v != nullptr && v[0] != '\0' && v[0] != '0';
}

// Everything the stream-control arguments ask for before the first launch.
struct StreamScope {
    at::cuda::CUDAStream compute, comm;
    bool switched = false;
    StreamScope(const StreamControl& sc, const at::cuda::CUDAStream& comm_stream)
        : compute(at::cuda::getCurrentCUDAStream()), comm(comm_stream) {
        if (sc.allocate_on_comm_stream) {
            at::cuda::setCurrentCUDAStream(comm);
            switched = true;
        }
        if (sc.previous_event.has_value()) sc.previous_event->stream_wait(comm);
        else stream_wait(comm, compute);
    }
    // Either hands back an event (async) or makes the compute stream wait for the comm stream.
    std::optional<EventHandle> finish(const StreamControl& sc, const std::vector<at::Tensor>& tensors) {
        std::optional<EventHandle> event;
        if (sc.async_with_compute_stream) {
            event = EventHandle(comm);
            // EP_AVOID_RECORD_STREAM=1: the event keeps the tensors alive instead (the caller holds the event until it
            // has waited on it); record_stream delays the reuse of a block by the caching allocator in a way that is
            // hard to predict (csrc/elastic/buffer.hpp:556-584 of the reference offers the same switch).
            static const bool avoid_record_stream = env_flag("EP_AVOID_RECORD_STREAM");
            for (const auto& t : tensors) {
                if (!t.defined() || !t.is_cuda()) continue;
                if (avoid_record_stream) {
                    event->keep_alive.push_back(t);
                    continue;
                }
                // (views of the heap are not owned by the caching allocator; record_stream ignores them)
                t.record_stream(comm);
                if (sc.allocate_on_comm_stream) t.record_stream(compute);
            }
        } else {
            stream_wait(compute, comm);
        }
        if (switched) at::cuda::setCurrentCUDAStream(compute);
        return event;
    }
};

at::TensorOptions opts(at::ScalarType dtype, int device) {
    return at::TensorOptions().dtype(dtype).device(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device)));
}

}  // namespace

// ============================================================================ construction
Runtime::Runtime(int rank, int num_ranks, int64_t num_bytes, double gpu_timeout_secs, double cpu_timeout_secs, int64_t num_cpu_bytes)
    : rank_(rank), num_ranks_(num_ranks), gpu_timeout_ns_(static_cast<uint64_t>(gpu_timeout_secs * 1e9)),
      cpu_timeout_secs_(cpu_timeout_secs), comm_stream_(at::cuda::getStreamFromPool(/*isHighPriority=*/true)) {
    EP_HOST_ASSERT(num_bytes >= static_cast<int64_t>(kCtlBytes));
    heap_ = std::make_unique<SymmetricHeap>(rank, num_ranks, align_up<size_t>(static_cast<size_t>(num_bytes), kHeapAlignment),
                                            SymmetricHeap::backend_from_env(), static_cast<size_t>(std::max<int64_t>(num_cpu_bytes, 0)));
    CUDA_RUNTIME_CHECK(cudaMalloc(reinterpret_cast<void**>(&local_ws_), kWsBytes));
    CUDA_RUNTIME_CHECK(cudaMemset(local_ws_, 0, kWsBytes));
    const size_t host_bytes = sizeof(uint64_t) * (kHostStatusWords + kHostCountWords);
    CUDA_RUNTIME_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&host_words_), host_bytes, cudaHostAllocMapped));
    std::memset(host_words_, 0, host_bytes);
    CUDA_RUNTIME_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&host_words_dev_), host_words_, 0));
    cudaDeviceProp prop;
    CUDA_RUNTIME_CHECK(cudaGetDeviceProperties(&prop, heap_->device()));
    num_device_sms_ = prop.multiProcessorCount;
    use_pdl_ = !env_flag("EP_DISABLE_PDL");
    smem_optin_ = static_cast<int>(prop.sharedMemPerBlockOptin);
    CUDA_RUNTIME_CHECK(cudaDeviceSynchronize());
}

Runtime::~Runtime() { destroy(); }

void Runtime::destroy() {
    if (destroyed_) return;
    destroyed_ = true;
    cudaDeviceSynchronize();
    heap_->release();
    if (local_ws_ != nullptr) cudaFree(local_ws_);
    if (host_words_ != nullptr) cudaFreeHost(host_words_);
    local_ws_ = nullptr;
    host_words_ = nullptr;
}

void Runtime::enable_profiling(int mode) {
    EP_HOST_ASSERT(mode >= 0 && mode <= 2);
    if (mode != 0 && prof_events_[0] == nullptr)
        for (auto& e : prof_events_) CUDA_RUNTIME_CHECK(cudaEventCreate(&e));
    profiling_ = mode;
    prof_valid_[0] = prof_valid_[1] = false;
}

std::vector<float> Runtime::last_timings() {
    std::vector<float> out(6, -1.f);
    for (int op = 0; op < 2; ++op) {
        if (!prof_valid_[op]) continue;
        CUDA_RUNTIME_CHECK(cudaEventSynchronize(prof_events_[3 * op + 2]));
        CUDA_RUNTIME_CHECK(cudaEventElapsedTime(&out[4 + op], prof_events_[3 * op], prof_events_[3 * op + 2]));
        if (prof_split_[op]) {
            CUDA_RUNTIME_CHECK(cudaEventElapsedTime(&out[2 * op], prof_events_[3 * op], prof_events_[3 * op + 1]));
            CUDA_RUNTIME_CHECK(cudaEventElapsedTime(&out[2 * op + 1], prof_events_[3 * op + 1], prof_events_[3 * op + 2]));
        }
    }
    return out;
}

std::vector<int64_t> Runtime::last_dispatch_phases() {
    CUDA_RUNTIME_CHECK(cudaDeviceSynchronize());
    uint64_t raw[8];
    CUDA_RUNTIME_CHECK(cudaMemcpy(raw, local_ws_ + kWsStamps, sizeof(raw), cudaMemcpyDeviceToHost));
    std::vector<int64_t> out;
    for (int i = 1; i < 8; ++i) out.push_back(static_cast<int64_t>(raw[i] - raw[0]));
    return out;
}

std::vector<int64_t> Runtime::last_timeline() {
    CUDA_RUNTIME_CHECK(cudaDeviceSynchronize());
    uint64_t raw[16];
    CUDA_RUNTIME_CHECK(cudaMemcpy(raw, reinterpret_cast<uint8_t*>(local_ws_) + kWsTimelineOffsetBytes, sizeof(raw), cudaMemcpyDeviceToHost));
    std::vector<int64_t> out;
    for (int i = 0; i < 8; ++i) out.push_back(raw[i] == 0 ? -1 : static_cast<int64_t>(raw[i] - raw[0]));
    // the low-latency combine kernel's phase stamps (block 0), relative to its own start
    for (int i = 8; i < 14; ++i) out.push_back(raw[i] == 0 ? -1 : static_cast<int64_t>(raw[i] - raw[8]));
    return out;
}

void Runtime::connect_local(const std::vector<std::shared_ptr<Runtime>>& runtimes) {
    std::vector<SymmetricHeap*> heaps;
    for (const auto& rt : runtimes) heaps.push_back(rt->heap_.get());
    for (const auto& rt : runtimes) rt->heap_->set_local_peers(heaps);
}

void Runtime::check_status() const {
    const uint64_t rec = *reinterpret_cast<volatile uint64_t*>(host_words_);
    if (rec == 0) return;
    const int code = static_cast<int>((rec >> 56) & 0xff);
    const int waiter = static_cast<int>((rec >> 44) & 0xfff);
    int peer = static_cast<int>((rec >> 32) & 0xfff);
    if (peer == 0xfff) peer = -1;
    std::ostringstream os;
    os << "EP device wait timed out on rank " << waiter << ": " << status_name(code) << " (awaited peer " << peer
       << ", tag " << static_cast<uint32_t>(rec) << ")";
    throw EPTimeoutError(os.str(), rec);
}

void Runtime::clear_status() {
    CUDA_RUNTIME_CHECK(cudaDeviceSynchronize());
    host_words_[0] = 0;
    CUDA_RUNTIME_CHECK(cudaMemset(local_ws_ + kWsPoison, 0, sizeof(uint64_t)));
    // the grid-barrier counter may be anywhere after a failed launch: restart it
    CUDA_RUNTIME_CHECK(cudaMemset(local_ws_, 0, kWsBytes));
    grid_bar_base = 0;
}

CommCtx Runtime::ctx() const {
    CommCtx c;
    c.rank = rank_;
    c.num_ranks = num_ranks_;
    for (int r = 0; r < kMaxRanks; ++r) c.heap[r] = r < num_ranks_ ? heap_->peer(r) : nullptr;
    c.local_ws = local_ws_;
    c.host_status = host_words_dev_;
    c.timeout_ns = gpu_timeout_ns_;
    return c;
}

at::Tensor Runtime::heap_tensor(int64_t offset, int64_t num_bytes) const {
    EP_HOST_ASSERT(offset >= 0 && offset + num_bytes <= static_cast<int64_t>(heap_->num_bytes()));
    return at::from_blob(heap_->base() + offset, {num_bytes}, opts(at::kByte, heap_->device()));
}

// ============================================================================ barrier
void Runtime::barrier(const std::vector<std::shared_ptr<Runtime>>& rts, bool use_comm_stream, bool with_cpu_sync) {
    EP_HOST_ASSERT(!rts.empty() && rts.size() <= kMaxVRanks);
    auto& rt0 = *rts[0];
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(rt0.heap_->device()));
    const auto compute = at::cuda::getCurrentCUDAStream();
    const auto stream = use_comm_stream ? rt0.comm_stream_ : compute;
    if (use_comm_stream) stream_wait(stream, compute);
    Multi<BarrierParams> m;
    m.num_vranks = static_cast<int>(rts.size());
    m.blocks_per_rank = 1;
    for (size_t v = 0; v < rts.size(); ++v) {
        EP_HOST_ASSERT(rts[v]->heap_->connected());
        m.r[v].c = rts[v]->ctx();
        m.r[v].epoch = ++rts[v]->barrier_epoch;
    }
    CUDA_RUNTIME_CHECK(launch_barrier(m, stream));
    ++rt0.num_launches_;
    if (use_comm_stream) stream_wait(compute, stream);
    if (with_cpu_sync) {
        CUDA_RUNTIME_CHECK(cudaStreamSynchronize(stream));
        for (const auto& rt : rts) rt->check_status();
    }
}

// ============================================================================ dispatch
std::vector<DispatchResult> Runtime::dispatch(const std::vector<std::shared_ptr<Runtime>>& rts, std::vector<DispatchArgs>& args) {
    const int V = static_cast<int>(rts.size());
    EP_HOST_ASSERT(V >= 1 && V <= kMaxVRanks && static_cast<int>(args.size()) == V);
    auto& rt0 = *rts[0];
    const int device = rt0.heap_->device();
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    StreamScope scope(args[0].sc, rt0.comm_stream_);
    const cudaStream_t stream = scope.comm.stream();

    const int R = rt0.num_ranks_;
    const auto& a0 = args[0];
    EP_HOST_ASSERT(a0.topk_idx.has_value());
    const int K = static_cast<int>(a0.topk_idx->size(1));
    const int H = static_cast<int>(a0.x.size(1));
    const int E = a0.num_experts, EL = E / R, T_max = a0.num_max_tokens;
    EP_HOST_ASSERT(E > 0 && E % R == 0 && E <= kMaxExperts && EL <= kMaxLocalExperts);
    EP_HOST_ASSERT(K >= 1 && K <= kMaxTopk && T_max > 0 && a0.expert_alignment >= 1);
    const bool quant = a0.quant_mode != kQuantNone;
    const int elem = static_cast<int>(a0.x.element_size());
    if (quant) EP_HOST_ASSERT_MSG(a0.x.scalar_type() == at::kBFloat16 && H % 128 == 0 && !a0.sf.has_value(),
                                  "fused FP8 dispatch wants a bf16 input with hidden % 128 == 0 and no scales");
    else EP_HOST_ASSERT(a0.x.scalar_type() == at::kBFloat16 || a0.x.scalar_type() == at::kFloat8_e4m3fn);
    const int src_row_bytes = H * elem;
    const int x_row_bytes = quant ? H : src_row_bytes;
    const int sf_packs = quant ? H / 128 : (a0.sf.has_value() ? static_cast<int>(a0.sf->size(1)) : 0);
    const int sf_bytes = sf_packs * 4;
    EP_HOST_ASSERT_MSG(src_row_bytes % 16 == 0 && x_row_bytes % 16 == 0, "hidden bytes must be a multiple of 16");
    EP_HOST_ASSERT(sf_bytes <= ceil_div(H, 128) * 4);
    const int meta_bytes = ht_meta_bytes(sf_bytes, K);
    const int rec_pitch = ht_record_pitch(x_row_bytes, sf_bytes, K);
    const HtLayout lay = ht_layout(R, T_max, H, K);
    EP_HOST_ASSERT_MSG(lay.end <= rt0.heap_->num_bytes(), "symmetric buffer too small for this dispatch");
    const at::ScalarType out_dtype = quant ? at::kFloat8_e4m3fn : a0.x.scalar_type();
    const at::ScalarType idx_dtype = a0.topk_idx->scalar_type();
    EP_HOST_ASSERT_MSG(idx_dtype == at::kLong || idx_dtype == at::kInt, "topk_idx must be int64 or int32");
    const bool has_sf = sf_packs > 0;
    const bool cached = a0.cached;
    EP_HOST_ASSERT_MSG(a0.num_sms > 0, "num_sms must be given (the Python front end fills in the SM model's value)");
    int num_sms = a0.num_sms;
    if (num_sms * V > rt0.num_device_sms_) num_sms = rt0.num_device_sms_ / V;

    Multi<DispatchParams> m;
    m.num_vranks = V;
    m.blocks_per_rank = num_sms;
    std::vector<DispatchResult> res(V);
    for (int v = 0; v < V; ++v) {
        auto& rt = *rts[v];
        auto& a = args[v];
        EP_HOST_ASSERT(rt.heap_->connected() && rt.num_ranks_ == R);
        EP_HOST_ASSERT(a.x.dim() == 2 && a.x.is_cuda() && a.x.size(1) == H && a.x.stride(1) == 1 && a.x.scalar_type() == a0.x.scalar_type());
        EP_HOST_ASSERT((a.x.stride(0) * elem) % 16 == 0 && reinterpret_cast<uintptr_t>(a.x.data_ptr()) % 16 == 0);
        EP_HOST_ASSERT(a.topk_idx.has_value() && a.topk_idx->scalar_type() == idx_dtype && a.topk_idx->is_contiguous() && a.topk_idx->size(1) == K);
        const int T = static_cast<int>(a.x.size(0));
        EP_HOST_ASSERT(T <= T_max && a.topk_idx->size(0) == T);
        EP_HOST_ASSERT(a.num_experts == E && a.num_max_tokens == T_max && a.cached == cached && a.do_expand == a0.do_expand &&
                       a.quant_mode == a0.quant_mode && a.expert_alignment == a0.expert_alignment);
        if (a.topk_weights.has_value())
            EP_HOST_ASSERT(a.topk_weights->scalar_type() == at::kFloat && a.topk_weights->is_contiguous() && a.topk_weights->size(0) == T && a.topk_weights->size(1) == K);
        if (has_sf && !quant) {
            EP_HOST_ASSERT(a.sf.has_value() && a.sf->dim() == 2 && a.sf->size(0) == T && a.sf->size(1) == sf_packs && a.sf->element_size() == 4);
        }
        DispatchParams& p = m.r[v];
        p.c = rt.ctx();
        p.num_tokens = T;
        p.num_topk = K;
        p.num_experts = E;
        p.num_local_experts = EL;
        p.num_max_tokens = T_max;
        p.src_row_bytes = src_row_bytes;
        p.x_row_bytes = x_row_bytes;
        p.sf_bytes = sf_bytes;
        p.meta_bytes = meta_bytes;
        p.rec_pitch = rec_pitch;
        p.quant_mode = a.quant_mode;
        p.expert_alignment = a.expert_alignment;
        p.do_expand = a.do_expand;
        p.cached = cached;
        p.idx32 = idx_dtype == at::kInt ? 1 : 0;
        p.smem_scratch_bytes = 0;    // filled in by the launcher
        p.x = static_cast<const uint8_t*>(a.x.data_ptr());
        p.x_stride_bytes = a.x.stride(0) * elem;
        p.sf = (has_sf && !quant) ? static_cast<const uint8_t*>(a.sf->data_ptr()) : nullptr;
        p.sf_token_stride = (has_sf && !quant) ? a.sf->stride(0) : 0;
        p.sf_pack_stride = (has_sf && !quant) ? a.sf->stride(1) : 0;
        p.topk_idx = a.topk_idx->data_ptr();
        p.topk_weights = a.topk_weights.has_value() ? a.topk_weights->data_ptr<float>() : nullptr;
        auto& r = res[v];
        if (cached) {
            EP_HOST_ASSERT(a.h_token_slot.has_value() && a.h_pair_row.has_value() && a.h_psum_rank.has_value() &&
                           a.h_psum_expert.has_value() && a.h_num_unaligned.has_value() && a.h_recv_src_metadata.has_value());
            EP_HOST_ASSERT(!a.cumulative_stats.has_value());
            r.token_slot = *a.h_token_slot;
            r.pair_row = *a.h_pair_row;
            r.psum_rank = *a.h_psum_rank;
            r.psum_expert = *a.h_psum_expert;
            r.num_unaligned = *a.h_num_unaligned;
            r.recv_src_metadata = *a.h_recv_src_metadata;
        } else {
            r.token_slot = at::empty({T, R}, opts(at::kInt, device));
            r.pair_row = at::empty({T, K}, opts(at::kInt, device));
            r.psum_rank = at::empty({R}, opts(at::kInt, device));
            r.psum_expert = at::empty({EL + 1}, opts(at::kInt, device));
            r.num_unaligned = at::empty({EL}, opts(at::kInt, device));
            r.count_matrix = at::empty({R, R}, opts(at::kInt, device));
        }
        p.token_slot = r.token_slot.data_ptr<int>();
        p.pair_row = r.pair_row.data_ptr<int>();
        p.psum_rank = r.psum_rank.data_ptr<int>();
        p.psum_expert = r.psum_expert.data_ptr<int>();
        p.num_unaligned = r.num_unaligned.data_ptr<int>();
        p.recv_stats = nullptr;
        p.count_matrix = r.count_matrix.defined() ? r.count_matrix.data_ptr<int>() : nullptr;
        if (a.cumulative_stats.has_value()) {
            EP_HOST_ASSERT(a.cumulative_stats->scalar_type() == at::kInt && a.cumulative_stats->numel() == EL && a.cumulative_stats->is_contiguous());
            p.recv_stats = a.cumulative_stats->data_ptr<int>();
        }
        // the counters of the runtime move only once the launch has happened (below)
        p.epoch = rt.dispatch_epoch + 1;
        p.off_recv = lay.dispatch_rec[p.epoch & 1];
        p.grid_bar_base = rt.grid_bar_base;
        p.host_counts = (a.do_cpu_sync && !cached) ? rt.host_words_dev_ + kHostStatusWords : nullptr;
    }

    DispatchLaunch launch;
    EP_HOST_ASSERT_MSG(plan_dispatch(m.r[0], num_sms, rt0.smem_optin_, &launch), "a token row does not fit into shared memory");
    rt0.prof_record(0, stream);
    CUDA_RUNTIME_CHECK(launch_dispatch(m, launch, stream));
    for (int v = 0; v < V; ++v) {
        ++rts[v]->dispatch_epoch;
        rts[v]->grid_bar_base += static_cast<uint64_t>(cached ? 1 : 2) * num_sms;
    }
    ++rt0.num_launches_;
    // an event between the two launches would serialise them (no programmatic overlap): only in split mode
    const bool split = rt0.profiling_ == 2;
    if (split) rt0.prof_record(1, stream);

    // ---- sizes of the outputs
    const int worst_rows = R * T_max;
    const int worst_expanded = align_up(R * T_max * std::min(K, EL) + EL * (a0.expert_alignment - 1), a0.expert_alignment);
    for (int v = 0; v < V; ++v) {
        auto& rt = *rts[v];
        auto& a = args[v];
        auto& r = res[v];
        r.num_sms = num_sms;
        if (cached) {
            r.num_recv_tokens = a.h_num_recv_tokens;
            r.num_expanded_tokens = a.h_num_expanded_tokens;
        } else if (a.do_cpu_sync) {
            // every count word carries the epoch of this dispatch: wait for each of them on its own
            volatile uint64_t* words = rt.host_words_ + kHostStatusWords;
            const uint32_t epoch = rt.dispatch_epoch;
            const auto start = std::chrono::steady_clock::now();
            auto wait_word = [&](int i) -> int {
                uint64_t v;
                int spins = 0;
                while (static_cast<uint32_t>((v = words[i]) >> 32) != epoch) {
                    if ((++spins & 1023) != 0) continue;
                    rt.check_status();
                    const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count();
                    if (waited > rt.cpu_timeout_secs_) throw EPTimeoutError("EP host wait for the received token counts timed out", 0);
                }
                return static_cast<int>(static_cast<uint32_t>(v));
            };
            r.num_recv_tokens = wait_word(0);
            r.num_expanded_tokens = wait_word(1);
            r.num_recv_tokens_per_expert_list.resize(EL);
            for (int le = 0; le < EL; ++le) r.num_recv_tokens_per_expert_list[le] = wait_word(2 + le);
        } else {
            r.num_recv_tokens = a.num_worst_tokens > 0 ? a.num_worst_tokens : worst_rows;
            EP_HOST_ASSERT_MSG(r.num_recv_tokens <= worst_rows, "num_worst_tokens exceeds ranks x num_max_tokens_per_rank");
            r.num_expanded_tokens = worst_expanded;
        }
    }

    // ---- outputs and the local epilogue
    std::vector<DispatchEpilogueParams> ep(V);
    std::vector<at::Tensor> touched;
    for (int v = 0; v < V; ++v) {
        auto& rt = *rts[v];
        auto& a = args[v];
        auto& r = res[v];
        const DispatchParams& p = m.r[v];
        const int N = r.num_recv_tokens;
        const int rows = a.do_expand ? r.num_expanded_tokens : N;
        const bool zero_copy = a.zero_copy && !a.do_expand;
        uint8_t* region = rt.heap_->base() + p.off_recv;
        bool sf_in_place = false;
        if (zero_copy) {
            // payload (and row-major scales) are read where they landed: strided views of the receive region
            r.recv_x = at::from_blob(region, {N, H}, {rec_pitch / static_cast<int64_t>(c10::elementSize(out_dtype)), 1}, opts(out_dtype, device));
        } else {
            r.recv_x = at::empty({rows, H}, opts(out_dtype, device));
        }
        if (has_sf) {
            const at::ScalarType sf_dtype = (!quant && a.sf->scalar_type() == at::kInt) ? at::kInt : at::kFloat;
            if (a.col_major_sf) {
                r.recv_sf = at::empty_strided({rows, sf_packs}, {1, align_up(std::max(rows, 1), 4)}, opts(sf_dtype, device));
            } else if (zero_copy) {
                r.recv_sf = at::from_blob(region + x_row_bytes, {N, sf_packs}, {rec_pitch / 4, 1}, opts(sf_dtype, device));
                sf_in_place = true;
            } else {
                r.recv_sf = at::empty({rows, sf_packs}, opts(sf_dtype, device));
            }
        }
        if (!a.do_expand) {
            r.recv_topk_idx = at::empty({N, K}, opts(idx_dtype, device));
            if (a.topk_weights.has_value()) r.recv_topk_weights = at::empty({N, K}, opts(at::kFloat, device));
        } else if (a.topk_weights.has_value()) {
            r.recv_topk_weights = at::empty({rows}, opts(at::kFloat, device));
        }
        if (!cached) r.recv_src_metadata = at::empty({N, K + 2}, opts(at::kInt, device));

        DispatchEpilogueParams& q = ep[v];
        q.c = p.c;
        q.epoch = p.epoch;
        q.wait_done = 1;
        q.num_ranks = R;
        q.num_topk = K;
        q.num_local_experts = EL;
        q.num_max_tokens = T_max;
        q.x_row_bytes = x_row_bytes;
        q.sf_bytes = sf_bytes;
        q.rec_pitch = rec_pitch;
        q.do_expand = a.do_expand;
        q.copy_x = zero_copy ? 0 : 1;
        q.expert_alignment = a.expert_alignment;
        q.do_zero_padding = a.do_zero_padding;
        q.write_metadata = cached ? 0 : 1;
        q.idx32 = p.idx32;
        q.region = region;
        q.psum_rank = p.psum_rank;
        q.psum_expert = p.psum_expert;
        q.num_unaligned = p.num_unaligned;
        q.recv_x = static_cast<uint8_t*>(r.recv_x.data_ptr());
        q.recv_sf = (has_sf && !sf_in_place) ? static_cast<uint8_t*>(r.recv_sf->data_ptr()) : nullptr;
        q.recv_sf_row_stride = has_sf ? r.recv_sf->stride(0) : 0;
        q.recv_sf_pack_stride = has_sf ? r.recv_sf->stride(1) : 0;
        q.recv_topk_idx = r.recv_topk_idx.has_value() ? r.recv_topk_idx->data_ptr() : nullptr;
        q.recv_topk_weights = r.recv_topk_weights.has_value() ? r.recv_topk_weights->data_ptr<float>() : nullptr;
        q.recv_src_metadata = r.recv_src_metadata.data_ptr<int>();
        q.num_out_rows = rows;
        q.num_idx_rows = static_cast<int>(r.recv_src_metadata.size(0));
        for (const at::Tensor& t : {r.recv_x, r.token_slot, r.pair_row, r.psum_rank, r.psum_expert, r.num_unaligned, r.recv_src_metadata,
                                    a.x, *a.topk_idx})
            touched.push_back(t);
        for (const auto& t : {r.recv_sf, r.recv_topk_idx, r.recv_topk_weights, a.sf, a.topk_weights, a.cumulative_stats})
            if (t.has_value()) touched.push_back(*t);
    }
    const bool gated = a0.sc.previous_event_before_epilogue.has_value();
    if (gated) a0.sc.previous_event_before_epilogue->stream_wait(scope.comm);
    const int epi_sms = std::max(1, rt0.num_device_sms_ / V);
    // programmatic dependent launch: the epilogue's blocks get resident while the dispatch kernel drains
    CUDA_RUNTIME_CHECK(launch_dispatch_epilogue(ep.data(), V, epi_sms, rt0.smem_optin_, stream,
                                                /*programmatic=*/!gated && !split && rt0.use_pdl_));
    ++rt0.num_launches_;
    rt0.prof_record(2, stream);
    rt0.prof_valid_[0] = rt0.profiling_ != 0;
    rt0.prof_split_[0] = split;

    auto event = scope.finish(a0.sc, touched);
    for (auto& r : res) r.event = event;
    return res;
}

// ============================================================================ combine
std::vector<CombineResult> Runtime::combine(const std::vector<std::shared_ptr<Runtime>>& rts, std::vector<CombineArgs>& args) {
    const int V = static_cast<int>(rts.size());
    EP_HOST_ASSERT(V >= 1 && V <= kMaxVRanks && static_cast<int>(args.size()) == V);
    auto& rt0 = *rts[0];
    const int device = rt0.heap_->device();
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    StreamScope scope(args[0].sc, rt0.comm_stream_);
    const cudaStream_t stream = scope.comm.stream();

    const int R = rt0.num_ranks_;
    const auto& a0 = args[0];
    const int K = static_cast<int>(a0.topk_idx.size(1));
    const int H = static_cast<int>(a0.x.size(1));
    const int E = a0.num_experts, EL = E / R, T_max = a0.num_max_tokens;
    EP_HOST_ASSERT(a0.x.scalar_type() == at::kBFloat16 && (H * 2) % 16 == 0);
    const HtLayout lay = ht_layout(R, T_max, H, K);
    EP_HOST_ASSERT_MSG(lay.end <= rt0.heap_->num_bytes(), "symmetric buffer too small for this combine");
    const bool rank_layout = !a0.do_expand || a0.allow_multiple_reduction;
    const int num_lanes = std::max(R, K);
    const at::ScalarType idx_dtype = a0.topk_idx.scalar_type();
    EP_HOST_ASSERT_MSG(idx_dtype == at::kLong || idx_dtype == at::kInt, "topk_idx must be int64 or int32");
    EP_HOST_ASSERT_MSG(a0.num_sms > 0, "num_sms must be given (the Python front end fills in the handle's value)");
    int num_sms = a0.num_sms;
    if (num_sms * V > rt0.num_device_sms_) num_sms = rt0.num_device_sms_ / V;
    const bool gated = a0.sc.previous_event_before_epilogue.has_value();
    const bool split = rt0.profiling_ == 2;
    // One rank: every token has at most one row (rank layout), so the send kernel can write the result itself.
    bool direct = R == 1 && rank_layout && !gated && !(a0.weighted && a0.do_expand);
    for (const auto& a : args) direct = direct && !a.bias0.has_value() && !a.bias1.has_value();
    // Reduce mode: 1 = arrival counters + the reduce kernel beside the send kernel (default with peers), 0 = the
    // reduce kernel after the send kernel.
    int mode = (direct || a0.fuse_reduce == 0) ? 0 : 1;
    for (const auto& a : args) if (!a.dst_slot.has_value() || !a.count_matrix.has_value()) mode = 0;
    if (gated) mode = 0;
    const int num_blocks = num_sms;
    const bool weighted = a0.weighted && a0.do_expand;
    if (weighted) EP_HOST_ASSERT_MSG(a0.topk_weights.has_value(), "a weighted combine needs the top-k weights of the expanded rows");

    Multi<CombineParams> m;
    m.num_vranks = V;
    m.blocks_per_rank = num_blocks;
    std::vector<CombineResult> res(V);
    std::vector<CombineEpilogueParams> ep(V);
    std::vector<at::Tensor> touched;
    for (int v = 0; v < V; ++v) {
        auto& rt = *rts[v];
        auto& a = args[v];
        EP_HOST_ASSERT(rt.heap_->connected());
        EP_HOST_ASSERT(a.x.dim() == 2 && a.x.is_cuda() && a.x.size(1) == H && a.x.stride(1) == 1 && a.x.scalar_type() == at::kBFloat16);
        EP_HOST_ASSERT((a.x.stride(0) * 2) % 16 == 0 && reinterpret_cast<uintptr_t>(a.x.data_ptr()) % 16 == 0);
        EP_HOST_ASSERT(a.recv_src_metadata.scalar_type() == at::kInt && a.recv_src_metadata.is_contiguous() && a.recv_src_metadata.size(1) == K + 2);
        EP_HOST_ASSERT(a.topk_idx.scalar_type() == idx_dtype && a.topk_idx.is_contiguous());
        EP_HOST_ASSERT(a.do_expand == a0.do_expand && a.num_max_tokens == T_max && a.num_experts == E && a.weighted == a0.weighted);
        const int T = static_cast<int>(a.topk_idx.size(0));
        if (a.topk_weights.has_value()) {
            EP_HOST_ASSERT(a.topk_weights->scalar_type() == at::kFloat && a.topk_weights->is_contiguous());
            if (a.do_expand) EP_HOST_ASSERT(a.topk_weights->dim() == 1);
            else EP_HOST_ASSERT(a.topk_weights->dim() == 2 && a.topk_weights->size(1) == K);
        }
        CombineParams& p = m.r[v];
        p.c = rt.ctx();
        p.num_topk = K;
        p.num_max_tokens = T_max;
        p.row_bytes = H * 2;
        p.do_expand = a.do_expand;
        p.num_lanes = num_lanes;
        p.use_rank_layout = rank_layout;
        p.weighted = weighted ? 1 : 0;
        p.x = static_cast<const uint8_t*>(a.x.data_ptr());
        p.x_stride_bytes = a.x.stride(0) * 2;
        p.topk_weights = a.topk_weights.has_value() ? a.topk_weights->data_ptr<float>() : nullptr;
        p.recv_src_metadata = a.recv_src_metadata.data_ptr<int>();
        p.psum_rank = a.psum_rank.data_ptr<int>();
        // the counters of the runtime move only once the launch has happened (below)
        p.epoch = rt.combine_epoch + 1;
        const int slot = p.epoch & 1;
        p.off_comb_x = lay.combine_x[slot];
        p.off_comb_w = lay.combine_w[slot];
        p.grid_bar_base = rt.grid_bar_base;
        p.num_send_blocks = num_sms;

        auto& r = res[v];
        r.combined_x = at::empty({T, H}, opts(at::kBFloat16, device));
        if (a.topk_weights.has_value()) r.combined_topk_weights = at::empty({T, K}, opts(at::kFloat, device));
        CombineEpilogueParams& q = ep[v];
        q.num_tokens = T;
        q.num_topk = K;
        q.num_ranks = R;
        q.num_local_experts = EL;
        q.num_max_tokens = T_max;
        q.hidden = H;
        q.num_lanes = num_lanes;
        q.use_rank_layout = rank_layout;
        q.idx32 = idx_dtype == at::kInt ? 1 : 0;
        q.weighted = (weighted && !rank_layout) ? 1 : 0;     // rank layout: the senders have applied the weights
        q.region_x = rt.heap_->base() + p.off_comb_x;
        q.region_w = a.topk_weights.has_value() ? reinterpret_cast<const float*>(rt.heap_->base() + p.off_comb_w) : nullptr;
        q.topk_idx = a.topk_idx.data_ptr();
        q.bias0 = nullptr;
        q.bias1 = nullptr;
        if (a.bias0.has_value()) {
            EP_HOST_ASSERT(a.bias0->scalar_type() == at::kBFloat16 && a.bias0->is_contiguous() && a.bias0->size(0) == T && a.bias0->size(1) == H);
            q.bias0 = static_cast<const uint8_t*>(a.bias0->data_ptr());
        }
        if (a.bias1.has_value()) {
            EP_HOST_ASSERT(a.bias1->scalar_type() == at::kBFloat16 && a.bias1->is_contiguous() && a.bias1->size(0) == T && a.bias1->size(1) == H);
            q.bias1 = static_cast<const uint8_t*>(a.bias1->data_ptr());
        }
        q.combined_x = static_cast<uint8_t*>(r.combined_x.data_ptr());
        q.combined_topk_weights = r.combined_topk_weights.has_value() ? r.combined_topk_weights->data_ptr<float>() : nullptr;
        q.c = p.c;
        q.epoch = p.epoch;
        q.arrivals = nullptr;
        q.flag_chunks = lay.combine_flag_chunks;
        q.dst_slot = nullptr;
        q.count_matrix = nullptr;
        q.local_ws = rt.local_ws_;
        p.fuse_reduce = mode;
        p.direct_out = direct ? 1 : 0;
        p.num_send_warps = 0;        // filled in by the launcher
        p.flag_chunks = lay.combine_flag_chunks;
        p.off_comb_flag = lay.combine_flag;
        if (mode != 0) {
            EP_HOST_ASSERT(a.dst_slot->scalar_type() == at::kInt && a.dst_slot->is_contiguous() && a.dst_slot->dim() == 2 &&
                           a.dst_slot->size(0) == T && a.dst_slot->size(1) == R);
            EP_HOST_ASSERT(a.count_matrix->scalar_type() == at::kInt && a.count_matrix->is_contiguous() && a.count_matrix->numel() == R * R);
            touched.push_back(*a.dst_slot);
            touched.push_back(*a.count_matrix);
            q.arrivals = reinterpret_cast<const uint32_t*>(rt.heap_->base() + lay.combine_flag) +
                         static_cast<size_t>(p.epoch & 1) * R * lay.combine_flag_chunks;
            q.dst_slot = a.dst_slot->data_ptr<int>();
            q.count_matrix = a.count_matrix->data_ptr<int>();
        }
        p.red = q;
        for (const at::Tensor& t : {r.combined_x, a.x, a.recv_src_metadata, a.topk_idx, a.psum_rank}) touched.push_back(t);
        for (const auto& t : {r.combined_topk_weights, a.topk_weights, a.bias0, a.bias1})
            if (t.has_value()) touched.push_back(*t);
    }
    CombineLaunch launch;
    EP_HOST_ASSERT_MSG(plan_combine(m.r[0], num_blocks, rt0.smem_optin_, &launch), "a token row does not fit into shared memory");
    rt0.prof_record(3, stream);
    CUDA_RUNTIME_CHECK(launch_combine(m, launch, stream));
    for (int v = 0; v < V; ++v) {
        ++rts[v]->combine_epoch;
        rts[v]->grid_bar_base += num_blocks;
    }
    ++rt0.num_launches_;
    if (split) rt0.prof_record(4, stream);
    if (gated) a0.sc.previous_event_before_epilogue->stream_wait(scope.comm);
    if (!direct) {
        // Arrival-driven: the reduce runs beside the send kernel, on the SMs that kernel leaves free (it is launched as
        // a programmatic dependent, so all send blocks are resident before the first reduce block starts).
        const bool beside = mode == 1 && !split && rt0.use_pdl_;
        const int free_sms = rt0.num_device_sms_ / V - num_sms;
        const int epi_sms = beside && free_sms >= 8 ? free_sms : std::max(1, rt0.num_device_sms_ / V);
        CUDA_RUNTIME_CHECK(launch_combine_epilogue(ep.data(), V, epi_sms, stream, beside));
        ++rt0.num_launches_;
    }
    rt0.prof_record(5, stream);
    rt0.prof_valid_[1] = rt0.profiling_ != 0;
    rt0.prof_split_[1] = split;
    auto event = scope.finish(a0.sc, touched);
    for (auto& r : res) r.event = event;
    return res;
}

}  // namespace ep
