// Host drivers of the low-latency dispatch / combine kernels and of the rank-mask API.
//
// Parity: csrc/legacy/buffer.hpp:1431-1748 of the reference (clean_low_latency_buffer,
// low_latency_dispatch, low_latency_combine, get_next_low_latency_combine_buffer, mask API) and
// csrc/legacy/config.hpp:122-188 (LowLatencyLayout, size hint).
#include <ATen/ops/empty.h>
#include <ATen/ops/from_blob.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "runtime.hpp"

namespace py = pybind11;

namespace ep {

namespace {

at::TensorOptions opts(at::ScalarType dtype, int device) {
    return at::TensorOptions().dtype(dtype).device(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device)));
}

struct LLDispatchIO {
    at::Tensor x, topk_idx;
    std::optional<at::Tensor> cumulative_stats, wait_stats;
    // outputs (allocated by the first call, passed again by the receive hook)
    at::Tensor packed_recv_x, packed_recv_count, src_info, layout_range;
    std::optional<at::Tensor> packed_recv_sf;
};

struct LLCombineIO {
    at::Tensor x, topk_idx, topk_weights, src_info, layout_range, combined_x;
    std::optional<at::Tensor> wait_stats;
    bool use_logfmt = false;   // send rows in the 10-bit log format (same for all emulated ranks of a call)
};

int64_t ll_buffer_size(int num_ranks, int num_max_tokens, int hidden, int num_experts) {
    return static_cast<int64_t>(ll_layout(num_ranks, num_max_tokens, hidden, num_experts).end);
}

// Launch-stream policy of the low-latency calls: with a receive hook the kernels run on the caller's
// stream (the caller overlaps them itself), otherwise on the communication stream.
struct LLStreams {
    at::cuda::CUDAStream compute, launch;
    bool on_comm;
    LLStreams(Runtime& rt, bool use_compute) : compute(at::cuda::getCurrentCUDAStream()), launch(use_compute ? compute : rt.comm_stream()), on_comm(!use_compute) {
        if (on_comm) stream_wait(launch, compute);
    }
    std::optional<EventHandle> finish(bool async_finish) {
        if (async_finish) return EventHandle(launch);
        if (on_comm) stream_wait(compute, launch);
        return std::nullopt;
    }
};

std::optional<EventHandle> ll_dispatch(const std::vector<std::shared_ptr<Runtime>>& rts, std::vector<LLDispatchIO*>& ios,
                                       int num_max_tokens, int num_experts, bool use_fp8, bool round_scale, bool use_ue8m0,
                                       int phases, int num_sms, bool shrink, bool async_finish, bool on_compute_stream) {
    const int V = static_cast<int>(rts.size());
    EP_HOST_ASSERT(V >= 1 && V <= kMaxVRanks && static_cast<int>(ios.size()) == V);
    auto& rt0 = *rts[0];
    const int device = rt0.heap().device();
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    LLStreams streams(rt0, on_compute_stream);
    const int R = rt0.num_ranks();
    const int H = static_cast<int>(ios[0]->x.size(1)), K = static_cast<int>(ios[0]->topk_idx.size(1));
    const int E = num_experts, EL = E / R, Tm = num_max_tokens;
    EP_HOST_ASSERT(E % R == 0 && E <= kMaxExperts && EL <= kMaxLocalExperts && K <= kMaxLLTopk && Tm >= 1 && Tm < 65536);
    EP_HOST_ASSERT_MSG(H % 128 == 0 && H <= 8192, "low-latency dispatch needs hidden % 128 == 0 and hidden <= 8192");
    if (use_ue8m0) EP_HOST_ASSERT_MSG(round_scale && use_fp8 && H % 512 == 0, "UE8M0 scales need round_scale, FP8 and hidden % 512 == 0");
    const LLLayout lay = ll_layout(R, Tm, H, E);
    EP_HOST_ASSERT_MSG(lay.end <= rt0.heap().num_bytes(), "symmetric buffer too small for low-latency mode");
    if (num_sms <= 0) num_sms = rt0.num_device_sms();   // latency-bound: one token / one (expert, source) pair per block
    if (num_sms * V > rt0.num_device_sms()) num_sms = rt0.num_device_sms() / V;

    Multi<LLDispatchParams> m;
    m.num_vranks = V;
    m.blocks_per_rank = num_sms;
    for (int v = 0; v < V; ++v) {
        auto& rt = *rts[v];
        auto& io = *ios[v];
        EP_HOST_ASSERT(io.x.scalar_type() == at::kBFloat16 && io.x.is_contiguous() && io.x.size(1) == H && io.x.size(0) <= Tm);
        EP_HOST_ASSERT((io.topk_idx.scalar_type() == at::kLong || io.topk_idx.scalar_type() == at::kInt) && io.topk_idx.is_contiguous() && io.topk_idx.size(0) == io.x.size(0) && io.topk_idx.size(1) == K);
        if (!io.packed_recv_x.defined()) {
            io.packed_recv_x = at::empty({EL, R * Tm, H}, opts(use_fp8 ? at::kFloat8_e4m3fn : at::kBFloat16, device));
            io.packed_recv_count = at::empty({EL}, opts(at::kInt, device));
            io.src_info = at::empty({EL, R * Tm}, opts(at::kInt, device));
            io.layout_range = at::empty({EL, R}, opts(at::kLong, device));
            if (use_fp8) {
                if (use_ue8m0) io.packed_recv_sf = at::empty({EL, H / 512, R * Tm}, opts(at::kInt, device)).transpose(1, 2);
                else io.packed_recv_sf = at::empty({EL, H / 128, R * Tm}, opts(at::kFloat, device)).transpose(1, 2);
            }
        }
        LLDispatchParams& p = m.r[v];
        p.c = rt.ctx();
        p.num_tokens = static_cast<int>(io.x.size(0));
        p.hidden = H;
        p.num_topk = K;
        p.num_experts = E;
        p.num_local_experts = EL;
        p.num_max_tokens = Tm;
        p.use_fp8 = use_fp8;
        p.round_scale = round_scale;
        p.use_ue8m0 = use_ue8m0;
        p.phases = phases;
        p.shrink = shrink;
        p.x = static_cast<const uint8_t*>(io.x.data_ptr());
        p.topk_idx = io.topk_idx.data_ptr();
        p.idx32 = io.topk_idx.scalar_type() == at::kInt ? 1 : 0;
        p.packed_recv_x = static_cast<uint8_t*>(io.packed_recv_x.data_ptr());
        p.packed_recv_sf = io.packed_recv_sf.has_value() ? static_cast<uint8_t*>(io.packed_recv_sf->data_ptr()) : nullptr;
        p.packed_recv_src_info = io.src_info.data_ptr<int>();
        p.packed_recv_layout_range = io.layout_range.data_ptr<int64_t>();
        p.packed_recv_count = io.packed_recv_count.data_ptr<int>();
        p.cumulative_stats = io.cumulative_stats.has_value() ? io.cumulative_stats->data_ptr<int>() : nullptr;
        p.wait_stats = io.wait_stats.has_value() ? io.wait_stats->data_ptr<int64_t>() : nullptr;
        for (int h = 0; h < 2; ++h) {
            p.off_recv_x[h] = lay.recv_x[h];
            p.off_recv_count[h] = lay.recv_count[h];
        }
    }
    CUDA_RUNTIME_CHECK(launch_ll_dispatch(m, num_sms, streams.launch.stream()));
    return streams.finish(async_finish);
}

std::optional<EventHandle> ll_combine(const std::vector<std::shared_ptr<Runtime>>& rts, std::vector<LLCombineIO*>& ios,
                                      int num_max_tokens, int num_experts, int phases, int num_sms, bool shrink,
                                      bool async_finish, bool on_compute_stream) {
    const int V = static_cast<int>(rts.size());
    EP_HOST_ASSERT(V >= 1 && V <= kMaxVRanks && static_cast<int>(ios.size()) == V);
    auto& rt0 = *rts[0];
    const int device = rt0.heap().device();
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    LLStreams streams(rt0, on_compute_stream);
    const int R = rt0.num_ranks();
    const int H = static_cast<int>(ios[0]->x.size(2)), K = static_cast<int>(ios[0]->topk_idx.size(1));
    const int E = num_experts, EL = E / R, Tm = num_max_tokens;
    EP_HOST_ASSERT(E % R == 0 && K <= kMaxLLTopk && K <= kMaxTopk && (H * 2) % 16 == 0);
    EP_HOST_ASSERT_MSG(!ios[0]->use_logfmt || H % 128 == 0, "LogFMT needs a hidden size that is a multiple of 128");
    const LLLayout lay = ll_layout(R, Tm, H, E);
    EP_HOST_ASSERT_MSG(lay.end <= rt0.heap().num_bytes(), "symmetric buffer too small for low-latency mode");
    if (num_sms <= 0) num_sms = rt0.num_device_sms();   // latency-bound: one token / one (expert, source) pair per block
    if (num_sms * V > rt0.num_device_sms()) num_sms = rt0.num_device_sms() / V;

    Multi<LLCombineParams> m;
    m.num_vranks = V;
    m.blocks_per_rank = num_sms;
    for (int v = 0; v < V; ++v) {
        auto& rt = *rts[v];
        auto& io = *ios[v];
        EP_HOST_ASSERT(io.x.scalar_type() == at::kBFloat16 && io.x.is_contiguous() && io.x.dim() == 3 && io.x.size(0) == EL &&
                       io.x.size(1) == R * Tm && io.x.size(2) == H);
        EP_HOST_ASSERT((io.topk_idx.scalar_type() == at::kLong || io.topk_idx.scalar_type() == at::kInt) && io.topk_idx.is_contiguous());
        EP_HOST_ASSERT(io.topk_weights.scalar_type() == at::kFloat && io.topk_weights.is_contiguous() && io.topk_weights.size(1) == K);
        const int T = static_cast<int>(io.topk_idx.size(0));
        if (!io.combined_x.defined()) io.combined_x = at::empty({T, H}, opts(at::kBFloat16, device));
        EP_HOST_ASSERT(io.combined_x.scalar_type() == at::kBFloat16 && io.combined_x.is_contiguous() && io.combined_x.size(0) == T && io.combined_x.size(1) == H);
        LLCombineParams& p = m.r[v];
        p.c = rt.ctx();
        p.num_tokens = T;
        p.hidden = H;
        p.num_topk = K;
        p.num_experts = E;
        p.num_local_experts = EL;
        p.num_max_tokens = Tm;
        p.phases = phases;
        p.shrink = shrink;
        p.use_logfmt = ios[0]->use_logfmt ? 1 : 0;
        p.x = static_cast<const uint8_t*>(io.x.data_ptr());
        p.topk_idx = io.topk_idx.data_ptr();
        p.idx32 = io.topk_idx.scalar_type() == at::kInt ? 1 : 0;
        p.topk_weights = io.topk_weights.data_ptr<float>();
        p.src_info = io.src_info.data_ptr<int>();
        p.layout_range = io.layout_range.data_ptr<int64_t>();
        p.combined_x = static_cast<uint8_t*>(io.combined_x.data_ptr());
        p.wait_stats = io.wait_stats.has_value() ? io.wait_stats->data_ptr<int64_t>() : nullptr;
        for (int h = 0; h < 2; ++h) {
            p.off_combine_x[h] = lay.combine_x[h];
            p.off_combine_flag[h] = lay.combine_flag[h];
        }
    }
    CUDA_RUNTIME_CHECK(launch_ll_combine(m, num_sms, rt0.smem_optin(), streams.launch.stream()));
    return streams.finish(async_finish);
}

// bf16 [EL, R * T_max, H] view of the staging half that the NEXT combine send may read from
at::Tensor ll_next_combine_buffer(Runtime& rt, int num_max_tokens, int hidden, int num_experts) {
    const int R = rt.num_ranks(), EL = num_experts / R;
    const LLLayout lay = ll_layout(R, num_max_tokens, hidden, num_experts);
    EP_HOST_ASSERT(lay.end <= rt.heap().num_bytes());
    uint64_t calls = 0;
    CUDA_RUNTIME_CHECK(cudaMemcpy(&calls, rt.local_ws() + kWsLLCalls + 2, sizeof(calls), cudaMemcpyDeviceToHost));
    const int half = static_cast<int>((calls + 1) & 1);
    return at::from_blob(rt.heap().base() + lay.send_x[half], {EL, R * num_max_tokens, hidden}, opts(at::kBFloat16, rt.heap().device()));
}

void ll_mask_update(Runtime& rt, int rank, bool mask) {
    CUDA_RUNTIME_CHECK(ll_update_mask(rt.local_ws(), rank, mask ? 1 : 0, at::cuda::getCurrentCUDAStream().stream()));
}
void ll_mask_clean(Runtime& rt) {
    CUDA_RUNTIME_CHECK(ll_update_mask(rt.local_ws(), -1, 0, at::cuda::getCurrentCUDAStream().stream()));
}
void ll_mask_query(Runtime& rt, at::Tensor out) {
    EP_HOST_ASSERT(out.scalar_type() == at::kInt && out.is_cuda() && out.numel() >= rt.num_ranks());
    CUDA_RUNTIME_CHECK(ll_query_mask(rt.local_ws(), out.data_ptr<int>(), rt.num_ranks(), at::cuda::getCurrentCUDAStream().stream()));
}

// Routing layout of `topk_idx` on the communication stream (legacy Buffer.get_dispatch_layout).
std::tuple<at::Tensor, at::Tensor, at::Tensor, std::optional<EventHandle>> get_dispatch_layout(
    Runtime& rt, const at::Tensor& topk_idx, int num_experts, std::optional<EventHandle> previous_event, bool async_finish,
    bool allocate_on_comm_stream) {
    EP_HOST_ASSERT(topk_idx.dim() == 2 && topk_idx.is_contiguous() && (topk_idx.scalar_type() == at::kLong || topk_idx.scalar_type() == at::kInt) && topk_idx.is_cuda());
    EP_HOST_ASSERT(num_experts > 0 && num_experts % rt.num_ranks() == 0 && num_experts <= kMaxExperts);
    const int device = rt.heap().device();
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    const auto compute = at::cuda::getCurrentCUDAStream();
    const auto comm = rt.comm_stream();
    if (allocate_on_comm_stream) at::cuda::setCurrentCUDAStream(comm);
    if (previous_event.has_value()) previous_event->stream_wait(comm);
    else stream_wait(comm, compute);
    const int T = static_cast<int>(topk_idx.size(0)), K = static_cast<int>(topk_idx.size(1)), R = rt.num_ranks();
    auto per_rank = at::empty({R}, opts(at::kInt, device));
    auto per_expert = at::empty({num_experts}, opts(at::kInt, device));
    auto in_rank = at::empty({T, R}, opts(at::kBool, device));
    CUDA_RUNTIME_CHECK(launch_dispatch_layout(topk_idx.data_ptr(), topk_idx.scalar_type() == at::kInt, T, K, R, num_experts, per_rank.data_ptr<int>(),
                                              per_expert.data_ptr<int>(), in_rank.data_ptr<bool>(), comm.stream()));
    std::optional<EventHandle> event;
    if (async_finish) {
        event = EventHandle(comm);
        for (const auto& t : {topk_idx, per_rank, per_expert, in_rank}) {
            t.record_stream(comm);
            if (allocate_on_comm_stream) t.record_stream(compute);
        }
    } else {
        stream_wait(compute, comm);
    }
    if (allocate_on_comm_stream) at::cuda::setCurrentCUDAStream(compute);
    return {per_rank, per_expert, in_rank, event};
}

}  // namespace

void register_ll_bindings(py::module_& m) {
    py::class_<LLDispatchIO>(m, "LLDispatchIO")
        .def(py::init<>())
        .def_readwrite("x", &LLDispatchIO::x)
        .def_readwrite("topk_idx", &LLDispatchIO::topk_idx)
        .def_readwrite("cumulative_stats", &LLDispatchIO::cumulative_stats)
        .def_readwrite("wait_stats", &LLDispatchIO::wait_stats)
        .def_readwrite("packed_recv_x", &LLDispatchIO::packed_recv_x)
        .def_readwrite("packed_recv_sf", &LLDispatchIO::packed_recv_sf)
        .def_readwrite("packed_recv_count", &LLDispatchIO::packed_recv_count)
        .def_readwrite("src_info", &LLDispatchIO::src_info)
        .def_readwrite("layout_range", &LLDispatchIO::layout_range);
    py::class_<LLCombineIO>(m, "LLCombineIO")
        .def(py::init<>())
        .def_readwrite("x", &LLCombineIO::x)
        .def_readwrite("topk_idx", &LLCombineIO::topk_idx)
        .def_readwrite("topk_weights", &LLCombineIO::topk_weights)
        .def_readwrite("src_info", &LLCombineIO::src_info)
        .def_readwrite("layout_range", &LLCombineIO::layout_range)
        .def_readwrite("combined_x", &LLCombineIO::combined_x)
        .def_readwrite("wait_stats", &LLCombineIO::wait_stats)
        .def_readwrite("use_logfmt", &LLCombineIO::use_logfmt);
    m.def("get_dispatch_layout", &get_dispatch_layout);
    m.def("ll_buffer_size", &ll_buffer_size);
    m.def("ll_dispatch", &ll_dispatch);
    m.def("ll_combine", &ll_combine);
    m.def("ll_next_combine_buffer", &ll_next_combine_buffer);
    m.def("ll_mask_update", &ll_mask_update);
    m.def("ll_mask_clean", &ll_mask_clean);
    m.def("ll_mask_query", &ll_mask_query);
    m.attr("LL_SEND") = static_cast<int>(kLLSend);
    m.attr("LL_RECV") = static_cast<int>(kLLRecv);
}

}  // namespace ep
