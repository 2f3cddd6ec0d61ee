// Python bindings of the native runtime (module deepep_b200._C).
//
// Parity: csrc/python_api.cpp:22-39 and the pybind blocks at csrc/elastic/buffer.hpp:1346-1380,
// csrc/legacy/buffer.hpp:1751-1792 of the reference.
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "runtime.hpp"

namespace py = pybind11;
using namespace ep;

void register_extra_bindings(py::module_& m);   // low latency, AGRS, PP, ops (other translation units)

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "B200-native expert-parallel communication runtime";

    py::register_exception<EPException>(m, "EPException");
    static py::exception<EPTimeoutError> timeout_exc(m, "EPTimeoutError");
    py::register_exception_translator([](std::exception_ptr p) {
        try {
            if (p) std::rethrow_exception(p);
        } catch (const EPTimeoutError& e) {
            timeout_exc(e.what());
        }
    });

    m.attr("MAX_RANKS") = kMaxRanks;
    m.attr("MAX_EXPERTS") = kMaxExperts;
    m.attr("MAX_LOCAL_EXPERTS") = kMaxLocalExperts;
    m.attr("MAX_TOPK") = kMaxTopk;
    m.attr("MAX_VRANKS") = kMaxVRanks;
    m.attr("HEAP_ALIGNMENT") = static_cast<int64_t>(kHeapAlignment);
    m.attr("CONTROL_BYTES") = static_cast<int64_t>(kCtlBytes);


    py::class_<EventHandle>(m, "EventHandle")
        .def(py::init<>())
        .def("current_stream_wait", &EventHandle::current_stream_wait);

    py::class_<StreamControl>(m, "StreamControl")
        .def(py::init<>())
        .def_readwrite("previous_event", &StreamControl::previous_event)
        .def_readwrite("previous_event_before_epilogue", &StreamControl::previous_event_before_epilogue)
        .def_readwrite("async_with_compute_stream", &StreamControl::async_with_compute_stream)
        .def_readwrite("allocate_on_comm_stream", &StreamControl::allocate_on_comm_stream);

    py::class_<DispatchArgs>(m, "DispatchArgs")
        .def(py::init<>())
        .def_readwrite("x", &DispatchArgs::x)
        .def_readwrite("sf", &DispatchArgs::sf)
        .def_readwrite("topk_idx", &DispatchArgs::topk_idx)
        .def_readwrite("topk_weights", &DispatchArgs::topk_weights)
        .def_readwrite("cumulative_stats", &DispatchArgs::cumulative_stats)
        .def_readwrite("num_experts", &DispatchArgs::num_experts)
        .def_readwrite("num_max_tokens", &DispatchArgs::num_max_tokens)
        .def_readwrite("expert_alignment", &DispatchArgs::expert_alignment)
        .def_readwrite("num_sms", &DispatchArgs::num_sms)
        .def_readwrite("quant_mode", &DispatchArgs::quant_mode)
        .def_readwrite("do_expand", &DispatchArgs::do_expand)
        .def_readwrite("do_zero_padding", &DispatchArgs::do_zero_padding)
        .def_readwrite("do_cpu_sync", &DispatchArgs::do_cpu_sync)
        .def_readwrite("zero_copy", &DispatchArgs::zero_copy)
        .def_readwrite("num_worst_tokens", &DispatchArgs::num_worst_tokens)
        .def_readwrite("col_major_sf", &DispatchArgs::col_major_sf)
        .def_readwrite("cached", &DispatchArgs::cached)
        .def_readwrite("h_token_slot", &DispatchArgs::h_token_slot)
        .def_readwrite("h_pair_row", &DispatchArgs::h_pair_row)
        .def_readwrite("h_psum_rank", &DispatchArgs::h_psum_rank)
        .def_readwrite("h_psum_expert", &DispatchArgs::h_psum_expert)
        .def_readwrite("h_num_unaligned", &DispatchArgs::h_num_unaligned)
        .def_readwrite("h_recv_src_metadata", &DispatchArgs::h_recv_src_metadata)
        .def_readwrite("h_num_recv_tokens", &DispatchArgs::h_num_recv_tokens)
        .def_readwrite("h_num_expanded_tokens", &DispatchArgs::h_num_expanded_tokens)
        .def_readwrite("sc", &DispatchArgs::sc);

    py::class_<DispatchResult>(m, "DispatchResult")
        .def_readonly("recv_x", &DispatchResult::recv_x)
        .def_readonly("recv_sf", &DispatchResult::recv_sf)
        .def_readonly("recv_topk_idx", &DispatchResult::recv_topk_idx)
        .def_readonly("recv_topk_weights", &DispatchResult::recv_topk_weights)
        .def_readonly("token_slot", &DispatchResult::token_slot)
        .def_readonly("pair_row", &DispatchResult::pair_row)
        .def_readonly("psum_rank", &DispatchResult::psum_rank)
        .def_readonly("psum_expert", &DispatchResult::psum_expert)
        .def_readonly("num_unaligned", &DispatchResult::num_unaligned)
        .def_readonly("recv_src_metadata", &DispatchResult::recv_src_metadata)
        .def_readonly("count_matrix", &DispatchResult::count_matrix)
        .def_readonly("num_recv_tokens", &DispatchResult::num_recv_tokens)
        .def_readonly("num_expanded_tokens", &DispatchResult::num_expanded_tokens)
        .def_readonly("num_sms", &DispatchResult::num_sms)
        .def_readonly("num_recv_tokens_per_expert_list", &DispatchResult::num_recv_tokens_per_expert_list)
        .def_readonly("event", &DispatchResult::event);

    py::class_<CombineArgs>(m, "CombineArgs")
        .def(py::init<>())
        .def_readwrite("x", &CombineArgs::x)
        .def_readwrite("topk_weights", &CombineArgs::topk_weights)
        .def_readwrite("bias0", &CombineArgs::bias0)
        .def_readwrite("bias1", &CombineArgs::bias1)
        .def_readwrite("recv_src_metadata", &CombineArgs::recv_src_metadata)
        .def_readwrite("topk_idx", &CombineArgs::topk_idx)
        .def_readwrite("psum_rank", &CombineArgs::psum_rank)
        .def_readwrite("num_experts", &CombineArgs::num_experts)
        .def_readwrite("num_max_tokens", &CombineArgs::num_max_tokens)
        .def_readwrite("num_sms", &CombineArgs::num_sms)
        .def_readwrite("do_expand", &CombineArgs::do_expand)
        .def_readwrite("allow_multiple_reduction", &CombineArgs::allow_multiple_reduction)
        .def_readwrite("weighted", &CombineArgs::weighted)
        .def_readwrite("dst_slot", &CombineArgs::dst_slot)
        .def_readwrite("count_matrix", &CombineArgs::count_matrix)
        .def_readwrite("fuse_reduce", &CombineArgs::fuse_reduce)
        .def_readwrite("sc", &CombineArgs::sc);

    py::class_<CombineResult>(m, "CombineResult")
        .def_readonly("combined_x", &CombineResult::combined_x)
        .def_readonly("combined_topk_weights", &CombineResult::combined_topk_weights)
        .def_readonly("event", &CombineResult::event);

    py::class_<Runtime, std::shared_ptr<Runtime>>(m, "Runtime")
        .def(py::init<int, int, int64_t, double, double, int64_t>(), py::arg("rank"), py::arg("num_ranks"), py::arg("num_bytes"),
             py::arg("gpu_timeout_secs") = 100.0, py::arg("cpu_timeout_secs") = 300.0, py::arg("num_cpu_bytes") = 0)
        .def("finish_export", &Runtime::finish_export)
        .def("heap_is_vmm", &Runtime::heap_is_vmm)
        .def_static("heap_backend_is_vmm", &Runtime::heap_backend_is_vmm)
        .def("destroy", &Runtime::destroy)
        .def("export_handle", [](const Runtime& rt) { return py::bytes(rt.export_handle()); })
        .def("open_peers", [](Runtime& rt, const std::vector<py::bytes>& handles) {
            std::vector<std::string> raw;
            for (const auto& h : handles) raw.push_back(static_cast<std::string>(h));
            rt.open_peers(raw);
        })
        .def_static("connect_local", &Runtime::connect_local)
        .def("status", &Runtime::status)
        .def("check_status", &Runtime::check_status)
        .def("clear_status", &Runtime::clear_status)
        .def("set_gpu_timeout", &Runtime::set_gpu_timeout)
        .def("enable_profiling", &Runtime::enable_profiling)
        .def("num_kernel_launches", &Runtime::num_kernel_launches)
        .def("last_timings", &Runtime::last_timings)
        .def("last_dispatch_phases", &Runtime::last_dispatch_phases)
        .def("last_timeline", &Runtime::last_timeline)
        .def("rank", &Runtime::rank)
        .def("num_ranks", &Runtime::num_ranks)
        .def("num_bytes", &Runtime::num_bytes)
        .def("num_device_sms", &Runtime::num_device_sms)
        .def("heap_tensor", &Runtime::heap_tensor)
        .def("comm_stream_ptr", [](const Runtime& rt) { return reinterpret_cast<uintptr_t>(rt.comm_stream().stream()); })
        .def("comm_stream_id", [](const Runtime& rt) {
            const auto s = rt.comm_stream();
            return std::make_tuple(static_cast<int64_t>(s.id()), static_cast<int64_t>(s.device_index()),
                                   static_cast<int64_t>(s.device_type()));
        })
        // The drivers may block on the host for a long time (the wait for the received counts, a stream
        // synchronisation): they run without the GIL so that Python threads of this process -- the heartbeat of the
        // failure detector among them -- keep running meanwhile.
        .def_static("barrier", &Runtime::barrier, py::arg("runtimes"), py::arg("use_comm_stream") = true, py::arg("with_cpu_sync") = false,
                    py::call_guard<py::gil_scoped_release>())
        .def_static("dispatch", &Runtime::dispatch, py::call_guard<py::gil_scoped_release>())
        .def_static("combine", &Runtime::combine, py::call_guard<py::gil_scoped_release>())
        .def_static("ht_buffer_size", &Runtime::ht_buffer_size);

    // A host-side wait of the given length without the GIL: what a driver does while it spins on the received counts
    // or synchronises a stream. Lets a CPU test check that Python threads (the heartbeat) keep running meanwhile.
    m.def("debug_blocking_host_wait", [](double seconds) {
        const auto end = std::chrono::steady_clock::now() + std::chrono::duration<double>(seconds);
        volatile uint64_t spins = 0;
        while (std::chrono::steady_clock::now() < end) ++spins;
        return static_cast<uint64_t>(spins);
    }, py::call_guard<py::gil_scoped_release>());

    register_extra_bindings(m);
}
