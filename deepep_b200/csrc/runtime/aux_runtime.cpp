// Host-side primitives for AGRS sessions, reduce-scatter, PP slot rings and Engram: copy-engine
// transfers into peer heaps, the flag wait / signal kernel, the slot reduction and the table gather.
// The session / ring bookkeeping that composes them lives in deepep_b200/parallel/{agrs,pp,engram}.py.
//
// Parity: csrc/elastic/buffer.hpp:210-524 of the reference (engram_write/fetch, pp_*, agrs_*, all_gather).
#include <ATen/cuda/CUDAContext.h>
#include <cstdlib>
#include <ATen/ops/empty.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "../kernels/aux_api.hpp"
#include "host_segment.hpp"
#include "runtime.hpp"
#include "stream_tools.hpp"

namespace py = pybind11;

namespace ep {

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// (wait offsets in the own heap, value to reach) then (signals: (peer, offset), value)
struct FlagSpec {
    std::vector<int64_t> wait_offsets;
    uint64_t wait_value = 0;
    std::vector<std::pair<int, int64_t>> signals;
    uint64_t signal_value = 0;
    int status_code = kStatusAgrs;
    bool signal_first = false;
};

bool stream_memops_enabled() { return stream_memops().available && stream_memops().waits; }

void flag_op(const std::vector<std::shared_ptr<Runtime>>& rts, const std::vector<FlagSpec>& specs) {
    EP_HOST_ASSERT(!rts.empty() && rts.size() == specs.size() && rts.size() <= kMaxVRanks);
    if (rts.size() == 1 && stream_memops_enabled()) {
        // one real rank per process: signal and wait as stream operations, no kernel, no SM
        auto& rt = *rts[0];
        const auto& s = specs[0];
        c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(rt.heap().device()));
        const cudaStream_t stream = cur_stream();
        auto signal = [&]() {
            for (const auto& [peer, off] : s.signals) {
                EP_HOST_ASSERT(peer >= 0 && peer < rt.num_ranks() && off >= 0 && off + 8 <= rt.num_bytes() && off % 8 == 0);
                EP_HOST_ASSERT(stream_memops().write(stream, reinterpret_cast<unsigned long long>(rt.heap().peer(peer) + off), s.signal_value, 0) == 0);
            }
        };
        auto wait = [&]() {
            for (const int64_t off : s.wait_offsets) {
                EP_HOST_ASSERT(off >= 0 && off + 8 <= rt.num_bytes() && off % 8 == 0);
                EP_HOST_ASSERT(stream_memops().wait(stream, reinterpret_cast<unsigned long long>(rt.heap().base() + off), s.wait_value, /*CU_STREAM_WAIT_VALUE_GEQ=*/0) == 0);
            }
        };
        if (s.signal_first) { signal(); wait(); } else { wait(); signal(); }
        return;
    }
    std::vector<aux::FlagOp> ops(rts.size());
    for (size_t v = 0; v < rts.size(); ++v) {
        auto& rt = *rts[v];
        const auto& s = specs[v];
        EP_HOST_ASSERT(s.wait_offsets.size() <= kMaxRanks && s.signals.size() <= kMaxRanks);
        aux::FlagOp& o = ops[v];
        o.c = rt.ctx();
        o.num_wait = static_cast<int>(s.wait_offsets.size());
        for (int i = 0; i < o.num_wait; ++i) {
            EP_HOST_ASSERT(s.wait_offsets[i] >= 0 && s.wait_offsets[i] + 8 <= rt.num_bytes() && s.wait_offsets[i] % 8 == 0);
            o.wait_ptrs[i] = reinterpret_cast<const uint64_t*>(rt.heap().base() + s.wait_offsets[i]);
        }
        o.wait_value = s.wait_value;
        o.num_signal = static_cast<int>(s.signals.size());
        for (int i = 0; i < o.num_signal; ++i) {
            const auto& [peer, off] = s.signals[i];
            EP_HOST_ASSERT(peer >= 0 && peer < rt.num_ranks() && off >= 0 && off + 8 <= rt.num_bytes() && off % 8 == 0);
            o.signal_ptrs[i] = reinterpret_cast<uint64_t*>(rt.heap().peer(peer) + off);
        }
        o.signal_value = s.signal_value;
        o.status_code = s.status_code;
        o.signal_first = s.signal_first ? 1 : 0;
    }
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(rts[0]->heap().device()));
    CUDA_RUNTIME_CHECK(aux::launch_flag_op(ops.data(), static_cast<int>(ops.size()), cur_stream()));
}

// copy-engine transfer of a contiguous tensor into a peer's heap (or the own heap with peer == rank)
void copy_to_heap(Runtime& rt, int peer, int64_t offset, const at::Tensor& src) {
    EP_HOST_ASSERT(src.is_cuda() && src.is_contiguous() && peer >= 0 && peer < rt.num_ranks());
    const int64_t bytes = src.numel() * src.element_size();
    EP_HOST_ASSERT(offset >= static_cast<int64_t>(kCtlBytes) && offset + bytes <= rt.num_bytes());
    if (bytes == 0) return;
    CUDA_RUNTIME_CHECK(cudaMemcpyAsync(rt.heap().peer(peer) + offset, src.data_ptr(), bytes, cudaMemcpyDeviceToDevice, cur_stream()));
}

// Several copy-engine transfers side by side (one side stream per copy, see FanOut). One binding call for all of them
// (the host cost of a call is of the order of a small copy).
void copy_fanout(Runtime& rt, const std::vector<std::tuple<int, int64_t, at::Tensor>>& copies) {
    if (copies.empty()) return;
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(rt.heap().device()));
    const cudaStream_t stream = cur_stream();
    if (copies.size() == 1) {
        copy_to_heap(rt, std::get<0>(copies[0]), std::get<1>(copies[0]), std::get<2>(copies[0]));
        return;
    }
    FanOut& f = fan_out(rt.heap().device());
    const int used = std::min<int>(FanOut::kFanStreams, static_cast<int>(copies.size()));
    f.fork(stream, used);
    for (size_t i = 0; i < copies.size(); ++i) {
        const auto& [peer, offset, src] = copies[i];
        EP_HOST_ASSERT(src.is_cuda() && src.is_contiguous() && peer >= 0 && peer < rt.num_ranks());
        const int64_t bytes = src.numel() * src.element_size();
        EP_HOST_ASSERT(offset >= static_cast<int64_t>(kCtlBytes) && offset + bytes <= rt.num_bytes());
        if (bytes == 0) continue;
        CUDA_RUNTIME_CHECK(cudaMemcpyAsync(rt.heap().peer(peer) + offset, src.data_ptr(), bytes, cudaMemcpyDeviceToDevice,
                                           f.streams[i % FanOut::kFanStreams]));
    }
    f.join(stream, used);
}

void copy_from_heap(Runtime& rt, int64_t offset, at::Tensor dst) {
    EP_HOST_ASSERT(dst.is_cuda() && dst.is_contiguous());
    const int64_t bytes = dst.numel() * dst.element_size();
    EP_HOST_ASSERT(offset >= static_cast<int64_t>(kCtlBytes) && offset + bytes <= rt.num_bytes());
    if (bytes == 0) return;
    CUDA_RUNTIME_CHECK(cudaMemcpyAsync(dst.data_ptr(), rt.heap().base() + offset, bytes, cudaMemcpyDeviceToDevice, cur_stream()));
}

// out = sum of `num_slots` equally shaped slots that start at `offset` in the own heap
void reduce_slots(Runtime& rt, int64_t offset, int64_t slot_stride_bytes, int num_slots, at::Tensor out) {
    EP_HOST_ASSERT(out.is_cuda() && out.is_contiguous() && (out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kFloat));
    const int64_t bytes = out.numel() * out.element_size();
    EP_HOST_ASSERT(offset >= static_cast<int64_t>(kCtlBytes) && offset + slot_stride_bytes * (num_slots - 1) + bytes <= rt.num_bytes());
    CUDA_RUNTIME_CHECK(aux::launch_reduce_slots(rt.heap().base() + offset, slot_stride_bytes, num_slots, out.data_ptr(), out.numel(),
                                                out.scalar_type() == at::kBFloat16, cur_stream()));
}

// rows of a table that is sharded over the ranks' heaps; returns (data, gathered scales or None)
std::vector<std::tuple<at::Tensor, std::optional<at::Tensor>>> engram_gather(
    const std::vector<std::shared_ptr<Runtime>>& rts, const std::vector<at::Tensor>& indices, int64_t table_offset, int entries_per_rank,
    int hidden, at::ScalarType dtype, const std::vector<std::optional<at::Tensor>>& sf_tables, bool col_major_sf, int num_sms,
    const std::vector<std::vector<std::shared_ptr<HostSegment>>>& host_tables) {
    const int V = static_cast<int>(rts.size());
    EP_HOST_ASSERT(V >= 1 && V <= kMaxVRanks && static_cast<int>(indices.size()) == V);
    auto& rt0 = *rts[0];
    const int device = rt0.heap().device();
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    const int elem = static_cast<int>(c10::elementSize(dtype));
    const int row_bytes = hidden * elem;
    EP_HOST_ASSERT(row_bytes % 16 == 0 && table_offset % 16 == 0 && table_offset >= static_cast<int64_t>(kCtlBytes));
    if (num_sms <= 0) num_sms = std::max(1, rt0.num_device_sms() / V / 4);
    std::vector<aux::EngramParams> params(V);
    std::vector<std::tuple<at::Tensor, std::optional<at::Tensor>>> out(V);
    for (int v = 0; v < V; ++v) {
        auto& rt = *rts[v];
        const auto& idx = indices[v];
        EP_HOST_ASSERT(idx.is_cuda() && idx.dim() == 2 && idx.scalar_type() == at::kInt && idx.is_contiguous());
        EP_HOST_ASSERT(!host_tables.empty() || table_offset + static_cast<int64_t>(entries_per_rank) * row_bytes <= rt.num_bytes());
        const int tokens = static_cast<int>(idx.size(0)), per_token = static_cast<int>(idx.size(1));
        auto data = at::empty({static_cast<int64_t>(tokens) * per_token, hidden}, idx.options().dtype(dtype));
        std::optional<at::Tensor> sf_out;
        aux::EngramParams& p = params[v];
        p.c = rt.ctx();
        p.indices = idx.data_ptr<int>();
        p.num_indices = tokens * per_token;
        p.entries_per_rank = entries_per_rank;
        p.row_bytes = row_bytes;
        // host_tables[v][r]: rank r's CPU segment as mapped by (virtual) rank v's process; empty = the shards are in the heaps
        const bool on_host = !host_tables.empty();
        EP_HOST_ASSERT(!on_host || (static_cast<int>(host_tables.size()) == V && static_cast<int>(host_tables[v].size()) == rt.num_ranks()));
        p.table_on_host = on_host ? 1 : 0;
        for (int r = 0; r < kMaxRanks; ++r) p.table[r] = nullptr;
        for (int r = 0; r < rt.num_ranks(); ++r) {
            if (on_host) {
                EP_HOST_ASSERT(static_cast<int64_t>(entries_per_rank) * row_bytes <= static_cast<int64_t>(host_tables[v][r]->num_bytes()));
                p.table[r] = host_tables[v][r]->device_ptr();
            } else {
                p.table[r] = rt.heap().peer(r) + table_offset;
            }
        }
        p.out = static_cast<uint8_t*>(data.data_ptr());
        p.sf_table = nullptr;
        p.sf_packs = 0;
        p.out_sf = nullptr;
        p.out_sf_token_stride = p.out_sf_pack_stride = 0;
        p.entries_per_token = std::max(per_token, 1);
        if (sf_tables[v].has_value()) {
            const auto& sf = *sf_tables[v];
            EP_HOST_ASSERT(sf.is_cuda() && sf.dim() == 2 && sf.is_contiguous() && sf.element_size() == 4);
            p.sf_table = static_cast<const uint32_t*>(sf.data_ptr());
            p.sf_packs = static_cast<int>(sf.size(1));
            const int64_t cols = static_cast<int64_t>(per_token) * p.sf_packs;
            if (col_major_sf) sf_out = at::empty({cols, align_up<int64_t>(std::max(tokens, 1), 4)}, sf.options()).t().slice(0, 0, tokens);
            else sf_out = at::empty({tokens, cols}, sf.options());
            p.out_sf = static_cast<uint32_t*>(sf_out->data_ptr());
            p.out_sf_token_stride = sf_out->stride(0);
            p.out_sf_pack_stride = sf_out->stride(1);
        }
        out[v] = {data, sf_out};
    }
    CUDA_RUNTIME_CHECK(aux::launch_engram_gather(params.data(), V, num_sms, rt0.smem_optin(), cur_stream()));
    return out;
}

}  // namespace

void register_aux_bindings(py::module_& m) {
    py::class_<FlagSpec>(m, "FlagSpec")
        .def(py::init<>())
        .def_readwrite("wait_offsets", &FlagSpec::wait_offsets)
        .def_readwrite("wait_value", &FlagSpec::wait_value)
        .def_readwrite("signals", &FlagSpec::signals)
        .def_readwrite("signal_value", &FlagSpec::signal_value)
        .def_readwrite("status_code", &FlagSpec::status_code)
        .def_readwrite("signal_first", &FlagSpec::signal_first);
    m.def("flag_op", &flag_op);
    m.def("stream_memops_enabled", &stream_memops_enabled);
    m.def("copy_to_heap", &copy_to_heap);
    m.def("copy_fanout", &copy_fanout);
    m.def("copy_from_heap", &copy_from_heap);
    m.def("reduce_slots", &reduce_slots);
    m.def("engram_gather", &engram_gather);
    py::class_<HostSegment, std::shared_ptr<HostSegment>>(m, "HostSegment")
        .def_static("create", &HostSegment::create)
        .def_static("open", &HostSegment::open)
        // the CPU segment of rank `r` inside a virtual-memory heap's address range
        .def_static("window", [](Runtime& rt, int r) {
            EP_HOST_ASSERT(rt.heap().num_cpu_bytes() > 0 && r >= 0 && r < rt.num_ranks() && rt.heap().cpu_segment(r) != nullptr);
            return HostSegment::window(rt.heap().cpu_segment(r), r == rt.rank() ? rt.heap().cpu_segment(r) : nullptr, rt.heap().num_cpu_bytes());
        })
        .def_property_readonly("name", &HostSegment::name)
        .def_property_readonly("num_bytes", &HostSegment::num_bytes)
        .def("device_ptr", [](const HostSegment& s) { return reinterpret_cast<int64_t>(s.device_ptr()); })
        .def("release", &HostSegment::release)
        // device tensor -> segment (asynchronous on the current stream) and a CPU view for checks
        .def("copy_from_device", [](HostSegment& s, const at::Tensor& src, int64_t offset) {
            EP_HOST_ASSERT(src.is_cuda() && src.is_contiguous() && offset >= 0);
            const int64_t bytes = src.numel() * src.element_size();
            EP_HOST_ASSERT(offset + bytes <= static_cast<int64_t>(s.num_bytes()));
            // (a segment inside a heap window is addressed through its device mapping)
            uint8_t* dst = s.host_ptr() != nullptr ? s.host_ptr() : s.device_ptr();
            CUDA_RUNTIME_CHECK(cudaMemcpyAsync(dst + offset, src.data_ptr(), bytes, cudaMemcpyDefault, cur_stream()));
        })
        .def("as_tensor", [](const std::shared_ptr<HostSegment>& s) {
            return at::from_blob(s->host_ptr(), {static_cast<int64_t>(s->num_bytes())}, [s](void*) {}, at::TensorOptions().dtype(at::kByte));
        });
    m.attr("CTL_AGRS_SIGNALS") = static_cast<int64_t>(kCtlAgrsSignals * 8);
    m.attr("CTL_PP_SIGNALS") = static_cast<int64_t>(kCtlPPSignals * 8);
    m.attr("MAX_AGRS_INFLIGHT") = kMaxAgrsInflight;
    m.attr("STATUS_AGRS") = static_cast<int>(kStatusAgrs);
    m.attr("STATUS_PP") = static_cast<int>(kStatusPP);
}

}  // namespace ep
