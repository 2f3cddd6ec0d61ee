// Host drivers of the fused tensor-parallel operators (all-gather -> GEMM, GEMM -> reduce-scatter).
#include <ATen/cuda/CUDAContext.h>
#include <cmath>
#include <cstdlib>
#include <ATen/ops/empty.h>
#include <ATen/ops/zeros.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "../kernels/aux_api.hpp"
#include "../kernels/tp_api.hpp"
#include "runtime.hpp"
#include "stream_tools.hpp"

namespace py = pybind11;

namespace ep {

namespace {

at::Tensor& tp_status(int device) {
    static std::map<int, at::Tensor> words;
    auto it = words.find(device);
    if (it == words.end())
        it = words.emplace(device, at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device))))).first;
    return it->second;
}

int tp_check_status() {
    int device = 0;
    CUDA_RUNTIME_CHECK(cudaGetDevice(&device));
    return tp_status(device).item<int>();
}

// C_r[R * Ml, N] = gather(A)[R * Ml, K] * B_r[N, K]^T, one launch for all listed (virtual) ranks.
// `gather_offsets` = the two halves of the gather buffer inside every heap (bytes from the heap base).
// `push`: 0 = decide here, 1 = push CTAs inside the kernel (bulk stores from SMs), 2 = copy engines: the shard goes out
// in groups of row chunks with one 2-D copy per peer and group on side streams, every chunk's arrival flag is a 64-bit
// stream write behind its copy, and ALL SMs run GEMM tiles, whose loader waits for those flags exactly as it waits for
// the flags of the push CTAs. The entry handshake (a peer's gather half may only be overwritten once that peer has
// entered this call) then runs as a one-block flag kernel ahead of the GEMM.
std::vector<at::Tensor> tp_ag_gemm(const std::vector<std::shared_ptr<Runtime>>& rts, const std::vector<at::Tensor>& a_local,
                                   const std::vector<at::Tensor>& b, const std::vector<int64_t>& gather_offsets, int num_comm_ctas,
                                   int num_sms, int push) {
    const int V = static_cast<int>(rts.size());
    EP_HOST_ASSERT(V >= 1 && V <= gemm::kTpMaxVRanks && static_cast<int>(a_local.size()) == V && static_cast<int>(b.size()) == V);
    EP_HOST_ASSERT(gather_offsets.size() == 2);
    auto& rt0 = *rts[0];
    const int device = rt0.heap().device();
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    const int R = rt0.num_ranks();
    const int Ml = static_cast<int>(a_local[0].size(0)), K = static_cast<int>(a_local[0].size(1)), N = static_cast<int>(b[0].size(0));
    const uint64_t half_bytes = static_cast<uint64_t>(R) * Ml * K * 2;
    if (num_sms <= 0) num_sms = rt0.num_device_sms() / V;
    // Copy engines need one real rank per process (the kernels of emulated ranks share one GPU and one stream), the
    // driver's stream writes, and at most 63 row chunks per source (flag word 63 is the entry word).
    const bool ce_possible = V == 1 && R > 1 && stream_memops().available && Ml % 128 == 0 && Ml / 128 <= 63;
    static const int env_push = [] { const char* v = std::getenv("EP_TP_PUSH"); return v == nullptr ? 0 : (v[0] == 's' ? 1 : (v[0] == 'c' ? 2 : 0)); }();
    if (push == 0) push = env_push;
    if (push == 0) {
        // Copy engines cost this call about 4 (R - 1) + 20 driver calls of 2.5 us on the host (measured: 539 us at TP8
        // before the copies and flag writes were batched); they pay where the GEMM outlasts that comfortably (TP2: 724
        // against 740 us, TP4: 427 against 459 us with push CTAs), else the push CTAs take the shard out.
        const double gemm_us = 2.0 * R * Ml * N * K / 1.4e15 * 1e6;
        const double host_us = 2.5 * (4.0 * (R - 1) + 20.0);
        push = gemm_us >= 2.0 * host_us ? 2 : 1;
    }
    const bool use_ce = push == 2 && ce_possible;
    if (use_ce) num_comm_ctas = 0;
    if (num_comm_ctas <= 0 && R > 1 && !use_ce) {
        // As few push CTAs as move the shard out within about half of the GEMM's time (every CTA taken from the GEMM
        // costs it 1 / #SMs of its rate): a push CTA was measured at about 40 GB/s, the GEMM at about 1.4 PFLOP/s.
        const double push_cta_seconds = static_cast<double>(R - 1) * Ml * K * 2 / 40e9;
        const double gemm_seconds = 2.0 * R * Ml * N * K / 1.4e15;
        int n = static_cast<int>(std::ceil(push_cta_seconds / (0.5 * gemm_seconds)));
        n = (std::max(8, std::min(n, 16)) + 1) & ~1;     // (four push CTAs were measured far slower than eight at TP2;
                                                         //  sixteen beat eight and thirty-two at TP4 and TP8)
        num_comm_ctas = std::min(n, std::max(2, (num_sms / 4) & ~1));
    }
    if (R == 1) num_comm_ctas = 0;
    std::vector<gemm::AgGemmParams> params(V);
    std::vector<const void*> bptr(V), gptr(V);
    std::vector<at::Tensor> outs(V);
    for (int v = 0; v < V; ++v) {
        auto& rt = *rts[v];
        const auto& a = a_local[v];
        EP_HOST_ASSERT(a.scalar_type() == at::kBFloat16 && a.dim() == 2 && a.stride(1) == 1 && a.size(0) == Ml && a.size(1) == K);
        EP_HOST_ASSERT(b[v].scalar_type() == at::kBFloat16 && b[v].is_contiguous() && b[v].size(0) == N && b[v].size(1) == K);
        EP_HOST_ASSERT((a.stride(0) * 2) % 16 == 0 && reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 == 0);
        const uint32_t epoch = ++rt.tp_ag_epoch;
        const uint64_t off = static_cast<uint64_t>(gather_offsets[epoch & 1]);
        EP_HOST_ASSERT_MSG(off + half_bytes <= rt.heap().num_bytes() && off >= kCtlBytes, "gather buffer does not fit the heap");
        outs[v] = at::empty({static_cast<int64_t>(R) * Ml, N}, a.options());
        gemm::AgGemmParams& p = params[v];
        p.c = rt.ctx();
        p.rows_per_rank = Ml;
        p.N = N;
        p.K = K;
        p.a_local = static_cast<const uint8_t*>(a.data_ptr());
        p.a_stride_bytes = a.stride(0) * 2;
        p.C = reinterpret_cast<__nv_bfloat16*>(outs[v].data_ptr());
        p.ldc = N;
        p.off_gather = off;
        p.epoch = epoch;
        p.num_comm_ctas = num_comm_ctas;
        p.error = tp_status(device).data_ptr<int>();
        bptr[v] = b[v].data_ptr();
        gptr[v] = rt.heap().base() + off;
    }
    const cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
    if (!use_ce) {
        CUDA_RUNTIME_CHECK(gemm::launch_ag_gemm(params.data(), bptr.data(), gptr.data(), V, num_sms, stream));
        return outs;
    }
    auto& rt = rt0;
    const gemm::AgGemmParams& p = params[0];
    const int me = rt.rank();
    // entry handshake, in stream order ahead of everything else of this call
    aux::FlagOp op{};
    op.c = rt.ctx();
    op.status_code = kStatusTileFlag;
    op.signal_first = 1;
    op.signal_value = op.wait_value = static_cast<uint64_t>(p.epoch) << 32;
    for (int r = 0; r < R; ++r) {
        if (r == me) continue;
        op.signal_ptrs[op.num_signal++] = reinterpret_cast<uint64_t*>(rt.heap().peer(r)) + kCtlTileFlags + me * 64 + 63;
        op.wait_ptrs[op.num_wait++] = reinterpret_cast<const uint64_t*>(rt.heap().base()) + kCtlTileFlags + r * 64 + 63;
    }
    CUDA_RUNTIME_CHECK(aux::launch_flag_op(&op, 1, stream));
    FanOut& f = fan_out(device);
    const int used = std::min<int>(FanOut::kFanStreams, R - 1);
    f.fork(stream, used);
    // the GEMM starts on the local chunks while the copies are queued
    CUDA_RUNTIME_CHECK(gemm::launch_ag_gemm(params.data(), bptr.data(), gptr.data(), V, num_sms, stream));
    const int chunks = Ml / 128;
    const int group = chunks >= 4 ? (chunks + 1) / 2 : 1;        // row chunks per copy: two copies per peer (the host
                                                                 // pays per driver call, the copy engine per byte)
    const size_t row_bytes = static_cast<size_t>(K) * 2;
    const uint64_t arrived = (static_cast<uint64_t>(p.epoch) << 32) | 1u;
    for (int c0 = 0; c0 < chunks; c0 += group) {
        const int c1 = std::min(chunks, c0 + group);
        for (int i = 0; i < R - 1; ++i) {
            const int peer = (me + 1 + i) % R;
            const cudaStream_t side = f.streams[i % FanOut::kFanStreams];
            uint8_t* dst = rt.heap().peer(peer) + p.off_gather + (static_cast<uint64_t>(me) * Ml + static_cast<uint64_t>(c0) * 128) * row_bytes;
            const uint8_t* src = p.a_local + static_cast<int64_t>(c0) * 128 * p.a_stride_bytes;
            if (static_cast<size_t>(p.a_stride_bytes) == row_bytes)
                CUDA_RUNTIME_CHECK(cudaMemcpyAsync(dst, src, row_bytes * static_cast<size_t>(c1 - c0) * 128, cudaMemcpyDeviceToDevice, side));
            else
                CUDA_RUNTIME_CHECK(cudaMemcpy2DAsync(dst, row_bytes, src, static_cast<size_t>(p.a_stride_bytes), row_bytes,
                                                     static_cast<size_t>(c1 - c0) * 128, cudaMemcpyDeviceToDevice, side));
            unsigned long long flags[64];
            for (int c = c0; c < c1; ++c)
                flags[c - c0] = reinterpret_cast<unsigned long long>(reinterpret_cast<uint64_t*>(rt.heap().peer(peer)) + kCtlTileFlags + me * 64 + c);
            stream_write_values(side, flags, c1 - c0, arrived);
        }
    }
    f.join(stream, used);
    return outs;
}

// out_r[Ml, N] = sum over ranks of (A_s[R * Ml, Kl] * B_s[N, Kl]^T) restricted to the rows of rank r.
// `partial_offsets` / `flag_offsets` = the two halves of the partial buffer and of its arrival counters.
std::vector<at::Tensor> tp_gemm_rs(const std::vector<std::shared_ptr<Runtime>>& rts, const std::vector<at::Tensor>& a,
                                   const std::vector<at::Tensor>& b, const std::vector<int64_t>& partial_offsets,
                                   const std::vector<int64_t>& flag_offsets, int num_sms) {
    const int V = static_cast<int>(rts.size());
    EP_HOST_ASSERT(V >= 1 && V <= gemm::kTpMaxVRanks && static_cast<int>(a.size()) == V && static_cast<int>(b.size()) == V);
    EP_HOST_ASSERT(partial_offsets.size() == 2 && flag_offsets.size() == 2);
    auto& rt0 = *rts[0];
    const int device = rt0.heap().device();
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    const int R = rt0.num_ranks();
    const int M = static_cast<int>(a[0].size(0)), K = static_cast<int>(a[0].size(1)), N = static_cast<int>(b[0].size(0));
    EP_HOST_ASSERT(M % R == 0);
    const int Ml = M / R;
    const uint64_t part_bytes = static_cast<uint64_t>(R) * Ml * N * 2;
    const uint64_t flag_bytes = static_cast<uint64_t>(R) * (Ml / 128) * (N / 256) * 8;
    if (num_sms <= 0) num_sms = rt0.num_device_sms() / V;
    std::vector<gemm::GemmRsParams> params(V);
    std::vector<const void*> aptr(V), bptr(V);
    std::vector<int64_t> astride(V);
    std::vector<at::Tensor> outs(V);
    for (int v = 0; v < V; ++v) {
        auto& rt = *rts[v];
        EP_HOST_ASSERT(a[v].scalar_type() == at::kBFloat16 && a[v].dim() == 2 && a[v].stride(1) == 1 && a[v].size(0) == M && a[v].size(1) == K);
        EP_HOST_ASSERT(b[v].scalar_type() == at::kBFloat16 && b[v].is_contiguous() && b[v].size(0) == N && b[v].size(1) == K);
        EP_HOST_ASSERT((a[v].stride(0) * 2) % 16 == 0 && reinterpret_cast<uintptr_t>(a[v].data_ptr()) % 16 == 0);
        // arrival counters only grow, so their meaning is tied to the first configuration used on this heap
        // (EP_TP_RS_FUSE_OWN=0 / 1 overrides the choice by rank count; the arrival counters of the own slot only move in
        // the unfused form, so the form is part of the configuration a buffer is tied to)
        const char* fuse_env = std::getenv("EP_TP_RS_FUSE_OWN");
        const int fuse_own = fuse_env != nullptr ? (fuse_env[0] == '1' ? 1 : 0) : (R <= 4 ? 1 : 0);
        const int64_t config = (static_cast<int64_t>(Ml) << 40) ^ (static_cast<int64_t>(N) << 20) ^ flag_offsets[0] ^ (flag_offsets[1] << 1) ^
                               (static_cast<int64_t>(fuse_own) << 62);
        if (rt.tp_rs_config == 0) rt.tp_rs_config = config;
        EP_HOST_ASSERT_MSG(rt.tp_rs_config == config, "GEMM->reduce-scatter on one buffer must keep its shape and offsets");
        const uint32_t epoch = ++rt.tp_rs_epoch;
        gemm::GemmRsParams& p = params[v];
        p.c = rt.ctx();
        p.rows_per_rank = Ml;
        p.N = N;
        p.K = K;
        outs[v] = at::empty({Ml, N}, a[v].options());
        p.out = reinterpret_cast<__nv_bfloat16*>(outs[v].data_ptr());
        p.ldo = N;
        for (int h = 0; h < 2; ++h) {
            p.off_partial[h] = static_cast<uint64_t>(partial_offsets[h]);
            p.off_flags[h] = static_cast<uint64_t>(flag_offsets[h]);
            EP_HOST_ASSERT(p.off_partial[h] + part_bytes <= rt.heap().num_bytes() && p.off_flags[h] + flag_bytes <= rt.heap().num_bytes());
            EP_HOST_ASSERT(p.off_partial[h] >= kCtlBytes && p.off_flags[h] >= kCtlBytes && p.off_partial[h] % 16 == 0 && p.off_flags[h] % 8 == 0);
        }
        p.epoch = epoch;
        p.flag_target = 4 * static_cast<int>((epoch + 1) / 2);   // four epilogue warps arrive per tile and call on this half
        p.fuse_own = fuse_own;
        p.error = tp_status(device).data_ptr<int>();
        aptr[v] = a[v].data_ptr();
        bptr[v] = b[v].data_ptr();
        astride[v] = a[v].stride(0) * 2;
    }
    CUDA_RUNTIME_CHECK(gemm::launch_gemm_rs(params.data(), aptr.data(), astride.data(), bptr.data(), V, num_sms,
                                            at::cuda::getCurrentCUDAStream().stream()));
    return outs;
}

}  // namespace

void register_tp_bindings(py::module_& m) {
    m.def("tp_ag_gemm", &tp_ag_gemm, py::arg("runtimes"), py::arg("a_local"), py::arg("b"), py::arg("gather_offsets"),
          py::arg("num_comm_ctas") = 0, py::arg("num_sms") = 0, py::arg("push") = 0);
    m.def("tp_gemm_rs", &tp_gemm_rs, py::arg("runtimes"), py::arg("a"), py::arg("b"), py::arg("partial_offsets"), py::arg("flag_offsets"),
          py::arg("num_sms") = 0);
    m.def("tp_check_status", &tp_check_status);
    m.attr("TP_MAX_VRANKS") = gemm::kTpMaxVRanks;
}

}  // namespace ep
