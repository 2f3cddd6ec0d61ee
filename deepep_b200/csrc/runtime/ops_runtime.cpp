// PyTorch-facing wrappers of the compute kernels (tcgen05 GEMM family, and the small hot ops).
// The reference library has no compute kernels; these exist for the fused MoE layer and the
// tensor-parallel fused operators built on the same runtime.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/ops/empty.h>
#include <ATen/ops/zeros.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <map>
#include <optional>

#include "../common/exception.hpp"
#include "../common/layout.hpp"
#include "../kernels/gemm_api.hpp"
#include "../kernels/ops_api.hpp"

namespace py = pybind11;

namespace ep {

namespace {

// one status word per device for the GEMM pipelines (0 = healthy)
at::Tensor& gemm_status(int device) {
    static std::map<int, at::Tensor> words;
    auto it = words.find(device);
    if (it == words.end())
        it = words.emplace(device, at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::Device(at::kCUDA, static_cast<c10::DeviceIndex>(device))))).first;
    return it->second;
}

int gemm_check_status() {
    int device = 0;
    CUDA_RUNTIME_CHECK(cudaGetDevice(&device));
    return gemm_status(device).item<int>();
}

at::Tensor gemm_impl(const at::Tensor& a, const at::Tensor& b, const std::optional<at::Tensor>& sfa, const std::optional<at::Tensor>& sfb,
                     const std::optional<at::Tensor>& group_end, int group_alignment, std::optional<at::Tensor> out, int num_sms,
                     bool pow2_scales) {
    EP_HOST_ASSERT(a.is_cuda() && b.is_cuda() && a.dim() == 2 && a.stride(1) == 1 && b.stride(-1) == 1);
    EP_HOST_ASSERT(b.dim() == 2 || b.is_contiguous());
    const bool fp8 = a.scalar_type() == at::kFloat8_e4m3fn;
    EP_HOST_ASSERT(fp8 || a.scalar_type() == at::kBFloat16);
    EP_HOST_ASSERT(b.scalar_type() == a.scalar_type());
    const bool grouped = b.dim() == 3;
    EP_HOST_ASSERT(b.dim() == 2 || b.dim() == 3);
    const int G = grouped ? static_cast<int>(b.size(0)) : 1;
    const int N = static_cast<int>(b.size(grouped ? 1 : 0)), K = static_cast<int>(b.size(grouped ? 2 : 1));
    const int M = static_cast<int>(a.size(0));
    EP_HOST_ASSERT(a.size(1) == K);
    const int elem = fp8 ? 1 : 2;
    EP_HOST_ASSERT((a.stride(0) * elem) % 16 == 0 && reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 == 0);
    EP_HOST_ASSERT_MSG(N % 128 == 0 && K % (fp8 ? 128 : 64) == 0, "N must be a multiple of 128 and K of 64 (bf16) / 128 (fp8)");
    const int device = a.get_device();
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    if (!out.has_value()) out = at::empty({M, N}, a.options().dtype(at::kBFloat16));
    EP_HOST_ASSERT(out->scalar_type() == at::kBFloat16 && out->size(0) == M && out->size(1) == N && out->stride(1) == 1 &&
                   (out->stride(0) * 2) % 16 == 0);
    if (M == 0) return *out;

    gemm::GemmParams p = {};
    p.M = M;
    p.N = N;
    p.K = K;
    p.num_groups = G;
    p.group_end = nullptr;
    p.group_alignment = std::max(group_alignment, 1);
    p.zero_gap = (grouped && p.group_alignment % 128 == 0) ? 1 : 0;
    if (grouped) {
        EP_HOST_ASSERT(group_end.has_value() && group_end->scalar_type() == at::kInt && group_end->is_contiguous() && group_end->numel() >= G);
        p.group_end = group_end->data_ptr<int>();
    }
    p.C = reinterpret_cast<__nv_bfloat16*>(out->data_ptr());
    p.ldc = out->stride(0);
    if (fp8) {
        EP_HOST_ASSERT(sfa.has_value() && sfb.has_value() && sfa->scalar_type() == at::kFloat && sfb->scalar_type() == at::kFloat);
        EP_HOST_ASSERT(sfa->dim() == 2 && sfa->size(0) == M && sfa->size(1) == K / 128);
        EP_HOST_ASSERT(sfb->is_contiguous() && sfb->numel() == static_cast<int64_t>(G) * (N / 128) * (K / 128));
        p.sfa = sfa->data_ptr<float>();
        p.sfa_row_stride = sfa->stride(0);
        p.sfa_k_stride = sfa->stride(1);
        p.sfb = sfb->data_ptr<float>();
        p.scales_pow2 = pow2_scales ? 1 : 0;
    }
    p.error = gemm_status(device).data_ptr<int>();
    p.timeout_ns = 10ull * 1000 * 1000 * 1000;
    const int sms = num_sms > 0 ? num_sms : at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const int64_t b_stride = (grouped ? b.stride(1) : b.stride(0)) * elem;
    EP_HOST_ASSERT(b_stride % 16 == 0 && reinterpret_cast<uintptr_t>(b.data_ptr()) % 16 == 0);
    CUDA_RUNTIME_CHECK(gemm::launch_gemm(p, a.data_ptr(), a.stride(0) * elem, b.data_ptr(), b_stride, fp8, sms,
                                         at::cuda::getCurrentCUDAStream().stream()));
    return *out;
}

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

// out[g] = a[:, range g] @ b[:, range g]^T for all groups in one launch (bf16): the k range of group g is
// [align(group_end[g-1], group_alignment), group_end[g]), read from the device array, no host synchronisation.
at::Tensor gemm_k_grouped(const at::Tensor& a, const at::Tensor& b, const at::Tensor& group_end, int num_groups, int group_alignment,
                          std::optional<at::Tensor> out, int num_sms) {
    EP_HOST_ASSERT(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1);
    EP_HOST_ASSERT(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && a.size(1) == b.size(1));
    const int M = static_cast<int>(a.size(0)), N = static_cast<int>(b.size(0)), K = static_cast<int>(a.size(1));
    EP_HOST_ASSERT_MSG(N % 128 == 0 && K % 64 == 0 && group_alignment % 64 == 0, "N must be a multiple of 128, K and the group alignment of 64");
    EP_HOST_ASSERT((a.stride(0) * 2) % 16 == 0 && (b.stride(0) * 2) % 16 == 0 && reinterpret_cast<uintptr_t>(a.data_ptr()) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(b.data_ptr()) % 16 == 0);
    EP_HOST_ASSERT(group_end.scalar_type() == at::kInt && group_end.is_contiguous() && group_end.numel() >= num_groups && num_groups >= 1);
    const int device = a.get_device();
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    if (!out.has_value()) out = at::empty({num_groups, M, N}, a.options());
    EP_HOST_ASSERT(out->scalar_type() == at::kBFloat16 && out->is_contiguous() && out->numel() == static_cast<int64_t>(num_groups) * M * N);
    gemm::GemmParams p = {};
    p.M = M;
    p.N = N;
    p.K = K;
    p.num_groups = num_groups;
    p.group_end = group_end.data_ptr<int>();
    p.group_alignment = group_alignment;
    p.zero_gap = 0;
    p.k_grouped = 1;
    p.c_group_stride = static_cast<int64_t>(M) * N;
    p.C = reinterpret_cast<__nv_bfloat16*>(out->data_ptr());
    p.ldc = N;
    p.error = gemm_status(device).data_ptr<int>();
    p.timeout_ns = 10ull * 1000 * 1000 * 1000;
    const int sms = num_sms > 0 ? num_sms : at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    CUDA_RUNTIME_CHECK(gemm::launch_gemm(p, a.data_ptr(), a.stride(0) * 2, b.data_ptr(), b.stride(0) * 2, false, sms, cur_stream()));
    return *out;
}

std::tuple<at::Tensor, at::Tensor> router_topk(const at::Tensor& logits, int num_topk) {
    EP_HOST_ASSERT(logits.is_cuda() && logits.dim() == 2 && logits.scalar_type() == at::kFloat && logits.is_contiguous());
    c10::cuda::CUDAGuard guard(logits.device());
    const int T = static_cast<int>(logits.size(0)), E = static_cast<int>(logits.size(1));
    auto idx = at::empty({T, num_topk}, logits.options().dtype(at::kLong));
    auto w = at::empty({T, num_topk}, logits.options());
    CUDA_RUNTIME_CHECK(ops::router_topk(logits.data_ptr<float>(), T, E, num_topk, idx.data_ptr<int64_t>(), w.data_ptr<float>(), cur_stream()));
    return {idx, w};
}

std::tuple<at::Tensor, at::Tensor> quant_1x128(const at::Tensor& x, bool pow2, bool col_major_sf) {
    EP_HOST_ASSERT(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.stride(1) == 1 && (x.stride(0) * 2) % 16 == 0);
    c10::cuda::CUDAGuard guard(x.device());
    const int M = static_cast<int>(x.size(0)), H = static_cast<int>(x.size(1));
    EP_HOST_ASSERT(H % 128 == 0);
    auto q = at::empty({M, H}, x.options().dtype(at::kFloat8_e4m3fn));
    at::Tensor sf = col_major_sf ? at::empty({H / 128, align_up(std::max(M, 1), 4)}, x.options().dtype(at::kFloat)).t().slice(0, 0, M)
                                 : at::empty({M, H / 128}, x.options().dtype(at::kFloat));
    CUDA_RUNTIME_CHECK(ops::quant_1x128(x.data_ptr(), x.stride(0) * 2, M, H, pow2, q.data_ptr(), sf.data_ptr<float>(), sf.stride(0),
                                        sf.stride(1), cur_stream()));
    return {q, sf};
}

at::Tensor dequant_1x128(const at::Tensor& q, const at::Tensor& sf) {
    EP_HOST_ASSERT(q.is_cuda() && q.dim() == 2 && q.scalar_type() == at::kFloat8_e4m3fn && q.is_contiguous() && sf.scalar_type() == at::kFloat);
    c10::cuda::CUDAGuard guard(q.device());
    const int M = static_cast<int>(q.size(0)), H = static_cast<int>(q.size(1));
    EP_HOST_ASSERT(H % 128 == 0 && sf.size(0) == M && sf.size(1) == H / 128);
    auto out = at::empty({M, H}, q.options().dtype(at::kBFloat16));
    CUDA_RUNTIME_CHECK(ops::dequant_1x128(q.data_ptr(), sf.data_ptr<float>(), sf.stride(0), sf.stride(1), M, H, out.data_ptr(), cur_stream()));
    return out;
}

// returns (out, scales or None)
std::tuple<at::Tensor, std::optional<at::Tensor>> swiglu(const at::Tensor& x, const std::optional<at::Tensor>& row_weight,
                                                          const std::optional<at::Tensor>& num_valid_rows, bool quant, bool pow2) {
    EP_HOST_ASSERT(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.size(1) % 16 == 0);
    c10::cuda::CUDAGuard guard(x.device());
    const int M = static_cast<int>(x.size(0)), I = static_cast<int>(x.size(1) / 2);
    const float* rw = nullptr;
    if (row_weight.has_value()) {
        EP_HOST_ASSERT(row_weight->scalar_type() == at::kFloat && row_weight->is_contiguous() && row_weight->numel() >= M);
        rw = row_weight->data_ptr<float>();
    }
    const int* nv = num_valid_rows.has_value() ? num_valid_rows->data_ptr<int>() : nullptr;
    at::Tensor out = at::empty({M, I}, x.options().dtype(quant ? at::kFloat8_e4m3fn : at::kBFloat16));
    std::optional<at::Tensor> sf;
    if (quant) sf = at::empty({M, I / 128}, x.options().dtype(at::kFloat));
    CUDA_RUNTIME_CHECK(ops::swiglu(x.data_ptr(), M, I, rw, nv, out.data_ptr(), quant, quant ? sf->data_ptr<float>() : nullptr,
                                   quant ? sf->stride(0) : 0, quant ? sf->stride(1) : 0, pow2, cur_stream()));
    return {out, sf};
}

// returns dx, or with `with_byproducts` (dx, weighted activation [rows, inter] bf16, gradient of the row weight [rows] fp32)
py::object swiglu_backward(const at::Tensor& x, const at::Tensor& dout, const std::optional<at::Tensor>& row_weight, bool with_byproducts) {
    EP_HOST_ASSERT(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && dout.scalar_type() == at::kBFloat16 && dout.is_contiguous());
    c10::cuda::CUDAGuard guard(x.device());
    const int M = static_cast<int>(x.size(0)), I = static_cast<int>(x.size(1) / 2);
    EP_HOST_ASSERT(dout.size(0) == M && dout.size(1) == I);
    if (row_weight.has_value()) EP_HOST_ASSERT(row_weight->scalar_type() == at::kFloat && row_weight->is_contiguous() && row_weight->numel() >= M);
    auto dx = at::empty_like(x);
    at::Tensor act, dweight;
    if (with_byproducts) {
        act = at::empty({M, I}, x.options());
        dweight = at::empty({M}, x.options().dtype(at::kFloat));
    }
    CUDA_RUNTIME_CHECK(ops::swiglu_backward(x.data_ptr(), dout.data_ptr(), M, I, row_weight.has_value() ? row_weight->data_ptr<float>() : nullptr,
                                            dx.data_ptr(), with_byproducts ? act.data_ptr() : nullptr,
                                            with_byproducts ? dweight.data_ptr<float>() : nullptr, cur_stream()));
    if (with_byproducts) return py::make_tuple(dx, act, dweight);
    return py::cast(dx);
}

at::Tensor transpose_bf16(const at::Tensor& x) {
    EP_HOST_ASSERT(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.stride(1) == 1);
    c10::cuda::CUDAGuard guard(x.device());
    auto out = at::empty({x.size(1), x.size(0)}, x.options());
    CUDA_RUNTIME_CHECK(ops::transpose_bf16(x.data_ptr(), x.stride(0), static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), out.data_ptr(),
                                           out.stride(0), cur_stream()));
    return out;
}

}  // namespace

void register_ops_bindings(py::module_& m) {
    m.def("router_topk", &router_topk);
    m.def("quant_1x128", &quant_1x128, py::arg("x"), py::arg("pow2") = false, py::arg("col_major_sf") = false);
    m.def("dequant_1x128", &dequant_1x128);
    m.def("swiglu", &swiglu, py::arg("x"), py::arg("row_weight") = py::none(), py::arg("num_valid_rows") = py::none(), py::arg("quant") = false,
          py::arg("pow2") = false);
    m.def("swiglu_backward", &swiglu_backward, py::arg("x"), py::arg("dout"), py::arg("row_weight") = py::none(),
          py::arg("with_byproducts") = false);
    m.def("transpose_bf16", &transpose_bf16);
    m.def("gemm", &gemm_impl, py::arg("a"), py::arg("b"), py::arg("sfa") = py::none(), py::arg("sfb") = py::none(),
          py::arg("group_end") = py::none(), py::arg("group_alignment") = 1, py::arg("out") = py::none(), py::arg("num_sms") = 0,
          py::arg("pow2_scales") = false,
          "C = A @ B^T on the tcgen05 tensor cores (bf16, or e4m3 with 1x128 / 128x128 block scales); 3-D B = grouped. "
          "pow2_scales: every scale is an exact power of two (round_scale quantisation), which lets the tensor core apply "
          "them itself (kind::mxf8f6f4.block_scale) when N is a multiple of 256 and K at most 8192");
    m.def("gemm_k_grouped", &gemm_k_grouped, py::arg("a"), py::arg("b"), py::arg("group_end"), py::arg("num_groups"),
          py::arg("group_alignment") = 128, py::arg("out") = py::none(), py::arg("num_sms") = 0,
          "C[g] = A[:, k range g] @ B[:, k range g]^T for all groups in one launch (bf16; the ranges come from a device array)");
    m.def("gemm_check_status", &gemm_check_status);
}

}  // namespace ep
