// Python bindings of the run-time compiler (see csrc/jit/jit.hpp).
#include <ATen/cuda/CUDAContext.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "../jit/jit.hpp"

namespace py = pybind11;

namespace ep {

namespace {

std::unique_ptr<jit::Compiler> g_compiler;
jit::KernelCache g_cache;

void jit_init(const std::string& cache_dir, const std::string& cuda_home, const std::string& include_root) {
    g_cache.clear();
    g_compiler = std::make_unique<jit::Compiler>(cache_dir, cuda_home, include_root);
}

jit::Compiler& compiler() {
    EP_HOST_ASSERT_MSG(g_compiler != nullptr, "call jit_init first");
    return *g_compiler;
}

}  // namespace

void register_jit_bindings(py::module_& m) {
    m.def("jit_init", &jit_init);
    m.def("jit_build", [](const std::string& name, const std::string& code) { return compiler().build(name, code); });
    m.def("jit_flags", []() { return compiler().flags(); });
    m.def("jit_num_compilations", []() { return compiler().num_compilations(); });
    m.def("jit_digest", &jit::digest);
    m.def("jit_launch", [](const std::string& cubin, std::tuple<int, int, int> grid, std::tuple<int, int, int> block, int smem_bytes,
                           const py::bytes& params, bool cooperative, int cluster_dim) {
        const std::string blob = params;
        auto lib = g_cache.get(cubin);
        lib->launch(dim3(std::get<0>(grid), std::get<1>(grid), std::get<2>(grid)), dim3(std::get<0>(block), std::get<1>(block), std::get<2>(block)),
                    smem_bytes, at::cuda::getCurrentCUDAStream().stream(), blob.data(), cooperative, cluster_dim);
    }, py::arg("cubin"), py::arg("grid"), py::arg("block"), py::arg("smem_bytes"), py::arg("params"), py::arg("cooperative") = false,
       py::arg("cluster_dim") = 1);
}

}  // namespace ep
