// Bindings of the subsystems that live next to the high-throughput EP core.
#include <pybind11/stl.h>
#include <torch/extension.h>

namespace py = pybind11;

namespace ep {
void register_ll_bindings(py::module_& m);
void register_ops_bindings(py::module_& m);
void register_tp_bindings(py::module_& m);
void register_aux_bindings(py::module_& m);
void register_jit_bindings(py::module_& m);
}

void register_extra_bindings(py::module_& m) {
    ep::register_ll_bindings(m);
    ep::register_ops_bindings(m);
    ep::register_tp_bindings(m);
    ep::register_aux_bindings(m);
    ep::register_jit_bindings(m);
}
