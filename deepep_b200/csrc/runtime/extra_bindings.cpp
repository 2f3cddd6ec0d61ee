// Bindings of the subsystems that live next to the high-throughput EP core.
#include <pybind11/stl.h>
#include <torch/extension.h>

namespace py = pybind11;

void register_extra_bindings(py::module_& m) { (void)m; }
