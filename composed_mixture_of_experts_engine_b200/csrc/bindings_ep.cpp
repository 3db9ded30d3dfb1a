// pybind11 registration of the expert-parallel peer-memory kernels (ep.cu).
#include <torch/extension.h>

void register_ep(pybind11::module_& m) { (void)m; }
