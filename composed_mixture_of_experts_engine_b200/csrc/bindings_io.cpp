// pybind11 registration of the checkpoint writer (odirect_writer.cpp).
#include <torch/extension.h>

void register_io(pybind11::module_& m) { (void)m; }
