// pybind11 registration of the attention kernels (attention.cu).
#include <torch/extension.h>

void register_attention(pybind11::module_& m) { (void)m; }
