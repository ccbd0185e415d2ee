// Bindings of the peer-memory (NVLink) communication kernels.
#include <torch/extension.h>

void bind_comm(pybind11::module_& m) { (void)m; }
