// Python bindings of the grouped expert GEMM (kept in its own translation unit so that kernel-side
// changes do not rebuild the runtime bindings).
#include <torch/extension.h>

#include "../kernels/gemm_api.h"

namespace py = pybind11;

void bind_gemm(py::module_& m) { (void)m; }
