// Bindings of the second kernel group (fp8, MLA, GGUF, fused tensor-/expert-parallel ops).
#include <torch/extension.h>
#include "b2/api.h"
namespace py = pybind11;

void bind_ops_extra(py::module_& m) { (void)m; }
