#include <pybind11/pybind11.h>
namespace py = pybind11;
void init_layerwise_bindings(py::module_& m) { (void)m; }
