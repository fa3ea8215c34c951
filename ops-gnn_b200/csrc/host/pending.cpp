// Bindings of operator families whose planners live in files still to be added.
#include <pybind11/pybind11.h>
namespace py = pybind11;
void BindScatter(py::module_&) {}
void BindGrouped(py::module_&) {}
