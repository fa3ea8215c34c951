// placeholder
#include <pybind11/pybind11.h>
namespace py = pybind11;
void BindSddmm(py::module_&) {}
void BindScatter(py::module_&) {}
void BindGrouped(py::module_&) {}
