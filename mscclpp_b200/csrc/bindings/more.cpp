// Bindings of components added after the first slice (channels, executor, proxy, ...).
#include "bindings.hpp"

namespace py = pybind11;

void registerMoreBindings(py::module_& m) { (void)m; }
