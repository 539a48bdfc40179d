// Split of the pybind11 module over several translation units (keeps each compile short).
#pragma once

#include <pybind11/pybind11.h>

void registerMoreBindings(pybind11::module_& m);
void registerCoreBindings(pybind11::module_& m);
void registerAlgorithmBindings(pybind11::module_& m);
