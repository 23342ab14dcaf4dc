// Registration hooks of the binding translation units (one per subsystem, compiled in parallel).
#pragma once
#include <torch/extension.h>
namespace sgb {
void register_sg2(pybind11::module_& m);
void register_dist(pybind11::module_& m);
void register_gemm(pybind11::module_& m);
void register_nn(pybind11::module_& m);
void register_llm(pybind11::module_& m);
}
