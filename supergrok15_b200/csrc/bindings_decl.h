// Registration hooks of the binding translation units (one per subsystem, compiled in parallel).
#pragma once
#include <torch/extension.h>
namespace sgb {
void register_sg2(pybind11::module_& m);
void register_dist(pybind11::module_& m);
void register_gemm(pybind11::module_& m);
void register_nn(pybind11::module_& m);
void register_llm(pybind11::module_& m);
void cpu_mt_apply(int op, const std::vector<std::vector<at::Tensor>>& roles, const std::vector<std::vector<double>>& ts, const std::vector<double>& f,
                  c10::optional<at::Tensor> clip, c10::optional<at::Tensor> dscal, c10::optional<at::Tensor> tscal, c10::optional<at::Tensor> W1,
                  c10::optional<at::Tensor> b1, c10::optional<at::Tensor> W2, c10::optional<at::Tensor> b2, int64_t hidden, bool write_grad,
                  c10::optional<at::Tensor> per_tensor_out);
void cpu_scalar_finalize(int op, const at::Tensor& per_tensor, int64_t n, at::Tensor out, double a0, double a1, double a2);
}
