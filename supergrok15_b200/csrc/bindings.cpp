// PyTorch bindings of the native launchers (pybind11 module `_C`).
//
// This is the host dispatch layer: it turns tensor lists into launch descriptors, splits them
// into launches, and enqueues everything on PyTorch's current CUDA stream.  Nothing here
// synchronises with the device or copies a scalar to the host.  (The reference's dispatch layer,
// csrc/ops.cpp:897-1087, does one host sync per reduction and launches on the legacy stream.)
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <vector>
#include "sg_native.h"
#include "bindings_decl.h"

namespace {

using at::Tensor;

int dtype_code(const Tensor& t) {
    switch (t.scalar_type()) {
        case at::kFloat: return sg::F32;
        case at::kBFloat16: return sg::BF16;
        case at::kHalf: return sg::F16;
        default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
    }
}

const float* fptr(const c10::optional<Tensor>& t) {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous(), "expected contiguous fp32 CUDA tensor");
    return t->data_ptr<float>();
}

// Number of CTAs a list of tensor sizes needs (also the length/3 of the partials array).
int64_t mt_num_blocks(const std::vector<int64_t>& numels) {
    int64_t b = 0;
    for (auto n : numels) b += (n + sg::MT_CHUNK - 1) / sg::MT_CHUNK;
    return b;
}

// roles[r] is either empty (role unused) or one tensor per parameter.  Roles 0/1 (param/grad) carry
// the launch dtype; every other role must be fp32 unless the op says otherwise.
void mt_apply(int op, const std::vector<std::vector<Tensor>>& roles, const std::vector<std::vector<double>>& ts,
              const std::vector<double>& f, c10::optional<Tensor> clip, c10::optional<Tensor> dscal,
              c10::optional<Tensor> tscal, c10::optional<Tensor> W1, c10::optional<Tensor> b1,
              c10::optional<Tensor> W2, c10::optional<Tensor> b2, int64_t hidden, bool write_grad,
              c10::optional<Tensor> partials, c10::optional<Tensor> per_tensor_out) {
    TORCH_CHECK(op >= 0 && op < sg::OP_COUNT, "bad op");
    TORCH_CHECK(roles.size() <= (size_t)sg::MT_NP, "too many roles");
    size_t n = 0;
    const Tensor* first = nullptr;
    for (size_t r = 0; r < roles.size(); ++r)
        if (!roles[r].empty()) {
            if (n == 0) n = roles[r].size();
            TORCH_CHECK(roles[r].size() == n, "role ", r, " has ", roles[r].size(), " tensors, expected ", n);
            if (!first && r <= 1) first = &roles[r][0];
        }
    if (n == 0) return;
    TORCH_CHECK(first != nullptr, "role 0 or 1 must be present");
    if (first->device().is_cpu()) {                 // fp32 CPU tensors: the C++ CPU kernels (csrc/cpu_kernels.cpp), same ops and formulas
        sgb::cpu_mt_apply(op, roles, ts, f, clip, dscal, tscal, W1, b1, W2, b2, hidden, write_grad, per_tensor_out);
        return;
    }
    TORCH_CHECK(first->is_cuda(), "mt_apply needs CUDA tensors");
    const int dt = dtype_code(*first);
    c10::cuda::CUDAGuard guard(first->device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();

    sg::MTParams p{};
    auto F = [&](size_t i) { return i < f.size() ? (float)f[i] : 0.f; };
    p.lr = F(0); p.beta1 = F(1); p.beta2 = F(2); p.eps = F(3); p.wd = F(4); p.alpha = F(5); p.lamb = F(6);
    p.rescale = F(7); p.extra0 = F(8); p.extra1 = F(9);
    p.clip = fptr(clip); p.dscal = fptr(dscal); p.tscal = fptr(tscal);
    p.W1 = fptr(W1); p.b1 = fptr(b1); p.W2 = fptr(W2); p.b2 = fptr(b2);
    p.hidden = (int)hidden; p.write_grad = write_grad ? 1 : 0;
    p.partials = partials.has_value() ? partials->data_ptr<float>() : nullptr;
    TORCH_CHECK(hidden <= 512, "meta-net hidden size > 512 not supported by the fused kernel");

    sg::MTArgs a{};
    int t_off = 0, blk_off = 0;
    auto flush = [&]() {
        if (a.n == 0) return;
        a.t_off = t_off; a.blk_off = blk_off;
        sg::mt_launch(op, dt, a, p, stream);
        if (per_tensor_out.has_value())
            sg::mt_finalize_per_tensor(a, p.partials, per_tensor_out->data_ptr<float>(), stream);
        t_off += a.n; blk_off += a.blk_start[a.n];
        a.n = 0; a.blk_start[0] = 0;
    };
    a.n = 0; a.blk_start[0] = 0;
    for (size_t i = 0; i < n; ++i) {
        int64_t numel = -1;
        bool skip = false;
        for (size_t r = 0; r < roles.size(); ++r) {
            if (roles[r].empty()) continue;
            const Tensor& t = roles[r][i];
            if (!t.defined()) { skip = true; break; }
            if (numel < 0) numel = t.numel();
            TORCH_CHECK(t.numel() == numel, "role ", r, " tensor ", i, " size mismatch");
            TORCH_CHECK(t.is_contiguous() && t.is_cuda(), "tensors must be contiguous CUDA tensors");
        }
        if (skip || numel <= 0) {     // keep tensor numbering: a zero-CTA entry
            numel = 0;
        }
        const int t = a.n;
        for (int r = 0; r < sg::MT_NP; ++r)
            a.ptr[r][t] = (!skip && (size_t)r < roles.size() && !roles[r].empty() && roles[r][i].defined())
                              ? roles[r][i].data_ptr() : nullptr;
        a.numel[t] = numel;
        a.blk_start[t + 1] = a.blk_start[t] + (int)((numel + sg::MT_CHUNK - 1) / sg::MT_CHUNK);
        for (int k = 0; k < sg::MT_NS; ++k)
            a.ts[t][k] = (i < ts.size() && (size_t)k < ts[i].size()) ? (float)ts[i][k] : 0.f;
        a.n += 1;
        if (a.n == sg::MT_MAX) flush();
    }
    flush();
}

void scalar_finalize(int op, const Tensor& per_tensor, int64_t n_tensors, Tensor out, double a0, double a1, double a2) {
    if (out.device().is_cpu()) { sgb::cpu_scalar_finalize(op, per_tensor, n_tensors, out, a0, a1, a2); return; }
    c10::cuda::CUDAGuard guard(out.device());
    sg::scalar_finalize(op, per_tensor.data_ptr<float>(), (int)n_tensors, out.data_ptr<float>(), (float)a0, (float)a1,
                        (float)a2, at::cuda::getCurrentCUDAStream());
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "supergrok15_b200 native kernels (sm_100a)";
    m.attr("MT_CHUNK") = sg::MT_CHUNK;
    m.def("mt_num_blocks", &mt_num_blocks);
    m.def("mt_apply", &mt_apply, py::arg("op"), py::arg("roles"), py::arg("ts"), py::arg("f"),
          py::arg("clip") = c10::nullopt, py::arg("dscal") = c10::nullopt, py::arg("tscal") = c10::nullopt,
          py::arg("W1") = c10::nullopt, py::arg("b1") = c10::nullopt, py::arg("W2") = c10::nullopt,
          py::arg("b2") = c10::nullopt, py::arg("hidden") = 0, py::arg("write_grad") = false,
          py::arg("partials") = c10::nullopt, py::arg("per_tensor_out") = c10::nullopt);
    m.def("scalar_finalize", &scalar_finalize);
    m.def("launch_count", []() { return sg::launch_count(); });
    m.def("bounds_check_enabled", []() { return sg::bounds_check_enabled(); });
    m.def("bounds_reset", []() { sg::bounds_reset(); });
    m.def("bounds_report", []() { int v[8]; sg::bounds_report(v); return std::vector<int64_t>(v, v + 8); });
    m.def("bounds_cap", [](int64_t bytes) { sg::bounds_cap((long long)bytes); });
    m.def("bounds_extent_of", [](const at::Tensor& t) { return (int64_t)sg::bounds_extent_of(t.data_ptr()); });
    // kernels that run from a replayed CUDA graph are not enqueued by a launcher: the owner of the graph adds them here
    m.def("add_launches", [](int64_t n) { sg::count_launch((int)n); });
    py::dict ops;
#define SG_OP(X) ops[#X] = (int)sg::X;
    SG_OP(OP_ADAMW) SG_OP(OP_LION) SG_OP(OP_GROKFAST_EMA) SG_OP(OP_GROKFAST_ADAMW) SG_OP(OP_GROKADAMW)
    SG_OP(OP_PRODIGY) SG_OP(OP_NEURALGROK) SG_OP(OP_SG15) SG_OP(OP_SG11_A) SG_OP(OP_SG11_B) SG_OP(OP_PERTURB)
    SG_OP(OP_RESTORE) SG_OP(OP_SHARP_RESTORE) SG_OP(OP_LOOKSAM_DIR) SG_OP(OP_LOOKSAM_ADJ) SG_OP(OP_MUON_MOMENTUM)
    SG_OP(OP_MUON_UPDATE) SG_OP(OP_SCALE) SG_OP(OP_SQNORM) SG_OP(OP_PRODIGY_REDUCE) SG_OP(OP_DIFF_SQNORM)
    SG_OP(SC_CLIP) SG_OP(SC_PRODIGY) SG_OP(SC_SG11_GATES) SG_OP(SC_SAM_SCALE) SG_OP(SC_LOOKSAM_NORMS)
    SG_OP(SC_MUON_NORMS) SG_OP(SC_SG2_CLIP) SG_OP(SC_SUM3)
#undef SG_OP
    m.attr("ops") = ops;
    sgb::register_sg2(m);
    sgb::register_dist(m);
    sgb::register_gemm(m);
    sgb::register_nn(m);
    sgb::register_llm(m);
}
