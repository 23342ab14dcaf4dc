// Bindings of the in-kernel collectives (peer pointers come from PyTorch symmetric memory handles).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "bindings_decl.h"
#include "mt_host.h"

namespace sg {
void dist_barrier(const PeerPtrs& pads, int rank, int world, uint32_t epoch, const uint32_t* dyn, int* status, unsigned long long timeout_ns,
                  int site, cudaStream_t s);
void dist_pull_reduce(int dtype, bool nvls, const PeerPtrs& grads, const void* mc, int world, int rank, int64_t off, int64_t n, float scale,
                      float* out, cudaStream_t s);
void dist_push(bool nvls, const PeerPtrs& params, void* mc, int world, int rank, int64_t off_bytes, int64_t n_bytes, cudaStream_t s);
void dist_fused_flat_step(int op, int gdtype, int pdtype, bool nvls, const PeerPtrs& grads, const PeerPtrs& params, const void* mc_grad,
                          void* mc_param, int world, int rank, int64_t off, int64_t n, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2, float gscale,
                          float* master, float* m, float* v, const float* dyn, bool push, cudaStream_t s);
void dist_scatter_slots(const PeerPtrs& slots, int world, int rank, const float* vec, int n, cudaStream_t s);
void dist_cast_push(int pdtype, const PeerPtrs& params, int world, int rank, int64_t off, int64_t n, const float* master, cudaStream_t s);
void dist_reduce_slots(const float* my_slots, int world, float* out, int n, float scale, cudaStream_t s);
void dist_bump(int* counter, cudaStream_t s);
}

namespace sgb {
namespace {
using at::Tensor;

sg::PeerPtrs peers(const std::vector<int64_t>& ptrs) {
    TORCH_CHECK(ptrs.size() <= (size_t)sg::MAX_RANKS, "at most ", sg::MAX_RANKS, " ranks per node");
    sg::PeerPtrs p{};
    for (size_t i = 0; i < ptrs.size(); ++i) p.p[i] = reinterpret_cast<void*>(static_cast<intptr_t>(ptrs[i]));
    return p;
}
void* vp(int64_t x) { return reinterpret_cast<void*>(static_cast<intptr_t>(x)); }
int dcode(const std::string& s) { return s == "f32" ? sg::F32 : (s == "bf16" ? sg::BF16 : sg::F16); }

const float* dyn_ptr(const c10::optional<Tensor>& dyn) {
    if (!dyn.has_value() || !dyn->defined()) return nullptr;
    TORCH_CHECK(dyn->is_cuda() && dyn->scalar_type() == at::kFloat && dyn->is_contiguous(), "dyn: contiguous fp32 CUDA table of step scalars");
    return dyn->data_ptr<float>();
}
// epoch: the epoch itself, or (with `dyn`) the offset added to the base epoch held in the device table of step scalars
void barrier(const std::vector<int64_t>& pads, int64_t rank, int64_t epoch, Tensor status, double timeout_s, int64_t site,
             c10::optional<Tensor> dyn) {
    c10::cuda::CUDAGuard guard(status.device());
    sg::dist_barrier(peers(pads), (int)rank, (int)pads.size(), (uint32_t)epoch, reinterpret_cast<const uint32_t*>(dyn_ptr(dyn)),
                     status.data_ptr<int>(), (unsigned long long)(timeout_s * 1e9), (int)site, at::cuda::getCurrentCUDAStream());
}
void pull_reduce(const std::string& dtype, bool nvls, const std::vector<int64_t>& grads, int64_t mc, int64_t rank, int64_t off, int64_t n,
                 double scale, Tensor out) {
    c10::cuda::CUDAGuard guard(out.device());
    TORCH_CHECK(out.scalar_type() == at::kFloat && out.numel() >= n, "out must be fp32 with >= n elements");
    sg::dist_pull_reduce(dcode(dtype), nvls, peers(grads), vp(mc), (int)grads.size(), (int)rank, off, n, (float)scale, out.data_ptr<float>(),
                         at::cuda::getCurrentCUDAStream());
}
void push(bool nvls, const std::vector<int64_t>& params, int64_t mc, int64_t rank, int64_t off_bytes, int64_t n_bytes, Tensor anchor) {
    c10::cuda::CUDAGuard guard(anchor.device());
    sg::dist_push(nvls, peers(params), vp(mc), (int)params.size(), (int)rank, off_bytes, n_bytes, at::cuda::getCurrentCUDAStream());
}
void fused_flat_step(int64_t op, const std::string& gdtype, const std::string& pdtype, const std::vector<int64_t>& grads,
                     const std::vector<int64_t>& params, int64_t rank, int64_t off, int64_t n, const std::vector<double>& f, Tensor master,
                     Tensor m, c10::optional<Tensor> v, bool nvls, int64_t mc_grad, int64_t mc_param, c10::optional<Tensor> dyn, bool push) {
    c10::cuda::CUDAGuard guard(master.device());
    TORCH_CHECK(off % 8 == 0 && n % 8 == 0, "shard offset and length must be multiples of 8 elements");
    TORCH_CHECK(f.size() >= 8, "f = lr beta1 beta2 eps wd bc1 bc2 gscale");
    TORCH_CHECK(!nvls || (mc_grad != 0 && mc_param != 0), "NVLS requested without multicast addresses");
    TORCH_CHECK(gdtype != "f16" && pdtype != "f16", "the fused flat step supports fp32 and bf16");
    sg::dist_fused_flat_step((int)op, dcode(gdtype), dcode(pdtype), nvls, peers(grads), peers(params), vp(mc_grad), vp(mc_param),
                             (int)grads.size(), (int)rank, off, n, (float)f[0],
                             (float)f[1], (float)f[2], (float)f[3], (float)f[4], (float)f[5], (float)f[6], (float)f[7], master.data_ptr<float>(),
                             m.data_ptr<float>(), v.has_value() ? v->data_ptr<float>() : nullptr, dyn_ptr(dyn), push, at::cuda::getCurrentCUDAStream());
}
void cast_push(const std::string& pdtype, const std::vector<int64_t>& params, int64_t rank, int64_t off, int64_t n, Tensor master) {
    c10::cuda::CUDAGuard guard(master.device());
    TORCH_CHECK(off % 8 == 0, "offset must be a multiple of 8 elements");
    sg::dist_cast_push(dcode(pdtype), peers(params), (int)params.size(), (int)rank, off, n, master.data_ptr<float>(), at::cuda::getCurrentCUDAStream());
}
void scatter_slots(const std::vector<int64_t>& slots, int64_t rank, Tensor vec) {
    c10::cuda::CUDAGuard guard(vec.device());
    sg::dist_scatter_slots(peers(slots), (int)slots.size(), (int)rank, vec.data_ptr<float>(), (int)vec.numel(), at::cuda::getCurrentCUDAStream());
}
void reduce_slots(Tensor my_slots, int64_t world, Tensor out, double scale) {
    c10::cuda::CUDAGuard guard(out.device());
    sg::dist_reduce_slots(my_slots.data_ptr<float>(), (int)world, out.data_ptr<float>(), (int)out.numel(), (float)scale,
                          at::cuda::getCurrentCUDAStream());
}
}  // namespace

void bump(Tensor counter) {
    TORCH_CHECK(counter.is_cuda() && counter.scalar_type() == at::kInt && counter.numel() >= 1, "counter: int32 CUDA tensor");
    c10::cuda::CUDAGuard guard(counter.device());
    sg::dist_bump(counter.data_ptr<int>(), at::cuda::getCurrentCUDAStream());
}

void register_dist(pybind11::module_& m) {
    m.def("dist_bump", &bump);
    m.def("dist_barrier", &barrier, py::arg("pads"), py::arg("rank"), py::arg("epoch"), py::arg("status"), py::arg("timeout_s"), py::arg("site"),
          py::arg("dyn") = c10::optional<Tensor>());
    m.def("dist_pull_reduce", &pull_reduce);
    m.def("dist_push", &push);
    m.def("dist_fused_flat_step", &fused_flat_step, py::arg("op"), py::arg("gdtype"), py::arg("pdtype"), py::arg("grads"), py::arg("params"),
          py::arg("rank"), py::arg("off"), py::arg("n"), py::arg("f"), py::arg("master"), py::arg("m"), py::arg("v"), py::arg("nvls") = false,
          py::arg("mc_grad") = 0, py::arg("mc_param") = 0, py::arg("dyn") = c10::optional<Tensor>(), py::arg("push") = true);
    m.def("dist_scatter_slots", &scatter_slots);
    m.def("dist_cast_push", &cast_push);
    m.def("dist_reduce_slots", &reduce_slots);
    m.attr("STATUS_TIMEOUT") = (int)sg::STATUS_TIMEOUT;
}
}  // namespace sgb
