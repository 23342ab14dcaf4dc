// Bindings of the model-side kernels (short-sequence attention, LayerNorm with residual).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "bindings_decl.h"
#include "mt_host.h"

namespace sg {
bool attn_small_supported(int S, int HD);
void attn_small(int dtype, bool bwd, const void* qkv, const void* dout, void* out, int B, int S, int H, int HD, bool causal, cudaStream_t st);
void ln_fwd(int dtype, bool rms, const void* x, const void* r, const void* gamma, const void* beta, void* z, void* y, float* stats, int64_t rows,
            int D, float eps, cudaStream_t st);
int ln_bwd_parts(int64_t rows);
void ln_bwd(int dtype, bool rms, const void* z, const void* dy, const void* gamma, const float* stats, const void* dz_in, void* dz, float* part,
            void* dgamma, void* dbeta, bool accumulate, int64_t rows, int D, cudaStream_t st);
int col_sum_parts(int64_t rows, int C, int elem_bytes);
void col_sum(int dtype, const void* x, int64_t ld, int64_t rows, int C, float* part, void* out, bool accumulate, cudaStream_t st);
}

namespace sgb {
namespace py = pybind11;
namespace {
using at::Tensor;

Tensor attn_small_fwd(const Tensor& qkv, int64_t H, bool causal) {
    TORCH_CHECK(qkv.is_cuda() && qkv.is_contiguous() && qkv.dim() == 3, "qkv must be a contiguous CUDA tensor [B, S, 3*D]");
    const int B = (int)qkv.size(0), S = (int)qkv.size(1);
    const int64_t D = qkv.size(2) / 3;
    const int HD = (int)(D / H);
    TORCH_CHECK(sg::attn_small_supported(S, HD), "attn_small supports S in {4,8} and head_dim in {32,64}");
    TORCH_CHECK(qkv.scalar_type() == at::kBFloat16 || qkv.scalar_type() == at::kFloat, "attn_small: bf16 or fp32");
    c10::cuda::CUDAGuard guard(qkv.device());
    Tensor out = at::empty({B, S, D}, qkv.options());
    sg::attn_small(dtype_code(qkv), false, qkv.data_ptr(), nullptr, out.data_ptr(), B, S, (int)H, HD, causal, at::cuda::getCurrentCUDAStream());
    return out;
}

Tensor attn_small_bwd(const Tensor& qkv, const Tensor& dout, int64_t H, bool causal) {
    const int B = (int)qkv.size(0), S = (int)qkv.size(1);
    const int64_t D = qkv.size(2) / 3;
    c10::cuda::CUDAGuard guard(qkv.device());
    Tensor d = dout.contiguous();
    Tensor dqkv = at::empty_like(qkv);
    sg::attn_small(dtype_code(qkv), true, qkv.data_ptr(), d.data_ptr(), dqkv.data_ptr(), B, S, (int)H, (int)(D / H), causal, at::cuda::getCurrentCUDAStream());
    return dqkv;
}

// returns (y, z, stats); z is x + r (the LayerNorm input, kept for backward); with no residual z aliases x
std::vector<Tensor> ln_fwd(const Tensor& x, const c10::optional<Tensor>& r, const Tensor& gamma, const c10::optional<Tensor>& beta, double eps,
                           bool rms) {
    TORCH_CHECK(gamma.scalar_type() == x.scalar_type(), "norm weight and input must have the same dtype");
    TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "x must be contiguous CUDA");
    const int D = (int)x.size(-1);
    TORCH_CHECK(D % 4 == 0, "LayerNorm width must be a multiple of 4");
    const int64_t rows = x.numel() / D;
    c10::cuda::CUDAGuard guard(x.device());
    Tensor y = at::empty_like(x);
    Tensor z = r.has_value() ? at::empty_like(x) : x;
    Tensor stats = at::empty({rows, 2}, x.options().dtype(at::kFloat));
    sg::ln_fwd(dtype_code(x), rms, x.data_ptr(), r.has_value() ? r->contiguous().data_ptr() : nullptr, gamma.data_ptr(),
               beta.has_value() ? beta->data_ptr() : nullptr, z.data_ptr(), y.data_ptr(), stats.data_ptr<float>(), rows, D, (float)eps,
               at::cuda::getCurrentCUDAStream());
    return {y, z, stats};
}

// returns (dz, dgamma, dbeta).  With dgamma_acc (and dbeta_acc) the parameter gradients are ADDED to those tensors (the parameters'
// own gradient buffers) instead of being returned: no temporary and no accumulation kernel afterwards.
std::vector<Tensor> ln_bwd(const Tensor& z, const Tensor& dy, const Tensor& gamma, const Tensor& stats, bool has_beta, bool rms,
                           const c10::optional<Tensor>& dz_in, const c10::optional<Tensor>& dgamma_acc, const c10::optional<Tensor>& dbeta_acc) {
    const int D = (int)z.size(-1);
    const int64_t rows = z.numel() / D;
    TORCH_CHECK((size_t)8 * 2 * D * sizeof(float) <= 200 * 1024, "LayerNorm width too large for the fused backward");
    c10::cuda::CUDAGuard guard(z.device());
    Tensor d = dy.contiguous();
    Tensor dz = at::empty_like(z);
    Tensor part = at::empty({(int64_t)sg::ln_bwd_parts(rows), 2, D}, z.options().dtype(at::kFloat));
    const bool acc = dgamma_acc.has_value();
    if (acc) {
        TORCH_CHECK(dgamma_acc->is_contiguous() && dgamma_acc->numel() == D && dgamma_acc->scalar_type() == z.scalar_type() &&
                    dgamma_acc->device() == z.device(), "ln_bwd: dgamma_acc must be a contiguous [D] tensor of the input's dtype and device");
        TORCH_CHECK(!has_beta || (dbeta_acc.has_value() && dbeta_acc->is_contiguous() && dbeta_acc->numel() == D &&
                                  dbeta_acc->scalar_type() == z.scalar_type() && dbeta_acc->device() == z.device()),
                    "ln_bwd: dbeta_acc must accompany dgamma_acc when the norm has a bias");
    }
    Tensor dgamma = acc ? *dgamma_acc : at::empty_like(gamma);
    Tensor dbeta = has_beta ? (acc ? *dbeta_acc : at::empty_like(gamma)) : Tensor();
    Tensor e = dz_in.has_value() ? dz_in->contiguous() : Tensor();
    sg::ln_bwd(dtype_code(z), rms, z.data_ptr(), d.data_ptr(), gamma.data_ptr(), stats.data_ptr<float>(), dz_in.has_value() ? e.data_ptr() : nullptr,
               dz.data_ptr(), part.data_ptr<float>(),
               dgamma.data_ptr(), has_beta ? dbeta.data_ptr() : nullptr, acc, rows, D, at::cuda::getCurrentCUDAStream());
    return {dz, dgamma, dbeta};
}

// column sums of x [rows, C] (innermost stride 1) in x's dtype, accumulated in fp32 in a fixed order: the bias gradient of a Linear layer.
// With acc the sums are ADDED to that tensor (the bias' own gradient buffer) and it is returned.
Tensor col_sum(const Tensor& x, const c10::optional<Tensor>& acc) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1, "col_sum needs a CUDA matrix whose innermost stride is 1");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kFloat || x.scalar_type() == at::kHalf, "col_sum: fp32, bf16 or fp16");
    const int64_t rows = x.size(0);
    const int C = (int)x.size(1);
    c10::cuda::CUDAGuard guard(x.device());
    if (acc.has_value())
        TORCH_CHECK(acc->is_contiguous() && acc->numel() == C && acc->scalar_type() == x.scalar_type() && acc->device() == x.device(),
                    "col_sum: acc must be a contiguous [C] tensor of x's dtype and device");
    Tensor out = acc.has_value() ? *acc : at::empty({C}, x.options());
    if (rows == 0 || C == 0) return acc.has_value() ? out : out.zero_();
    Tensor part = at::empty({(int64_t)sg::col_sum_parts(rows, C, (int)x.element_size()), C}, x.options().dtype(at::kFloat));
    sg::col_sum(dtype_code(x), x.data_ptr(), x.stride(0), rows, C, part.data_ptr<float>(), out.data_ptr(), acc.has_value(), at::cuda::getCurrentCUDAStream());
    return out;
}
}  // namespace

void register_nn(pybind11::module_& m) {
    m.def("attn_small_fwd", &attn_small_fwd);
    m.def("attn_small_bwd", &attn_small_bwd);
    m.def("attn_small_supported", [](int64_t S, int64_t HD) { return sg::attn_small_supported((int)S, (int)HD); });
    m.def("col_sum", &col_sum, py::arg("x"), py::arg("acc") = c10::optional<Tensor>());
    m.def("ln_fwd", &ln_fwd, py::arg("x"), py::arg("residual"), py::arg("gamma"), py::arg("beta"), py::arg("eps"), py::arg("rms") = false);
    m.def("ln_bwd", &ln_bwd, py::arg("z"), py::arg("dy"), py::arg("gamma"), py::arg("stats"), py::arg("has_beta"), py::arg("rms") = false,
          py::arg("dz_in") = c10::optional<Tensor>(), py::arg("dgamma_acc") = c10::optional<Tensor>(), py::arg("dbeta_acc") = c10::optional<Tensor>());
}
}  // namespace sgb
