// Bindings of the tcgen05 GEMM.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "bindings_decl.h"
#include "mt_host.h"

namespace sg {
void gemm_plain_tile_coords(int tile, int n_tiles_m, int n_tiles_n, int* mt, int* nt);
int gemm_bf16_tn(const void* A, int lda, const void* B, int ldb, int M, int N, int K, float alpha, float beta, const void* D, int ldd,
                 bool d_bf16, const void* bias, bool bias_bf16, float diag, int act, void* C, int ldc, bool c_bf16, void* C2, int ldc2,
                 float* splitk_ws, int64_t splitk_ws_floats, int* err, cudaStream_t s, bool a_t, bool b_t);
int gemm_bf16_tn_allgather(const void* A, int lda, const PeerPtrs& w_peers, int rank, int world, int M, int N, int K, void* C, int ldc,
                           bool c_bf16, int* counters, void* sched, int epoch, int n_copy, int* err, cudaStream_t s, float alpha,
                           float beta, const void* D, int ldd, bool d_bf16, float diag, int diag_off, void* C2, int ldc2, const int* epoch_ptr);
int gemm_bf16_tn_reducescatter(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const PeerPtrs& slots, const PeerPtrs& flags,
                               int rank, int world, void* c_local, int ldc, int epoch, unsigned long long timeout_ns, int* err, cudaStream_t s,
                               const int* epoch_ptr);
}

namespace sgb {
namespace {
using at::Tensor;

// out = act(alpha * a @ b.T + beta * d + bias + diag * I);  a [M,K], b [N,K] bf16 row-major (last stride 1, row stride multiple of 8).
// out: bf16 or fp32 [M,N]; out_t (optional): [N,M] receives the transposed result.
void gemm_tn(const Tensor& a, const Tensor& b, Tensor out, double alpha, double beta, const c10::optional<Tensor>& d,
             const c10::optional<Tensor>& bias, double diag, int64_t act, const c10::optional<Tensor>& out_t, Tensor err,
             const c10::optional<Tensor>& splitk_ws, bool a_t, bool b_t) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda(), "gemm_tn needs CUDA tensors");
    TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "gemm_tn operands must be bf16");
    // a_t: a is stored [K, M]; b_t: b is stored [K, N]
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(a_t ? 0 : 1) == b.size(b_t ? 0 : 1), "shape mismatch: a [M,K] (or [K,M]), b [N,K] (or [K,N])");
    TORCH_CHECK(!a_t || b_t, "a_t without b_t is not supported");
    TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1, "innermost stride must be 1");
    TORCH_CHECK(a.stride(0) % 8 == 0 && b.stride(0) % 8 == 0, "row strides must be multiples of 8 elements (16 bytes)");
    TORCH_CHECK((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(b.data_ptr()) & 15) == 0, "operands must be 16-byte aligned");
    const int M = (int)a.size(a_t ? 1 : 0), N = (int)b.size(b_t ? 1 : 0), K = (int)a.size(a_t ? 0 : 1);
    TORCH_CHECK(out.size(0) == M && out.size(1) == N, "out must be [M,N]");
    const bool c_bf16 = out.scalar_type() == at::kBFloat16;
    TORCH_CHECK(c_bf16 || out.scalar_type() == at::kFloat, "out must be bf16 or fp32");
    if (d.has_value()) TORCH_CHECK(d->size(0) == M && d->size(1) == N && d->stride(1) == 1, "d must be [M,N]");
    if (out_t.has_value()) TORCH_CHECK(out_t->size(0) == N && out_t->size(1) == M && out_t->stride(1) == 1 && out_t->scalar_type() == out.scalar_type(), "out_t must be [N,M] of out's dtype");
    c10::cuda::CUDAGuard guard(a.device());
    const int rc = sg::gemm_bf16_tn(a.data_ptr(), (int)a.stride(0), b.data_ptr(), (int)b.stride(0), M, N, K, (float)alpha, (float)beta,
                                    d.has_value() ? d->data_ptr() : nullptr, d.has_value() ? (int)d->stride(0) : 0,
                                    d.has_value() && d->scalar_type() == at::kBFloat16, bias.has_value() ? bias->data_ptr() : nullptr,
                                    bias.has_value() && bias->scalar_type() == at::kBFloat16, (float)diag, (int)act, out.data_ptr(), (int)out.stride(0),
                                    c_bf16, out_t.has_value() ? out_t->data_ptr() : nullptr, out_t.has_value() ? (int)out_t->stride(0) : 0,
                                    splitk_ws.has_value() ? splitk_ws->data_ptr<float>() : nullptr, splitk_ws.has_value() ? splitk_ws->numel() : 0,
                                    err.data_ptr<int>(), at::cuda::getCurrentCUDAStream(), a_t, b_t);
    TORCH_CHECK(rc == 0, "gemm_tn launch failed (code ", rc, ")");
}

// out = a @ Wfull.T where Wfull [N, K] is assembled inside the kernel from the row shards held by `world` ranks:
// w_ptrs[r] is the address of rank r's [N, K] bf16 buffer (peer-mapped symmetric memory; w_ptrs[rank] is the local one).
// Optional epilogue: out = alpha * acc + beta * d + diag * [m + diag_off == n]; out_t [N, M] receives the transposed result.
void gemm_tn_allgather(const Tensor& a, const std::vector<int64_t>& w_ptrs, int64_t rank, int64_t N, Tensor out, Tensor counters, int64_t epoch,
                       int64_t n_copy, Tensor err, double alpha, double beta, const c10::optional<Tensor>& d, double diag, int64_t diag_off,
                       const c10::optional<Tensor>& out_t, const c10::optional<Tensor>& epoch_dev) {
    TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kBFloat16 && a.dim() == 2 && a.stride(1) == 1 && a.stride(0) % 8 == 0, "a must be bf16 [M,K]");
    const int world = (int)w_ptrs.size();
    TORCH_CHECK(world >= 1 && world <= sg::MAX_RANKS && rank >= 0 && rank < world, "bad rank / world");
    const int M = (int)a.size(0), K = (int)a.size(1);
    TORCH_CHECK(out.size(0) == M && out.size(1) == N && out.stride(1) == 1, "out must be [M,N]");
    TORCH_CHECK(N % (world * 32) == 0, "N must be a multiple of 32 * world");
    TORCH_CHECK(counters.is_cuda() && counters.scalar_type() == at::kInt && counters.numel() >= (N + 255) / 256 + 2 &&
                (reinterpret_cast<uintptr_t>(counters.data_ptr()) & 7) == 0, "counters: int32 [2 + ceil(N/256)], 8-byte aligned");
    TORCH_CHECK(n_copy >= 1 && n_copy <= 148 && (epoch >= 1 || epoch_dev.has_value()), "n_copy in [1,148], epoch >= 1");
    const int* ep_ptr = nullptr;
    if (epoch_dev.has_value()) {
        TORCH_CHECK(epoch_dev->is_cuda() && epoch_dev->scalar_type() == at::kInt && epoch_dev->numel() >= 1, "epoch_dev: int32 CUDA tensor");
        ep_ptr = epoch_dev->data_ptr<int>();
    }
    sg::PeerPtrs w{};
    for (int r = 0; r < world; ++r) {
        TORCH_CHECK(w_ptrs[r] != 0 && (w_ptrs[r] & 15) == 0, "weight buffers must be mapped and 16-byte aligned");
        w.p[r] = reinterpret_cast<void*>(w_ptrs[r]);
    }
    c10::cuda::CUDAGuard guard(a.device());
    const bool c_bf16 = out.scalar_type() == at::kBFloat16;
    if (d.has_value()) TORCH_CHECK(d->size(0) == M && d->size(1) == N && d->stride(1) == 1, "d must be [M,N]");
    if (out_t.has_value()) TORCH_CHECK(out_t->size(0) == N && out_t->size(1) == M && out_t->stride(1) == 1 && out_t->scalar_type() == out.scalar_type(), "out_t must be [N,M] of out's dtype");
    const int rc = sg::gemm_bf16_tn_allgather(a.data_ptr(), (int)a.stride(0), w, (int)rank, world, M, (int)N, K, out.data_ptr(), (int)out.stride(0),
                                              c_bf16, counters.data_ptr<int>() + 2, counters.data_ptr<int>(), (int)epoch, (int)n_copy, err.data_ptr<int>(),
                                              at::cuda::getCurrentCUDAStream(), (float)alpha, (float)beta, d.has_value() ? d->data_ptr() : nullptr,
                                              d.has_value() ? (int)d->stride(0) : 0, d.has_value() && d->scalar_type() == at::kBFloat16, (float)diag,
                                              (int)diag_off, out_t.has_value() ? out_t->data_ptr() : nullptr, out_t.has_value() ? (int)out_t->stride(0) : 0, ep_ptr);
    TORCH_CHECK(rc == 0, "gemm_tn_allgather launch failed (code ", rc, ")");
}

// out [M / world, N] = this rank's rows of sum_r a_r @ b_r.T (K sharded over the ranks); slot_ptrs / flag_ptrs: every rank's buffers.
void gemm_tn_reducescatter(const Tensor& a, const Tensor& b, const std::vector<int64_t>& slot_ptrs, const std::vector<int64_t>& flag_ptrs,
                           int64_t rank, Tensor out, int64_t epoch, double timeout_s, Tensor err, const c10::optional<Tensor>& epoch_dev) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "operands must be CUDA bf16");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1) && a.stride(1) == 1 && b.stride(1) == 1 && a.stride(0) % 8 == 0 &&
                b.stride(0) % 8 == 0, "a [M,K], b [N,K], rows 16-byte aligned");
    const int world = (int)slot_ptrs.size();
    TORCH_CHECK(world >= 1 && world <= sg::MAX_RANKS && (int)flag_ptrs.size() == world && rank >= 0 && rank < world, "bad rank / world");
    const int M = (int)a.size(0), N = (int)b.size(0), K = (int)a.size(1);
    TORCH_CHECK(M % (world * 128) == 0 && N % 64 == 0, "M must be a multiple of 128 * world and N of 64");
    TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.size(0) == M / world && out.size(1) == N && out.stride(1) == 1 && out.stride(0) % 8 == 0,
                "out must be bf16 [M / world, N]");
    sg::PeerPtrs sl{}, fl{};
    for (int r = 0; r < world; ++r) { sl.p[r] = reinterpret_cast<void*>(slot_ptrs[r]); fl.p[r] = reinterpret_cast<void*>(flag_ptrs[r]); }
    c10::cuda::CUDAGuard guard(a.device());
    const int rc = sg::gemm_bf16_tn_reducescatter(a.data_ptr(), (int)a.stride(0), b.data_ptr(), (int)b.stride(0), M, N, K, sl, fl, (int)rank, world,
                                                  out.data_ptr(), (int)out.stride(0), (int)epoch, (unsigned long long)(timeout_s * 1e9),
                                                  err.data_ptr<int>(), at::cuda::getCurrentCUDAStream(),
                                                  epoch_dev.has_value() ? epoch_dev->data_ptr<int>() : nullptr);
    TORCH_CHECK(rc == 0, "gemm_tn_reducescatter launch failed (code ", rc, ")");
}
}  // namespace

void register_gemm(pybind11::module_& m) {
    m.def("gemm_tile_order", [](int64_t n_tiles_m, int64_t n_tiles_n) {          // the plain GEMM's tile order, for host-side checks
        std::vector<std::pair<int64_t, int64_t>> order;
        for (int64_t t = 0; t < n_tiles_m * n_tiles_n; ++t) {
            int mt = 0, nt = 0;
            sg::gemm_plain_tile_coords((int)t, (int)n_tiles_m, (int)n_tiles_n, &mt, &nt);
            order.emplace_back(mt, nt);
        }
        return order;
    });
    m.def("gemm_tn", &gemm_tn, py::arg("a"), py::arg("b"), py::arg("out"), py::arg("alpha") = 1.0, py::arg("beta") = 0.0,
          py::arg("d") = c10::nullopt, py::arg("bias") = c10::nullopt, py::arg("diag") = 0.0, py::arg("act") = 0,
          py::arg("out_t") = c10::nullopt, py::arg("err"), py::arg("splitk_ws") = c10::nullopt, py::arg("a_t") = false, py::arg("b_t") = false);
    m.def("gemm_tn_reducescatter", &gemm_tn_reducescatter, py::arg("a"), py::arg("b"), py::arg("slot_ptrs"), py::arg("flag_ptrs"), py::arg("rank"),
          py::arg("out"), py::arg("epoch"), py::arg("timeout_s"), py::arg("err"), py::arg("epoch_dev") = c10::nullopt);
    m.def("gemm_tn_allgather", &gemm_tn_allgather, py::arg("a"), py::arg("w_ptrs"), py::arg("rank"), py::arg("N"), py::arg("out"),
          py::arg("counters"), py::arg("epoch"), py::arg("n_copy"), py::arg("err"), py::arg("alpha") = 1.0, py::arg("beta") = 0.0,
          py::arg("d") = c10::nullopt, py::arg("diag") = 0.0, py::arg("diag_off") = 0, py::arg("out_t") = c10::nullopt,
          py::arg("epoch_dev") = c10::nullopt);
}
}  // namespace sgb
