// Bindings of the decoder-model kernels (rotary embedding, SwiGLU, GELU, embedding, cross-entropy).
#include <cmath>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "bindings_decl.h"
#include "mt_host.h"

namespace sg {
void rope(int dtype, const void* x, void* y, const float* cosT, const float* sinT, int64_t B, int S, int H, int HD, bool backward, cudaStream_t st);
void swiglu(int dtype, bool backward, const void* g, const void* u, const void* dy, void* out0, void* out1, int64_t n, cudaStream_t st);
void gelu(int dtype, bool backward, const void* x, const void* dy, void* y, int64_t n, cudaStream_t st);
void embed_fwd(int dtype, const int64_t* ids, const void* W, void* out, int64_t T_tok, int D, int V, cudaStream_t st);
void embed_keys(const int64_t* ids, uint32_t* keys, uint32_t* vals, int64_t T_tok, int V, cudaStream_t st);
void embed_bwd(int dtype, const uint32_t* keys, const uint32_t* vals, const void* dout, void* dW, int64_t T_tok, int D, cudaStream_t st);
bool embed_bwd_small_ok(int64_t T_tok, int V);
int embed_bwd_table_splits(int64_t T_tok, int D, int V);
void embed_bwd_table(int dtype, const int64_t* ids, const void* dout, float* part, void* dW, int64_t T_tok, int D, int V, int S, bool accumulate,
                     cudaStream_t st);
void embed_bwd_small(int dtype, const int64_t* ids, const void* dout, void* dW, int64_t T_tok, int D, int V, bool accumulate, cudaStream_t st);
void ce_fwd(int dtype, const void* logits, const int64_t* target, float* lse, float* loss, float* mean_out, int64_t rows, int V, int64_t ignore_index,
            cudaStream_t st);
void ce_bwd(int dtype, const void* logits, const int64_t* target, const float* lse, const float* mean_out, const float* gout, void* dlogits,
            int64_t rows, int V, int64_t ignore_index, cudaStream_t st);
bool flash_attn_supported(int S, int HD);
int flash_attn_fwd(const void* q, const void* k, const void* v, int64_t ld, void* out, int64_t ld_o, float* lse, int B, int S, int H, int HD,
                   float scale, bool causal, int variant, int* err, cudaStream_t st);
int flash_attn_bwd(const void* q, const void* k, const void* v, int64_t ld, const void* o, const void* dout, int64_t ld_o, const float* lse,
                   float* delta, void* dq, void* dk, void* dv, int B, int S, int H, int HD, float scale, bool causal, int* err, cudaStream_t st);
}

namespace sgb {
namespace py = pybind11;
namespace {
using at::Tensor;

void check_act(const Tensor& x, const char* what) {
    TORCH_CHECK(x.is_cuda() && x.is_contiguous(), what, ": contiguous CUDA tensor expected");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kFloat || x.scalar_type() == at::kHalf, what, ": bf16, fp16 or fp32");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, what, ": storage must be 16-byte aligned");
}

// x: [B, S, H, HD] -> rotated copy (backward = true applies the inverse rotation to a gradient)
Tensor rope(const Tensor& x, const Tensor& cosT, const Tensor& sinT, bool backward) {
    check_act(x, "rope");
    TORCH_CHECK(x.dim() == 4, "rope: x must be [B, S, H, HD]");
    const int64_t B = x.size(0);
    const int S = (int)x.size(1), H = (int)x.size(2), HD = (int)x.size(3);
    TORCH_CHECK(HD % 8 == 0, "rope: head_dim must be a multiple of 8");
    TORCH_CHECK(cosT.is_cuda() && cosT.scalar_type() == at::kFloat && cosT.is_contiguous() && cosT.size(0) >= S && cosT.size(1) == HD / 2 &&
                sinT.is_cuda() && sinT.scalar_type() == at::kFloat && sinT.is_contiguous() && sinT.sizes() == cosT.sizes(),
                "rope: cos/sin must be contiguous fp32 CUDA tables [>=S, HD/2]");
    c10::cuda::CUDAGuard guard(x.device());
    Tensor y = at::empty_like(x);
    sg::rope(dtype_code(x), x.data_ptr(), y.data_ptr(), cosT.data_ptr<float>(), sinT.data_ptr<float>(), B, S, H, HD, backward,
             at::cuda::getCurrentCUDAStream());
    return y;
}

Tensor swiglu_fwd(const Tensor& g, const Tensor& u) {
    check_act(g, "swiglu"); check_act(u, "swiglu");
    TORCH_CHECK(g.sizes() == u.sizes() && g.scalar_type() == u.scalar_type() && g.numel() % 8 == 0, "swiglu: equal shapes, numel multiple of 8");
    c10::cuda::CUDAGuard guard(g.device());
    Tensor y = at::empty_like(g);
    sg::swiglu(dtype_code(g), false, g.data_ptr(), u.data_ptr(), nullptr, y.data_ptr(), nullptr, g.numel(), at::cuda::getCurrentCUDAStream());
    return y;
}

std::vector<Tensor> swiglu_bwd(const Tensor& g, const Tensor& u, const Tensor& dy_) {
    Tensor dy = dy_.contiguous();
    check_act(dy, "swiglu");
    c10::cuda::CUDAGuard guard(g.device());
    Tensor dg = at::empty_like(g), du = at::empty_like(u);
    sg::swiglu(dtype_code(g), true, g.data_ptr(), u.data_ptr(), dy.data_ptr(), dg.data_ptr(), du.data_ptr(), g.numel(), at::cuda::getCurrentCUDAStream());
    return {dg, du};
}

Tensor gelu_fwd(const Tensor& x) {
    check_act(x, "gelu");
    TORCH_CHECK(x.numel() % 8 == 0, "gelu: numel multiple of 8");
    c10::cuda::CUDAGuard guard(x.device());
    Tensor y = at::empty_like(x);
    sg::gelu(dtype_code(x), false, x.data_ptr(), nullptr, y.data_ptr(), x.numel(), at::cuda::getCurrentCUDAStream());
    return y;
}
Tensor gelu_bwd(const Tensor& x, const Tensor& dy_) {
    Tensor dy = dy_.contiguous();
    check_act(dy, "gelu");
    c10::cuda::CUDAGuard guard(x.device());
    Tensor dx = at::empty_like(x);
    sg::gelu(dtype_code(x), true, x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel(), at::cuda::getCurrentCUDAStream());
    return dx;
}

Tensor embedding_fwd(const Tensor& ids, const Tensor& W) {
    check_act(W, "embedding");
    TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "embedding: ids must be contiguous int64 CUDA");
    const int D = (int)W.size(1), V = (int)W.size(0);
    TORCH_CHECK((D * W.element_size()) % 16 == 0, "embedding: row bytes must be a multiple of 16");
    c10::cuda::CUDAGuard guard(W.device());
    auto shape = ids.sizes().vec();
    shape.push_back(D);
    Tensor out = at::empty(shape, W.options());
    sg::embed_fwd(dtype_code(W), ids.data_ptr<int64_t>(), W.data_ptr(), out.data_ptr(), ids.numel(), D, V, at::cuda::getCurrentCUDAStream());
    return out;
}

// Deterministic gradient of the gather: stable radix sort of the token ids (the framework's own sort), then one warp per id run.
// Gradient of the table.  With acc the result is ADDED to that tensor (the table's own gradient buffer), which is returned.
Tensor embedding_bwd(const Tensor& ids, const Tensor& dout_, int64_t V, const c10::optional<Tensor>& acc) {
    Tensor dout = dout_.contiguous();
    check_act(dout, "embedding");
    const int D = (int)dout.size(-1);
    const int64_t T_tok = ids.numel();
    TORCH_CHECK(D % 8 == 0 && T_tok < (int64_t)1 << 31, "embedding: width multiple of 8, fewer than 2^31 tokens");
    if (acc.has_value())
        TORCH_CHECK(acc->is_contiguous() && acc->dim() == 2 && acc->size(0) == V && acc->size(1) == D && acc->scalar_type() == dout.scalar_type() &&
                    acc->device() == dout.device(), "embedding_bwd: acc must be a contiguous [V, D] tensor of the gradient's dtype and device");
    c10::cuda::CUDAGuard guard(dout.device());
    auto st = at::cuda::getCurrentCUDAStream();
    auto io = dout.options().dtype(at::kInt);
    if (const int S = sg::embed_bwd_table_splits(T_tok, D, (int)V)) {     // table fits shared memory: per-split tables + ordered sum
        Tensor out = acc.has_value() ? *acc : at::empty({V, D}, dout.options());
        Tensor part = at::empty({S, V, D}, dout.options().dtype(at::kFloat));
        sg::embed_bwd_table(dtype_code(dout), ids.data_ptr<int64_t>(), dout.data_ptr(), part.data_ptr<float>(), out.data_ptr(), T_tok, D, (int)V, S,
                            acc.has_value(), st);
        return out;
    }
    if (sg::embed_bwd_small_ok(T_tok, (int)V)) {                         // small table: one kernel, no sort, no zero fill
        Tensor out = acc.has_value() ? *acc : at::empty({V, D}, dout.options());
        sg::embed_bwd_small(dtype_code(dout), ids.data_ptr<int64_t>(), dout.data_ptr(), out.data_ptr(), T_tok, D, (int)V, acc.has_value(), st);
        return out;
    }
    if (acc.has_value()) return acc->add_(embedding_bwd(ids, dout, V, c10::nullopt));
    Tensor dW = at::zeros({V, D}, dout.options());
    if (T_tok == 0) return dW;
    Tensor kv = at::empty({4, T_tok}, io);
    const int64_t nb = (int64_t)sg::sg2_sort_blocks(T_tok);
    Tensor hist = at::empty({256 * nb + 256}, io);
    Tensor seg = at::zeros({2}, dout.options().dtype(at::kLong));          // one segment: offsets are only read when there are several
    auto* k0 = reinterpret_cast<uint32_t*>(kv.data_ptr<int>());
    uint32_t* k1 = k0 + T_tok; uint32_t* v0 = k1 + T_tok; uint32_t* v1 = v0 + T_tok;
    auto* h = reinterpret_cast<uint32_t*>(hist.data_ptr<int>());
    sg::embed_keys(ids.data_ptr<int64_t>(), k0, v0, T_tok, (int)V, st);
    int cur = 0;
    sg::sg2_segmented_sort(k0, k1, v0, v1, h, h + 256 * nb, seg.data_ptr<int64_t>(), 1, T_tok, &cur, st);
    sg::embed_bwd(dtype_code(dout), cur ? k1 : k0, cur ? v1 : v0, dout.data_ptr(), dW.data_ptr(), T_tok, D, st);
    return dW;
}

// returns (mean loss [1], lse [rows], mean_out [2] = {mean, 1/count})
std::vector<Tensor> ce_fwd(const Tensor& logits, const Tensor& target, int64_t ignore_index) {
    check_act(logits, "cross_entropy");
    TORCH_CHECK(logits.dim() == 2 && logits.size(1) % 8 == 0, "cross_entropy: logits [rows, V] with V a multiple of 8");
    TORCH_CHECK(target.is_cuda() && target.scalar_type() == at::kLong && target.is_contiguous() && target.numel() == logits.size(0),
                "cross_entropy: target must be contiguous int64 CUDA [rows]");
    c10::cuda::CUDAGuard guard(logits.device());
    const int64_t rows = logits.size(0);
    auto fo = logits.options().dtype(at::kFloat);
    Tensor lse = at::empty({rows}, fo), loss = at::empty({rows}, fo), mean_out = at::zeros({2}, fo);
    sg::ce_fwd(dtype_code(logits), logits.data_ptr(), target.data_ptr<int64_t>(), lse.data_ptr<float>(), loss.data_ptr<float>(),
               mean_out.data_ptr<float>(), rows, (int)logits.size(1), ignore_index, at::cuda::getCurrentCUDAStream());
    return {mean_out.narrow(0, 0, 1).reshape({}), lse, mean_out};
}

Tensor ce_bwd(const Tensor& logits, const Tensor& target, const Tensor& lse, const Tensor& mean_out, const Tensor& gout, int64_t ignore_index) {
    c10::cuda::CUDAGuard guard(logits.device());
    Tensor g = gout.to(at::kFloat).contiguous();
    Tensor d = at::empty_like(logits);
    sg::ce_bwd(dtype_code(logits), logits.data_ptr(), target.data_ptr<int64_t>(), lse.data_ptr<float>(), mean_out.data_ptr<float>(),
               g.data_ptr<float>(), d.data_ptr(), logits.size(0), (int)logits.size(1), ignore_index, at::cuda::getCurrentCUDAStream());
    return d;
}

// q, k, v: bf16 [B, S, H, HD] views whose position stride is a common `ld` and whose heads are adjacent (stride HD); returns (out, lse)
void check_qkv(const Tensor& t, const Tensor& q, const char* what) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 4 && t.sizes() == q.sizes(), what, ": bf16 CUDA [B, S, H, HD]");
    TORCH_CHECK(t.stride(3) == 1 && t.stride(2) == t.size(3) && t.stride(1) == q.stride(1) && t.stride(0) == t.size(1) * t.stride(1) &&
                t.stride(1) % 8 == 0 && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, what, ": unsupported strides");
}

std::vector<Tensor> flash_fwd(const Tensor& q, const Tensor& k, const Tensor& v, bool causal, Tensor err, int64_t variant) {
    check_qkv(q, q, "q"); check_qkv(k, q, "k"); check_qkv(v, q, "v");
    const int B = (int)q.size(0), S = (int)q.size(1), H = (int)q.size(2), HD = (int)q.size(3);
    TORCH_CHECK(sg::flash_attn_supported(S, HD), "flash attention: S must be a multiple of 128 and head_dim 64 or 128");
    c10::cuda::CUDAGuard guard(q.device());
    Tensor out = at::empty({B, S, H, HD}, q.options());
    Tensor lse = at::empty({B, H, S}, q.options().dtype(at::kFloat));
    const int rc = sg::flash_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(1), out.data_ptr(), (int64_t)H * HD, lse.data_ptr<float>(), B, S,
                                      H, HD, 1.f / std::sqrt((float)HD), causal, (int)variant, err.data_ptr<int>(), at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(rc == 0, "flash_fwd launch failed (code ", rc, ")");
    return {out, lse};
}

// gradients of flash_fwd: returns (dq, dk, dv), contiguous [B, S, H, HD]
std::vector<Tensor> flash_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& lse, const Tensor& dout_, bool causal,
                              Tensor err) {
    check_qkv(q, q, "q"); check_qkv(k, q, "k"); check_qkv(v, q, "v");
    Tensor dout = dout_.contiguous();
    TORCH_CHECK(out.is_contiguous() && out.sizes() == q.sizes() && dout.sizes() == q.sizes() && dout.scalar_type() == at::kBFloat16 &&
                out.scalar_type() == at::kBFloat16, "out / dout must be contiguous bf16 [B, S, H, HD]");
    const int B = (int)q.size(0), S = (int)q.size(1), H = (int)q.size(2), HD = (int)q.size(3);
    TORCH_CHECK(lse.is_contiguous() && lse.scalar_type() == at::kFloat && lse.numel() == (int64_t)B * H * S, "lse: fp32 [B, H, S]");
    c10::cuda::CUDAGuard guard(q.device());
    Tensor dq = at::empty({B, S, H, HD}, q.options()), dk = at::empty({B, S, H, HD}, q.options()), dv = at::empty({B, S, H, HD}, q.options());
    Tensor delta = at::empty({B, H, S}, lse.options());
    const int rc = sg::flash_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(1), out.data_ptr(), dout.data_ptr(), (int64_t)H * HD,
                                      lse.data_ptr<float>(), delta.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, S, H, HD,
                                      1.f / std::sqrt((float)HD), causal, err.data_ptr<int>(), at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(rc == 0, "flash_bwd launch failed (code ", rc, "): q ", q.data_ptr(), " ld ", q.stride(1), " dout ", dout.data_ptr(), " B ", B, " S ", S, " H ", H,
                " HD ", HD);
    return {dq, dk, dv};
}
}  // namespace

void register_llm(pybind11::module_& m) {
    m.def("rope", &rope, py::arg("x"), py::arg("cos"), py::arg("sin"), py::arg("backward") = false);
    m.def("swiglu_fwd", &swiglu_fwd);
    m.def("swiglu_bwd", &swiglu_bwd);
    m.def("gelu_fwd", &gelu_fwd);
    m.def("gelu_bwd", &gelu_bwd);
    m.def("embedding_fwd", &embedding_fwd);
    m.def("embedding_bwd_table_splits", [](int64_t tokens, int64_t D, int64_t V) { return (int64_t)sg::embed_bwd_table_splits(tokens, (int)D, (int)V); });
    m.def("embedding_bwd", &embedding_bwd, py::arg("ids"), py::arg("dout"), py::arg("vocab"), py::arg("acc") = c10::optional<Tensor>());
    m.def("flash_fwd", &flash_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("causal"), py::arg("err"), py::arg("variant") = 3);
    m.def("flash_bwd", &flash_bwd);
    m.def("flash_supported", [](int64_t S, int64_t HD) { return sg::flash_attn_supported((int)S, (int)HD); });
    m.def("ce_fwd", &ce_fwd);
    m.def("ce_bwd", &ce_bwd);
}
}  // namespace sgb
