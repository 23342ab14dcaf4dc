// Bindings of the SuperGrok v2 step pipeline (sort, scan, element step).
#include <cstring>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include "bindings_decl.h"
#include "mt_host.h"
#include "sg2_routing_math.h"
#include "sg2_gru_math.h"

namespace sg {
void sg2_upload_weights(const float* packed_dev, cudaStream_t s);
void sg2_sqnorm(int dtype, const MTArgs& a, float* partials, cudaStream_t s);
void sg2_prep(int dtype, bool packed_src, const MTArgs& a, const float* tclip, float* g_packed, float* s_packed, uint32_t* keys, uint32_t* vals,
              cudaStream_t s);
void sg2_pull_sqnorm(int dtype, const MTArgs& a, const PeerPtrs& bases, int world, int rank, void* local_base, float scale, float* g_packed,
                     float* partials, cudaStream_t s);
void sg2_gather(const uint32_t* vals_sorted, const float* g_packed, const float* s_packed, float* gs_sorted, int64_t total, cudaStream_t s);
void sg2_scan(const void* items_dev, int n_items, int dir1_start, const void* tds_dev, int n_td, bool any_multi, const float* gs_sorted,
              const uint32_t* vals_sorted, float* agg, float* carry, float* ctx, const int* status, cudaStream_t s);
void sg2_elem(int dtype, const MTArgs& a, float beta2, float eps, float rescale, const float* dyn, const float* w_global, const int* status,
              const float* g_packed,
              const float* s_packed, const float* ctx, int* expert_counts, int n_peers, void* local_base, void* const* peer_base,
              cudaStream_t s);
size_t sg2_item_bytes();
size_t sg2_td_bytes();
size_t sg2_bilevel_smem_bytes();
int sg2_bilevel_ng();
int sg2_bilevel_tile();
void sg2_scan_backward(const void* items_dev, int n_items, int dir1_start, const void* tds_dev, int n_td, const int64_t* snap_base_dev,
                       const float* gs_sorted, const uint32_t* vals_sorted, const float* dctx, const float* carry, float* agg, float* dcarry,
                       float* snaps, float* partial, float* grads, int snap_every, cudaStream_t s);
}

namespace sg {
void sg2_recycle(int* counts, float* W1, float* b1, float* W2, float* b2, float* const* keyA, float* const* keyB, float threshold,
                 uint32_t seed, uint32_t call, int* info, cudaStream_t s);
}

namespace sg {
bool routed_experts_supported(int heads, int E, int hidden, int topk);
int routed_experts_bwd_ctas(int64_t n, int heads);
int routed_experts_fwd(const float* g, const int* ia, const int* ib, const float* wa, const float* wb, const float* W1, const float* b1,
                       const float* W2, const float* b2, int64_t n, int heads, int E, int pk, float* total, cudaStream_t s);
int routed_experts_bwd(const float* g, const int* ia, const int* ib, const float* wa, const float* wb, const float* W1, const float* b1,
                       const float* W2, const float* b2, const float* dtotal, int64_t n, int heads, int E, int pk, float* dwa, float* dwb,
                       float* partial, float* dparams, cudaStream_t s);
}

namespace sg {
bool routing_supported(int heads, int P, int pk, int d_model, int topk);
int routing_bwd_ctas(int64_t n, int heads);
int routing_ng(int heads, int P, int pk);
int routing_fwd(const float* pin, const float* Wq, const float* KA, const float* KB, int64_t n, int heads, int P, int pk, int* ia, int* ib,
                float* wa, float* wb, cudaStream_t s);
int routing_bwd(const float* pin, const float* Wq, const float* KA, const float* KB, const int* ia, const int* ib, const float* wa, const float* wb,
                const float* dwa, const float* dwb, int64_t n, int heads, int P, int pk, float* dpin, float* partial, float* dparams, cudaStream_t s);
}

namespace sg {
int gru_ng(int IN);
bool gru_supported(int IN, int hidden);
int gru_bwd_ctas(int64_t n);
int gru_fwd(const float* x, const float* h, const float* W, const float* b, int64_t n, int IN, float* hn, cudaStream_t s);
int gru_bwd(const float* x, const float* h, const float* W, const float* b, const float* dhn, int64_t n, int IN, float* dx, float* partial,
            float* dparams, cudaStream_t s);
}

namespace sgb {
namespace {
using at::Tensor;
using TL = std::vector<Tensor>;

uint32_t* u32(const Tensor& t) { return reinterpret_cast<uint32_t*>(t.data_ptr()); }

// ws: dict of workspace tensors allocated by the caller (see ops/sg2.py for the sizes).
// pull_bases (optional): base address of every rank's gradient buffer; `grads` are then this rank's tensors inside its own buffer
// (base pull_bases[pull_rank]) and the first kernel reduces the W copies itself (reduce-scatter fused into the pipeline).
// stage: 0 = everything, 1 = norm + clip + keys only, 2 = sort + gather only (per-phase timing).
int64_t sg2_prepare(const TL& grads, const TL& sharps, const std::vector<int64_t>& offsets, int64_t total, Tensor seg_off, double clip,
                    py::dict ws, const std::vector<int64_t>& pull_bases, int64_t pull_rank, double pull_scale, int64_t stage) {
    TORCH_CHECK(!grads.empty(), "no gradients");
    c10::cuda::CUDAGuard guard(grads[0].device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const int dt = dtype_code(grads[0]);
    auto W = [&](const char* k) { return ws[k].cast<Tensor>(); };
    Tensor partials = W("partials"), tnorm = W("tnorm"), tclip = W("tclip"), g = W("g"), s = W("s");
    Tensor k0 = W("keys0"), k1 = W("keys1"), v0 = W("vals0"), v1 = W("vals1"), hist = W("hist"), tot = W("tot"), gs = W("gs");
    const int n = (int)grads.size();
    const bool pull = !pull_bases.empty();
    if (stage != 2) {
        if (pull) {
            TORCH_CHECK(pull_bases.size() <= (size_t)sg::MAX_RANKS && pull_rank >= 0 && pull_rank < (int64_t)pull_bases.size(), "bad peer table");
            sg::PeerPtrs bases{};
            for (size_t r = 0; r < pull_bases.size(); ++r) bases.p[r] = reinterpret_cast<void*>(static_cast<intptr_t>(pull_bases[r]));
            const int64_t esz = grads[0].element_size();
            for (const Tensor& t : grads) {
                const int64_t d = reinterpret_cast<char*>(t.data_ptr()) - reinterpret_cast<char*>(bases.p[pull_rank]);
                TORCH_CHECK(d >= 0 && d % 16 == 0 && (int)dtype_code(t) == dt && t.element_size() == esz,
                            "pulled gradients must be 16-byte aligned slices of this rank's gradient buffer, all of one dtype");
            }
            for_each_launch({{}, grads}, {}, &offsets, [&](sg::MTArgs& a) {
                sg::sg2_pull_sqnorm(dt, a, bases, (int)pull_bases.size(), (int)pull_rank, bases.p[pull_rank], (float)pull_scale,
                                    g.data_ptr<float>(), partials.data_ptr<float>(), st);
                sg::mt_finalize_per_tensor(a, partials.data_ptr<float>(), tnorm.data_ptr<float>(), st);
            });
        } else {
            for_each_launch({{}, grads}, {}, nullptr, [&](sg::MTArgs& a) {
                sg::sg2_sqnorm(dt, a, partials.data_ptr<float>(), st);
                sg::mt_finalize_per_tensor(a, partials.data_ptr<float>(), tnorm.data_ptr<float>(), st);
            });
        }
        sg::scalar_finalize(sg::SC_SG2_CLIP, tnorm.data_ptr<float>(), n, tclip.data_ptr<float>(), (float)clip, 0.f, 0.f, st);
        for_each_launch({{}, grads, sharps}, {}, &offsets, [&](sg::MTArgs& a) {
            sg::sg2_prep(dt, pull, a, tclip.data_ptr<float>(), g.data_ptr<float>(), s.data_ptr<float>(), u32(k0), u32(v0), st);
        });
        if (stage == 1) return 0;
    }
    int cur = 0;
    sg::sg2_segmented_sort(u32(k0), u32(k1), u32(v0), u32(v1), u32(hist), u32(tot), seg_off.data_ptr<int64_t>(), n, total, &cur, st);
    const uint32_t* vs = cur ? u32(v1) : u32(v0);
    sg::sg2_gather(vs, g.data_ptr<float>(), s.data_ptr<float>(), gs.data_ptr<float>(), total, st);
    return cur;
}

const int* status_ptr(const c10::optional<Tensor>& st) {
    if (!st.has_value() || !st->defined()) return nullptr;
    TORCH_CHECK(st->is_cuda() && st->scalar_type() == at::kInt && st->numel() >= 1, "status: int32 CUDA tensor");
    return st->data_ptr<int>();
}

void sg2_scan(Tensor items, int64_t n_items, int64_t dir1_start, Tensor tds, int64_t n_td, bool any_multi, int64_t sorted_buf, py::dict ws,
              c10::optional<Tensor> status) {
    c10::cuda::CUDAGuard guard(items.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    auto W = [&](const char* k) { return ws[k].cast<Tensor>(); };
    const uint32_t* vs = sorted_buf ? u32(W("vals1")) : u32(W("vals0"));
    sg::sg2_scan(items.data_ptr(), (int)n_items, (int)dir1_start, tds.data_ptr(), (int)n_td, any_multi, W("gs").data_ptr<float>(), vs,
                 W("agg").data_ptr<float>(), W("carry").data_ptr<float>(), W("ctx").data_ptr<float>(), status_ptr(status), st);
}

// masters: empty, or one fp32 tensor per parameter.  peer_ptrs: base addresses of the peers' parameter buffers (same layout as
// the local buffer starting at local_base); the updated parameters are also stored there (all-gather fused into the step).
// dyn: device table of step scalars (sg_native.h: DYN_*); packed: the packed meta-net weights (global-memory copy).
void sg2_elem(const TL& params, const TL& ms, const TL& vs, const TL& mus, const TL& grus, const TL& masters, Tensor dyn, Tensor packed,
              const std::vector<int64_t>& offsets, double beta2, double eps, double rescale, c10::optional<Tensor> expert_counts, py::dict ws,
              int64_t local_base, const std::vector<int64_t>& peer_ptrs, c10::optional<Tensor> status) {
    c10::cuda::CUDAGuard guard(params[0].device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const int dt = dtype_code(params[0]);
    auto W = [&](const char* k) { return ws[k].cast<Tensor>(); };
    Tensor g = W("g"), s = W("s"), ctx = W("ctx");
    TORCH_CHECK(dyn.is_cuda() && dyn.scalar_type() == at::kFloat && dyn.is_contiguous() &&
                dyn.numel() >= sg::DYN_TS + 4 * (int64_t)params.size(), "dyn: fp32 table of at least 16 + 4 * tensors words");
    TORCH_CHECK(packed.is_cuda() && packed.scalar_type() == at::kFloat && packed.is_contiguous() && packed.numel() == sg::SG2Pack::TOTAL,
                "packed meta-net weights expected");
    int* ec = expert_counts.has_value() ? expert_counts->data_ptr<int>() : nullptr;
    TORCH_CHECK(peer_ptrs.size() <= 8, "at most 8 peers");
    void* peers[8] = {nullptr};
    for (size_t r = 0; r < peer_ptrs.size(); ++r) peers[r] = reinterpret_cast<void*>(static_cast<intptr_t>(peer_ptrs[r]));
    if (!peer_ptrs.empty())
        for (const Tensor& t : params)
            TORCH_CHECK((reinterpret_cast<char*>(t.data_ptr()) - reinterpret_cast<char*>(static_cast<intptr_t>(local_base))) % 16 == 0,
                        "pushed parameters must be 16-byte aligned slices of the parameter buffer");
    for_each_launch({params, ms, vs, mus, grus, masters}, {}, &offsets, [&](sg::MTArgs& a) {
        sg::sg2_elem(dt, a, (float)beta2, (float)eps, (float)rescale, dyn.data_ptr<float>(), packed.data_ptr<float>(), status_ptr(status), g.data_ptr<float>(),
                     s.data_ptr<float>(), ctx.data_ptr<float>(), ec, (int)peer_ptrs.size(),
                     reinterpret_cast<void*>(static_cast<intptr_t>(local_base)), peers, st);
    });
}

// dst[0 .. n) = 32-bit words: `uints` first, then the bit patterns of `floats` (the per-step scalar table; no host buffer is kept)
void write_table(Tensor dst, const std::vector<int64_t>& uints, const std::vector<double>& floats) {
    TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && dst.element_size() == 4 && dst.numel() >= (int64_t)(uints.size() + floats.size()),
                "table too small");
    c10::cuda::CUDAGuard guard(dst.device());
    std::vector<uint32_t> w(uints.size() + floats.size());
    for (size_t i = 0; i < uints.size(); ++i) w[i] = (uint32_t)uints[i];
    for (size_t i = 0; i < floats.size(); ++i) { const float f = (float)floats[i]; memcpy(&w[uints.size() + i], &f, 4); }
    sg::write_words(reinterpret_cast<uint32_t*>(dst.data_ptr()), w.data(), (int)w.size(), at::cuda::getCurrentCUDAStream());
}

// Adjoint of the scan: dctx [total,16] -> grads [2, NG] (see csrc/sg2_bilevel.cuh for the layout).  Must follow a forward scan on the
// same plan / workspace (it re-uses gs, vals and the chunk carry-in states of that forward).
void sg2_scan_backward(Tensor items, int64_t n_items, int64_t dir1_start, Tensor tds, int64_t n_td, Tensor snap_base, int64_t sorted_buf,
                       Tensor dctx, py::dict ws, Tensor snaps, Tensor partial, Tensor grads, int64_t snap_every) {
    c10::cuda::CUDAGuard guard(items.device());
    auto W = [&](const char* k) { return ws[k].cast<Tensor>(); };
    TORCH_CHECK(dctx.is_contiguous() && dctx.scalar_type() == at::kFloat, "dctx must be contiguous fp32");
    const uint32_t* vs = sorted_buf ? u32(W("vals1")) : u32(W("vals0"));
    sg::sg2_scan_backward(items.data_ptr(), (int)n_items, (int)dir1_start, tds.data_ptr(), (int)n_td, snap_base.data_ptr<int64_t>(),
                          W("gs").data_ptr<float>(), vs, dctx.data_ptr<float>(), W("carry").data_ptr<float>(), W("agg").data_ptr<float>(),
                          W("dcarry").data_ptr<float>(), snaps.data_ptr<float>(), partial.data_ptr<float>(), grads.data_ptr<float>(),
                          (int)snap_every, at::cuda::getCurrentCUDAStream());
}

void sg2_upload_weights(Tensor packed) {
    TORCH_CHECK(packed.is_cuda() && packed.scalar_type() == at::kFloat && packed.numel() == sg::SG2Pack::TOTAL && packed.is_contiguous(),
                "packed weights must be a contiguous fp32 CUDA vector of ", sg::SG2Pack::TOTAL, " floats");
    c10::cuda::CUDAGuard guard(packed.device());
    sg::sg2_upload_weights(packed.data_ptr<float>(), at::cuda::getCurrentCUDAStream());
}

// stand-alone stable segmented argsort of |x| (testing / bilevel): returns the index of the buffer holding the result
int64_t sg2_sort(Tensor keys0, Tensor keys1, Tensor vals0, Tensor vals1, Tensor hist, Tensor tot, Tensor seg_off, int64_t n_seg, int64_t total) {
    c10::cuda::CUDAGuard guard(keys0.device());
    int cur = 0;
    sg::sg2_segmented_sort(u32(keys0), u32(keys1), u32(vals0), u32(vals1), u32(hist), u32(tot), seg_off.data_ptr<int64_t>(), (int)n_seg, total,
                           &cur, at::cuda::getCurrentCUDAStream());
    return cur;
}

py::dict sg2_layout() {
    py::dict d;
    using P = sg::SG2Pack;
#define L(X) d[#X] = (int)P::X;
    L(IN_W) L(IN_B) L(DIR0) L(DIR1) L(D_INPROJ) L(D_DTW) L(D_DTB) L(D_BW) L(D_CW) L(D_ALOG) L(D_D) L(D_ROPE) L(D_OUT) L(DIR_SIZE)
    L(GRU_WZ) L(GRU_WR) L(GRU_WH) L(GRU_BZ) L(GRU_BR) L(GRU_BH) L(PQ) L(KA) L(KB) L(EW1) L(EB1) L(EW2) L(EB2) L(TOTAL) L(NET) L(A_X) L(A_Z) L(A_DT) L(A_B) L(A_C) L(AFF_SIZE) L(AFF0) L(AFF1)
#undef L
    d["item_bytes"] = (int)sg::sg2_item_bytes();
    d["td_bytes"] = (int)sg::sg2_td_bytes();
    d["sort_tile"] = 4096;
    return d;
}

// Device-side expert recycling: the parameters are modified in place, the counts are cleared; nothing is read back.
void sg2_recycle_b(at::Tensor counts, at::Tensor W1, at::Tensor b1, at::Tensor W2, at::Tensor b2, std::vector<at::Tensor> keys_a,
                   std::vector<at::Tensor> keys_b, double threshold, int64_t seed, int64_t call, at::Tensor info) {
    TORCH_CHECK(counts.is_cuda() && counts.scalar_type() == at::kInt && counts.numel() == sg::SG2_NE && counts.is_contiguous(), "counts: int32 [144]");
    auto chk = [](const at::Tensor& t, int64_t n, const char* what) {
        TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous() && t.numel() == n, what, ": contiguous fp32 CUDA tensor of ", n, " elements");
    };
    chk(W1, sg::SG2_NE * sg::SG2_EH, "W1"); chk(b1, sg::SG2_NE * sg::SG2_EH, "b1"); chk(W2, sg::SG2_NE * sg::SG2_EH, "W2"); chk(b2, sg::SG2_NE, "b2");
    TORCH_CHECK((int)keys_a.size() == sg::SG2_HEADS && (int)keys_b.size() == sg::SG2_HEADS, "four heads of sub-keys expected");
    float* ka[sg::SG2_HEADS]; float* kb[sg::SG2_HEADS];
    for (int h = 0; h < sg::SG2_HEADS; ++h) {
        chk(keys_a[h], sg::SG2_PK * 4, "keys_a"); chk(keys_b[h], sg::SG2_PK * 4, "keys_b");
        ka[h] = keys_a[h].data_ptr<float>(); kb[h] = keys_b[h].data_ptr<float>();
    }
    TORCH_CHECK(info.is_cuda() && info.scalar_type() == at::kInt && info.numel() >= 2, "info: int32 [2]");
    c10::cuda::CUDAGuard guard(counts.device());
    sg::sg2_recycle(counts.data_ptr<int>(), W1.data_ptr<float>(), b1.data_ptr<float>(), W2.data_ptr<float>(), b2.data_ptr<float>(), ka, kb,
                    (float)threshold, (uint32_t)seed, (uint32_t)call, info.data_ptr<int>(), at::cuda::getCurrentCUDAStream());
}

// ---- routed expert evaluation of the bilevel tail (csrc/sg2_experts.cu)
struct XShape { int64_t n; int heads, E, hidden; };
XShape routed_check(const Tensor& g, const Tensor& ia, const Tensor& ib, const Tensor& wa, const Tensor& wb, const Tensor& W1, const Tensor& b1,
                    const Tensor& W2, const Tensor& b2) {
    auto f32 = [](const Tensor& t, const char* nm) { TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kFloat, nm, ": contiguous fp32 CUDA tensor"); };
    auto i32 = [](const Tensor& t, const char* nm) { TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kInt, nm, ": contiguous int32 CUDA tensor"); };
    f32(g, "g"); f32(wa, "wa"); f32(wb, "wb"); f32(W1, "W1"); f32(b1, "b1"); f32(W2, "W2"); f32(b2, "b2"); i32(ia, "ia"); i32(ib, "ib");
    TORCH_CHECK(g.dim() == 1 && ia.dim() == 3 && ia.size(0) == g.size(0) && ia.size(2) == 4, "ia must be [n, heads, 4]");
    TORCH_CHECK(ib.sizes() == ia.sizes() && wa.sizes() == ia.sizes() && wb.sizes() == ia.sizes(), "ia, ib, wa, wb must have the same shape");
    TORCH_CHECK(W1.dim() == 2 && b1.sizes() == W1.sizes() && W2.sizes() == W1.sizes() && b2.dim() == 1 && b2.size(0) == W1.size(0), "expert tables: W1, b1, W2 [E, hidden], b2 [E]");
    XShape s{g.size(0), (int)ia.size(1), (int)W1.size(0), (int)W1.size(1)};
    TORCH_CHECK(sg::routed_experts_supported(s.heads, s.E, s.hidden, 4), "routed_experts: unsupported configuration (heads ", s.heads, ", experts ", s.E, ", hidden ", s.hidden, ")");
    return s;
}

Tensor routed_experts_fwd(const Tensor& g, const Tensor& ia, const Tensor& ib, const Tensor& wa, const Tensor& wb, const Tensor& W1, const Tensor& b1,
                          const Tensor& W2, const Tensor& b2, int64_t pk) {
    const XShape s = routed_check(g, ia, ib, wa, wb, W1, b1, W2, b2);
    c10::cuda::CUDAGuard guard(g.device());
    Tensor total = at::empty({s.n}, g.options());
    const int rc = sg::routed_experts_fwd(g.data_ptr<float>(), ia.data_ptr<int>(), ib.data_ptr<int>(), wa.data_ptr<float>(), wb.data_ptr<float>(),
                                          W1.data_ptr<float>(), b1.data_ptr<float>(), W2.data_ptr<float>(), b2.data_ptr<float>(), s.n, s.heads, s.E,
                                          (int)pk, total.data_ptr<float>(), at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(rc == 0, "routed_experts_fwd launch failed (code ", rc, ")");
    return total;
}

// returns (d wa, d wb, d [W1 | b1 | W2 | b2] flat)
std::vector<Tensor> routed_experts_bwd(const Tensor& g, const Tensor& ia, const Tensor& ib, const Tensor& wa, const Tensor& wb, const Tensor& W1,
                                       const Tensor& b1, const Tensor& W2, const Tensor& b2, int64_t pk, const Tensor& dtotal) {
    const XShape s = routed_check(g, ia, ib, wa, wb, W1, b1, W2, b2);
    TORCH_CHECK(dtotal.is_cuda() && dtotal.is_contiguous() && dtotal.scalar_type() == at::kFloat && dtotal.numel() == s.n, "dtotal: fp32 [n]");
    c10::cuda::CUDAGuard guard(g.device());
    const int64_t ng = 3 * (int64_t)s.E * s.hidden + s.E;
    Tensor dwa = at::empty_like(wa), dwb = at::empty_like(wb);
    Tensor partial = at::empty({(int64_t)sg::routed_experts_bwd_ctas(s.n, s.heads), ng}, g.options());
    Tensor dparams = at::empty({ng}, g.options());
    const int rc = sg::routed_experts_bwd(g.data_ptr<float>(), ia.data_ptr<int>(), ib.data_ptr<int>(), wa.data_ptr<float>(), wb.data_ptr<float>(),
                                          W1.data_ptr<float>(), b1.data_ptr<float>(), W2.data_ptr<float>(), b2.data_ptr<float>(),
                                          dtotal.data_ptr<float>(), s.n, s.heads, s.E, (int)pk, dwa.data_ptr<float>(), dwb.data_ptr<float>(),
                                          partial.data_ptr<float>(), dparams.data_ptr<float>(), at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(rc == 0, "routed_experts_bwd launch failed (code ", rc, ")");
    return {dwa, dwb, dparams};
}

// ---- product-key routing of the bilevel tail (csrc/sg2_routing.cu on CUDA; the same arithmetic, csrc/sg2_routing_math.h, in a loop on CPU)
struct RShape { int64_t n; int heads, P, pk; };
RShape routing_check(const Tensor& pin, const Tensor& Wq, const Tensor& KA, const Tensor& KB) {
    for (const Tensor* t : {&pin, &Wq, &KA, &KB})
        TORCH_CHECK(t->is_contiguous() && t->scalar_type() == at::kFloat && t->device() == pin.device(), "routing: contiguous fp32 tensors on one device");
    TORCH_CHECK(pin.dim() == 2 && Wq.dim() == 2 && Wq.size(1) == pin.size(1) && Wq.size(0) % sg::routing::RD == 0, "pin [n, P], Wq [heads * 8, P]");
    RShape s{pin.size(0), (int)(Wq.size(0) / sg::routing::RD), (int)pin.size(1), (int)KA.size(1)};
    TORCH_CHECK(KA.dim() == 3 && KA.size(0) == s.heads && KA.size(2) == sg::routing::RH && KB.sizes() == KA.sizes(), "KA, KB [heads, pk, 4]");
    TORCH_CHECK(sg::routing_supported(s.heads, s.P, s.pk, sg::routing::RD, sg::routing::RK), "routing: unsupported configuration");
    return s;
}

// returns (ia, ib int32 [n, heads, 4], wa, wb fp32 [n, heads, 4])
std::vector<Tensor> routing_fwd(const Tensor& pin, const Tensor& Wq, const Tensor& KA, const Tensor& KB) {
    const RShape s = routing_check(pin, Wq, KA, KB);
    auto io = pin.options().dtype(at::kInt);
    Tensor ia = at::empty({s.n, s.heads, 4}, io), ib = at::empty({s.n, s.heads, 4}, io);
    Tensor wa = at::empty({s.n, s.heads, 4}, pin.options()), wb = at::empty({s.n, s.heads, 4}, pin.options());
    if (pin.is_cuda()) {
        c10::cuda::CUDAGuard guard(pin.device());
        const int rc = sg::routing_fwd(pin.data_ptr<float>(), Wq.data_ptr<float>(), KA.data_ptr<float>(), KB.data_ptr<float>(), s.n, s.heads, s.P, s.pk,
                                       ia.data_ptr<int>(), ib.data_ptr<int>(), wa.data_ptr<float>(), wb.data_ptr<float>(), at::cuda::getCurrentCUDAStream());
        TORCH_CHECK(rc == 0, "routing_fwd launch failed (code ", rc, ")");
        return {ia, ib, wa, wb};
    }
    const float *x = pin.data_ptr<float>(), *wq = Wq.data_ptr<float>(), *ka = KA.data_ptr<float>(), *kb = KB.data_ptr<float>();
    for (int64_t e = 0; e < s.n; ++e)
        for (int h = 0; h < s.heads; ++h) {
            float q[sg::routing::RD];
            const int64_t r = (e * s.heads + h) * 4;
            sg::routing::route_fwd(x + e * s.P, s.P, wq + h * sg::routing::RD * s.P, ka + h * s.pk * 4, kb + h * s.pk * 4, s.pk, q,
                                   ia.data_ptr<int>() + r, ib.data_ptr<int>() + r, wa.data_ptr<float>() + r, wb.data_ptr<float>() + r);
        }
    return {ia, ib, wa, wb};
}

// returns (d pin [n, P], d [Wq | KA | KB] flat)
std::vector<Tensor> routing_bwd(const Tensor& pin, const Tensor& Wq, const Tensor& KA, const Tensor& KB, const Tensor& ia, const Tensor& ib,
                                const Tensor& wa, const Tensor& wb, const Tensor& dwa, const Tensor& dwb) {
    const RShape s = routing_check(pin, Wq, KA, KB);
    for (const Tensor* t : {&wa, &wb, &dwa, &dwb})
        TORCH_CHECK(t->is_contiguous() && t->scalar_type() == at::kFloat && t->numel() == s.n * s.heads * 4 && t->device() == pin.device(), "wa, wb, dwa, dwb: fp32 [n, heads, 4]");
    for (const Tensor* t : {&ia, &ib})
        TORCH_CHECK(t->is_contiguous() && t->scalar_type() == at::kInt && t->numel() == s.n * s.heads * 4 && t->device() == pin.device(), "ia, ib: int32 [n, heads, 4]");
    const int ng = sg::routing_ng(s.heads, s.P, s.pk);
    Tensor dpin = at::empty_like(pin), dparams = at::empty({ng}, pin.options());
    if (pin.is_cuda()) {
        c10::cuda::CUDAGuard guard(pin.device());
        Tensor partial = at::empty({(int64_t)sg::routing_bwd_ctas(s.n, s.heads), ng}, pin.options());
        const int rc = sg::routing_bwd(pin.data_ptr<float>(), Wq.data_ptr<float>(), KA.data_ptr<float>(), KB.data_ptr<float>(), ia.data_ptr<int>(),
                                       ib.data_ptr<int>(), wa.data_ptr<float>(), wb.data_ptr<float>(), dwa.data_ptr<float>(), dwb.data_ptr<float>(), s.n,
                                       s.heads, s.P, s.pk, dpin.data_ptr<float>(), partial.data_ptr<float>(), dparams.data_ptr<float>(),
                                       at::cuda::getCurrentCUDAStream());
        TORCH_CHECK(rc == 0, "routing_bwd launch failed (code ", rc, ")");
        return {dpin, dparams};
    }
    using namespace sg::routing;
    const float *x = pin.data_ptr<float>(), *wq = Wq.data_ptr<float>(), *ka = KA.data_ptr<float>(), *kb = KB.data_ptr<float>();
    const int n_wq = s.heads * RD * s.P, n_k = s.heads * s.pk * RH;
    std::vector<double> acc(ng, 0.0);
    float* dp = dpin.data_ptr<float>();
    for (int64_t e = 0; e < s.n; ++e) {
        for (int j = 0; j < s.P; ++j) dp[e * s.P + j] = 0.f;
        for (int h = 0; h < s.heads; ++h) {
            const int64_t r = (e * s.heads + h) * 4;
            float q[RD], dt[2 * RK], dq[RD];
            query(x + e * s.P, s.P, wq + h * RD * s.P, q);
            route_bwd(ia.data_ptr<int>() + r, ib.data_ptr<int>() + r, wa.data_ptr<float>() + r, wb.data_ptr<float>() + r, dwa.data_ptr<float>() + r,
                      dwb.data_ptr<float>() + r, ka + h * s.pk * RH, kb + h * s.pk * RH, dt, dq);
            for (int o = 0; o < RD; ++o)
                for (int j = 0; j < s.P; ++j) {
                    dp[e * s.P + j] += wq[(h * RD + o) * s.P + j] * dq[o];
                    acc[(h * RD + o) * s.P + j] += (double)dq[o] * x[e * s.P + j];
                }
            for (int k = 0; k < RK; ++k)
                for (int d = 0; d < RH; ++d) {
                    acc[n_wq + (h * s.pk + ia.data_ptr<int>()[r + k]) * RH + d] += (double)dt[k] * q[d];
                    acc[n_wq + n_k + (h * s.pk + ib.data_ptr<int>()[r + k]) * RH + d] += (double)dt[RK + k] * q[RH + d];
                }
        }
    }
    float* out = dparams.data_ptr<float>();
    for (int i = 0; i < ng; ++i) out[i] = (float)acc[i];
    return {dpin, dparams};
}

// ---- per-element GRU of the meta-net (csrc/sg2_gru.cu on CUDA; the same arithmetic, csrc/sg2_gru_math.h, in a loop on CPU)
int gru_check(const Tensor& x, const Tensor& h, const Tensor& W, const Tensor& b) {
    for (const Tensor* t : {&x, &h, &W, &b})
        TORCH_CHECK(t->is_contiguous() && t->scalar_type() == at::kFloat && t->device() == x.device(), "gru: contiguous fp32 tensors on one device");
    const int IN = (int)x.size(1);
    TORCH_CHECK(x.dim() == 2 && h.dim() == 2 && h.size(0) == x.size(0) && h.size(1) == sg::gru::GH, "x [n, IN], h [n, 4]");
    TORCH_CHECK(W.numel() == 3 * sg::gru::GH * (IN + sg::gru::GH) && b.numel() == 3 * sg::gru::GH, "W [3, 4, IN + 4], b [3, 4]");
    TORCH_CHECK(sg::gru_supported(IN, (int)h.size(1)), "gru: unsupported width");
    return IN;
}

Tensor gru_fwd(const Tensor& x, const Tensor& h, const Tensor& W, const Tensor& b) {
    const int IN = gru_check(x, h, W, b);
    const int64_t n = x.size(0);
    Tensor hn = at::empty_like(h);
    if (x.is_cuda()) {
        c10::cuda::CUDAGuard guard(x.device());
        const int rc = sg::gru_fwd(x.data_ptr<float>(), h.data_ptr<float>(), W.data_ptr<float>(), b.data_ptr<float>(), n, IN, hn.data_ptr<float>(),
                                   at::cuda::getCurrentCUDAStream());
        TORCH_CHECK(rc == 0, "gru_fwd launch failed (code ", rc, ")");
        return hn;
    }
    using namespace sg::gru;
    for (int64_t e = 0; e < n; ++e) {
        float z[GH], r[GH], c[GH];
        gru_gates(x.data_ptr<float>() + e * IN, h.data_ptr<float>() + e * GH, IN, W.data_ptr<float>(), b.data_ptr<float>(), z, r, c, hn.data_ptr<float>() + e * GH);
    }
    return hn;
}

// returns (d x [n, IN], d [W | b] flat)
std::vector<Tensor> gru_bwd(const Tensor& x, const Tensor& h, const Tensor& W, const Tensor& b, const Tensor& dhn) {
    const int IN = gru_check(x, h, W, b);
    const int64_t n = x.size(0);
    TORCH_CHECK(dhn.is_contiguous() && dhn.scalar_type() == at::kFloat && dhn.sizes() == h.sizes() && dhn.device() == x.device(), "dhn: fp32 [n, 4]");
    const int ng = sg::gru_ng(IN);
    Tensor dx = at::empty_like(x), dparams = at::empty({ng}, x.options());
    if (x.is_cuda()) {
        c10::cuda::CUDAGuard guard(x.device());
        Tensor partial = at::empty({(int64_t)sg::gru_bwd_ctas(n), ng}, x.options());
        const int rc = sg::gru_bwd(x.data_ptr<float>(), h.data_ptr<float>(), W.data_ptr<float>(), b.data_ptr<float>(), dhn.data_ptr<float>(), n, IN,
                                   dx.data_ptr<float>(), partial.data_ptr<float>(), dparams.data_ptr<float>(), at::cuda::getCurrentCUDAStream());
        TORCH_CHECK(rc == 0, "gru_bwd launch failed (code ", rc, ")");
        return {dx, dparams};
    }
    using namespace sg::gru;
    const int P = IN + GH, nw = 3 * GH * P;
    std::vector<double> acc(ng, 0.0);
    for (int64_t e = 0; e < n; ++e) {
        const float* xe = x.data_ptr<float>() + e * IN;
        const float* he = h.data_ptr<float>() + e * GH;
        float dpre[3 * GH], rh[GH];
        gru_adjoint(xe, he, IN, W.data_ptr<float>(), b.data_ptr<float>(), dhn.data_ptr<float>() + e * GH, dpre, rh, dx.data_ptr<float>() + e * IN);
        for (int gi = 0; gi < 3 * GH; ++gi) {
            for (int j = 0; j < P; ++j) {
                const float src = j < IN ? xe[j] : (gi >= 2 * GH ? rh[j - IN] : he[j - IN]);
                acc[gi * P + j] += (double)dpre[gi] * src;
            }
            acc[nw + gi] += dpre[gi];
        }
    }
    for (int i = 0; i < ng; ++i) dparams.data_ptr<float>()[i] = (float)acc[i];
    return {dx, dparams};
}
}  // namespace

void register_sg2(pybind11::module_& m) {
    m.def("sg2_gru_supported", [](int64_t IN, int64_t hidden) { return sg::gru_supported((int)IN, (int)hidden); });
    m.def("sg2_gru_fwd", &gru_fwd);
    m.def("sg2_gru_bwd", &gru_bwd);
    m.def("sg2_routing_supported", [](int64_t heads, int64_t P, int64_t pk, int64_t d_model, int64_t topk) {
        return sg::routing_supported((int)heads, (int)P, (int)pk, (int)d_model, (int)topk); });
    m.def("sg2_routing_fwd", &routing_fwd);
    m.def("sg2_routing_bwd", &routing_bwd);
    m.def("sg2_routed_experts_supported", [](int64_t heads, int64_t E, int64_t hidden, int64_t topk) {
        return sg::routed_experts_supported((int)heads, (int)E, (int)hidden, (int)topk); });
    m.def("sg2_routed_experts_fwd", &routed_experts_fwd);
    m.def("sg2_routed_experts_bwd", &routed_experts_bwd);
    m.def("sg2_prepare", &sg2_prepare, py::arg("grads"), py::arg("sharps"), py::arg("offsets"), py::arg("total"), py::arg("seg_off"),
          py::arg("clip"), py::arg("ws"), py::arg("pull_bases") = std::vector<int64_t>(), py::arg("pull_rank") = 0,
          py::arg("pull_scale") = 1.0, py::arg("stage") = 0);
    m.def("write_table", &write_table);
    m.attr("DYN_TS") = (int)sg::DYN_TS; m.attr("DYN_LR") = (int)sg::DYN_LR; m.attr("DYN_WD") = (int)sg::DYN_WD;
    m.attr("DYN_LAMB") = (int)sg::DYN_LAMB; m.attr("DYN_EPOCH") = (int)sg::DYN_EPOCH;
    m.def("sg2_scan", &sg2_scan, py::arg("items"), py::arg("n_items"), py::arg("dir1_start"), py::arg("tds"), py::arg("n_td"), py::arg("any_multi"),
          py::arg("sorted_buf"), py::arg("ws"), py::arg("status") = c10::optional<Tensor>());
    m.def("sg2_elem", &sg2_elem, py::arg("params"), py::arg("ms"), py::arg("vs"), py::arg("mus"), py::arg("grus"), py::arg("masters"),
          py::arg("dyn"), py::arg("packed"), py::arg("offsets"), py::arg("beta2"), py::arg("eps"), py::arg("rescale"),
          py::arg("expert_counts"), py::arg("ws"), py::arg("local_base") = 0, py::arg("peer_ptrs") = std::vector<int64_t>(),
          py::arg("status") = c10::optional<Tensor>());
    m.def("sg2_upload_weights", &sg2_upload_weights);
    m.def("sg2_sort", &sg2_sort);
    m.def("sg2_layout", &sg2_layout);
    m.def("sg2_scan_ctas_per_sm", []() { return sg::sg2_scan_ctas_per_sm(); });
    m.def("sg2_recycle", &sg2_recycle_b, py::arg("counts"), py::arg("W1"), py::arg("b1"), py::arg("W2"), py::arg("b2"), py::arg("keys_a"),
          py::arg("keys_b"), py::arg("threshold"), py::arg("seed"), py::arg("call"), py::arg("info"));
    m.def("sg2_scan_backward", &sg2_scan_backward, py::arg("items"), py::arg("n_items"), py::arg("dir1_start"), py::arg("tds"), py::arg("n_td"),
          py::arg("snap_base"), py::arg("sorted_buf"), py::arg("dctx"), py::arg("ws"), py::arg("snaps"), py::arg("partial"), py::arg("grads"),
          py::arg("snap_every") = 1);
    m.def("sg2_bilevel_info", []() { py::dict d; d["ng"] = sg::sg2_bilevel_ng(); d["tile"] = sg::sg2_bilevel_tile();
                                     d["smem"] = (int64_t)sg::sg2_bilevel_smem_bytes(); return d; });
    m.def("sg2_sort_blocks", [](int64_t total) { return (int64_t)sg::sg2_sort_blocks(total); });
}
}  // namespace sgb
