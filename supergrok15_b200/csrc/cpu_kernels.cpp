// C++ CPU counterparts of the multi-tensor optimizer kernels (fp32 tensors), op for op and formula for formula the same as
// csrc/mt_kernels.cu: they are the native CPU path of the element-wise optimizers (the reference ships CPU fallbacks of its
// kernels in csrc/ops.cpp) and a second, independent oracle for the CUDA kernels.  Work is split into the same 8,192-element
// chunks as on the GPU; chunks run under at::parallel_for and every reduction adds its chunk partials in index order, so the
// result does not depend on the number of threads.
#include <ATen/Parallel.h>
#include <torch/extension.h>
#include <cmath>
#include <vector>
#include "sg_native.h"

namespace sgb {
namespace {
using at::Tensor;

inline float adam_update(float p, float fg, float& m, float& v, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2) {
    m = b1 * m + (1.f - b1) * fg;
    v = b2 * v + (1.f - b2) * fg * fg;
    const float denom = std::sqrt(v / bc2) + eps;
    return p * (1.f - lr * wd) - (lr / bc1) * m / denom;
}
inline float lion_update(float p, float g, float& m, float lr, float b1, float b2, float wd) {
    const float c = b1 * m + (1.f - b1) * g;
    const float s = (c > 0.f) ? 1.f : ((c < 0.f) ? -1.f : 0.f);
    m = b2 * m + (1.f - b2) * g;
    return p - lr * (s + wd * p);
}
// ---- the sharpness MLP over a block of elements -------------------------------------------------------------------------------
// Per element the MLP costs `hidden` exponentials; element by element through std::exp that is most of a CPU step of SuperGrok
// v1.5 / v1.1.  Here the hidden units are the outer loop and a block of elements the inner one, with a polynomial exponential
// (Cody-Waite reduction, degree-5 polynomial, relative error below 2e-7), so the inner loop is plain arithmetic that the compiler
// vectorises (measured on a 2.7 GHz Xeon, 422,755 elements x 32 hidden units, one thread: 112 ms element by element, 14.5 ms
// in blocks with AVX2); an AVX2 clone is chosen at load time where the CPU has it (same arithmetic, same results).  Each element
// still adds its hidden units in index order.  The clamp must compile to min / max instructions: written as comparisons the
// loop stayed scalar.
constexpr int MLP_BLOCK = 64;

__attribute__((always_inline)) inline float poly_expf(float x) {
    x = __builtin_fminf(__builtin_fmaxf(x, -87.f), 88.f);               // min / max instructions under the flags of sharp_mlp_block
    const float t = x * 1.44269504088896341f;
    const int k = (int)(t + __builtin_copysignf(0.5f, t));             // round to nearest, as a conversion the vectoriser knows
    const float kf = (float)k;
    const float r = (x - kf * 0.693359375f) - kf * -2.12194440e-4f;
    float p = 1.9875691500e-4f;
    p = p * r + 1.3981999507e-3f;
    p = p * r + 8.3334519073e-3f;
    p = p * r + 4.1665795894e-2f;
    p = p * r + 1.6666665459e-1f;
    p = p * r + 5.0000001201e-1f;
    const float y = p * r * r + r + 1.f;
    union { int32_t i; float f; } s;
    s.i = (k + 127) << 23;
    return y * s.f;
}

__attribute__((target_clones("avx2", "default"), optimize("O3", "no-trapping-math", "no-math-errno", "finite-math-only")))
void sharp_mlp_block(const float* __restrict__ g, const float* __restrict__ s, int nb, const float* __restrict__ W1, const float* __restrict__ b1,
                     const float* __restrict__ W2, float b2, int H, float* __restrict__ out) {
    for (int b = 0; b < nb; ++b) out[b] = b2;
    for (int h = 0; h < H; ++h) {
        const float w0 = W1[2 * h], w1 = W1[2 * h + 1], bb = b1[h], w2 = W2[h];
        for (int b = 0; b < nb; ++b) {
            const float z = w0 * g[b] + (w1 * s[b] + bb);
            out[b] += w2 * (z / (1.f + poly_expf(-1.702f * z)));
        }
    }
}

// the NeuralGrok amplifier (1 -> hidden -> 1, ReLU) over a block of elements, same scheme
__attribute__((target_clones("avx2", "default"), optimize("O3", "no-trapping-math", "no-math-errno", "finite-math-only")))
void amp_mlp_block(const float* __restrict__ g, int nb, const float* __restrict__ W1, const float* __restrict__ b1, const float* __restrict__ W2,
                   float b2, int H, float* __restrict__ out) {
    for (int b = 0; b < nb; ++b) out[b] = b2;
    for (int h = 0; h < H; ++h) {
        const float w1 = W1[h], bb = b1[h], w2 = W2[h];
        for (int b = 0; b < nb; ++b) out[b] += w2 * __builtin_fmaxf(w1 * g[b] + bb, 0.f);
    }
}

const float* fp(const c10::optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr<float>() : nullptr; }

struct Prm {
    float lr, beta1, beta2, eps, wd, alpha, lamb, rescale, extra0, extra1;
    const float *clip, *dscal, *tscal, *W1, *b1, *W2, *b2;
    int hidden, write_grad;
};

// one chunk [lo, hi) of tensor t; returns up to three partial sums
void run_chunk(int op, float* const P[6], const float ts[4], const Prm& q, int t_global, int64_t lo, int64_t hi, float acc[3]) {
    using namespace sg;
    float *P0 = P[0], *P1 = P[1], *P2 = P[2], *P3 = P[3], *P4 = P[4], *P5 = P[5];
    const float clip = q.clip ? q.clip[0] : 1.f;
    const float lr = q.lr, b1 = q.beta1, b2 = q.beta2, eps = q.eps, wd = q.wd;
    const int H = q.hidden;
    const float b2s = q.b2 ? q.b2[0] : 0.f;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f;
    if (op == OP_SG15 || op == OP_SG11_A) {                           // the two ops with the sharpness MLP: block by block
        const float* S = op == OP_SG15 ? P5 : P3;
        float gb[MLP_BLOCK], out[MLP_BLOCK];
        for (int64_t i0 = lo; i0 < hi; i0 += MLP_BLOCK) {
            const int nb = (int)(hi - i0 < MLP_BLOCK ? hi - i0 : MLP_BLOCK);
            for (int b = 0; b < nb; ++b) gb[b] = P1[i0 + b] * clip;
            sharp_mlp_block(gb, S + i0, nb, q.W1, q.b1, q.W2, b2s, H, out);
            for (int b = 0; b < nb; ++b) {
                const int64_t i = i0 + b;
                const float g = gb[b];
                if (op == OP_SG15) {
                    P4[i] = ts[0] * P4[i] + (1.f - ts[0]) * g;
                    const float sgd = g + q.rescale * out[b];
                    P0[i] = adam_update(P0[i], sgd + q.lamb * P4[i], P2[i], P3[i], lr, ts[1], b2, eps, wd, ts[2], ts[3]);
                } else {
                    P2[i] = ts[0] * P2[i] + (1.f - ts[0]) * g;
                    const float sm = g + q.rescale * out[b];
                    P4[i] = sm;
                    a0 = std::fma(sm, P2[i], a0); a1 = std::fma(sm, sm, a1); a2 = std::fma(P2[i], P2[i], a2);
                }
                if (q.write_grad) P1[i] = g;
            }
        }
        acc[0] = a0; acc[1] = a1; acc[2] = a2;
        return;
    }
    if (op == OP_NEURALGROK) {
        float gb[MLP_BLOCK], out[MLP_BLOCK];
        for (int64_t i0 = lo; i0 < hi; i0 += MLP_BLOCK) {
            const int nb = (int)(hi - i0 < MLP_BLOCK ? hi - i0 : MLP_BLOCK);
            for (int b = 0; b < nb; ++b) gb[b] = P1[i0 + b] * clip;
            amp_mlp_block(gb, nb, q.W1, q.b1, q.W2, b2s, H, out);
            for (int b = 0; b < nb; ++b) {
                const int64_t i = i0 + b;
                const float ag = gb[b] * (q.alpha * out[b] + q.rescale);
                P0[i] = adam_update(P0[i], ag, P2[i], P3[i], lr, b1, b2, eps, wd, ts[0], ts[1]);
                if (q.write_grad) P1[i] = gb[b];
            }
        }
        acc[0] = acc[1] = acc[2] = 0.f;
        return;
    }
    for (int64_t i = lo; i < hi; ++i) {
        switch (op) {
            case OP_ADAMW: P0[i] = adam_update(P0[i], P1[i] * clip, P2[i], P3[i], lr, b1, b2, eps, wd, ts[0], ts[1]); break;
            case OP_LION: P0[i] = lion_update(P0[i], P1[i] * clip, P2[i], lr, b1, b2, wd); break;
            case OP_GROKFAST_EMA: P2[i] = q.alpha * P2[i] + (1.f - q.alpha) * P1[i]; P1[i] += q.lamb * P2[i]; break;
            case OP_GROKFAST_ADAMW: case OP_GROKADAMW: {
                const float gg = P1[i] * clip;
                P4[i] = q.alpha * P4[i] + (1.f - q.alpha) * gg;
                const float am = gg + q.lamb * P4[i];
                P0[i] = adam_update(P0[i], am, P2[i], P3[i], lr, b1, b2, eps, wd, ts[0], ts[1]);
                if (q.write_grad) P1[i] = (op == OP_GROKFAST_ADAMW) ? am : gg;
                break;
            }
            case OP_PRODIGY: {
                const float d = q.dscal[0], dg = d * P1[i];
                P4[i] = b2 * P4[i] + (1.f - b2) * dg * dg;
                P2[i] = b1 * P2[i] + (1.f - b1) * dg;
                P3[i] = b2 * P3[i] + (1.f - b2) * dg * dg;
                P0[i] = P0[i] * (1.f - lr * d * wd) - (lr / ts[0]) * P2[i] / (std::sqrt(P3[i] / ts[1]) + d * eps);
                break;
            }
            case OP_SG11_B: P0[i] = adam_update(P0[i], P1[i] + q.tscal[t_global] * P4[i], P2[i], P3[i], lr, ts[0], b2, eps, wd, ts[1], ts[2]); break;
            case OP_PERTURB: P2[i] = P0[i]; P0[i] = std::fma(q.dscal[0], P1[i], P0[i]); break;
            case OP_RESTORE: P0[i] = P2[i]; break;
            case OP_SHARP_RESTORE: P4[i] = std::fabs(P3[i] - P1[i]); P0[i] = P2[i]; break;
            case OP_LOOKSAM_DIR: { const float inv = q.tscal[2 * t_global]; if (inv > 0.f) P2[i] = (P3[i] - P1[i]) * inv; break; }
            case OP_LOOKSAM_ADJ: P1[i] = std::fma(q.alpha * q.tscal[2 * t_global + 1], P2[i], P1[i]); break;
            case OP_MUON_MOMENTUM: P2[i] = std::fma(q.alpha, P2[i], P1[i]); a0 = std::fma(P2[i], P2[i], a0); break;
            case OP_MUON_UPDATE: P0[i] = std::fma(q.extra0, P1[i], P0[i]) * q.extra1; break;
            case OP_SCALE: P1[i] *= (q.dscal ? q.dscal[0] : q.extra0); break;
            case OP_SQNORM: a0 = std::fma(P1[i], P1[i], a0); break;
            case OP_PRODIGY_REDUCE: a0 = std::fma(P1[i], P0[i] - P2[i], a0); a1 += P3[i]; break;
            case OP_DIFF_SQNORM: { const float d = P2[i] - P1[i]; a0 = std::fma(d, d, a0); a1 = std::fma(P1[i], P1[i], a1); break; }
            default: break;
        }
    }
    acc[0] = a0; acc[1] = a1; acc[2] = a2;
}
}  // namespace

// Same contract as mt_apply for CUDA tensors; every tensor must be a contiguous fp32 CPU tensor.
void cpu_mt_apply(int op, const std::vector<std::vector<Tensor>>& roles, const std::vector<std::vector<double>>& ts, const std::vector<double>& f,
                  c10::optional<Tensor> clip, c10::optional<Tensor> dscal, c10::optional<Tensor> tscal, c10::optional<Tensor> W1,
                  c10::optional<Tensor> b1, c10::optional<Tensor> W2, c10::optional<Tensor> b2, int64_t hidden, bool write_grad,
                  c10::optional<Tensor> per_tensor_out) {
    size_t n = 0;
    for (const auto& r : roles) if (!r.empty()) { n = r.size(); break; }
    if (n == 0) return;
    auto F = [&](size_t i) { return i < f.size() ? (float)f[i] : 0.f; };
    Prm q{F(0), F(1), F(2), F(3), F(4), F(5), F(6), F(7), F(8), F(9), fp(clip), fp(dscal), fp(tscal), fp(W1), fp(b1), fp(W2), fp(b2),
          (int)hidden, write_grad ? 1 : 0};
    float* out = per_tensor_out.has_value() ? per_tensor_out->data_ptr<float>() : nullptr;
    for (size_t t = 0; t < n; ++t) {
        float* P[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
        int64_t numel = -1;
        bool skip = false;
        for (size_t r = 0; r < roles.size() && r < 6; ++r) {
            if (roles[r].empty()) continue;
            TORCH_CHECK(roles[r].size() == n, "role ", r, " has ", roles[r].size(), " tensors, expected ", n);
            const Tensor& x = roles[r][t];
            if (!x.defined()) { skip = true; break; }
            TORCH_CHECK(x.device().is_cpu() && x.scalar_type() == at::kFloat && x.is_contiguous(), "CPU kernels take contiguous fp32 tensors");
            if (numel < 0) numel = x.numel();
            TORCH_CHECK(x.numel() == numel, "role ", r, " tensor ", t, " size mismatch");
            P[r] = x.data_ptr<float>();
        }
        float tsv[4] = {0.f, 0.f, 0.f, 0.f};
        if (t < ts.size()) for (size_t k = 0; k < ts[t].size() && k < 4; ++k) tsv[k] = (float)ts[t][k];
        float tot[3] = {0.f, 0.f, 0.f};
        if (!skip && numel > 0) {
            const int64_t chunks = (numel + sg::MT_CHUNK - 1) / sg::MT_CHUNK;
            std::vector<float> part(3 * (size_t)chunks);
            at::parallel_for(0, chunks, 1, [&](int64_t c0, int64_t c1) {
                for (int64_t c = c0; c < c1; ++c) {
                    const int64_t lo = c * sg::MT_CHUNK, hi = std::min<int64_t>(numel, lo + sg::MT_CHUNK);
                    run_chunk(op, P, tsv, q, (int)t, lo, hi, &part[3 * (size_t)c]);
                }
            });
            for (int64_t c = 0; c < chunks; ++c) { tot[0] += part[3 * c]; tot[1] += part[3 * c + 1]; tot[2] += part[3 * c + 2]; }
        }
        if (out) { out[3 * t] = tot[0]; out[3 * t + 1] = tot[1]; out[3 * t + 2] = tot[2]; }
    }
}

void cpu_scalar_finalize(int op, const Tensor& per_tensor, int64_t n, Tensor out_t, double a0d, double a1d, double a2d) {
    using namespace sg;
    const float* pt = per_tensor.data_ptr<float>();
    float* out = out_t.data_ptr<float>();
    const float a0 = (float)a0d, a1 = (float)a1d, a2 = (float)a2d;
    if (op == SC_CLIP || op == SC_SAM_SCALE || op == SC_PRODIGY || op == SC_SUM3) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f;
        for (int64_t t = 0; t < n; ++t) { s0 += pt[3 * t]; s1 += pt[3 * t + 1]; s2 += pt[3 * t + 2]; }
        if (op == SC_SUM3) { out[0] = s0; out[1] = s1; out[2] = s2; }
        else if (op == SC_CLIP) { const float norm = std::sqrt(s0); out[0] = s0; out[1] = (norm > a0) ? a0 / (norm + 1e-6f) : 1.f; out[2] = norm; }
        else if (op == SC_SAM_SCALE) out[0] = a0 / (std::sqrt(s0) + 1e-12f);
        else { float d = out[0]; if (s1 > 1e-30f) d = std::fmax(d, std::fabs(s0) / (s1 + 1e-12f)); out[0] = d; }
        return;
    }
    for (int64_t t = 0; t < n; ++t) {
        if (op == SC_SG11_GATES) {
            const float cosv = pt[3 * t] / (std::sqrt(pt[3 * t + 1]) * std::sqrt(pt[3 * t + 2]) + 1e-8f);
            const float gate = 1.f / (1.f + std::exp(-a0 * cosv));
            out[t] = (a1 > 0.f) ? a1 * gate * a2 : 0.f;
            out[n + t] = gate;
        } else if (op == SC_LOOKSAM_NORMS) {
            const float dn = std::sqrt(pt[3 * t]);
            out[2 * t] = (dn < 1e-12f) ? 0.f : 1.f / dn;
            out[2 * t + 1] = std::sqrt(pt[3 * t + 1]);
        } else if (op == SC_MUON_NORMS) {
            out[t] = 1.f / (std::sqrt(pt[3 * t]) + 1e-7f);
        } else if (op == SC_SG2_CLIP) {
            const float norm = std::sqrt(pt[3 * t]);
            out[t] = (norm > a0) ? a0 / (norm + 1e-12f) : 1.f;
        }
    }
}

}  // namespace sgb
