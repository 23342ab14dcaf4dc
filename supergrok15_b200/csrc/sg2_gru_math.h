// The per-element GRU of the SuperGrok v2 meta-net (reference mamba3_peer_metanet.py:163-192), forward and adjoint, per element:
// the arithmetic shared by the CUDA kernels (csrc/sg2_gru.cu) and their C++ CPU loop (csrc/bindings_sg2.cpp).
//
//   xh = [x, h]            z = sigmoid(Wz xh + bz)        r = sigmoid(Wr xh + br)
//   xr = [x, r * h]        c = tanh(Wh xr + bh)           h' = (1 - z) * h + z * c
// W: [3][HID][IN + HID] (z, r, candidate), b: [3][HID].  The adjoint takes d h' and returns d x and the three pre-activation
// gradients (the parameter gradients are their outer products with xh, xh and xr); the previous state h is data here.
#pragma once
#include <math.h>

#ifdef __CUDACC__
#define SG_HD __host__ __device__ __forceinline__
#else
#define SG_HD inline
#endif

namespace sg {
namespace gru {

constexpr int GH = 4;             // hidden width
constexpr int GIN_MAX = 28;       // inputs (2 + 2 * d_model = 18 by default)

SG_HD float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }

// z, r, c [GH] and the new state hn [GH]
SG_HD void gru_gates(const float* x, const float* h, int IN, const float* W, const float* b, float* z, float* r, float* c, float* hn) {
    const int P = IN + GH;
    for (int i = 0; i < GH; ++i) {
        float az = b[i], ar = b[GH + i];
        for (int j = 0; j < IN; ++j) { az = fmaf(W[i * P + j], x[j], az); ar = fmaf(W[(GH + i) * P + j], x[j], ar); }
        for (int j = 0; j < GH; ++j) { az = fmaf(W[i * P + IN + j], h[j], az); ar = fmaf(W[(GH + i) * P + IN + j], h[j], ar); }
        z[i] = sigmoidf_(az);
        r[i] = sigmoidf_(ar);
    }
    for (int i = 0; i < GH; ++i) {
        float ac = b[2 * GH + i];
        for (int j = 0; j < IN; ++j) ac = fmaf(W[(2 * GH + i) * P + j], x[j], ac);
        for (int j = 0; j < GH; ++j) ac = fmaf(W[(2 * GH + i) * P + IN + j], r[j] * h[j], ac);
        c[i] = tanhf(ac);
        hn[i] = (1.f - z[i]) * h[i] + z[i] * c[i];
    }
}

// dpre [3][GH]: gradients of the z, r and candidate pre-activations; rh [GH] = r * h; dx [IN]
SG_HD void gru_adjoint(const float* x, const float* h, int IN, const float* W, const float* b, const float* dhn, float* dpre, float* rh, float* dx) {
    const int P = IN + GH;
    float z[GH], r[GH], c[GH], hn[GH];
    gru_gates(x, h, IN, W, b, z, r, c, hn);
    float drh[GH];
    for (int j = 0; j < GH; ++j) { rh[j] = r[j] * h[j]; drh[j] = 0.f; }
    for (int j = 0; j < IN; ++j) dx[j] = 0.f;
    for (int i = 0; i < GH; ++i) {
        dpre[i] = dhn[i] * (c[i] - h[i]) * z[i] * (1.f - z[i]);                     // through z
        dpre[2 * GH + i] = dhn[i] * z[i] * (1.f - c[i] * c[i]);                       // through the candidate
    }
    for (int i = 0; i < GH; ++i) {
        const float dc = dpre[2 * GH + i];
        for (int j = 0; j < IN; ++j) dx[j] = fmaf(W[(2 * GH + i) * P + j], dc, dx[j]);
        for (int j = 0; j < GH; ++j) drh[j] = fmaf(W[(2 * GH + i) * P + IN + j], dc, drh[j]);
    }
    for (int i = 0; i < GH; ++i) dpre[GH + i] = drh[i] * h[i] * r[i] * (1.f - r[i]);  // through r
    for (int i = 0; i < GH; ++i) {
        const float dz = dpre[i], dr = dpre[GH + i];
        for (int j = 0; j < IN; ++j) dx[j] = fmaf(W[i * P + j], dz, fmaf(W[(GH + i) * P + j], dr, dx[j]));
    }
}

}  // namespace gru
}  // namespace sg
