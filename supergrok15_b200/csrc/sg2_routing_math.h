// Product-key routing of the SuperGrok v2 bilevel (soft top-k) path, per (element, head): the arithmetic shared by the CUDA
// kernels (csrc/sg2_routing.cu) and their C++ CPU counterpart (csrc/cpu_kernels.cpp), which is what the CPU tests check.
//
//   q = Wq_h . pin                      (8 x P)                     P = gru_hidden + 2 * d_model + 2 = 22 by default
//   sA[r] = <KA_h[r], q[0:4]>,  sB[r] = <KB_h[r], q[4:8]>           r < pk
//   (tA, ia) = top-4 of sA,  wa = softmax(10 * tA);  same for B     (reference mamba3_peer_metanet.py:372-435)
// Backward, given d wa and d wb:  d t = 10 * w * (d w - <w, d w>),  d q[0:4] = sum_k d tA[k] * KA_h[ia[k]],  d KA_h[ia[k]] += d tA[k] * q[0:4],
// d pin += Wq_h^T d q,  d Wq_h += d q (x) pin.  The selection itself carries no gradient.
#pragma once
#include <math.h>

#ifdef __CUDACC__
#define SG_HD __host__ __device__ __forceinline__
#else
#define SG_HD inline
#endif

namespace sg {
namespace routing {

constexpr int RK = 4;            // keys kept per sub-key
constexpr int RH = 4;            // half of the query width (one sub-key)
constexpr int RD = 2 * RH;       // query width (the meta-net's d_model)
constexpr int RPK_MAX = 16;      // rows of a sub-key table
constexpr int RP_MAX = 32;       // width of the routing input

// q[o] = sum_j Wq_h[o * P + j] * pin[j]
SG_HD void query(const float* pin, int P, const float* Wq_h, float* q) {
    for (int o = 0; o < RD; ++o) {
        float a = 0.f;
        for (int j = 0; j < P; ++j) a = fmaf(Wq_h[o * P + j], pin[j], a);
        q[o] = a;
    }
}

// top-4 rows of keys [pk][4] by score against qh [4] (ties and NaN: the lower index wins), softmax(10 * score) over them
SG_HD void top4_softmax(const float* qh, const float* keys, int pk, int* idx, float* w) {
    float sc[RPK_MAX];
    for (int r = 0; r < pk; ++r) sc[r] = fmaf(keys[r * RH + 3], qh[3], fmaf(keys[r * RH + 2], qh[2], fmaf(keys[r * RH + 1], qh[1], keys[r * RH] * qh[0])));
    unsigned used = 0u;
    float top[RK];
    for (int k = 0; k < RK; ++k) {
        int bi = -1;
        float best = 0.f;
        for (int r = 0; r < pk; ++r)
            if (!((used >> r) & 1u) && (bi < 0 || sc[r] > best)) { best = sc[r]; bi = r; }
        if (bi < 0) bi = 0;                                   // pk < 4: repeat row 0
        used |= 1u << bi;
        idx[k] = bi;
        top[k] = best;
    }
    float e[RK], s = 0.f;
    for (int k = 0; k < RK; ++k) { e[k] = expf(10.f * (top[k] - top[0])); s += e[k]; }
    for (int k = 0; k < RK; ++k) w[k] = e[k] / s;
}

SG_HD void route_fwd(const float* pin, int P, const float* Wq_h, const float* KA_h, const float* KB_h, int pk, float* q, int* ia, int* ib,
                     float* wa, float* wb) {
    query(pin, P, Wq_h, q);
    top4_softmax(q, KA_h, pk, ia, wa);
    top4_softmax(q + RH, KB_h, pk, ib, wb);
}

// dt[0:4] / dt[4:8]: gradients of the selected A / B scores; dq [8]
SG_HD void route_bwd(const int* ia, const int* ib, const float* wa, const float* wb, const float* dwa, const float* dwb, const float* KA_h,
                     const float* KB_h, float* dt, float* dq) {
    float da = 0.f, db = 0.f;
    for (int k = 0; k < RK; ++k) { da = fmaf(wa[k], dwa[k], da); db = fmaf(wb[k], dwb[k], db); }
    for (int k = 0; k < RK; ++k) { dt[k] = 10.f * wa[k] * (dwa[k] - da); dt[RK + k] = 10.f * wb[k] * (dwb[k] - db); }
    for (int d = 0; d < RH; ++d) {
        float a = 0.f, b = 0.f;
        for (int k = 0; k < RK; ++k) { a = fmaf(dt[k], KA_h[ia[k] * RH + d], a); b = fmaf(dt[RK + k], KB_h[ib[k] * RH + d], b); }
        dq[d] = a;
        dq[RH + d] = b;
    }
}

}  // namespace routing
}  // namespace sg
