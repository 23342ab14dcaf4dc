// Routed expert evaluation of the SuperGrok v2 bilevel (soft top-k) path, forward and backward (sm_100a).
//
// After the product-key routing every head of an element holds 4 row keys (ia, weight wa) and 4 column keys (ib, wb); the 16
// experts e = ia*pk + ib are evaluated on the element's scalar gradient g with weight wa*wb:
//     total[n] = sum_h sum_a sum_b wa[n,h,a] * wb[n,h,b] * expert_e(g[n]),   expert_e(g) = b2[e] + sum_j relu(g*W1[e,j] + b1[e,j]) * W2[e,j]
// The PyTorch formulation of this step (reference grokking_optimizers/supergrok2.py:717-807 evaluates it per head with
// gathered expert weights; a dense variant evaluates all 144 experts for every element) materialises [n, 144, 16] tensors in
// the forward and the backward pass; here nothing but the routing tables crosses HBM.
//
// Backward: d wa / d wb per element, and the expert-parameter gradients summed over all elements WITHOUT atomics: a tile of
// elements first scatters dtotal*wa*wb into a dense [elements, experts] table in shared memory (head after head, so the
// order of additions is fixed), then every thread owns up to nine fixed (expert, hidden unit) pairs - their weights in
// registers - and walks the tile's elements; per-CTA sums go to a partial buffer that a second kernel adds in CTA order.
#include "sg_native.h"

namespace sg {
namespace {

constexpr int XH = 16;            // expert hidden width
constexpr int XK = 4;             // keys kept per sub-key (top-4 x top-4 = 16 experts per head)
constexpr int XTHREADS = 256;
constexpr int XMAXQ = 9;          // (expert, hidden) pairs per thread in the backward pass: experts <= 16 * XMAXQ = 144
constexpr int XPAD = XH + 1;      // shared-memory row pitch of the expert tables (different experts fall into different banks)

struct XParams {                  // shared-memory copy of the expert tables
    float* w1; float* b1; float* w2; float* b2;
};

__device__ __forceinline__ XParams load_params(float* sm, const float* __restrict__ W1, const float* __restrict__ b1,
                                               const float* __restrict__ W2, const float* __restrict__ b2, int E) {
    XParams p{sm, sm + E * XPAD, sm + 2 * E * XPAD, sm + 3 * E * XPAD};
    for (int i = threadIdx.x; i < E * XH; i += XTHREADS) {
        const int e = i / XH, j = i % XH;
        p.w1[e * XPAD + j] = W1[i];
        p.b1[e * XPAD + j] = b1[i];
        p.w2[e * XPAD + j] = W2[i];
    }
    for (int i = threadIdx.x; i < E; i += XTHREADS) p.b2[i] = b2[i];
    return p;
}

__device__ __forceinline__ float expert_eval(const XParams& p, int e, float g) {
    float o = p.b2[e];
    const float* w1 = p.w1 + e * XPAD; const float* bb = p.b1 + e * XPAD; const float* w2 = p.w2 + e * XPAD;
#pragma unroll
    for (int j = 0; j < XH; ++j) o = fmaf(fmaxf(fmaf(g, w1[j], bb[j]), 0.f), w2[j], o);
    return o;
}

// one thread per (element, head); the heads of an element are added in head order by the thread of head 0
__global__ void __launch_bounds__(XTHREADS) routed_experts_fwd_kernel(const float* __restrict__ g, const int4* __restrict__ ia,
                                                                      const int4* __restrict__ ib, const float4* __restrict__ wa,
                                                                      const float4* __restrict__ wb, const float* __restrict__ W1,
                                                                      const float* __restrict__ b1, const float* __restrict__ W2,
                                                                      const float* __restrict__ b2, int64_t n, int heads, int E, int pk,
                                                                      float* __restrict__ total) {
    extern __shared__ float sm[];
    const XParams p = load_params(sm, W1, b1, W2, b2, E);
    float* s_tot = sm + 3 * E * XPAD + E;
    __syncthreads();
    const int epc = XTHREADS / heads;                                   // elements per CTA
    const int le = threadIdx.x / heads, h = threadIdx.x % heads;
    const int64_t elem = (int64_t)blockIdx.x * epc + le;
    float t = 0.f;
    if (le < epc && elem < n) {
        const float gv = g[elem];
        const int64_t r = elem * heads + h;
        const int4 a4 = ia[r], b4 = ib[r];
        const float4 wa4 = wa[r], wb4 = wb[r];
        const int av[XK] = {a4.x, a4.y, a4.z, a4.w}, bv[XK] = {b4.x, b4.y, b4.z, b4.w};
        const float wav[XK] = {wa4.x, wa4.y, wa4.z, wa4.w}, wbv[XK] = {wb4.x, wb4.y, wb4.z, wb4.w};
#pragma unroll
        for (int a = 0; a < XK; ++a)
#pragma unroll
            for (int b = 0; b < XK; ++b) {
                int e = av[a] * pk + bv[b];
                e = e < 0 ? 0 : (e >= E ? E - 1 : e);
                t = fmaf(wav[a] * wbv[b], expert_eval(p, e, gv), t);
            }
    }
    s_tot[threadIdx.x] = t;
    __syncthreads();
    if (h == 0 && le < epc && elem < n) {
        float s = 0.f;
        for (int k = 0; k < heads; ++k) s += s_tot[threadIdx.x + k];
        total[elem] = s;
    }
}

// Persistent CTAs over tiles of XTHREADS / heads elements.  partial: [gridDim.x, 3*E*XH + E] (dW1, db1, dW2, db2).
__global__ void __launch_bounds__(XTHREADS) routed_experts_bwd_kernel(const float* __restrict__ g, const int4* __restrict__ ia,
                                                                      const int4* __restrict__ ib, const float4* __restrict__ wa,
                                                                      const float4* __restrict__ wb, const float* __restrict__ W1,
                                                                      const float* __restrict__ b1, const float* __restrict__ W2,
                                                                      const float* __restrict__ b2, const float* __restrict__ dtotal,
                                                                      int64_t n, int heads, int E, int pk, float4* __restrict__ dwa,
                                                                      float4* __restrict__ dwb, float* __restrict__ partial) {
    extern __shared__ float sm[];
    const XParams p = load_params(sm, W1, b1, W2, b2, E);
    const int epc = XTHREADS / heads;
    float* s_g = sm + 3 * E * XPAD + E;                                 // [epc]
    float* s_route = s_g + XTHREADS;                                    // [epc][E]
    __syncthreads();
    const int le = threadIdx.x / heads, h = threadIdx.x % heads;
    // the (expert, hidden unit) pairs of this thread: hidden unit j is fixed, experts e0 + 16 q
    const int j = threadIdx.x & (XH - 1), e0 = threadIdx.x / XH;
    float w1r[XMAXQ], b1r[XMAXQ], w2r[XMAXQ], aw1[XMAXQ], ab1[XMAXQ], aw2[XMAXQ], ab2[XMAXQ];
#pragma unroll
    for (int q = 0; q < XMAXQ; ++q) {
        const int e = e0 + (XTHREADS / XH) * q;
        const bool in = e < E;
        w1r[q] = in ? p.w1[e * XPAD + j] : 0.f;
        b1r[q] = in ? p.b1[e * XPAD + j] : 0.f;
        w2r[q] = in ? p.w2[e * XPAD + j] : 0.f;
        aw1[q] = ab1[q] = aw2[q] = ab2[q] = 0.f;
    }
    const int64_t tiles = (n + epc - 1) / epc;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t elem = tile * epc + le;
        const bool live = le < epc && elem < n;
        int ev[XK * XK];
        float cv[XK * XK];
        float dt = 0.f;
        if (live) {
            const float gv = g[elem];
            dt = dtotal[elem];
            const int64_t r = elem * heads + h;
            const int4 a4 = ia[r], b4 = ib[r];
            const float4 wa4 = wa[r], wb4 = wb[r];
            const int av[XK] = {a4.x, a4.y, a4.z, a4.w}, bv[XK] = {b4.x, b4.y, b4.z, b4.w};
            const float wav[XK] = {wa4.x, wa4.y, wa4.z, wa4.w}, wbv[XK] = {wb4.x, wb4.y, wb4.z, wb4.w};
            float da[XK] = {0.f, 0.f, 0.f, 0.f}, db[XK] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int a = 0; a < XK; ++a)
#pragma unroll
                for (int b = 0; b < XK; ++b) {
                    int e = av[a] * pk + bv[b];
                    e = e < 0 ? 0 : (e >= E ? E - 1 : e);
                    const float dw = dt * expert_eval(p, e, gv);       // d total / d (wa*wb) times the incoming gradient
                    da[a] = fmaf(dw, wbv[b], da[a]);
                    db[b] = fmaf(dw, wav[a], db[b]);
                    ev[a * XK + b] = e;
                    cv[a * XK + b] = dt * wav[a] * wbv[b];
                }
            dwa[r] = make_float4(da[0], da[1], da[2], da[3]);
            dwb[r] = make_float4(db[0], db[1], db[2], db[3]);
            if (h == 0) s_g[le] = gv;
        } else if (h == 0 && le < epc) {
            s_g[le] = 0.f;
        }
        for (int i = threadIdx.x; i < epc * E; i += XTHREADS) s_route[i] = 0.f;
        __syncthreads();
        // head after head: within one head the 16 experts of an element are distinct when its keys are (top-k indices are);
        // repeated keys would still be added by one thread, in a fixed order
        for (int hh = 0; hh < heads; ++hh) {
            if (live && h == hh) {
#pragma unroll
                for (int k = 0; k < XK * XK; ++k) s_route[le * E + ev[k]] += cv[k];
            }
            __syncthreads();
        }
        const int64_t left = n - tile * epc;
        const int cnt = left < epc ? (int)left : epc;
        for (int m = 0; m < cnt; ++m) {
            const float gm = s_g[m];
            const float* rt = s_route + m * E;
#pragma unroll
            for (int q = 0; q < XMAXQ; ++q) {
                const int e = e0 + (XTHREADS / XH) * q;
                if (e < E) {
                    const float c = rt[e];
                    if (c != 0.f) {
                        const float z = fmaf(gm, w1r[q], b1r[q]);
                        const float on = z > 0.f ? 1.f : 0.f;
                        aw2[q] = fmaf(c, z * on, aw2[q]);
                        const float dz = c * w2r[q] * on;
                        aw1[q] = fmaf(dz, gm, aw1[q]);
                        ab1[q] += dz;
                        ab2[q] += c;
                    }
                }
            }
        }
        __syncthreads();                                               // the tables are rewritten by the next tile
    }
    float* out = partial + (int64_t)blockIdx.x * (3 * E * XH + E);
#pragma unroll
    for (int q = 0; q < XMAXQ; ++q) {
        const int e = e0 + (XTHREADS / XH) * q;
        if (e < E) {
            out[e * XH + j] = aw1[q];
            out[E * XH + e * XH + j] = ab1[q];
            out[2 * E * XH + e * XH + j] = aw2[q];
            if (j == 0) out[3 * E * XH + e] = ab2[q];
        }
    }
}

__global__ void __launch_bounds__(256) routed_experts_reduce_kernel(const float* __restrict__ partial, int parts, int ng, float* __restrict__ out) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= ng) return;
    float t = 0.f;
    for (int p = 0; p < parts; ++p) t += partial[(int64_t)p * ng + i];
    out[i] = t;
}

size_t fwd_smem(int E) { return (size_t)(3 * E * XPAD + E + XTHREADS) * sizeof(float); }
size_t bwd_smem(int E, int heads) { return (size_t)(3 * E * XPAD + E + XTHREADS + (XTHREADS / heads) * E) * sizeof(float); }

}  // namespace

bool routed_experts_supported(int heads, int E, int hidden, int topk) {
    return hidden == XH && topk == XK && heads >= 1 && heads <= 16 && E >= 1 && E <= (XTHREADS / XH) * XMAXQ && bwd_smem(E, heads) <= 200 * 1024;
}

// CTAs of the backward pass = rows of `partial` ([ctas, 3*E*16 + E] floats)
int routed_experts_bwd_ctas(int64_t n, int heads) {
    const int epc = XTHREADS / heads;
    const int64_t tiles = (n + epc - 1) / epc;
    const int64_t cap = 2 * 148;
    return (int)(tiles < cap ? (tiles < 1 ? 1 : tiles) : cap);
}

int routed_experts_fwd(const float* g, const int* ia, const int* ib, const float* wa, const float* wb, const float* W1, const float* b1,
                       const float* W2, const float* b2, int64_t n, int heads, int E, int pk, float* total, cudaStream_t s) {
    if (n <= 0) return 0;
    const size_t smem = fwd_smem(E);
    if (cudaFuncSetAttribute(routed_experts_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
    const int epc = XTHREADS / heads;
    count_launch();
    routed_experts_fwd_kernel<<<(unsigned)((n + epc - 1) / epc), XTHREADS, smem, s>>>(
        g, (const int4*)ia, (const int4*)ib, (const float4*)wa, (const float4*)wb, W1, b1, W2, b2, n, heads, E, pk, total);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int routed_experts_bwd(const float* g, const int* ia, const int* ib, const float* wa, const float* wb, const float* W1, const float* b1,
                       const float* W2, const float* b2, const float* dtotal, int64_t n, int heads, int E, int pk, float* dwa, float* dwb,
                       float* partial, float* dparams, cudaStream_t s) {
    const int ng = 3 * E * XH + E;
    if (n <= 0) return cudaMemsetAsync(dparams, 0, (size_t)ng * sizeof(float), s) == cudaSuccess ? 0 : 3;
    const size_t smem = bwd_smem(E, heads);
    if (cudaFuncSetAttribute(routed_experts_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
    const int ctas = routed_experts_bwd_ctas(n, heads);
    count_launch(2);
    routed_experts_bwd_kernel<<<ctas, XTHREADS, smem, s>>>(g, (const int4*)ia, (const int4*)ib, (const float4*)wa, (const float4*)wb, W1, b1, W2, b2,
                                                          dtotal, n, heads, E, pk, (float4*)dwa, (float4*)dwb, partial);
    routed_experts_reduce_kernel<<<(ng + 255) / 256, 256, 0, s>>>(partial, ctas, ng, dparams);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace sg
