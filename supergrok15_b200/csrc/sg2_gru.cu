// The meta-net's per-element GRU as kernels (sm_100a): forward, and the adjoint used by the bilevel path.  Arithmetic:
// csrc/sg2_gru_math.h.  One thread per element; in the adjoint a CTA keeps its 256 elements' inputs, gated states and
// pre-activation gradients in shared memory, every thread owns up to two fixed weight / bias outputs and walks the elements in
// order, sums stay in registers across tiles, one partial row per CTA, a second kernel adds the rows in CTA order (no atomics).
#include "sg_native.h"
#include "sg2_gru_math.h"

namespace sg {
namespace {
using namespace gru;

constexpr int GT = 256;
constexpr int GMAXO = 2;                               // outputs per thread: 3 * GH * (IN + GH + 1) <= 512

__device__ __forceinline__ void stage(float* sm, const float* __restrict__ W, const float* __restrict__ b, int IN) {
    const int nw = 3 * GH * (IN + GH);
    for (int i = threadIdx.x; i < nw; i += GT) sm[i] = W[i];
    for (int i = threadIdx.x; i < 3 * GH; i += GT) sm[nw + i] = b[i];
}

// CIN > 0: the input width is a compile-time constant (loops unroll, the per-element arrays stay in registers); 0: run-time width
template <int CIN>
__global__ void __launch_bounds__(GT) gru_fwd_kernel(const float* __restrict__ x, const float* __restrict__ h, const float* __restrict__ W,
                                                     const float* __restrict__ b, int64_t n, int IN_rt, float* __restrict__ hn) {
    const int IN = CIN > 0 ? CIN : IN_rt;
    extern __shared__ float sm[];
    stage(sm, W, b, IN);
    __syncthreads();
    const int64_t e = (int64_t)blockIdx.x * GT + threadIdx.x;
    if (e >= n) return;
    float xv[CIN > 0 ? CIN : GIN_MAX], hv[GH], z[GH], r[GH], c[GH], o[GH];
#pragma unroll
    for (int j = 0; j < IN; ++j) xv[j] = x[e * IN + j];
    const float4 h4 = *reinterpret_cast<const float4*>(h + e * GH);
    hv[0] = h4.x; hv[1] = h4.y; hv[2] = h4.z; hv[3] = h4.w;
    gru_gates(xv, hv, IN, sm, sm + 3 * GH * (IN + GH), z, r, c, o);
    *reinterpret_cast<float4*>(hn + e * GH) = make_float4(o[0], o[1], o[2], o[3]);
}

// partial: [gridDim.x, 3*GH*(IN+GH) + 3*GH]   (d W | d b)
template <int CIN>
__global__ void __launch_bounds__(GT) gru_bwd_kernel(const float* __restrict__ x, const float* __restrict__ h, const float* __restrict__ W,
                                                     const float* __restrict__ b, const float* __restrict__ dhn, int64_t n, int IN_rt,
                                                     float* __restrict__ dx, float* __restrict__ partial) {
    const int IN = CIN > 0 ? CIN : IN_rt;
    extern __shared__ float sm[];
    const int P = IN + GH, nw = 3 * GH * P, ng = nw + 3 * GH;
    const int pitch = IN + 2 * GH + 3 * GH + 1;                  // x | h | r*h | dpre, odd pitch
    float* s_el = sm + ng;                                        // [GT][pitch]
    stage(sm, W, b, IN);
    float acc[GMAXO];
#pragma unroll
    for (int u = 0; u < GMAXO; ++u) acc[u] = 0.f;
    __syncthreads();
    const int64_t tiles = (n + GT - 1) / GT;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t e = tile * GT + threadIdx.x;
        const int64_t left = n - tile * GT;
        const int cnt = left < GT ? (int)left : GT;
        if (e < n) {
            float xv[CIN > 0 ? CIN : GIN_MAX], hv[GH], dh[GH], dpre[3 * GH], rh[GH], dxv[CIN > 0 ? CIN : GIN_MAX];
#pragma unroll
            for (int j = 0; j < IN; ++j) xv[j] = x[e * IN + j];
            const float4 h4 = *reinterpret_cast<const float4*>(h + e * GH), d4 = *reinterpret_cast<const float4*>(dhn + e * GH);
            hv[0] = h4.x; hv[1] = h4.y; hv[2] = h4.z; hv[3] = h4.w;
            dh[0] = d4.x; dh[1] = d4.y; dh[2] = d4.z; dh[3] = d4.w;
            gru_adjoint(xv, hv, IN, sm, sm + nw, dh, dpre, rh, dxv);
#pragma unroll
            for (int j = 0; j < IN; ++j) dx[e * IN + j] = dxv[j];
            float* row = s_el + threadIdx.x * pitch;
#pragma unroll
            for (int j = 0; j < IN; ++j) row[j] = xv[j];
#pragma unroll
            for (int j = 0; j < GH; ++j) { row[IN + j] = hv[j]; row[IN + GH + j] = rh[j]; }
#pragma unroll
            for (int j = 0; j < 3 * GH; ++j) row[IN + 2 * GH + j] = dpre[j];
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < GMAXO; ++u) {
            const int id = threadIdx.x + u * GT;
            if (id < ng) {
                float a = acc[u];
                if (id < nw) {
                    const int gi = id / P, j = id % P;            // gi = gate * GH + hidden unit
                    // the candidate's input is [x, r*h]; the z and r gates read [x, h]
                    const int src = (gi >= 2 * GH && j >= IN) ? j + GH : j;
                    for (int m = 0; m < cnt; ++m) a = fmaf(s_el[m * pitch + IN + 2 * GH + gi], s_el[m * pitch + src], a);
                } else {
                    const int gi = id - nw;
                    for (int m = 0; m < cnt; ++m) a += s_el[m * pitch + IN + 2 * GH + gi];
                }
                acc[u] = a;
            }
        }
        __syncthreads();
    }
    float* out = partial + (int64_t)blockIdx.x * ng;
#pragma unroll
    for (int u = 0; u < GMAXO; ++u) { const int id = threadIdx.x + u * GT; if (id < ng) out[id] = acc[u]; }
}

__global__ void __launch_bounds__(256) gru_reduce_kernel(const float* __restrict__ partial, int parts, int ng, float* __restrict__ out) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= ng) return;
    float t = 0.f;
    for (int p = 0; p < parts; ++p) t += partial[(int64_t)p * ng + i];
    out[i] = t;
}
}  // namespace

int gru_ng(int IN) { return 3 * gru::GH * (IN + gru::GH) + 3 * gru::GH; }
bool gru_supported(int IN, int hidden) { return hidden == gru::GH && IN >= 1 && IN <= gru::GIN_MAX && gru_ng(IN) <= GMAXO * GT; }
int gru_bwd_ctas(int64_t n) {
    const int64_t tiles = (n + GT - 1) / GT;
    return (int)(tiles < 1 ? 1 : (tiles < 4 * 148 ? tiles : 4 * 148));
}

int gru_fwd(const float* x, const float* h, const float* W, const float* b, int64_t n, int IN, float* hn, cudaStream_t s) {
    if (n <= 0) return 0;
    count_launch();
    const unsigned grid = (unsigned)((n + GT - 1) / GT);
    const size_t smem = (size_t)gru_ng(IN) * sizeof(float);
    if (IN == 18) gru_fwd_kernel<18><<<grid, GT, smem, s>>>(x, h, W, b, n, IN, hn);          // 2 + 2 * d_model of the default meta-net
    else gru_fwd_kernel<0><<<grid, GT, smem, s>>>(x, h, W, b, n, IN, hn);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int gru_bwd(const float* x, const float* h, const float* W, const float* b, const float* dhn, int64_t n, int IN, float* dx, float* partial,
            float* dparams, cudaStream_t s) {
    const int ng = gru_ng(IN);
    if (n <= 0) return cudaMemsetAsync(dparams, 0, (size_t)ng * sizeof(float), s) == cudaSuccess ? 0 : 3;
    const size_t smem = (size_t)(ng + GT * (IN + 5 * gru::GH + 1)) * sizeof(float);
    // the adjoint keeps the run-time width: fully unrolled for 18 inputs it needs 255 registers and spills (-Xptxas -v)
    if (cudaFuncSetAttribute(gru_bwd_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
    const int ctas = gru_bwd_ctas(n);
    count_launch(2);
    gru_bwd_kernel<0><<<ctas, GT, smem, s>>>(x, h, W, b, dhn, n, IN, dx, partial);
    gru_reduce_kernel<<<(ng + 255) / 256, 256, 0, s>>>(partial, ctas, ng, dparams);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace sg
