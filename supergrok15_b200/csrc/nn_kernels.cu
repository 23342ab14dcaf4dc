// Model-side kernels for the small-sequence transformers of the grokking tasks (sm_100a):
//   * causal multi-head attention for very short sequences (S <= 8) - one warp per (batch, head), the whole
//     S x S score matrix lives in registers; forward and backward (scores recomputed, nothing saved but q,k,v);
//   * LayerNorm with fused residual add, forward and backward (deterministic two-stage column reduction for
//     the weight / bias gradients, no atomics).
// They replace nn.MultiheadAttention / nn.LayerNorm of the reference model (grokking_race_v2.py:310-331); library
// flash-attention kernels are tuned for long sequences and take ~2.5 ms per layer on a [8192, 8, 4, 64] problem
// whose memory traffic is worth ~20 us.
#include "sg_native.h"
#include "optim_math.cuh"

namespace sg {
namespace {

template <typename T, int EPL> struct LaneVec;       // EPL consecutive head-dim elements owned by one lane
template <> struct LaneVec<__nv_bfloat16, 2> {
    static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float (&v)[2]) {
        const __nv_bfloat162 t = *reinterpret_cast<const __nv_bfloat162*>(p);
        v[0] = __bfloat162float(t.x); v[1] = __bfloat162float(t.y);
    }
    static __device__ __forceinline__ void st(__nv_bfloat16* p, const float (&v)[2]) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
    }
};
template <> struct LaneVec<__nv_bfloat16, 1> {
    static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float (&v)[1]) { v[0] = __bfloat162float(*p); }
    static __device__ __forceinline__ void st(__nv_bfloat16* p, const float (&v)[1]) { *p = __float2bfloat16_rn(v[0]); }
};
template <> struct LaneVec<float, 2> {
    static __device__ __forceinline__ void ld(const float* p, float (&v)[2]) { const float2 t = *reinterpret_cast<const float2*>(p); v[0] = t.x; v[1] = t.y; }
    static __device__ __forceinline__ void st(float* p, const float (&v)[2]) { *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]); }
};
template <> struct LaneVec<float, 1> {
    static __device__ __forceinline__ void ld(const float* p, float (&v)[1]) { v[0] = *p; }
    static __device__ __forceinline__ void st(float* p, const float (&v)[1]) { *p = v[0]; }
};

// qkv [B, S, 3, H, HD] (HD = 32*EPL), out [B, S, H, HD]; one warp per (b, h); causal; scale = 1/sqrt(HD)
template <typename T, int S, int EPL, bool CAUSAL>
__global__ void __launch_bounds__(256) attn_small_fwd_kernel(const T* __restrict__ qkv, T* __restrict__ out, int B, int H, float scale) {
    const int lane = threadIdx.x & 31;
    const int64_t w = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (w >= (int64_t)B * H) return;
    const int b = (int)(w / H), h = (int)(w % H);
    constexpr int HD = 32 * EPL;
    const int64_t D = (int64_t)H * HD;
    float q[S][EPL], k[S][EPL], v[S][EPL];
#pragma unroll
    for (int s = 0; s < S; ++s) {
        const T* base = qkv + ((int64_t)(b * S + s) * 3) * D + (int64_t)h * HD + lane * EPL;
        LaneVec<T, EPL>::ld(base, q[s]); LaneVec<T, EPL>::ld(base + D, k[s]); LaneVec<T, EPL>::ld(base + 2 * D, v[s]);
    }
    float sc[S][S];
#pragma unroll
    for (int i = 0; i < S; ++i)
#pragma unroll
        for (int j = 0; j < S; ++j) {
            if (CAUSAL && j > i) { sc[i][j] = 0.f; continue; }
            float d = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) d = fmaf(q[i][e], k[j][e], d);
            sc[i][j] = warp_sum(d) * scale;
        }
#pragma unroll
    for (int i = 0; i < S; ++i) {
        const int jm = CAUSAL ? i : S - 1;
        float mx = sc[i][0];
#pragma unroll
        for (int j = 1; j < S; ++j) if (j <= jm) mx = fmaxf(mx, sc[i][j]);
        float den = 0.f;
#pragma unroll
        for (int j = 0; j < S; ++j) if (j <= jm) { sc[i][j] = __expf(sc[i][j] - mx); den += sc[i][j]; }
        const float inv = 1.f / den;
        float o[EPL];
#pragma unroll
        for (int e = 0; e < EPL; ++e) o[e] = 0.f;
#pragma unroll
        for (int j = 0; j < S; ++j) if (j <= jm) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) o[e] = fmaf(sc[i][j] * inv, v[j][e], o[e]);
        }
        LaneVec<T, EPL>::st(out + (int64_t)(b * S + i) * D + (int64_t)h * HD + lane * EPL, o);
    }
}

template <typename T, int S, int EPL, bool CAUSAL>
__global__ void __launch_bounds__(256) attn_small_bwd_kernel(const T* __restrict__ qkv, const T* __restrict__ dout, T* __restrict__ dqkv,
                                                             int B, int H, float scale) {
    const int lane = threadIdx.x & 31;
    const int64_t w = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (w >= (int64_t)B * H) return;
    const int b = (int)(w / H), h = (int)(w % H);
    constexpr int HD = 32 * EPL;
    const int64_t D = (int64_t)H * HD;
    float q[S][EPL], k[S][EPL], v[S][EPL], dO[S][EPL];
#pragma unroll
    for (int s = 0; s < S; ++s) {
        const T* base = qkv + ((int64_t)(b * S + s) * 3) * D + (int64_t)h * HD + lane * EPL;
        LaneVec<T, EPL>::ld(base, q[s]); LaneVec<T, EPL>::ld(base + D, k[s]); LaneVec<T, EPL>::ld(base + 2 * D, v[s]);
        LaneVec<T, EPL>::ld(dout + (int64_t)(b * S + s) * D + (int64_t)h * HD + lane * EPL, dO[s]);
    }
    float p[S][S], dp[S][S];
#pragma unroll
    for (int i = 0; i < S; ++i)
#pragma unroll
        for (int j = 0; j < S; ++j) {
            if (CAUSAL && j > i) { p[i][j] = 0.f; dp[i][j] = 0.f; continue; }
            float d = 0.f, e2 = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) { d = fmaf(q[i][e], k[j][e], d); e2 = fmaf(dO[i][e], v[j][e], e2); }
            p[i][j] = warp_sum(d) * scale;
            dp[i][j] = warp_sum(e2);
        }
    float dq[S][EPL], dk[S][EPL], dv[S][EPL];
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int e = 0; e < EPL; ++e) { dq[s][e] = 0.f; dk[s][e] = 0.f; dv[s][e] = 0.f; }
#pragma unroll
    for (int i = 0; i < S; ++i) {
        const int jm = CAUSAL ? i : S - 1;
        float mx = p[i][0];
#pragma unroll
        for (int j = 1; j < S; ++j) if (j <= jm) mx = fmaxf(mx, p[i][j]);
        float den = 0.f;
#pragma unroll
        for (int j = 0; j < S; ++j) if (j <= jm) { p[i][j] = __expf(p[i][j] - mx); den += p[i][j]; }
        const float inv = 1.f / den;
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < S; ++j) if (j <= jm) { p[i][j] *= inv; dot = fmaf(p[i][j], dp[i][j], dot); }
#pragma unroll
        for (int j = 0; j < S; ++j) if (j <= jm) {
            const float ds = p[i][j] * (dp[i][j] - dot) * scale;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                dv[j][e] = fmaf(p[i][j], dO[i][e], dv[j][e]);
                dq[i][e] = fmaf(ds, k[j][e], dq[i][e]);
                dk[j][e] = fmaf(ds, q[i][e], dk[j][e]);
            }
        }
    }
#pragma unroll
    for (int s = 0; s < S; ++s) {
        T* base = dqkv + ((int64_t)(b * S + s) * 3) * D + (int64_t)h * HD + lane * EPL;
        LaneVec<T, EPL>::st(base, dq[s]); LaneVec<T, EPL>::st(base + D, dk[s]); LaneVec<T, EPL>::st(base + 2 * D, dv[s]);
    }
}

// ---------------------------------------------------------------------------------------------------- LayerNorm
// z = x (+ r); y = (z - mean) * rstd * gamma (+ beta).  One warp per row; rows of D <= 8192 elements.
// RMS = true is RMSNorm: the mean is taken as zero (y = z * rsqrt(mean(z^2) + eps) * gamma) and there is no beta.
template <typename T, bool RMS>
__global__ void __launch_bounds__(256) ln_fwd_kernel(const T* __restrict__ x, const T* __restrict__ r, const T* __restrict__ gamma,
                                                     const T* __restrict__ beta, T* __restrict__ z, T* __restrict__ y,
                                                     float* __restrict__ stats, int64_t rows, int D, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const T* xr = x + row * D;
    const T* rr = r ? r + row * D : nullptr;
    float s = 0.f, ss = 0.f;
    for (int c = lane * 4; c < D; c += 128) {
        float a[4], bres[4];
        ld4<T>(xr, c, (D - c >= 4) ? 4 : D - c, true, a);
        if (rr) { ld4<T>(rr, c, (D - c >= 4) ? 4 : D - c, true, bres);
#pragma unroll
            for (int k = 0; k < 4; ++k) a[k] = Cvt<T>::to(Cvt<T>::from(a[k] + bres[k])); }
#pragma unroll
        for (int k = 0; k < 4; ++k) { s += a[k]; ss = fmaf(a[k], a[k], ss); }
    }
    s = warp_sum(s); ss = warp_sum(ss);
    const float mean = RMS ? 0.f : s / D;
    const float var = fmaxf(ss / D - mean * mean, 0.f);
    const float rstd = rsqrtf(var + eps);
    if (lane == 0) { stats[2 * row] = mean; stats[2 * row + 1] = rstd; }
    for (int c = lane * 4; c < D; c += 128) {
        const int cnt = (D - c >= 4) ? 4 : D - c;
        float a[4], bres[4], g[4], bb[4], o[4];
        ld4<T>(xr, c, cnt, true, a);
        if (rr) { ld4<T>(rr, c, cnt, true, bres);
#pragma unroll
            for (int k = 0; k < 4; ++k) a[k] = Cvt<T>::to(Cvt<T>::from(a[k] + bres[k]));
            st4<T>(z + row * D, c, cnt, true, a); }
        ld4<T>(gamma, c, cnt, true, g);
        if (beta) ld4<T>(beta, c, cnt, true, bb);
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = (a[k] - mean) * rstd * g[k] + (beta ? bb[k] : 0.f);
        st4<T>(y + row * D, c, cnt, true, o);
    }
}

// dz = rstd * (dy*g - mean_c(dy*g) - xhat * mean_c(dy*g*xhat)); per-CTA partial sums of dgamma / dbeta over its rows.
constexpr int LN_ROWS_PER_CTA = 64;
template <typename T, bool RMS>
__global__ void __launch_bounds__(256) ln_bwd_kernel(const T* __restrict__ z, const T* __restrict__ dy, const T* __restrict__ gamma,
                                                     const float* __restrict__ stats, const T* __restrict__ dz_in, T* __restrict__ dz,
                                                     float* __restrict__ part, int64_t rows, int D) {
    extern __shared__ float sm[];                       // [8 warps][2][D]  per-warp column partials
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    float* pg = sm + (size_t)w * 2 * D;
    float* pb = pg + D;
    for (int c = lane; c < D; c += 32) { pg[c] = 0.f; pb[c] = 0.f; }
    const int64_t row0 = (int64_t)blockIdx.x * LN_ROWS_PER_CTA;
    for (int rr = w; rr < LN_ROWS_PER_CTA; rr += 8) {
        const int64_t row = row0 + rr;
        if (row >= rows) break;
        const float mean = stats[2 * row], rstd = stats[2 * row + 1];
        float s1 = 0.f, s2 = 0.f;
        for (int c = lane * 4; c < D; c += 128) {
            const int cnt = (D - c >= 4) ? 4 : D - c;
            float a[4], d[4], g[4];
            ld4<T>(z + row * D, c, cnt, true, a); ld4<T>(dy + row * D, c, cnt, true, d); ld4<T>(gamma, c, cnt, true, g);
#pragma unroll
            for (int k = 0; k < 4; ++k) if (k < cnt) {
                const float xh = (a[k] - mean) * rstd, dg = d[k] * g[k];
                s1 += dg; s2 = fmaf(dg, xh, s2);
                pg[c + k] = fmaf(d[k], xh, pg[c + k]); pb[c + k] += d[k];
            }
        }
        s1 = RMS ? 0.f : warp_sum(s1) / D; s2 = warp_sum(s2) / D;
        for (int c = lane * 4; c < D; c += 128) {
            const int cnt = (D - c >= 4) ? 4 : D - c;
            float a[4], d[4], g[4], o[4];
            ld4<T>(z + row * D, c, cnt, true, a); ld4<T>(dy + row * D, c, cnt, true, d); ld4<T>(gamma, c, cnt, true, g);
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float xh = (a[k] - mean) * rstd; o[k] = rstd * (d[k] * g[k] - s1 - xh * s2); }
            if (dz_in) {                                 // gradient that reached z directly (z is also the residual stream)
                float e[4];
                ld4<T>(dz_in + row * D, c, cnt, true, e);
#pragma unroll
                for (int k = 0; k < 4; ++k) o[k] += e[k];
            }
            st4<T>(dz + row * D, c, cnt, true, o);
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < D; c += 256) {
        float a = 0.f, b = 0.f;
#pragma unroll
        for (int ww = 0; ww < 8; ++ww) { a += sm[(size_t)ww * 2 * D + c]; b += sm[(size_t)ww * 2 * D + D + c]; }
        part[((int64_t)blockIdx.x * 2) * D + c] = a;
        part[((int64_t)blockIdx.x * 2 + 1) * D + c] = b;
    }
}


// ---------------------------------------------------------------------------------------------------- wide rows
// Variants for rows of exactly 32 * VEC * NCH elements (VEC = 16 bytes of T per lane, NCH in {1,2,4,8}): every access is 16 bytes
// per lane, the forward keeps the row in registers between the statistics and the output pass, and the backward keeps each
// lane's slice of the weight (and bias) gradient in registers over all the rows a warp visits - no shared-memory read-modify-
// write per element - before one fixed-order reduction over the eight warps.
template <typename T> struct RowVec {
    static constexpr int VEC = 16 / sizeof(T);
    static __device__ __forceinline__ void ld(const T* p, float (&v)[VEC]) {
        const uint4 t = *reinterpret_cast<const uint4*>(p);
        const T* h = reinterpret_cast<const T*>(&t);
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[k] = Cvt<T>::to(h[k]);
    }
    static __device__ __forceinline__ void st(T* p, const float (&v)[VEC]) {
        uint4 t;
        T* h = reinterpret_cast<T*>(&t);
#pragma unroll
        for (int k = 0; k < VEC; ++k) h[k] = Cvt<T>::from(v[k]);
        *reinterpret_cast<uint4*>(p) = t;
    }
};

template <typename T, bool RMS, int NCH>
__global__ void __launch_bounds__(256) norm_fwd_wide_kernel(const T* __restrict__ x, const T* __restrict__ r, const T* __restrict__ gamma,
                                                            const T* __restrict__ beta, T* __restrict__ z, T* __restrict__ y,
                                                            float* __restrict__ stats, int64_t rows, float eps) {
    constexpr int VEC = RowVec<T>::VEC, D = 32 * VEC * NCH;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    float a[NCH][VEC];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int col = (c * 32 + lane) * VEC;
        RowVec<T>::ld(x + row * D + col, a[c]);
        if (r) {
            float b[VEC];
            RowVec<T>::ld(r + row * D + col, b);
#pragma unroll
            for (int k = 0; k < VEC; ++k) a[c][k] = Cvt<T>::to(Cvt<T>::from(a[c][k] + b[k]));
            RowVec<T>::st(z + row * D + col, a[c]);
        }
#pragma unroll
        for (int k = 0; k < VEC; ++k) { s += a[c][k]; ss = fmaf(a[c][k], a[c][k], ss); }
    }
    s = warp_sum(s); ss = warp_sum(ss);
    const float mean = RMS ? 0.f : s / D;
    const float rstd = rsqrtf(fmaxf(ss / D - mean * mean, 0.f) + eps);
    if (lane == 0) { stats[2 * row] = mean; stats[2 * row + 1] = rstd; }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int col = (c * 32 + lane) * VEC;
        float g[VEC], bb[VEC], o[VEC];
        RowVec<T>::ld(gamma + col, g);
        if (beta) RowVec<T>::ld(beta + col, bb);
#pragma unroll
        for (int k = 0; k < VEC; ++k) o[k] = (a[c][k] - mean) * rstd * g[k] + (beta ? bb[k] : 0.f);
        RowVec<T>::st(y + row * D + col, o);
    }
}

template <typename T, bool RMS, int NCH>
__global__ void __launch_bounds__(256) norm_bwd_wide_kernel(const T* __restrict__ z, const T* __restrict__ dy, const T* __restrict__ gamma,
                                                            const float* __restrict__ stats, const T* __restrict__ dz_in, T* __restrict__ dz,
                                                            float* __restrict__ part, int64_t rows) {
    constexpr int VEC = RowVec<T>::VEC, D = 32 * VEC * NCH;
    extern __shared__ float sm[];                       // [8 warps][D]
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    float ag[NCH][VEC], ab[RMS ? 1 : NCH][VEC];        // gamma is re-read per row (4 KB, stays in L1): registers go to the accumulators
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int k = 0; k < VEC; ++k) { ag[c][k] = 0.f; if (!RMS) ab[c][k] = 0.f; }
    for (int64_t row = (int64_t)blockIdx.x * 8 + w; row < rows; row += (int64_t)gridDim.x * 8) {
        const float mean = stats[2 * row], rstd = stats[2 * row + 1];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const int col = (c * 32 + lane) * VEC;
            float a[VEC], d[VEC], g[VEC];
            RowVec<T>::ld(z + row * D + col, a); RowVec<T>::ld(dy + row * D + col, d); RowVec<T>::ld(gamma + col, g);
#pragma unroll
            for (int k = 0; k < VEC; ++k) { const float xh = (a[k] - mean) * rstd, dg = d[k] * g[k]; s1 += dg; s2 = fmaf(dg, xh, s2); }
            if (NCH >= 8 && (c & 1)) asm volatile("" ::: "memory");      // keep the unrolled loads from being hoisted all at once (register pressure)
        }
        s1 = RMS ? 0.f : warp_sum(s1) / D; s2 = warp_sum(s2) / D;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {                 // second pass: the row is re-read through L1
            const int col = (c * 32 + lane) * VEC;
            float a[VEC], d[VEC], o[VEC], g[VEC];
            RowVec<T>::ld(z + row * D + col, a); RowVec<T>::ld(dy + row * D + col, d); RowVec<T>::ld(gamma + col, g);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                const float xh = (a[k] - mean) * rstd;
                o[k] = rstd * (d[k] * g[k] - s1 - xh * s2);
                ag[c][k] = fmaf(d[k], xh, ag[c][k]);
                if (!RMS) ab[c][k] += d[k];
            }
            if (dz_in) {
                float e[VEC];
                RowVec<T>::ld(dz_in + row * D + col, e);
#pragma unroll
                for (int k = 0; k < VEC; ++k) o[k] += e[k];
            }
            RowVec<T>::st(dz + row * D + col, o);
            if (NCH >= 8) asm volatile("" ::: "memory");
        }
    }
    // fixed-order reduction over the eight warps, first the weight gradient, then (LayerNorm) the bias gradient
#pragma unroll 1
    for (int which = 0; which < (RMS ? 1 : 2); ++which) {
        __syncthreads();
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int k = 0; k < VEC; ++k) sm[w * D + (c * 32 + lane) * VEC + k] = which == 0 ? ag[c][k] : ab[RMS ? 0 : c][k];
        __syncthreads();
        for (int col = threadIdx.x; col < D; col += 256) {
            float acc = 0.f;
#pragma unroll
            for (int ww = 0; ww < 8; ++ww) acc += sm[ww * D + col];
            part[((int64_t)blockIdx.x * 2 + which) * D + col] = acc;
        }
    }
    if (RMS) for (int col = threadIdx.x; col < D; col += 256) part[((int64_t)blockIdx.x * 2 + 1) * D + col] = 0.f;
}

// Second stage of the parameter gradients: column c of dgamma / dbeta is the sum of its n_part partial rows.  A CTA owns 32
// columns; its 32 warps take the partial rows p = warp, warp + 32, ... and the 32 sub-sums are added in warp order, so the
// result does not depend on timing.  (D / 32 CTAs only: with 8 warps per CTA the kernel took 9 us for 296 partial rows of 512 columns.)
constexpr int LN_RED_WARPS = 32;
template <typename T>
__global__ void __launch_bounds__(32 * LN_RED_WARPS) ln_bwd_reduce_kernel(const float* __restrict__ part, int n_part, int D, T* __restrict__ dgamma,
                                                                          T* __restrict__ dbeta, bool accumulate) {
    __shared__ float sh[2][LN_RED_WARPS][33];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    float a = 0.f, b = 0.f;
    if (c < D) {
        int p = w;
        for (; p + 3 * LN_RED_WARPS < n_part; p += 4 * LN_RED_WARPS) {
            float va[4], vb[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                va[u] = part[((int64_t)(p + LN_RED_WARPS * u) * 2) * D + c];
                vb[u] = part[((int64_t)(p + LN_RED_WARPS * u) * 2 + 1) * D + c];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) { a += va[u]; b += vb[u]; }
        }
        for (; p < n_part; p += LN_RED_WARPS) { a += part[((int64_t)p * 2) * D + c]; b += part[((int64_t)p * 2 + 1) * D + c]; }
    }
    sh[0][w][lane] = a; sh[1][w][lane] = b;
    __syncthreads();
    if (w == 0 && c < D) {
        a = 0.f; b = 0.f;
#pragma unroll
        for (int k = 0; k < LN_RED_WARPS; ++k) { a += sh[0][k][lane]; b += sh[1][k][lane]; }
        // accumulate: dgamma / dbeta are the parameters' gradient buffers and already hold other contributions of this step
        if (accumulate) { a += Cvt<T>::to(dgamma[c]); if (dbeta) b += Cvt<T>::to(dbeta[c]); }
        dgamma[c] = Cvt<T>::from(a);
        if (dbeta) dbeta[c] = Cvt<T>::from(b);
    }
}

}  // namespace

bool attn_small_supported(int S, int HD) { return (S == 4 || S == 8) && (HD == 32 || HD == 64); }

template <typename T>
static void attn_dispatch(bool bwd, const T* qkv, const T* dout, T* out, int B, int S, int H, int HD, bool causal, cudaStream_t st) {
    const float scale = 1.f / sqrtf((float)HD);
    const unsigned blocks = (unsigned)(((int64_t)B * H + 7) / 8);
    count_launch();
#define GO(SV, EV, CV) \
    if (bwd) attn_small_bwd_kernel<T, SV, EV, CV><<<blocks, 256, 0, st>>>(qkv, dout, out, B, H, scale); \
    else attn_small_fwd_kernel<T, SV, EV, CV><<<blocks, 256, 0, st>>>(qkv, out, B, H, scale);
#define GO2(SV, EV) if (causal) { GO(SV, EV, true) } else { GO(SV, EV, false) }
    if (S == 4 && HD == 64) { GO2(4, 2) } else if (S == 4 && HD == 32) { GO2(4, 1) }
    else if (S == 8 && HD == 64) { GO2(8, 2) } else { GO2(8, 1) }
#undef GO2
#undef GO
}

void attn_small(int dtype, bool bwd, const void* qkv, const void* dout, void* out, int B, int S, int H, int HD, bool causal, cudaStream_t st) {
    if (dtype == BF16) attn_dispatch<__nv_bfloat16>(bwd, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)dout, (__nv_bfloat16*)out, B, S, H, HD, causal, st);
    else attn_dispatch<float>(bwd, (const float*)qkv, (const float*)dout, (float*)out, B, S, H, HD, causal, st);
}

constexpr int WIDE_GRID = 148 * 2;
static int wide_nch(int D, int elem_bytes) {            // rows of 32 * (16 / elem_bytes) * NCH elements take the wide kernels
    const int unit = 32 * (16 / elem_bytes);
    if (D % unit) return 0;
    const int n = D / unit;
    return (n == 1 || n == 2 || n == 4 || n == 8) ? n : 0;          // 16 chunks would need 128+ accumulator registers per lane
}
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
static void ln_fwd_t(bool rms, const void* x, const void* r, const void* gamma, const void* beta, void* z, void* y, float* stats, int64_t rows, int D,
                     float eps, cudaStream_t st) {
    const unsigned blocks = (unsigned)((rows + 7) / 8);
    const int nch = wide_nch(D, (int)sizeof(T));
    if (nch && aligned16(x) && aligned16(r) && aligned16(gamma) && aligned16(beta) && aligned16(z) && aligned16(y)) {
#define WIDE_F(N) \
        if (rms) norm_fwd_wide_kernel<T, true, N><<<blocks, 256, 0, st>>>((const T*)x, (const T*)r, (const T*)gamma, nullptr, (T*)z, (T*)y, stats, rows, eps); \
        else norm_fwd_wide_kernel<T, false, N><<<blocks, 256, 0, st>>>((const T*)x, (const T*)r, (const T*)gamma, (const T*)beta, (T*)z, (T*)y, stats, rows, eps);
        switch (nch) { case 1: WIDE_F(1) break; case 2: WIDE_F(2) break; case 4: WIDE_F(4) break; default: WIDE_F(8) break; }
#undef WIDE_F
        return;
    }
    if (rms) ln_fwd_kernel<T, true><<<blocks, 256, 0, st>>>((const T*)x, (const T*)r, (const T*)gamma, nullptr, (T*)z, (T*)y, stats, rows, D, eps);
    else ln_fwd_kernel<T, false><<<blocks, 256, 0, st>>>((const T*)x, (const T*)r, (const T*)gamma, (const T*)beta, (T*)z, (T*)y, stats, rows, D, eps);
}

void ln_fwd(int dtype, bool rms, const void* x, const void* r, const void* gamma, const void* beta, void* z, void* y, float* stats, int64_t rows,
            int D, float eps, cudaStream_t st) {
    count_launch();
    if (dtype == BF16) ln_fwd_t<__nv_bfloat16>(rms, x, r, gamma, beta, z, y, stats, rows, D, eps, st);
    else ln_fwd_t<float>(rms, x, r, gamma, beta, z, y, stats, rows, D, eps, st);
}

// CTA partials of the weight / bias gradient: enough for either backward kernel
static int wide_grid(int64_t rows) { const int64_t b = (rows + 7) / 8; return (int)(b < WIDE_GRID ? b : WIDE_GRID); }
int ln_bwd_parts(int64_t rows) {
    const int a = (int)((rows + LN_ROWS_PER_CTA - 1) / LN_ROWS_PER_CTA), b = wide_grid(rows);
    return a > b ? a : b;
}

template <typename T>
static void ln_bwd_t(bool rms, const void* z, const void* dy, const void* gamma, const float* stats, const void* dz_in, void* dz, float* part,
                     void* dgamma, void* dbeta, bool accumulate, int64_t rows, int D, cudaStream_t st) {
    const int nch = wide_nch(D, (int)sizeof(T));
    if (nch && aligned16(z) && aligned16(dy) && aligned16(gamma) && aligned16(dz_in) && aligned16(dz)) {
        const int grid = wide_grid(rows);
        const size_t smw = (size_t)8 * D * sizeof(float);
#define WIDE_B2(R, N) \
        { cudaFuncSetAttribute(norm_bwd_wide_kernel<T, R, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smw); \
          norm_bwd_wide_kernel<T, R, N><<<grid, 256, smw, st>>>((const T*)z, (const T*)dy, (const T*)gamma, stats, (const T*)dz_in, (T*)dz, part, rows); }
#define WIDE_B(N) if (rms) WIDE_B2(true, N) else WIDE_B2(false, N)
        switch (nch) { case 1: WIDE_B(1) break; case 2: WIDE_B(2) break; case 4: WIDE_B(4) break; default: WIDE_B(8) break; }
#undef WIDE_B
#undef WIDE_B2
        ln_bwd_reduce_kernel<T><<<(D + 31) / 32, 32 * LN_RED_WARPS, 0, st>>>(part, grid, D, (T*)dgamma, (T*)dbeta, accumulate);
        return;
    }
    const int parts = (int)((rows + LN_ROWS_PER_CTA - 1) / LN_ROWS_PER_CTA);
    const size_t smem = (size_t)8 * 2 * D * sizeof(float);
    if (rms) {
        cudaFuncSetAttribute(ln_bwd_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ln_bwd_kernel<T, true><<<parts, 256, smem, st>>>((const T*)z, (const T*)dy, (const T*)gamma, stats, (const T*)dz_in, (T*)dz, part, rows, D);
    } else {
        cudaFuncSetAttribute(ln_bwd_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ln_bwd_kernel<T, false><<<parts, 256, smem, st>>>((const T*)z, (const T*)dy, (const T*)gamma, stats, (const T*)dz_in, (T*)dz, part, rows, D);
    }
    ln_bwd_reduce_kernel<T><<<(D + 31) / 32, 32 * LN_RED_WARPS, 0, st>>>(part, parts, D, (T*)dgamma, (T*)dbeta, accumulate);
}

void ln_bwd(int dtype, bool rms, const void* z, const void* dy, const void* gamma, const float* stats, const void* dz_in, void* dz, float* part,
            void* dgamma, void* dbeta, bool accumulate, int64_t rows, int D, cudaStream_t st) {
    count_launch(2);
    if (dtype == BF16) ln_bwd_t<__nv_bfloat16>(rms, z, dy, gamma, stats, dz_in, dz, part, dgamma, dbeta, accumulate, rows, D, st);
    else ln_bwd_t<float>(rms, z, dy, gamma, stats, dz_in, dz, part, dgamma, dbeta, accumulate, rows, D, st);
}


// ---------------------------------------------------------------------------------------------------------------------------
// Column sums of a row-major [rows, C] matrix: the bias gradient of a Linear layer (db = sum over tokens of dy).  Two stages in
// a fixed order (no atomics): CTA (bx, by) sums rows [by * rows_per_cta, ...) of a slab of 32 sixteen-byte vectors, eight row
// lanes per column vector with fp32 accumulators, and writes one partial row; the second kernel adds the partial rows in order.
namespace {
template <typename T>
__global__ void __launch_bounds__(256) col_sum_part_kernel(const T* __restrict__ x, int64_t ld, int64_t rows, int C, int64_t rows_per_cta,
                                                           bool vec, float* __restrict__ part) {
    constexpr int VEC = 16 / (int)sizeof(T);
    __shared__ float sh[8][32 * VEC + 1];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c0 = (blockIdx.x * 32 + tx) * VEC;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_cta;
    const int64_t r1 = r0 + rows_per_cta < rows ? r0 + rows_per_cta : rows;
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
    if (c0 < C) {
        if (vec) {
            int64_t r = r0 + ty;
            for (; r + 24 < r1; r += 32) {                    // four independent 16-byte loads in flight per thread
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const uint4*>(x + (r + 8 * u) * ld + c0);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const T* e = reinterpret_cast<const T*>(&v[u]);
#pragma unroll
                    for (int j = 0; j < VEC; ++j) acc[j] += Cvt<T>::to(e[j]);
                }
            }
            for (; r < r1; r += 8) {
                const uint4 v = *reinterpret_cast<const uint4*>(x + r * ld + c0);
                const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
                for (int j = 0; j < VEC; ++j) acc[j] += Cvt<T>::to(e[j]);
            }
        } else {
            for (int64_t r = r0 + ty; r < r1; r += 8)
#pragma unroll
                for (int j = 0; j < VEC; ++j)
                    if (c0 + j < C) acc[j] += Cvt<T>::to(x[r * ld + c0 + j]);
        }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) sh[ty][tx * VEC + j] = acc[j];
    __syncthreads();
    for (int c = threadIdx.x; c < 32 * VEC; c += 256) {
        const int col = blockIdx.x * 32 * VEC + c;
        if (col < C) {
            float t = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) t += sh[k][c];
            part[(int64_t)blockIdx.y * C + col] = t;
        }
    }
}

// Second stage: 32 columns per CTA; warp w adds the partial rows w, w + 8, ... and the 8 sub-sums are added in warp order.
template <typename T>
__global__ void __launch_bounds__(256) col_sum_final_kernel(const float* __restrict__ part, int parts, int C, T* __restrict__ out,
                                                            bool accumulate) {
    __shared__ float sh[8][33];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    float t = 0.f;
    if (c < C) {
        int p = w;
        for (; p + 24 < parts; p += 32) {
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = part[(int64_t)(p + 8 * u) * C + c];
#pragma unroll
            for (int u = 0; u < 4; ++u) t += v[u];
        }
        for (; p < parts; p += 8) t += part[(int64_t)p * C + c];
    }
    sh[w][lane] = t;
    __syncthreads();
    if (w == 0 && c < C) {
        t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += sh[k][lane];
        if (accumulate) t += Cvt<T>::to(out[c]);
        out[c] = Cvt<T>::from(t);
    }
}
}  // namespace

// number of partial rows the first stage writes for a [rows, C] input (the caller provides parts * C floats of scratch)
int col_sum_parts(int64_t rows, int C, int elem_bytes) {
    const int vecw = 32 * (16 / elem_bytes);
    const int bx = (C + vecw - 1) / vecw;
    int64_t parts = (4 * 148 + bx - 1) / bx;
    const int64_t max_parts = (rows + 63) / 64;
    if (parts > max_parts) parts = max_parts;
    return parts < 1 ? 1 : (int)parts;
}

void col_sum(int dtype, const void* x, int64_t ld, int64_t rows, int C, float* part, void* out, bool accumulate, cudaStream_t st) {
    const int es = dtype == F32 ? 4 : 2;
    const int parts = col_sum_parts(rows, C, es);
    const int64_t rpc = (rows + parts - 1) / parts;
    const int vecw = 32 * (16 / es);
    const dim3 grid((C + vecw - 1) / vecw, parts);
    const bool vec = C % (16 / es) == 0 && (ld * es) % 16 == 0 && aligned16(x);
    count_launch(2);
    if (dtype == BF16) {
        col_sum_part_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ld, rows, C, rpc, vec, part);
        col_sum_final_kernel<__nv_bfloat16><<<(C + 31) / 32, 256, 0, st>>>(part, parts, C, (__nv_bfloat16*)out, accumulate);
    } else if (dtype == F16) {
        col_sum_part_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, ld, rows, C, rpc, vec, part);
        col_sum_final_kernel<__half><<<(C + 31) / 32, 256, 0, st>>>(part, parts, C, (__half*)out, accumulate);
    } else {
        col_sum_part_kernel<float><<<grid, 256, 0, st>>>((const float*)x, ld, rows, C, rpc, vec, part);
        col_sum_final_kernel<float><<<(C + 31) / 32, 256, 0, st>>>(part, parts, C, (float*)out, accumulate);
    }
}

}  // namespace sg
