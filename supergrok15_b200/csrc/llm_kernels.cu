// Memory-bound model kernels of the Llama-style decoder (sm_100a): rotary position embedding, SwiGLU, GELU, embedding gather and its
// deterministic gradient, and softmax cross-entropy.  Each replaces a chain of PyTorch element-wise / reduction launches used by
// the reference models (grokking_race_v2.py:310-331, :452 builds them from nn.Embedding, F.gelu and F.cross_entropy) with ONE pass
// over the data at 16 bytes per lane; every reduction has a fixed order (no floating-point atomics).
#include "sg_native.h"
#include "optim_math.cuh"
#include <cfloat>

namespace sg {
namespace {

template <typename T> struct Vec8 {                       // 8 elements = 16 bytes (bf16/fp16) or 32 bytes (fp32)
    static __device__ __forceinline__ void ld(const T* p, float (&v)[8]) {
        if constexpr (sizeof(T) == 2) {
            const uint4 t = *reinterpret_cast<const uint4*>(p);
            const T* h = reinterpret_cast<const T*>(&t);
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = Cvt<T>::to(h[k]);
        } else {
            const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
    }
    static __device__ __forceinline__ void st(T* p, const float (&v)[8]) {
        if constexpr (sizeof(T) == 2) {
            uint4 t;
            T* h = reinterpret_cast<T*>(&t);
#pragma unroll
            for (int k = 0; k < 8; ++k) h[k] = Cvt<T>::from(v[k]);
            *reinterpret_cast<uint4*>(p) = t;
        } else {
            reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
            reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
    }
};

// ------------------------------------------------------------------------------------------------ rotary embedding
// x, y: [B, S, H, HD] (the projection output viewed per head); pairs are (2i, 2i+1); cs: [S, HD/2] cos and sin tables (fp32).
// sign = +1 rotates by the position angle, -1 by its negative (the backward pass: the Jacobian of a rotation is its transpose).
template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const T* __restrict__ x, T* __restrict__ y, const float* __restrict__ cosT,
                                                   const float* __restrict__ sinT, int64_t n_vec, int S, int H, int HD, float sign) {
    const int vec_per_head = HD / 8;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += (int64_t)gridDim.x * blockDim.x) {
        const int hv = (int)(v % vec_per_head);
        const int64_t bsh = v / vec_per_head;
        const int s = (int)((bsh / H) % S);
        float a[8], o[8];
        Vec8<T>::ld(x + v * 8, a);
        const float4 c = *reinterpret_cast<const float4*>(cosT + (int64_t)s * (HD / 2) + hv * 4);
        const float4 sn = *reinterpret_cast<const float4*>(sinT + (int64_t)s * (HD / 2) + hv * 4);
        const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x * sign, sn.y * sign, sn.z * sign, sn.w * sign};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            o[2 * k] = a[2 * k] * cc[k] - a[2 * k + 1] * ss[k];
            o[2 * k + 1] = a[2 * k] * ss[k] + a[2 * k + 1] * cc[k];
        }
        Vec8<T>::st(y + v * 8, o);
    }
}

// ------------------------------------------------------------------------------------------------ SwiGLU / GELU
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const T* __restrict__ g, const T* __restrict__ u, T* __restrict__ y, int64_t n_vec) {
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += (int64_t)gridDim.x * blockDim.x) {
        float a[8], b[8], o[8];
        Vec8<T>::ld(g + v * 8, a); Vec8<T>::ld(u + v * 8, b);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = Cvt<T>::to(Cvt<T>::from(a[k] * sigmoidf_(a[k]))) * b[k];   // silu rounded like the unfused chain
        Vec8<T>::st(y + v * 8, o);
    }
}
template <typename T>
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const T* __restrict__ g, const T* __restrict__ u, const T* __restrict__ dy,
                                                         T* __restrict__ dg, T* __restrict__ du, int64_t n_vec) {
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += (int64_t)gridDim.x * blockDim.x) {
        float a[8], b[8], d[8], og[8], ou[8];
        Vec8<T>::ld(g + v * 8, a); Vec8<T>::ld(u + v * 8, b); Vec8<T>::ld(dy + v * 8, d);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float sg = sigmoidf_(a[k]);
            ou[k] = d[k] * a[k] * sg;
            og[k] = d[k] * b[k] * sg * (1.f + a[k] * (1.f - sg));
        }
        Vec8<T>::st(dg + v * 8, og); Vec8<T>::st(du + v * 8, ou);
    }
}

// erf GELU; bwd = true writes dy * gelu'(x).  fp32 tensors use erff.  16-bit tensors use the rational approximation
// erf(z) = 1 - (a1 t + ... + a5 t^5) exp(-z^2), t = 1 / (1 + p z), z >= 0 (absolute error 1.5e-7, far below half an ulp of a
// 16-bit result), whose exponential exp(-x^2 / 2) is the one the derivative needs anyway: two special-function results and
// nine FMAs per element instead of erff's ~25 instructions (backward 103 -> 87 us at 32,768 x 2,048 bf16).
template <typename T, bool BWD>
__device__ __forceinline__ void gelu8(const float (&a)[8], const float (&d)[8], float (&o)[8]) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        float cdf, e;
        if constexpr (sizeof(T) == 2) {
            const float z = fabsf(a[k]) * 0.70710678118654752f;
            e = __expf(-z * z);
            const float t = __fdividef(1.f, fmaf(0.3275911f, z, 1.f));      // approximate reciprocal: one special-function result
            const float poly = t * fmaf(t, fmaf(t, fmaf(t, fmaf(t, 1.061405429f, -1.453152027f), 1.421413741f), -0.284496736f), 0.254829592f);
            const float half_tail = 0.5f * poly * e;                 // (1 - erf(|z|)) / 2
            cdf = a[k] >= 0.f ? 1.f - half_tail : half_tail;
        } else {
            cdf = 0.5f * (1.f + erff(a[k] * 0.70710678118654752f));
            if (BWD) e = __expf(-0.5f * a[k] * a[k]);
        }
        if (BWD) o[k] = d[k] * (cdf + a[k] * 0.3989422804014327f * e);
        else o[k] = a[k] * cdf;
    }
}

template <typename T, bool BWD>
__global__ void __launch_bounds__(256) gelu_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ y, int64_t n_vec) {
    // one 16-byte vector per thread and iteration; four in flight per thread were measured no faster forward and slower backward
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n_vec; v += (int64_t)gridDim.x * blockDim.x) {
        float a[8], d[8], o[8];
        Vec8<T>::ld(x + v * 8, a);
        if (BWD) Vec8<T>::ld(dy + v * 8, d);
        gelu8<T, BWD>(a, d, o);
        Vec8<T>::st(y + v * 8, o);
    }
}

// ------------------------------------------------------------------------------------------------ embedding
// out[t, :] = W[ids[t], :]; one warp per token, D a multiple of 8.
template <typename T>
__global__ void __launch_bounds__(256) embed_fwd_kernel(const int64_t* __restrict__ ids, const T* __restrict__ W, T* __restrict__ out,
                                                        int64_t T_tok, int D, int V) {
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= T_tok) return;
    int64_t id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);                     // clamp: never read outside the table
    const uint4* src = reinterpret_cast<const uint4*>(W + id * D);
    uint4* dst = reinterpret_cast<uint4*>(out + t * D);
    const int nv = D * (int)sizeof(T) / 16;
    for (int c = lane; c < nv; c += 32) dst[c] = src[c];
}

__global__ void __launch_bounds__(256) embed_keys_kernel(const int64_t* __restrict__ ids, uint32_t* __restrict__ keys, uint32_t* __restrict__ vals,
                                                         int64_t T_tok, int V) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T_tok) return;
    const int64_t id = ids[t];
    keys[t] = (uint32_t)(id < 0 ? 0 : (id >= V ? V - 1 : id));
    vals[t] = (uint32_t)t;
}

// Gradient of the gather: the token positions arrive sorted by id (stable), so every row of dW is the sum of one contiguous run,
// added in position order by ONE warp (fixed order: bitwise reproducible).  dW is zero-filled by the caller.
template <typename T>
__global__ void __launch_bounds__(256) embed_bwd_kernel(const uint32_t* __restrict__ keys, const uint32_t* __restrict__ vals,
                                                        const T* __restrict__ dout, T* __restrict__ dW, int64_t T_tok, int D) {
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= T_tok) return;
    const uint32_t key = keys[i];
    if (i > 0 && keys[i - 1] == key) return;                       // not the start of a run
    int64_t end = i + 1;
    while (end < T_tok && keys[end] == key) ++end;
    for (int c = lane * 8; c < D; c += 256) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int64_t j = i; j < end; ++j) {
            float d[8];
            Vec8<T>::ld(dout + (int64_t)vals[j] * D + c, d);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += d[k];
        }
        Vec8<T>::st(dW + (int64_t)key * D + c, acc);
    }
}

// Small tables (vocabulary x tokens <= 2^24, the modular-arithmetic models): no sort.  CTA (v, slab) owns row v of dW and 256 of its
// columns.  Its 8 warps split the token positions into 8 contiguous ranges; a warp reads 32 ids at a time, finds the positions whose
// id is v with a ballot and adds their rows of dout in position order (lane = 8 columns); the 8 range sums are then added in warp
// order.  Every CTA reads all ids (from L2), which is what limits the table size.  accumulate: dW already holds other contributions.
template <typename T>
__global__ void __launch_bounds__(256) embed_bwd_small_kernel(const int64_t* __restrict__ ids, const T* __restrict__ dout, T* __restrict__ dW,
                                                              int64_t T_tok, int D, int V, bool accumulate) {
    __shared__ float sh[8][256 + 8];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int v = blockIdx.x;
    const int c = blockIdx.y * 256 + lane * 8;
    const int64_t per = ((T_tok + 7) / 8 + 31) / 32 * 32;              // positions per warp, a multiple of 32
    const int64_t t0 = w * per, t1 = (t0 + per < T_tok) ? t0 + per : T_tok;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int64_t t = t0; t < t1; t += 32) {
        int64_t id = (t + lane < t1) ? ids[t + lane] : -1;
        if (id >= V) id = V - 1;                                       // same clamp as the forward gather
        if (id < 0 && t + lane < t1) id = 0;
        unsigned m = __ballot_sync(0xffffffffu, id == v);
        while (m) {
            const int k = __ffs(m) - 1;
            m &= m - 1;
            if (c < D) {
                float d[8];
                Vec8<T>::ld(dout + (t + k) * D + c, d);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += d[j];
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) sh[w][lane * 8 + j] = acc[j];
    __syncthreads();
    if (w == 0 && c < D) {
        float o[8];
        if (accumulate) Vec8<T>::ld(dW + (int64_t)v * D + c, o);
        else {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = 0.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k)
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += sh[k][lane * 8 + j];
        Vec8<T>::st(dW + (int64_t)v * D + c, o);
    }
}

// Tables of at most EMB_TAB_V rows (the modular-arithmetic vocabularies) whatever the token statistics: the kernel above walks the
// matches of one id serially, and in those datasets two ids ("op", "=") occur in every sequence.  Here CTA (split s, slab) walks a
// contiguous range of token positions in order; thread c adds dout[t][slab * 256 + c] into ITS column of a [V][256] fp32 table in
// shared memory (row = id of token t): no conflicts, no atomics, a fixed order.  The S partial tables are then added in split order.
constexpr int EMB_TAB_V = 208;                     // 208 x 256 x 4 B = 208 KB of shared memory
template <typename T>
__global__ void __launch_bounds__(256) embed_bwd_table_kernel(const int64_t* __restrict__ ids, const T* __restrict__ dout, float* __restrict__ part,
                                                              int64_t T_tok, int D, int V, int S) {
    extern __shared__ float tab[];                 // [V][256]; thread c only ever touches column c
    const int c = blockIdx.y * 256 + threadIdx.x;
    for (int v = 0; v < V; ++v) tab[v * 256 + threadIdx.x] = 0.f;
    const int64_t per = (T_tok + S - 1) / S;
    const int64_t t0 = (int64_t)blockIdx.x * per, t1 = (t0 + per < T_tok) ? t0 + per : T_tok;
    if (c < D) {
        int64_t t = t0;
        for (; t + 8 <= t1; t += 8) {              // eight rows in flight; the table is updated in position order
            int id[8]; float x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                int64_t i = ids[t + u];
                id[u] = (int)(i < 0 ? 0 : (i >= V ? V - 1 : i));
                x[u] = Cvt<T>::to(dout[(t + u) * D + c]);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) tab[id[u] * 256 + threadIdx.x] += x[u];
        }
        for (; t < t1; ++t) {
            int64_t i = ids[t];
            const int id = (int)(i < 0 ? 0 : (i >= V ? V - 1 : i));
            tab[id * 256 + threadIdx.x] += Cvt<T>::to(dout[t * D + c]);
        }
        for (int v = 0; v < V; ++v) part[((int64_t)blockIdx.x * V + v) * D + c] = tab[v * 256 + threadIdx.x];
    }
}

template <typename T>
__global__ void __launch_bounds__(256) embed_bwd_table_reduce_kernel(const float* __restrict__ part, T* __restrict__ dW, int64_t VD, int S, bool accumulate) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= VD) return;
    float a = 0.f;
    for (int s = 0; s < S; ++s) a += part[(int64_t)s * VD + i];
    if (accumulate) a += Cvt<T>::to(dW[i]);
    dW[i] = Cvt<T>::from(a);
}

// ------------------------------------------------------------------------------------------------ cross-entropy
// One CTA per row of logits [rows, V] (V a multiple of 8).  Forward: log-sum-exp (online max) and the row loss lse - x[target];
// rows whose target equals ignore_index contribute nothing.
template <typename T>
__global__ void __launch_bounds__(256) ce_fwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ target, float* __restrict__ lse,
                                                     float* __restrict__ loss, int V, int64_t ignore_index) {
    __shared__ float red_m[8], red_s[8];
    const int64_t row = blockIdx.x;
    const T* x = logits + row * V;
    float m = -FLT_MAX, s = 0.f;
    for (int c = threadIdx.x * 8; c < V; c += 256 * 8) {
        float a[8];
        Vec8<T>::ld(x + c, a);
        float mm = a[0];
#pragma unroll
        for (int k = 1; k < 8; ++k) mm = fmaxf(mm, a[k]);
        const float nm = fmaxf(m, mm);
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += __expf(a[k] - nm);
        s = s * __expf(m - nm) + t;
        m = nm;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
        const float nm = fmaxf(m, om);
        s = s * __expf(m - nm) + os * __expf(om - nm);
        m = nm;
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { red_m[w] = m; red_s[w] = s; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float M = red_m[0], S = red_s[0];
        for (int ww = 1; ww < 8; ++ww) {
            const float nm = fmaxf(M, red_m[ww]);
            S = S * __expf(M - nm) + red_s[ww] * __expf(red_m[ww] - nm);
            M = nm;
        }
        const float l = M + logf(S);
        lse[row] = l;
        const int64_t t = target[row];
        loss[row] = (t == ignore_index || t < 0 || t >= V) ? 0.f : l - Cvt<T>::to(x[t]);
    }
}

// out[0] = mean loss over the counted rows, out[1] = 1 / max(count, 1): single CTA, fixed order.
__global__ void __launch_bounds__(256) ce_mean_kernel(const float* __restrict__ loss, const int64_t* __restrict__ target, int64_t rows, int V,
                                                      int64_t ignore_index, float* __restrict__ out) {
    __shared__ float red[32];
    float s = 0.f, n = 0.f;
    for (int64_t r = threadIdx.x; r < rows; r += 256) {
        const int64_t t = target[r];
        if (!(t == ignore_index || t < 0 || t >= V)) { s += loss[r]; n += 1.f; }
    }
    const float S = block_sum(s, red);
    const float Nn = block_sum(n, red);
    if (threadIdx.x == 0) { const float inv = 1.f / fmaxf(Nn, 1.f); out[0] = S * inv; out[1] = inv; }
}

// dlogits[row, c] = (softmax - onehot) * gout * inv_count  (zero for ignored rows)
template <typename T>
__global__ void __launch_bounds__(256) ce_bwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ target, const float* __restrict__ lse,
                                                     const float* __restrict__ mean_out, const float* __restrict__ gout, T* __restrict__ dlogits,
                                                     int V, int64_t ignore_index) {
    const int64_t row = blockIdx.x;
    const int64_t t = target[row];
    const bool ignored = (t == ignore_index || t < 0 || t >= V);
    const float scale = ignored ? 0.f : gout[0] * mean_out[1];
    const float l = lse[row];
    const T* x = logits + row * V;
    T* d = dlogits + row * V;
    for (int c = threadIdx.x * 8; c < V; c += 256 * 8) {
        float a[8], o[8];
        Vec8<T>::ld(x + c, a);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = (__expf(a[k] - l) - ((int64_t)(c + k) == t ? 1.f : 0.f)) * scale;
        Vec8<T>::st(d + c, o);
    }
}

int ew_grid(int64_t n_vec) {
    const int64_t b = (n_vec + 255) / 256;
    return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace

#define DISPATCH_T(dtype, ...) \
    if ((dtype) == BF16) { using T = __nv_bfloat16; __VA_ARGS__ } else if ((dtype) == F16) { using T = __half; __VA_ARGS__ } else { using T = float; __VA_ARGS__ }

void rope(int dtype, const void* x, void* y, const float* cosT, const float* sinT, int64_t B, int S, int H, int HD, bool backward, cudaStream_t st) {
    const int64_t n_vec = B * S * H * (HD / 8);
    if (n_vec <= 0) return;
    count_launch();
    DISPATCH_T(dtype, rope_kernel<T><<<ew_grid(n_vec), 256, 0, st>>>((const T*)x, (T*)y, cosT, sinT, n_vec, S, H, HD, backward ? -1.f : 1.f);)
}

void swiglu(int dtype, bool backward, const void* g, const void* u, const void* dy, void* out0, void* out1, int64_t n, cudaStream_t st) {
    const int64_t n_vec = n / 8;
    if (n_vec <= 0) return;
    count_launch();
    DISPATCH_T(dtype,
        if (backward) swiglu_bwd_kernel<T><<<ew_grid(n_vec), 256, 0, st>>>((const T*)g, (const T*)u, (const T*)dy, (T*)out0, (T*)out1, n_vec);
        else swiglu_fwd_kernel<T><<<ew_grid(n_vec), 256, 0, st>>>((const T*)g, (const T*)u, (T*)out0, n_vec);)
}

void gelu(int dtype, bool backward, const void* x, const void* dy, void* y, int64_t n, cudaStream_t st) {
    const int64_t n_vec = n / 8;
    if (n_vec <= 0) return;
    count_launch();
    DISPATCH_T(dtype,
        if (backward) gelu_kernel<T, true><<<ew_grid(n_vec), 256, 0, st>>>((const T*)x, (const T*)dy, (T*)y, n_vec);
        else gelu_kernel<T, false><<<ew_grid(n_vec), 256, 0, st>>>((const T*)x, nullptr, (T*)y, n_vec);)
}

void embed_fwd(int dtype, const int64_t* ids, const void* W, void* out, int64_t T_tok, int D, int V, cudaStream_t st) {
    if (T_tok <= 0) return;
    count_launch();
    DISPATCH_T(dtype, embed_fwd_kernel<T><<<(unsigned)((T_tok + 7) / 8), 256, 0, st>>>(ids, (const T*)W, (T*)out, T_tok, D, V);)
}

void embed_keys(const int64_t* ids, uint32_t* keys, uint32_t* vals, int64_t T_tok, int V, cudaStream_t st) {
    if (T_tok <= 0) return;
    count_launch();
    embed_keys_kernel<<<(unsigned)((T_tok + 255) / 256), 256, 0, st>>>(ids, keys, vals, T_tok, V);
}

void embed_bwd(int dtype, const uint32_t* keys, const uint32_t* vals, const void* dout, void* dW, int64_t T_tok, int D, cudaStream_t st) {
    if (T_tok <= 0) return;
    count_launch();
    DISPATCH_T(dtype, embed_bwd_kernel<T><<<(unsigned)((T_tok + 7) / 8), 256, 0, st>>>(keys, vals, (const T*)dout, (T*)dW, T_tok, D);)
}

// splits of the token range for the table kernel: enough CTAs to fill the GPU, at least 64 positions each
int embed_bwd_table_splits(int64_t T_tok, int D, int V) {
    if (V <= 0 || V > EMB_TAB_V || T_tok <= 0) return 0;
    const int slabs = (D + 255) / 256;
    int64_t S = (2 * 148 + slabs - 1) / slabs;
    if (S > 64) S = 64;
    if (S > (T_tok + 63) / 64) S = (T_tok + 63) / 64;
    return (int)(S < 1 ? 1 : S);
}

void embed_bwd_table(int dtype, const int64_t* ids, const void* dout, float* part, void* dW, int64_t T_tok, int D, int V, int S, bool accumulate,
                     cudaStream_t st) {
    count_launch(2);
    const dim3 grid((unsigned)S, (unsigned)((D + 255) / 256));
    const size_t smem = (size_t)V * 256 * sizeof(float);
    const int64_t VD = (int64_t)V * D;
    DISPATCH_T(dtype,
        cudaFuncSetAttribute(embed_bwd_table_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        embed_bwd_table_kernel<T><<<grid, 256, smem, st>>>(ids, (const T*)dout, part, T_tok, D, V, S);
        embed_bwd_table_reduce_kernel<T><<<(unsigned)((VD + 255) / 256), 256, 0, st>>>(part, (T*)dW, VD, S, accumulate);)
}

bool embed_bwd_small_ok(int64_t T_tok, int V) { return V > 0 && V <= 65535 && T_tok * (int64_t)V <= ((int64_t)1 << 24); }

void embed_bwd_small(int dtype, const int64_t* ids, const void* dout, void* dW, int64_t T_tok, int D, int V, bool accumulate, cudaStream_t st) {
    if (V <= 0 || D <= 0) return;
    count_launch();
    const dim3 grid((unsigned)V, (unsigned)((D + 255) / 256));
    DISPATCH_T(dtype, embed_bwd_small_kernel<T><<<grid, 256, 0, st>>>(ids, (const T*)dout, (T*)dW, T_tok, D, V, accumulate);)
}

void ce_fwd(int dtype, const void* logits, const int64_t* target, float* lse, float* loss, float* mean_out, int64_t rows, int V, int64_t ignore_index,
            cudaStream_t st) {
    if (rows <= 0) return;
    count_launch(2);
    DISPATCH_T(dtype, ce_fwd_kernel<T><<<(unsigned)rows, 256, 0, st>>>((const T*)logits, target, lse, loss, V, ignore_index);)
    ce_mean_kernel<<<1, 256, 0, st>>>(loss, target, rows, V, ignore_index, mean_out);
}

void ce_bwd(int dtype, const void* logits, const int64_t* target, const float* lse, const float* mean_out, const float* gout, void* dlogits,
            int64_t rows, int V, int64_t ignore_index, cudaStream_t st) {
    if (rows <= 0) return;
    count_launch();
    DISPATCH_T(dtype, ce_bwd_kernel<T><<<(unsigned)rows, 256, 0, st>>>((const T*)logits, target, lse, mean_out, gout, (T*)dlogits, V, ignore_index);)
}

}  // namespace sg
