// Per-element optimizer arithmetic shared by the local multi-tensor kernels and the fused
// reduce-scatter + step kernels.  All state is fp32.  Formulas follow the reference kernels
// (csrc/lion_kernels.cu:20, grokadamw_kernels.cu:42, prodigy_kernels.cu:50,
//  neuralgrok_kernels.cu:244, supergrok15_kernels.cu:323, supergrok11_kernels.cu:37,109).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace sg {

__device__ __forceinline__ float adam_update(float p, float fg, float& m, float& v, float lr, float b1, float b2,
                                              float eps, float wd, float bc1, float bc2) {
    m = b1 * m + (1.f - b1) * fg;
    v = b2 * v + (1.f - b2) * fg * fg;
    const float denom = sqrtf(v / bc2) + eps;
    return p * (1.f - lr * wd) - (lr / bc1) * m / denom;
}

__device__ __forceinline__ float lion_update(float p, float g, float& m, float lr, float b1, float b2, float wd) {
    const float c = b1 * m + (1.f - b1) * g;
    const float s = (c > 0.f) ? 1.f : ((c < 0.f) ? -1.f : 0.f);
    m = b2 * m + (1.f - b2) * g;
    return p - lr * (s + wd * p);
}

__device__ __forceinline__ float fast_gelu(float z) { return z / (1.f + __expf(-1.702f * z)); }

// 2 -> H -> 1 meta-net of SuperGrok v1.1 / v1.5, weights in shared memory: sW1 [H][2], sb1 [H], sW2 [H], sb2 [1]
__device__ __forceinline__ float sharp_mlp(float g, float s, const float* sW1, const float* sb1, const float* sW2,
                                           float b2, int H) {
    float acc = b2;
#pragma unroll 4
    for (int h = 0; h < H; ++h) {
        const float z = fmaf(sW1[2 * h], g, fmaf(sW1[2 * h + 1], s, sb1[h]));
        acc = fmaf(sW2[h], fast_gelu(z), acc);
    }
    return acc;
}

// 1 -> H -> 1 ReLU amplifier of NeuralGrok: sW1 [H], sb1 [H], sW2 [H]
__device__ __forceinline__ float amp_mlp(float g, const float* sW1, const float* sb1, const float* sW2, float b2,
                                         int H) {
    float acc = b2;
#pragma unroll 4
    for (int h = 0; h < H; ++h) acc = fmaf(sW2[h], fmaxf(fmaf(sW1[h], g, sb1[h]), 0.f), acc);
    return acc;
}

// ---- typed vector access -----------------------------------------------------------------
template <typename T> struct Cvt;
template <> struct Cvt<float> {
    static __device__ __forceinline__ float to(float x) { return x; }
    static __device__ __forceinline__ float from(float x) { return x; }
};
template <> struct Cvt<__nv_bfloat16> {
    static __device__ __forceinline__ float to(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 from(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Cvt<__half> {
    static __device__ __forceinline__ float to(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from(float x) { return __float2half_rn(x); }
};

template <typename T>
__device__ __forceinline__ bool vec_ok(const void* p) {
    return (reinterpret_cast<uintptr_t>(p) & (sizeof(T) * 4 - 1)) == 0;
}

// loads up to 4 consecutive elements starting at element i (cnt valid); vec => aligned 4-wide access allowed
template <typename T>
__device__ __forceinline__ void ld4(const void* base, int64_t i, int cnt, bool vec, float v[4]) {
    const T* p = reinterpret_cast<const T*>(base) + i;
    if (vec && cnt == 4) {
        if constexpr (sizeof(T) == 4) {
            const float4 t = *reinterpret_cast<const float4*>(p);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
            const uint2 t = *reinterpret_cast<const uint2*>(p);
            const T* h = reinterpret_cast<const T*>(&t);
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = Cvt<T>::to(h[k]);
        }
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = (k < cnt) ? Cvt<T>::to(p[k]) : 0.f;
    }
}

template <typename T>
__device__ __forceinline__ void st4(void* base, int64_t i, int cnt, bool vec, const float v[4]) {
    T* p = reinterpret_cast<T*>(base) + i;
    if (vec && cnt == 4) {
        if constexpr (sizeof(T) == 4) {
            *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
            uint2 t;
            T* h = reinterpret_cast<T*>(&t);
#pragma unroll
            for (int k = 0; k < 4; ++k) h[k] = Cvt<T>::from(v[k]);
            *reinterpret_cast<uint2*>(p) = t;
        }
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (k < cnt) p[k] = Cvt<T>::from(v[k]);
    }
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// deterministic block sum (fixed tree); result valid in thread 0.  `red` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float x, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    x = warp_sum(x);
    __syncthreads();
    if (lane == 0) red[w] = x;
    __syncthreads();
    float r = 0.f;
    if (w == 0) {
        r = (lane < nw) ? red[lane] : 0.f;
        r = warp_sum(r);
    }
    return r;
}

}  // namespace sg
