// Vector access helpers for the in-kernel collectives: 16-byte loads of a gradient shard from every rank's buffer
// (plain peer loads over NVLink, all issued before the first is consumed, or one NVLS multimem.ld_reduce on the multicast
// address), packing of fp32 results into the low-precision parameter dtype.  Shared by the flat fused step
// (csrc/dist_kernels.cu) and by the SuperGrok v2 pipeline, whose first kernel pulls the gradients itself (csrc/sg2_kernels.cu).
#pragma once
#include "comm.cuh"
#include "optim_math.cuh"

namespace sg {

template <typename T> struct Vec8;      // 16-byte vector of a gradient dtype
template <> struct Vec8<float> { static constexpr int N = 4; };
template <> struct Vec8<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct Vec8<__half> { static constexpr int N = 8; };

template <typename T, int N>
__device__ __forceinline__ void acc_vec(const uint4& v, float (&acc)[N]) {
    const T* h = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int k = 0; k < N; ++k) acc[k] += Cvt<T>::to(h[k]);
}

// Remote accesses are ONE 16-byte (or 8-byte) access per lane with the lanes of a warp contiguous: a vector is 8 elements when
// both buffers hold 16-bit values and 4 elements as soon as one of them is fp32.  (Two 16-byte accesses per lane at a 32-byte
// stride touch every 32-byte sector twice with half of it; over NVLink that halves the useful bandwidth - measured.)
template <typename T, int N>
__device__ __forceinline__ void vload(const T* p, float (&v)[N]) {
    if constexpr (sizeof(T) * N == 16) {
        const uint4 t = *reinterpret_cast<const uint4*>(p);
        const T* h = reinterpret_cast<const T*>(&t);
#pragma unroll
        for (int k = 0; k < N; ++k) v[k] = Cvt<T>::to(h[k]);
    } else {
        static_assert(sizeof(T) * N == 8, "vector of 8 or 16 bytes");
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const T* h = reinterpret_cast<const T*>(&t);
#pragma unroll
        for (int k = 0; k < N; ++k) v[k] = Cvt<T>::to(h[k]);
    }
}
template <typename T, int N>
__device__ __forceinline__ void vpack(const float (&v)[N], uint4& o) {
    T* h = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int k = 0; k < N; ++k) h[k] = Cvt<T>::from(v[k]);
}
template <typename T, int N>
__device__ __forceinline__ void vstore_packed(T* p, const uint4& o) {
    if constexpr (sizeof(T) * N == 16) *reinterpret_cast<uint4*>(p) = o;
    else *reinterpret_cast<uint2*>(p) = make_uint2(o.x, o.y);
}

// Gradient fetch for one vector.  P2P: all W peer loads are issued before any of them is consumed (W is a compile-time constant so
// the loop unrolls; with a runtime trip count the first add would stall the warp and serialise the remote loads).
// NVLS: ONE multimem.ld_reduce per 16 bytes on the multicast address - the NVSwitch adds the W copies.
template <typename G, int N, bool NVLS, int W>
__device__ __forceinline__ void fetch_grad(const PeerPtrs& grads, const void* mc_grad, int world, int rank, int64_t elem, float (&g)[N]) {
    if constexpr (NVLS && sizeof(G) * N == 16) {
        const char* a = reinterpret_cast<const char*>(mc_grad) + elem * sizeof(G);
        if constexpr (sizeof(G) == 2) {
            const uint4 t = multimem_ld_reduce_bf16x8(a);
            const G* h = reinterpret_cast<const G*>(&t);
#pragma unroll
            for (int k = 0; k < N; ++k) g[k] = Cvt<G>::to(h[k]);
        } else {
            const float4 t0 = multimem_ld_reduce_f32x4(a);
            g[0] = t0.x; g[1] = t0.y; g[2] = t0.z; g[3] = t0.w;
        }
        return;
    }
#pragma unroll
    for (int k = 0; k < N; ++k) g[k] = 0.f;
    if constexpr (W > 0) {
        float raw[W][N];
#pragma unroll
        for (int kk = 0; kk < W; ++kk) vload<G, N>(reinterpret_cast<const G*>(grads.p[(rank + kk) % W]) + elem, raw[kk]);
#pragma unroll
        for (int kk = 0; kk < W; ++kk)
#pragma unroll
            for (int k = 0; k < N; ++k) g[k] += raw[kk][k];
    } else {
        for (int kk = 0; kk < world; ++kk) {
            float raw[N];
            vload<G, N>(reinterpret_cast<const G*>(grads.p[(rank + kk) % world]) + elem, raw);
#pragma unroll
            for (int k = 0; k < N; ++k) g[k] += raw[k];
        }
    }
}

}  // namespace sg
