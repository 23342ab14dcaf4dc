// In-kernel collectives for the ZeRO-sharded optimizer step (sm_100a, NVLink 5 / NVSwitch).
//
// Every rank owns a shard of the optimizer state.  Gradients live in a buffer that every peer has mapped
// (symmetric memory); so do the low-precision parameters.  The kernels here read the peers' gradient shards
// with plain 16-byte peer loads (or one NVLS multimem.ld_reduce on the multicast address), reduce in fp32
// registers, run the optimizer arithmetic on the owner's fp32 master / moments, and store the updated
// low-precision parameters into every peer's parameter buffer (or one multimem.st): reduce-scatter, step and
// all-gather are one pass over the shard and nothing round-trips through HBM in between.
// A path that calls NCCL reduce_scatter / all_gather around a local kernel exists only as the baseline
// (parallel/engine.py, comm="nccl").
//
// Cross-GPU ordering uses epoch flags in a signal pad with st.release.sys / ld.acquire.sys; waits are bounded.
#include "sg_native.h"
#include "comm.cuh"
#include "optim_math.cuh"

namespace sg {
namespace {

// ---- barrier: rank r publishes `epoch` in slot r of every pad, then waits for all slots of its own pad ----
__global__ void barrier_kernel(PeerPtrs pads, int rank, int world, uint32_t epoch, int* status, unsigned long long timeout_ns, int site) {
    const int r = threadIdx.x;
    if (r < world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t*>(pads.p[r]) + rank, epoch);
        if (!wait_flag_ge(reinterpret_cast<uint32_t*>(pads.p[rank]) + r, epoch, timeout_ns))
            atomicCAS(status, STATUS_OK, STATUS_TIMEOUT | (r << 8) | (site << 16));
        __threadfence_system();
    }
}

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

// ---- all-gather push: copy [off, off+n) of the local parameter buffer into every peer's buffer ----
template <bool NVLS>
__global__ void __launch_bounds__(256) push_kernel(PeerPtrs params, void* mc_param, int world, int rank, int64_t off_bytes, int64_t n_bytes) {
    const int64_t nv = n_bytes / 16;
    const char* src = reinterpret_cast<const char*>(params.p[rank]) + off_bytes;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nv; v += (int64_t)gridDim.x * blockDim.x) {
        const uint4 t = reinterpret_cast<const uint4*>(src)[v];
        if (NVLS) {
            multimem_st_u32x4(reinterpret_cast<char*>(mc_param) + off_bytes + v * 16, t);
        } else {
            for (int k = 1; k < world; ++k) {
                const int r = (rank + k) % world;
                reinterpret_cast<uint4*>(reinterpret_cast<char*>(params.p[r]) + off_bytes)[v] = t;
            }
        }
    }
    for (int64_t i = nv * 16 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_bytes; i += (int64_t)gridDim.x * blockDim.x)
        for (int k = 1; k < world; ++k) {
            const int r = (rank + k) % world;
            (reinterpret_cast<char*>(params.p[r]) + off_bytes)[i] = src[i];
        }
}

// ---- fused reduce-scatter + optimizer step + all-gather on a flat shard (single pass) ----
// OP 0: AdamW, OP 1: Lion.  Gradient dtype G (buffer of every rank), parameter dtype T (buffer of every rank),
// fp32 master / moments local to the owner.  off/n in elements, multiples of 8.
struct FlatStep {
    float lr, beta1, beta2, eps, wd, bc1, bc2, gscale;
    float* master; float* m; float* v;      // local shard arrays (index 0 = element `off`)
};

// Gradient fetch for one 8-element vector.  P2P: all W peer loads are issued before any of them is consumed (W is a compile-time
// constant so the loop unrolls; with a runtime trip count the first add would stall the warp and serialise the remote loads).
// NVLS: ONE multimem.ld_reduce per 16 bytes on the multicast address - the NVSwitch adds the W copies, so each rank receives its
// shard once instead of W-1 times.
template <typename G, bool NVLS, int W>
__device__ __forceinline__ void fetch_grad8(const PeerPtrs& grads, const void* mc_grad, int world, int rank, int64_t elem, float (&g)[8]) {
    constexpr int Q = sizeof(G) == 2 ? 1 : 2;                         // 16-byte pieces per 8 elements
    if (NVLS) {
        const char* a = reinterpret_cast<const char*>(mc_grad) + elem * sizeof(G);
        if constexpr (sizeof(G) == 2) {
            const uint4 t = multimem_ld_reduce_bf16x8(a);
            const G* h = reinterpret_cast<const G*>(&t);
#pragma unroll
            for (int k = 0; k < 8; ++k) g[k] = Cvt<G>::to(h[k]);
        } else {
            const float4 t0 = multimem_ld_reduce_f32x4(a), t1 = multimem_ld_reduce_f32x4(a + 16);
            g[0] = t0.x; g[1] = t0.y; g[2] = t0.z; g[3] = t0.w; g[4] = t1.x; g[5] = t1.y; g[6] = t1.z; g[7] = t1.w;
        }
        return;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = 0.f;
    if constexpr (W > 0) {
        uint4 raw[W][Q];
#pragma unroll
        for (int kk = 0; kk < W; ++kk) {
            const int r = (rank + kk) % W;                            // a different first peer on every rank
            const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const G*>(grads.p[r]) + elem);
#pragma unroll
            for (int q = 0; q < Q; ++q) raw[kk][q] = src[q];
        }
#pragma unroll
        for (int kk = 0; kk < W; ++kk) {
            const G* h = reinterpret_cast<const G*>(&raw[kk][0]);
#pragma unroll
            for (int k = 0; k < 8; ++k) g[k] += Cvt<G>::to(h[k]);
        }
    } else {
        for (int kk = 0; kk < world; ++kk) {
            const int r = (rank + kk) % world;
            const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const G*>(grads.p[r]) + elem);
            uint4 raw[Q];
#pragma unroll
            for (int q = 0; q < Q; ++q) raw[q] = src[q];
            const G* h = reinterpret_cast<const G*>(&raw[0]);
#pragma unroll
            for (int k = 0; k < 8; ++k) g[k] += Cvt<G>::to(h[k]);
        }
    }
}

// Fused reduce-scatter + optimizer step + all-gather over the flat shard [off, off+n).  U vectors are fetched before the first is
// consumed (memory-level parallelism for the long-latency multimem loads).  NVLS: the updated parameters leave as ONE multimem.st
// per 16 bytes (the switch replicates them to every rank).
template <int OP, typename G, typename T, bool NVLS, int W>
__global__ void __launch_bounds__(256) fused_rs_step_ag_kernel(PeerPtrs grads, PeerPtrs params, const void* mc_grad, void* mc_param,
                                                               int world, int rank, int64_t off, int64_t n, FlatStep st) {
    constexpr int N = 8;
    constexpr int U = NVLS ? 4 : 1;
    const int64_t nv = n / N;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t v0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v0 < nv; v0 += stride * U) {
        float gg[U][N];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t v = v0 + u * stride;
            if (v < nv) fetch_grad8<G, NVLS, W>(grads, mc_grad, world, rank, off + v * N, gg[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t v = v0 + u * stride;
            if (v >= nv) break;
            float (&g)[N] = gg[u];
            float p[N], mm[N], vv[N];
            const int64_t i0 = v * N;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const float4 a = reinterpret_cast<const float4*>(st.master + i0)[q];
                p[4 * q] = a.x; p[4 * q + 1] = a.y; p[4 * q + 2] = a.z; p[4 * q + 3] = a.w;
                const float4 b = reinterpret_cast<const float4*>(st.m + i0)[q];
                mm[4 * q] = b.x; mm[4 * q + 1] = b.y; mm[4 * q + 2] = b.z; mm[4 * q + 3] = b.w;
                if (OP == 0) {
                    const float4 c = reinterpret_cast<const float4*>(st.v + i0)[q];
                    vv[4 * q] = c.x; vv[4 * q + 1] = c.y; vv[4 * q + 2] = c.z; vv[4 * q + 3] = c.w;
                }
            }
#pragma unroll
            for (int k = 0; k < N; ++k) {
                const float gs = g[k] * st.gscale;
                if (OP == 0) p[k] = adam_update(p[k], gs, mm[k], vv[k], st.lr, st.beta1, st.beta2, st.eps, st.wd, st.bc1, st.bc2);
                else         p[k] = lion_update(p[k], gs, mm[k], st.lr, st.beta1, st.beta2, st.wd);
            }
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                reinterpret_cast<float4*>(st.master + i0)[q] = make_float4(p[4 * q], p[4 * q + 1], p[4 * q + 2], p[4 * q + 3]);
                reinterpret_cast<float4*>(st.m + i0)[q] = make_float4(mm[4 * q], mm[4 * q + 1], mm[4 * q + 2], mm[4 * q + 3]);
                if (OP == 0) reinterpret_cast<float4*>(st.v + i0)[q] = make_float4(vv[4 * q], vv[4 * q + 1], vv[4 * q + 2], vv[4 * q + 3]);
            }
            // all-gather: the updated low-precision parameters go straight to every rank's buffer
            uint4 o[2];
            constexpr int QO = sizeof(T) == 2 ? 1 : 2;
            if constexpr (sizeof(T) == 2) {
                T* h = reinterpret_cast<T*>(&o[0]);
#pragma unroll
                for (int k = 0; k < N; ++k) h[k] = Cvt<T>::from(p[k]);
            } else {
                o[0] = make_uint4(__float_as_uint(p[0]), __float_as_uint(p[1]), __float_as_uint(p[2]), __float_as_uint(p[3]));
                o[1] = make_uint4(__float_as_uint(p[4]), __float_as_uint(p[5]), __float_as_uint(p[6]), __float_as_uint(p[7]));
            }
            if (NVLS) {
                char* d = reinterpret_cast<char*>(mc_param) + (off + i0) * sizeof(T);
#pragma unroll
                for (int q = 0; q < QO; ++q) multimem_st_u32x4(d + 16 * q, o[q]);
            } else {
                for (int kk = 0; kk < world; ++kk) {
                    const int r = (rank + kk) % world;
                    uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<T*>(params.p[r]) + off + i0);
#pragma unroll
                    for (int q = 0; q < QO; ++q) d[q] = o[q];
                }
            }
        }
    }
}

// ---- reduce-scatter pull: out[i] = scale * sum_r grad_r[off + i], i in [0, n) ----
// grads.p[r] is rank r's gradient buffer (same layout everywhere).  off is a multiple of 8 elements.
template <typename T, bool NVLS, int W>
__global__ void __launch_bounds__(256) pull_reduce_kernel(PeerPtrs grads, const void* mc_grad, int world, int rank, int64_t off, int64_t n,
                                                          float scale, float* __restrict__ out) {
    constexpr int U = NVLS ? 4 : 1;
    const int64_t nv = n / 8;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t v0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v0 < nv; v0 += stride * U) {
        float g[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (v0 + u * stride < nv) fetch_grad8<T, NVLS, W>(grads, mc_grad, world, rank, off + (v0 + u * stride) * 8, g[u]);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t v = v0 + u * stride;
            if (v >= nv) break;
            float4* o = reinterpret_cast<float4*>(out + v * 8);
            o[0] = make_float4(g[u][0] * scale, g[u][1] * scale, g[u][2] * scale, g[u][3] * scale);
            o[1] = make_float4(g[u][4] * scale, g[u][5] * scale, g[u][6] * scale, g[u][7] * scale);
        }
    }
    // tail (n not a multiple of 8): scalar peer loads
    for (int64_t i = nv * 8 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float a = 0.f;
        for (int r = 0; r < world; ++r) a += Cvt<T>::to(reinterpret_cast<const T*>(grads.p[r])[off + i]);
        out[i] = a * scale;
    }
}

// ---- all-gather fused with the fp32 -> low-precision cast: master[0..n) -> every rank's parameter buffer at element `off` ----
template <typename T>
__global__ void __launch_bounds__(256) cast_push_kernel(PeerPtrs params, int world, int rank, int64_t off, int64_t n,
                                                        const float* __restrict__ master) {
    const int64_t nv = n / 8;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nv; v += (int64_t)gridDim.x * blockDim.x) {
        const float4 a = reinterpret_cast<const float4*>(master)[2 * v], b = reinterpret_cast<const float4*>(master)[2 * v + 1];
        const float p[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        if constexpr (sizeof(T) == 2) {
            uint4 o;
            T* h = reinterpret_cast<T*>(&o);
#pragma unroll
            for (int k = 0; k < 8; ++k) h[k] = Cvt<T>::from(p[k]);
            for (int kk = 0; kk < world; ++kk) {
                const int r = (rank + kk) % world;
                *reinterpret_cast<uint4*>(reinterpret_cast<T*>(params.p[r]) + off + v * 8) = o;
            }
        } else {
            for (int kk = 0; kk < world; ++kk) {
                const int r = (rank + kk) % world;
                float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(params.p[r]) + off + v * 8);
                d[0] = a; d[1] = b;
            }
        }
    }
    for (int64_t i = nv * 8 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        for (int r = 0; r < world; ++r) reinterpret_cast<T*>(params.p[r])[off + i] = Cvt<T>::from(master[i]);
}

// ---- small deterministic all-reduce (sum) through per-rank slots: every rank ends with bitwise identical results ----
// slots.p[r] is rank r's scratch [world][n]; rank `rank` writes its vector into slot `rank` of every peer, a barrier
// follows (separate launch), then reduce_slots sums the slots in rank order.
__global__ void __launch_bounds__(256) scatter_slots_kernel(PeerPtrs slots, int world, int rank, const float* __restrict__ vec, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float x = vec[i];
        for (int r = 0; r < world; ++r) reinterpret_cast<float*>(slots.p[r])[(int64_t)rank * n + i] = x;
    }
}
__global__ void __launch_bounds__(256) reduce_slots_kernel(const float* __restrict__ my_slots, int world, float* __restrict__ out, int n, float scale) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float a = 0.f;
        for (int r = 0; r < world; ++r) a += my_slots[(int64_t)r * n + i];
        out[i] = a * scale;
    }
}

int grid_for(int64_t work_items) {
    const int64_t b = (work_items + 255) / 256;
    const int64_t cap = 148 * 8;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

void dist_barrier(const PeerPtrs& pads, int rank, int world, uint32_t epoch, int* status, unsigned long long timeout_ns, int site, cudaStream_t s) {
    count_launch();
    barrier_kernel<<<1, 32, 0, s>>>(pads, rank, world, epoch, status, timeout_ns, site);
}

void dist_pull_reduce(int dtype, bool nvls, const PeerPtrs& grads, const void* mc, int world, int rank, int64_t off, int64_t n, float scale,
                      float* out, cudaStream_t s) {
    if (n <= 0) return;
    count_launch();
    const int g = grid_for(n / 8);
#define LAUNCH(T) \
    if (nvls) pull_reduce_kernel<T, true, 0><<<g, 256, 0, s>>>(grads, mc, world, rank, off, n, scale, out); \
    else if (world == 8) pull_reduce_kernel<T, false, 8><<<g, 256, 0, s>>>(grads, mc, world, rank, off, n, scale, out); \
    else if (world == 4) pull_reduce_kernel<T, false, 4><<<g, 256, 0, s>>>(grads, mc, world, rank, off, n, scale, out); \
    else if (world == 2) pull_reduce_kernel<T, false, 2><<<g, 256, 0, s>>>(grads, mc, world, rank, off, n, scale, out); \
    else pull_reduce_kernel<T, false, 0><<<g, 256, 0, s>>>(grads, mc, world, rank, off, n, scale, out);
    switch (dtype) { case F32: LAUNCH(float) break; case BF16: LAUNCH(__nv_bfloat16) break; default: LAUNCH(__half) break; }
#undef LAUNCH
}

void dist_push(bool nvls, const PeerPtrs& params, void* mc, int world, int rank, int64_t off_bytes, int64_t n_bytes, cudaStream_t s) {
    if (n_bytes <= 0 || world <= 1) return;
    count_launch();
    const int g = grid_for(n_bytes / 16);
    if (nvls) push_kernel<true><<<g, 256, 0, s>>>(params, mc, world, rank, off_bytes, n_bytes);
    else push_kernel<false><<<g, 256, 0, s>>>(params, mc, world, rank, off_bytes, n_bytes);
}

void dist_fused_flat_step(int op, int gdtype, int pdtype, bool nvls, const PeerPtrs& grads, const PeerPtrs& params, const void* mc_grad,
                          void* mc_param, int world, int rank, int64_t off, int64_t n, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2, float gscale,
                          float* master, float* m, float* v, cudaStream_t s) {
    if (n <= 0) return;
    count_launch();
    FlatStep st{lr, beta1, beta2, eps, wd, bc1, bc2, gscale, master, m, v};
    const int g = grid_for(n / 8);
#define L3(OPV, G, T, NV, WW) fused_rs_step_ag_kernel<OPV, G, T, NV, WW><<<g, 256, 0, s>>>(grads, params, mc_grad, mc_param, world, rank, off, n, st)
#define L2(OPV, G, T) \
    if (nvls) L3(OPV, G, T, true, 0); \
    else if (world == 8) L3(OPV, G, T, false, 8); \
    else if (world == 4) L3(OPV, G, T, false, 4); \
    else if (world == 2) L3(OPV, G, T, false, 2); \
    else L3(OPV, G, T, false, 0)
#define L1(OPV) \
    if (gdtype == BF16 && pdtype == BF16) { L2(OPV, __nv_bfloat16, __nv_bfloat16); } \
    else if (gdtype == F32 && pdtype == BF16) { L2(OPV, float, __nv_bfloat16); } \
    else if (gdtype == F32 && pdtype == F32) { L2(OPV, float, float); } \
    else { L2(OPV, __nv_bfloat16, float); }
    if (op == 0) { L1(0) } else { L1(1) }
#undef L1
#undef L2
#undef L3
}

void dist_cast_push(int pdtype, const PeerPtrs& params, int world, int rank, int64_t off, int64_t n, const float* master, cudaStream_t s) {
    if (n <= 0) return;
    count_launch();
    const int g = grid_for(n / 8);
    switch (pdtype) {
        case F32:  cast_push_kernel<float><<<g, 256, 0, s>>>(params, world, rank, off, n, master); break;
        case BF16: cast_push_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(params, world, rank, off, n, master); break;
        default:   cast_push_kernel<__half><<<g, 256, 0, s>>>(params, world, rank, off, n, master); break;
    }
}

void dist_scatter_slots(const PeerPtrs& slots, int world, int rank, const float* vec, int n, cudaStream_t s) {
    if (n > 0) count_launch();
    if (n > 0) scatter_slots_kernel<<<grid_for(n), 256, 0, s>>>(slots, world, rank, vec, n);
}
void dist_reduce_slots(const float* my_slots, int world, float* out, int n, float scale, cudaStream_t s) {
    if (n > 0) count_launch();
    if (n > 0) reduce_slots_kernel<<<grid_for(n), 256, 0, s>>>(my_slots, world, out, n, scale);
}

}  // namespace sg
