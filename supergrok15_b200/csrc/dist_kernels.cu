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
#include <cstdlib>
#include "comm.cuh"
#include "optim_math.cuh"
#include "peer_fetch.cuh"

namespace sg {
namespace {

// ---- barrier: rank r publishes `epoch` in slot r of every pad, then waits for all slots of its own pad ----
// The epoch is `epoch` itself, or, when `dyn` is given, the step's base epoch in the device table of step scalars plus `epoch`:
// a barrier captured in a CUDA graph then advances with every replay (the host rewrites the table before each one).
// A rank whose status word already records a timeout still publishes its epoch (its peers are not held up) but does not wait.
__global__ void barrier_kernel(PeerPtrs pads, int rank, int world, uint32_t epoch, const uint32_t* __restrict__ dyn, int* status,
                               unsigned long long timeout_ns, int site) {
    const int r = threadIdx.x;
    if (dyn) epoch += dyn[DYN_EPOCH];
    if (r < world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t*>(pads.p[r]) + rank, epoch);
        const bool failed = (*reinterpret_cast<volatile int*>(status) & 0xff) != STATUS_OK;
        if (!failed && !wait_flag_ge(reinterpret_cast<uint32_t*>(pads.p[rank]) + r, epoch, timeout_ns))
            atomicCAS(status, STATUS_OK, STATUS_TIMEOUT | (r << 8) | (site << 16));
        __threadfence_system();
    }
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
    const float* dyn;                       // optional device table: lr at DYN_LR, bc1 / bc2 at DYN_TS + 2 / + 3 (CUDA-graph replays)
};

template <typename G, typename T> struct VecN { static constexpr int value = (sizeof(G) == 2 && sizeof(T) == 2) ? 8 : 4; };

// Fused reduce-scatter + optimizer step + all-gather over the flat shard [off, off+n).  NVLS: the updated parameters leave as ONE
// multimem.st per 16 bytes (the switch replicates them to every rank); NVLS needs 16-byte vectors of both buffers (same dtype).
template <int OP, typename G, typename T, bool NVLS, int W, int U>
__global__ void __launch_bounds__(256) fused_rs_step_ag_kernel(PeerPtrs grads, PeerPtrs params, const void* mc_grad, void* mc_param,
                                                               int world, int rank, int64_t off, int64_t n, FlatStep st, int n_push) {
    constexpr int N = VecN<G, T>::value;
    const int64_t nv = n / N;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (st.dyn) { st.lr = st.dyn[DYN_LR]; st.bc1 = st.dyn[DYN_TS + 2]; st.bc2 = st.dyn[DYN_TS + 3]; }
    for (int64_t v0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v0 < nv; v0 += stride * U) {
        // local state first, remote gradients second: every load of this iteration is in flight before the first use stalls the warp
        float pp[U][N], ms[U][N], vs[U][N], gg[U][N];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t v = v0 + u * stride;
            if (v >= nv) continue;
            const int64_t i0 = v * N;
#pragma unroll
            for (int q = 0; q < N / 4; ++q) {
                const float4 a = __ldcs(reinterpret_cast<const float4*>(st.master + i0) + q);
                pp[u][4 * q] = a.x; pp[u][4 * q + 1] = a.y; pp[u][4 * q + 2] = a.z; pp[u][4 * q + 3] = a.w;
                const float4 b = __ldcs(reinterpret_cast<const float4*>(st.m + i0) + q);
                ms[u][4 * q] = b.x; ms[u][4 * q + 1] = b.y; ms[u][4 * q + 2] = b.z; ms[u][4 * q + 3] = b.w;
                if (OP == 0) {
                    const float4 c = __ldcs(reinterpret_cast<const float4*>(st.v + i0) + q);
                    vs[u][4 * q] = c.x; vs[u][4 * q + 1] = c.y; vs[u][4 * q + 2] = c.z; vs[u][4 * q + 3] = c.w;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t v = v0 + u * stride;
            if (v < nv) fetch_grad<G, N, NVLS, W>(grads, mc_grad, world, rank, off + v * N, gg[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t v = v0 + u * stride;
            if (v >= nv) break;
            float (&g)[N] = gg[u];
            float (&p)[N] = pp[u];
            float (&mm)[N] = ms[u];
            float (&vv)[N] = vs[u];
            const int64_t i0 = v * N;
#pragma unroll
            for (int k = 0; k < N; ++k) {
                const float gs = g[k] * st.gscale;
                if (OP == 0) p[k] = adam_update(p[k], gs, mm[k], vv[k], st.lr, st.beta1, st.beta2, st.eps, st.wd, st.bc1, st.bc2);
                else         p[k] = lion_update(p[k], gs, mm[k], st.lr, st.beta1, st.beta2, st.wd);
            }
#pragma unroll
            for (int q = 0; q < N / 4; ++q) {
                __stcs(reinterpret_cast<float4*>(st.master + i0) + q, make_float4(p[4 * q], p[4 * q + 1], p[4 * q + 2], p[4 * q + 3]));
                __stcs(reinterpret_cast<float4*>(st.m + i0) + q, make_float4(mm[4 * q], mm[4 * q + 1], mm[4 * q + 2], mm[4 * q + 3]));
                if (OP == 0) __stcs(reinterpret_cast<float4*>(st.v + i0) + q, make_float4(vv[4 * q], vv[4 * q + 1], vv[4 * q + 2], vv[4 * q + 3]));
            }
            // all-gather: the updated parameters go straight to every rank's buffer
            uint4 o;
            vpack<T, N>(p, o);
            // n_push = world: every rank's buffer (all-gather fused into the step); n_push = 1: only this rank's own buffer (the
            // peers fetch these rows from inside the first GEMM that consumes the weight)
            if (NVLS && sizeof(T) * N == 16 && n_push == world) {
                multimem_st_u32x4(reinterpret_cast<char*>(mc_param) + (off + i0) * sizeof(T), o);
            } else {
                for (int kk = 0; kk < n_push; ++kk)
                    vstore_packed<T, N>(reinterpret_cast<T*>(params.p[(rank + kk) % world]) + off + i0, o);
            }
        }
    }
}

// ---- reduce-scatter pull: out[i] = scale * sum_r grad_r[off + i], i in [0, n) ----
// grads.p[r] is rank r's gradient buffer (same layout everywhere).  off is a multiple of 8 elements.
template <typename T, bool NVLS, int W>
__global__ void __launch_bounds__(256) pull_reduce_kernel(PeerPtrs grads, const void* mc_grad, int world, int rank, int64_t off, int64_t n,
                                                          float scale, float* __restrict__ out) {
    constexpr int N = 16 / sizeof(T);
    constexpr int U = NVLS ? 4 : 2;
    const int64_t nv = n / N;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t v0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v0 < nv; v0 += stride * U) {
        float g[U][N];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (v0 + u * stride < nv) fetch_grad<T, N, NVLS, W>(grads, mc_grad, world, rank, off + (v0 + u * stride) * N, g[u]);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t v = v0 + u * stride;
            if (v >= nv) break;
#pragma unroll
            for (int q = 0; q < N / 4; ++q)
                __stcs(reinterpret_cast<float4*>(out + v * N) + q, make_float4(g[u][4 * q] * scale, g[u][4 * q + 1] * scale, g[u][4 * q + 2] * scale, g[u][4 * q + 3] * scale));
        }
    }
    // tail (n not a multiple of the vector): scalar peer loads
    for (int64_t i = nv * N + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float a = 0.f;
        for (int r = 0; r < world; ++r) a += Cvt<T>::to(reinterpret_cast<const T*>(grads.p[r])[off + i]);
        out[i] = a * scale;
    }
}

// ---- all-gather fused with the fp32 -> low-precision cast: master[0..n) -> every rank's parameter buffer at element `off` ----
template <typename T>
__global__ void __launch_bounds__(256) cast_push_kernel(PeerPtrs params, int world, int rank, int64_t off, int64_t n,
                                                        const float* __restrict__ master) {
    constexpr int N = 16 / sizeof(T);                    // one 16-byte store per lane and destination
    const int64_t nv = n / N;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nv; v += (int64_t)gridDim.x * blockDim.x) {
        float p[N];
#pragma unroll
        for (int q = 0; q < N / 4; ++q) {
            const float4 a = __ldcs(reinterpret_cast<const float4*>(master + v * N) + q);
            p[4 * q] = a.x; p[4 * q + 1] = a.y; p[4 * q + 2] = a.z; p[4 * q + 3] = a.w;
        }
        uint4 o;
        vpack<T, N>(p, o);
        for (int kk = 0; kk < world; ++kk)
            vstore_packed<T, N>(reinterpret_cast<T*>(params.p[(rank + kk) % world]) + off + v * N, o);
    }
    for (int64_t i = nv * N + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
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

// one thread: *p += 1.  The call counters of the fused GEMMs and the epoch of the barriers live in device memory when the sequence
// is replayed from a CUDA graph; this kernel, captured in the same graph, advances them.
__global__ void bump_kernel(int* p) { *p += 1; }

int grid_for(int64_t work_items) {
    const int64_t b = (work_items + 255) / 256;
    const int64_t cap = 148 * 8;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

void dist_bump(int* counter, cudaStream_t s) {
    count_launch();
    bump_kernel<<<1, 1, 0, s>>>(counter);
}

void dist_barrier(const PeerPtrs& pads, int rank, int world, uint32_t epoch, const uint32_t* dyn, int* status, unsigned long long timeout_ns,
                  int site, cudaStream_t s) {
    count_launch();
    barrier_kernel<<<1, 32, 0, s>>>(pads, rank, world, epoch, dyn, status, timeout_ns, site);
}

void dist_pull_reduce(int dtype, bool nvls, const PeerPtrs& grads, const void* mc, int world, int rank, int64_t off, int64_t n, float scale,
                      float* out, cudaStream_t s) {
    if (n <= 0) return;
    count_launch();
    const int g = grid_for(n / 4);
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
                          float* master, float* m, float* v, const float* dyn, bool push, cudaStream_t s) {
    if (n <= 0) return;
    const int n_push = push ? world : 1;
    count_launch();
    FlatStep st{lr, beta1, beta2, eps, wd, bc1, bc2, gscale, master, m, v, dyn};
    if (nvls && gdtype != pdtype) nvls = false;              // the multimem path needs 16-byte vectors of both buffers
    // Tuning knobs (read once): vectors in flight per thread and CTAs per SM of the grid.
    static const int unroll = [] { const char* e = getenv("SG_FUSED_UNROLL"); const int u = e ? atoi(e) : 0; return (u == 1 || u == 2 || u == 4) ? u : 0; }();
    static const int ctas = [] { const char* e = getenv("SG_FUSED_CTAS"); const int c = e ? atoi(e) : 0; return (c >= 1 && c <= 32) ? c : 8; }();
    const int u_sel = unroll ? unroll : (nvls ? 4 : 2);
    const int64_t want = (n / 4 + 255) / 256;
    const int g = (int)(want < 1 ? 1 : (want > 148LL * ctas ? 148LL * ctas : want));
#define L4(OPV, G, T, NV, WW, UU) fused_rs_step_ag_kernel<OPV, G, T, NV, WW, UU><<<g, 256, 0, s>>>(grads, params, mc_grad, mc_param, world, rank, off, n, st, n_push)
#define L3(OPV, G, T, NV, WW) \
    if (u_sel == 4) L4(OPV, G, T, NV, WW, 4); else if (u_sel == 2) L4(OPV, G, T, NV, WW, 2); else L4(OPV, G, T, NV, WW, 1)
#define L2(OPV, G, T) \
    if (nvls) { L3(OPV, G, T, true, 0); } \
    else if (world == 8) { L3(OPV, G, T, false, 8); } \
    else if (world == 4) { L3(OPV, G, T, false, 4); } \
    else if (world == 2) { L3(OPV, G, T, false, 2); } \
    else { L3(OPV, G, T, false, 0); }
#define L1(OPV) \
    if (gdtype == BF16 && pdtype == BF16) { L2(OPV, __nv_bfloat16, __nv_bfloat16); } \
    else if (gdtype == F32 && pdtype == BF16) { L2(OPV, float, __nv_bfloat16); } \
    else if (gdtype == F32 && pdtype == F32) { L2(OPV, float, float); } \
    else { L2(OPV, __nv_bfloat16, float); }
    if (op == 0) { L1(0) } else { L1(1) }
#undef L1
#undef L2
#undef L3
#undef L4
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
