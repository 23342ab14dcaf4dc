// Multi-tensor element-wise optimizer kernels for sm_100a.
//
// One launch covers every tensor of a parameter group: the launch descriptor (pointer tables,
// sizes, per-tensor scalars, CTA ranges) travels as a kernel parameter.  Global scalars that
// the reference fetches to the host between kernels (clip coefficient, Prodigy d_lr, cosine
// gates, SAM scale; reference csrc/ops.cpp:23-76, 449-478, 619, 644) are produced by a
// reduction kernel and read back from device memory by the step kernel, so a step never
// synchronises the host.  Reductions are two-stage with a fixed summation order (no float
// atomics): results are bitwise reproducible run to run.
#include "sg_native.h"
#include "optim_math.cuh"
#include <atomic>

namespace sg {

namespace {

#ifdef GROK_BOUNDS_CHECK
// Checked build (-DGROK_BOUNDS_CHECK, this file only): every element access of the multi-tensor kernel is compared with the
// number of bytes that are really addressable from its base pointer.  That extent does not come from the launch descriptor (which
// is what is being checked) but from the driver: before a launch the host asks cuMemGetAddressRange for the allocation that
// holds each pointer and uploads "end of allocation - pointer" to g_extent.  An access past it is NOT made: the lanes read zeros /
// drop the store, and the first violation is recorded in g_viol {count, op, role, tensor, index low 31 bits, index >> 31, 1 =
// store}.  Nothing traps and the context stays usable.  With PyTorch's caching allocator an allocation is a whole segment, so
// the check is exact only under PYTORCH_NO_CUDA_MEMORY_CACHING=1 (one cudaMalloc per tensor).
__device__ unsigned long long g_extent[MT_NP][MT_MAX];
__device__ int g_viol[8];

struct CPtr {
    void* p; unsigned long long bytes; int role, t, op;
    __device__ __forceinline__ operator void*() const { return p; }
};

__device__ __forceinline__ bool checked_ok(const CPtr& P, int64_t i, int cnt, size_t esz, int store) {
    if (P.bytes == 0 || (unsigned long long)(i + cnt) * esz <= P.bytes) return true;        // 0: extent unknown (not a device allocation)
    if (atomicAdd(&g_viol[0], 1) == 0) {
        g_viol[1] = P.op; g_viol[2] = P.role; g_viol[3] = P.t; g_viol[4] = (int)(i & 0x7fffffff); g_viol[5] = (int)(i >> 31); g_viol[6] = store;
    }
    return false;
}

template <typename T>
__device__ __forceinline__ void ld4(const CPtr& P, int64_t i, int cnt, bool vec, float v[4]) {
    if (checked_ok(P, i, cnt, sizeof(T), 0)) { sg::ld4<T>((const void*)P.p, i, cnt, vec, v); return; }
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = 0.f;
}

template <typename T>
__device__ __forceinline__ void st4(const CPtr& P, int64_t i, int cnt, bool vec, const float v[4]) {
    if (checked_ok(P, i, cnt, sizeof(T), 1)) sg::st4<T>((void*)P.p, i, cnt, vec, v);
}
#define MT_PTR(r) CPtr{a.ptr[r][t], g_extent[r][t], r, t, OP}
#else
#define MT_PTR(r) a.ptr[r][t]
#endif

struct Loc { int t; int64_t begin, end; };

__device__ __forceinline__ Loc locate(const MTArgs& a) {
    int lo = 0, hi = a.n;                     // find t with blk_start[t] <= blockIdx.x < blk_start[t+1]
    const int b = blockIdx.x;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (a.blk_start[mid] <= b) lo = mid; else hi = mid;
    }
    Loc l;
    l.t = lo;
    l.begin = (int64_t)(b - a.blk_start[lo]) * MT_CHUNK;
    const int64_t n = a.numel[lo];
    l.end = (l.begin + MT_CHUNK < n) ? l.begin + MT_CHUNK : n;
    return l;
}

template <int OP, typename T>
__global__ void __launch_bounds__(MT_THREADS) mt_kernel(const __grid_constant__ MTArgs a,
                                                        const __grid_constant__ MTParams prm) {
    __shared__ float red[32];
    extern __shared__ float smem[];           // MLP weights (SG15 / SG11_A / NEURALGROK)
    const Loc L = locate(a);
    const int t = L.t;
    const auto P0 = MT_PTR(0); const auto P1 = MT_PTR(1); const auto P2 = MT_PTR(2); const auto P3 = MT_PTR(3);
    const auto P4 = MT_PTR(4); const auto P5 = MT_PTR(5);
    const float ts0 = a.ts[t][0], ts1 = a.ts[t][1], ts2 = a.ts[t][2], ts3 = a.ts[t][3];
    const float clip = prm.clip ? *prm.clip : 1.f;
    const int H = prm.hidden;
    float b2s = 0.f;
    if constexpr (OP == OP_SG15 || OP == OP_SG11_A) {
        for (int i = threadIdx.x; i < 2 * H; i += MT_THREADS) smem[i] = prm.W1[i];
        for (int i = threadIdx.x; i < H; i += MT_THREADS) { smem[2 * H + i] = prm.b1[i]; smem[3 * H + i] = prm.W2[i]; }
        b2s = prm.b2[0];
        __syncthreads();
    }
    if constexpr (OP == OP_NEURALGROK) {
        for (int i = threadIdx.x; i < H; i += MT_THREADS) {
            smem[i] = prm.W1[i]; smem[H + i] = prm.b1[i]; smem[2 * H + i] = prm.W2[i];
        }
        b2s = prm.b2[0];
        __syncthreads();
    }
    const bool vT = vec_ok<T>(P0) && vec_ok<T>(P1);
    const bool vF = vec_ok<float>(P2) && vec_ok<float>(P3) && vec_ok<float>(P4) && vec_ok<float>(P5) &&
                    vec_ok<float>(P0) && vec_ok<float>(P1);
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f;
    const float lr = prm.lr, b1 = prm.beta1, b2 = prm.beta2, eps = prm.eps, wd = prm.wd;

    for (int64_t i = L.begin + (int64_t)threadIdx.x * 4; i < L.end; i += MT_THREADS * 4) {
        const int cnt = (L.end - i >= 4) ? 4 : (int)(L.end - i);
        float p[4], g[4], x2[4], x3[4], x4[4], x5[4];
        if constexpr (OP == OP_ADAMW) {
            ld4<T>(P0, i, cnt, vT, p); ld4<T>(P1, i, cnt, vT, g); ld4<float>(P2, i, cnt, vF, x2); ld4<float>(P3, i, cnt, vF, x3);
#pragma unroll
            for (int k = 0; k < 4; ++k) p[k] = adam_update(p[k], g[k] * clip, x2[k], x3[k], lr, b1, b2, eps, wd, ts0, ts1);
            st4<T>(P0, i, cnt, vT, p); st4<float>(P2, i, cnt, vF, x2); st4<float>(P3, i, cnt, vF, x3);
        } else if constexpr (OP == OP_LION) {
            ld4<T>(P0, i, cnt, vT, p); ld4<T>(P1, i, cnt, vT, g); ld4<float>(P2, i, cnt, vF, x2);
#pragma unroll
            for (int k = 0; k < 4; ++k) p[k] = lion_update(p[k], g[k] * clip, x2[k], lr, b1, b2, wd);
            st4<T>(P0, i, cnt, vT, p); st4<float>(P2, i, cnt, vF, x2);
        } else if constexpr (OP == OP_GROKFAST_EMA) {
            ld4<T>(P1, i, cnt, vT, g); ld4<float>(P2, i, cnt, vF, x2);
#pragma unroll
            for (int k = 0; k < 4; ++k) { x2[k] = prm.alpha * x2[k] + (1.f - prm.alpha) * g[k]; g[k] += prm.lamb * x2[k]; }
            st4<T>(P1, i, cnt, vT, g); st4<float>(P2, i, cnt, vF, x2);
        } else if constexpr (OP == OP_GROKFAST_ADAMW || OP == OP_GROKADAMW) {
            ld4<T>(P0, i, cnt, vT, p); ld4<T>(P1, i, cnt, vT, g); ld4<float>(P2, i, cnt, vF, x2); ld4<float>(P3, i, cnt, vF, x3);
            ld4<float>(P4, i, cnt, vF, x4);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float gg = g[k] * clip;
                x4[k] = prm.alpha * x4[k] + (1.f - prm.alpha) * gg;
                const float am = gg + prm.lamb * x4[k];
                if constexpr (OP == OP_GROKFAST_ADAMW) {
                    // the amplified gradient is rounded to the gradient dtype before Adam reads it,
                    // as in the two-kernel reference sequence (grokfast.py:124-132)
                    g[k] = Cvt<T>::to(Cvt<T>::from(am));
                    p[k] = adam_update(p[k], g[k], x2[k], x3[k], lr, b1, b2, eps, wd, ts0, ts1);
                } else {
                    g[k] = gg;
                    p[k] = adam_update(p[k], am, x2[k], x3[k], lr, b1, b2, eps, wd, ts0, ts1);
                }
            }
            st4<T>(P0, i, cnt, vT, p); st4<float>(P2, i, cnt, vF, x2); st4<float>(P3, i, cnt, vF, x3); st4<float>(P4, i, cnt, vF, x4);
            if (prm.write_grad) st4<T>(P1, i, cnt, vT, g);
        } else if constexpr (OP == OP_PRODIGY) {
            const float d = prm.dscal[0];
            ld4<T>(P0, i, cnt, vT, p); ld4<T>(P1, i, cnt, vT, g); ld4<float>(P2, i, cnt, vF, x2); ld4<float>(P3, i, cnt, vF, x3);
            ld4<float>(P4, i, cnt, vF, x4);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float dg = d * g[k];
                x4[k] = b2 * x4[k] + (1.f - b2) * dg * dg;
                x2[k] = b1 * x2[k] + (1.f - b1) * dg;
                x3[k] = b2 * x3[k] + (1.f - b2) * dg * dg;
                p[k] = p[k] * (1.f - lr * d * wd) - (lr / ts0) * x2[k] / (sqrtf(x3[k] / ts1) + d * eps);
            }
            st4<T>(P0, i, cnt, vT, p); st4<float>(P2, i, cnt, vF, x2); st4<float>(P3, i, cnt, vF, x3); st4<float>(P4, i, cnt, vF, x4);
        } else if constexpr (OP == OP_NEURALGROK) {
            ld4<T>(P0, i, cnt, vT, p); ld4<T>(P1, i, cnt, vT, g); ld4<float>(P2, i, cnt, vF, x2); ld4<float>(P3, i, cnt, vF, x3);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                g[k] *= clip;
                const float ag = g[k] * (prm.alpha * amp_mlp(g[k], smem, smem + H, smem + 2 * H, b2s, H) + prm.rescale);
                p[k] = adam_update(p[k], ag, x2[k], x3[k], lr, b1, b2, eps, wd, ts0, ts1);
            }
            st4<T>(P0, i, cnt, vT, p); st4<float>(P2, i, cnt, vF, x2); st4<float>(P3, i, cnt, vF, x3);
            if (prm.write_grad) st4<T>(P1, i, cnt, vT, g);
        } else if constexpr (OP == OP_SG15) {
            ld4<T>(P0, i, cnt, vT, p); ld4<T>(P1, i, cnt, vT, g); ld4<float>(P2, i, cnt, vF, x2); ld4<float>(P3, i, cnt, vF, x3);
            ld4<float>(P4, i, cnt, vF, x4); ld4<float>(P5, i, cnt, vF, x5);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                g[k] *= clip;
                x4[k] = ts0 * x4[k] + (1.f - ts0) * g[k];
                const float sgd = g[k] + prm.rescale * sharp_mlp(g[k], x5[k], smem, smem + 2 * H, smem + 3 * H, b2s, H);
                const float fg = sgd + prm.lamb * x4[k];
                p[k] = adam_update(p[k], fg, x2[k], x3[k], lr, ts1, b2, eps, wd, ts2, ts3);
            }
            st4<T>(P0, i, cnt, vT, p); st4<float>(P2, i, cnt, vF, x2); st4<float>(P3, i, cnt, vF, x3); st4<float>(P4, i, cnt, vF, x4);
            if (prm.write_grad) st4<T>(P1, i, cnt, vT, g);
        } else if constexpr (OP == OP_SG11_A) {
            ld4<T>(P1, i, cnt, vT, g); ld4<float>(P2, i, cnt, vF, x2); ld4<float>(P3, i, cnt, vF, x3);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                g[k] *= clip;
                x2[k] = ts0 * x2[k] + (1.f - ts0) * g[k];
                x4[k] = g[k] + prm.rescale * sharp_mlp(g[k], x3[k], smem, smem + 2 * H, smem + 3 * H, b2s, H);
                if (k < cnt) { acc0 = fmaf(x4[k], x2[k], acc0); acc1 = fmaf(x4[k], x4[k], acc1); acc2 = fmaf(x2[k], x2[k], acc2); }
            }
            st4<float>(P2, i, cnt, vF, x2); st4<float>(P4, i, cnt, vF, x4);
            if (prm.write_grad) st4<T>(P1, i, cnt, vT, g);
        } else if constexpr (OP == OP_SG11_B) {
            const float lamb_eff = prm.tscal[a.t_off + t];
            ld4<T>(P0, i, cnt, vT, p); ld4<float>(P1, i, cnt, vF, g); ld4<float>(P2, i, cnt, vF, x2); ld4<float>(P3, i, cnt, vF, x3);
            ld4<float>(P4, i, cnt, vF, x4);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                p[k] = adam_update(p[k], g[k] + lamb_eff * x4[k], x2[k], x3[k], lr, ts0, b2, eps, wd, ts1, ts2);
            st4<T>(P0, i, cnt, vT, p); st4<float>(P2, i, cnt, vF, x2); st4<float>(P3, i, cnt, vF, x3);
        } else if constexpr (OP == OP_PERTURB) {
            const float sc = prm.dscal[0];
            ld4<T>(P0, i, cnt, vT, p); ld4<T>(P1, i, cnt, vT, g);
            st4<float>(P2, i, cnt, vF, p);
#pragma unroll
            for (int k = 0; k < 4; ++k) p[k] = fmaf(sc, g[k], p[k]);
            st4<T>(P0, i, cnt, vT, p);
        } else if constexpr (OP == OP_RESTORE) {
            ld4<float>(P2, i, cnt, vF, x2);
            st4<T>(P0, i, cnt, vT, x2);
        } else if constexpr (OP == OP_SHARP_RESTORE) {
            ld4<T>(P1, i, cnt, vT, g); ld4<float>(P2, i, cnt, vF, x2); ld4<T>(P3, i, cnt, vec_ok<T>(P3), x3);
#pragma unroll
            for (int k = 0; k < 4; ++k) x4[k] = fabsf(x3[k] - g[k]);
            st4<float>(P4, i, cnt, vF, x4); st4<T>(P0, i, cnt, vT, x2);
        } else if constexpr (OP == OP_LOOKSAM_DIR) {
            const float inv = prm.tscal[2 * (a.t_off + t)];
            if (inv > 0.f) {
                ld4<T>(P1, i, cnt, vT, g); ld4<T>(P3, i, cnt, vec_ok<T>(P3), x3);
#pragma unroll
                for (int k = 0; k < 4; ++k) x2[k] = (x3[k] - g[k]) * inv;
                st4<float>(P2, i, cnt, vF, x2);
            }
        } else if constexpr (OP == OP_LOOKSAM_ADJ) {
            const float gn = prm.tscal[2 * (a.t_off + t) + 1];
            ld4<T>(P1, i, cnt, vT, g); ld4<float>(P2, i, cnt, vF, x2);
#pragma unroll
            for (int k = 0; k < 4; ++k) g[k] = fmaf(prm.alpha * gn, x2[k], g[k]);
            st4<T>(P1, i, cnt, vT, g);
        } else if constexpr (OP == OP_MUON_MOMENTUM) {
            ld4<T>(P1, i, cnt, vT, g); ld4<float>(P2, i, cnt, vF, x2);
#pragma unroll
            for (int k = 0; k < 4; ++k) { x2[k] = fmaf(prm.alpha, x2[k], g[k]); if (k < cnt) acc0 = fmaf(x2[k], x2[k], acc0); }
            st4<float>(P2, i, cnt, vF, x2);
        } else if constexpr (OP == OP_MUON_UPDATE) {
            ld4<T>(P0, i, cnt, vT, p); ld4<float>(P1, i, cnt, vF, g);
#pragma unroll
            for (int k = 0; k < 4; ++k) p[k] = fmaf(prm.extra0, g[k], p[k]) * prm.extra1;
            st4<T>(P0, i, cnt, vT, p);
        } else if constexpr (OP == OP_SCALE) {
            const float sc = prm.dscal ? prm.dscal[0] : prm.extra0;
            ld4<T>(P1, i, cnt, vT, g);
#pragma unroll
            for (int k = 0; k < 4; ++k) g[k] *= sc;
            st4<T>(P1, i, cnt, vT, g);
        } else if constexpr (OP == OP_SQNORM) {
            ld4<T>(P1, i, cnt, vT, g);
#pragma unroll
            for (int k = 0; k < 4; ++k) acc0 = fmaf(g[k], g[k], acc0);
        } else if constexpr (OP == OP_PRODIGY_REDUCE) {
            ld4<T>(P0, i, cnt, vT, p); ld4<T>(P1, i, cnt, vT, g); ld4<float>(P2, i, cnt, vF, x2); ld4<float>(P3, i, cnt, vF, x3);
#pragma unroll
            for (int k = 0; k < 4; ++k) { acc0 = fmaf(g[k], p[k] - x2[k], acc0); acc1 += x3[k]; }
        } else if constexpr (OP == OP_DIFF_SQNORM) {
            ld4<T>(P1, i, cnt, vT, g); ld4<T>(P2, i, cnt, vec_ok<T>(P2), x2);
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float d = x2[k] - g[k]; acc0 = fmaf(d, d, acc0); acc1 = fmaf(g[k], g[k], acc1); }
        }
    }
    if constexpr (OP == OP_SG11_A || OP == OP_MUON_MOMENTUM || OP == OP_SQNORM || OP == OP_PRODIGY_REDUCE ||
                  OP == OP_DIFF_SQNORM) {
        const float r0 = block_sum(acc0, red);
        const float r1 = block_sum(acc1, red);
        const float r2 = block_sum(acc2, red);
        if (threadIdx.x == 0) {
            float* o = prm.partials + 3 * (int64_t)(a.blk_off + blockIdx.x);
            o[0] = r0; o[1] = r1; o[2] = r2;
        }
    }
}

template <int OP>
void launch_typed(int dtype, const MTArgs& a, const MTParams& p, cudaStream_t s) {
    const int blocks = a.blk_start[a.n];
    if (blocks <= 0) return;
    size_t sm = 0;
    if (OP == OP_SG15 || OP == OP_SG11_A) sm = (size_t)(4 * p.hidden) * sizeof(float);
    if (OP == OP_NEURALGROK) sm = (size_t)(3 * p.hidden) * sizeof(float);
    switch (dtype) {
        case F32:  mt_kernel<OP, float><<<blocks, MT_THREADS, sm, s>>>(a, p); break;
        case BF16: mt_kernel<OP, __nv_bfloat16><<<blocks, MT_THREADS, sm, s>>>(a, p); break;
        default:   mt_kernel<OP, __half><<<blocks, MT_THREADS, sm, s>>>(a, p); break;
    }
}

__global__ void finalize_per_tensor_kernel(const __grid_constant__ MTArgs a, const float* __restrict__ partials,
                                           float* __restrict__ out) {
    const int t = blockIdx.x;
    const int b0 = a.blk_start[t], b1 = a.blk_start[t + 1];
    float s0 = 0.f, s1 = 0.f, s2 = 0.f;
    for (int b = b0 + threadIdx.x; b < b1; b += 32) {
        const float* q = partials + 3 * (int64_t)(a.blk_off + b);
        s0 += q[0]; s1 += q[1]; s2 += q[2];
    }
    s0 = warp_sum(s0); s1 = warp_sum(s1); s2 = warp_sum(s2);
    if (threadIdx.x == 0) {
        float* o = out + 3 * (int64_t)(a.t_off + t);
        o[0] = s0; o[1] = s1; o[2] = s2;
    }
}

__global__ void scalar_finalize_kernel(int op, const float* __restrict__ pt, int n, float* __restrict__ out, float a0,
                                       float a1, float a2) {
    // one warp; per-tensor entries are summed lane-strided then tree-reduced (fixed order)
    const int lane = threadIdx.x;
    if (op == SC_CLIP || op == SC_SAM_SCALE || op == SC_PRODIGY || op == SC_SUM3) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f;
        for (int t = lane; t < n; t += 32) { s0 += pt[3 * t]; s1 += pt[3 * t + 1]; s2 += pt[3 * t + 2]; }
        s0 = warp_sum(s0); s1 = warp_sum(s1); s2 = warp_sum(s2);
        if (lane == 0 && op == SC_SUM3) { out[0] = s0; out[1] = s1; out[2] = s2; }
        if (lane == 0 && op != SC_SUM3) {
            if (op == SC_CLIP) {
                const float norm = sqrtf(s0);
                out[0] = s0; out[1] = (norm > a0) ? a0 / (norm + 1e-6f) : 1.f; out[2] = norm;
            } else if (op == SC_SAM_SCALE) {
                out[0] = a0 / (sqrtf(s0) + 1e-12f);
            } else {
                float d = out[0];
                if (s1 > 1e-30f) d = fmaxf(d, fabsf(s0) / (s1 + 1e-12f));
                out[0] = d;
            }
        }
    } else {
        for (int t = lane; t < n; t += 32) {
            if (op == SC_SG11_GATES) {
                const float cosv = pt[3 * t] / (sqrtf(pt[3 * t + 1]) * sqrtf(pt[3 * t + 2]) + 1e-8f);
                const float gate = 1.f / (1.f + expf(-a0 * cosv));
                out[t] = (a1 > 0.f) ? a1 * gate * a2 : 0.f;          // a0 temperature, a1 ramp, a2 lambda
                out[n + t] = gate;
            } else if (op == SC_LOOKSAM_NORMS) {
                const float dn = sqrtf(pt[3 * t]);
                out[2 * t] = (dn < 1e-12f) ? 0.f : 1.f / dn;
                out[2 * t + 1] = sqrtf(pt[3 * t + 1]);
            } else if (op == SC_MUON_NORMS) {
                out[t] = 1.f / (sqrtf(pt[3 * t]) + 1e-7f);
            } else if (op == SC_SG2_CLIP) {
                const float norm = sqrtf(pt[3 * t]);
                out[t] = (norm > a0) ? a0 / (norm + 1e-12f) : 1.f;
            }
        }
    }
}

}  // namespace

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

#ifdef GROK_BOUNDS_CHECK
namespace {
using AddressRangeFn = int (*)(unsigned long long*, size_t*, unsigned long long);
long long g_cap = -1;                                  // test hook: upper limit on every extent (bytes), -1 = none

AddressRangeFn address_range_fn() {
    static AddressRangeFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
        return (AddressRangeFn)f;
    }();
    return fn;
}

unsigned long long extent_of(const void* ptr) {
    AddressRangeFn fn = address_range_fn();
    unsigned long long base = 0;
    size_t size = 0;
    if (!ptr || !fn || fn(&base, &size, (unsigned long long)(uintptr_t)ptr) != 0) return 0;
    unsigned long long e = base + size - (unsigned long long)(uintptr_t)ptr;
    if (g_cap >= 0 && e > (unsigned long long)g_cap) e = (unsigned long long)g_cap;
    return e;
}

// The table is one device symbol shared by all launches: wait for the stream (an earlier launch may still read it), then copy.
// A launch recorded into a CUDA graph keeps whatever the table holds when the graph runs, so it goes unchecked (zeros).
void upload_extents(const MTArgs& a, cudaStream_t s) {
    static unsigned long long host[MT_NP][MT_MAX];
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(s, &cap);
    if (cap != cudaStreamCaptureStatusNone) return;
    for (int r = 0; r < MT_NP; ++r)
        for (int t = 0; t < MT_MAX; ++t) host[r][t] = (t < a.n) ? extent_of(a.ptr[r][t]) : 0;
    cudaStreamSynchronize(s);
    cudaMemcpyToSymbol(g_extent, host, sizeof(host));
}
}  // namespace
bool bounds_check_enabled() { return true; }
void bounds_reset() { int z[8] = {0, 0, 0, 0, 0, 0, 0, 0}; cudaDeviceSynchronize(); cudaMemcpyToSymbol(g_viol, z, sizeof(z)); }
void bounds_report(int out[8]) { cudaDeviceSynchronize(); cudaMemcpyFromSymbol(out, g_viol, 8 * sizeof(int)); }
void bounds_cap(long long bytes) { g_cap = bytes; }
long long bounds_extent_of(const void* ptr) { return (long long)extent_of(ptr); }
#else
bool bounds_check_enabled() { return false; }
void bounds_reset() {}
void bounds_report(int out[8]) { for (int k = 0; k < 8; ++k) out[k] = 0; }
void bounds_cap(long long) {}
long long bounds_extent_of(const void*) { return 0; }
#endif

void mt_launch(int op, int dtype, const MTArgs& a, const MTParams& p, cudaStream_t s) {
    if (a.blk_start[a.n] > 0) count_launch();
#ifdef GROK_BOUNDS_CHECK
    if (a.blk_start[a.n] > 0) upload_extents(a, s);
#endif
    switch (op) {
#define SG_CASE(X) case X: launch_typed<X>(dtype, a, p, s); break;
        SG_CASE(OP_ADAMW) SG_CASE(OP_LION) SG_CASE(OP_GROKFAST_EMA) SG_CASE(OP_GROKFAST_ADAMW) SG_CASE(OP_GROKADAMW)
        SG_CASE(OP_PRODIGY) SG_CASE(OP_NEURALGROK) SG_CASE(OP_SG15) SG_CASE(OP_SG11_A) SG_CASE(OP_SG11_B)
        SG_CASE(OP_PERTURB) SG_CASE(OP_RESTORE) SG_CASE(OP_SHARP_RESTORE) SG_CASE(OP_LOOKSAM_DIR)
        SG_CASE(OP_LOOKSAM_ADJ) SG_CASE(OP_MUON_MOMENTUM) SG_CASE(OP_MUON_UPDATE) SG_CASE(OP_SCALE)
        SG_CASE(OP_SQNORM) SG_CASE(OP_PRODIGY_REDUCE) SG_CASE(OP_DIFF_SQNORM)
#undef SG_CASE
        default: break;
    }
}

void mt_finalize_per_tensor(const MTArgs& a, const float* partials, float* out, cudaStream_t s) {
    if (a.n <= 0) return;
    count_launch();
    finalize_per_tensor_kernel<<<a.n, 32, 0, s>>>(a, partials, out);
}

void scalar_finalize(int op, const float* per_tensor, int n_tensors, float* out, float a0, float a1, float a2,
                     cudaStream_t s) {
    count_launch();
    scalar_finalize_kernel<<<1, 32, 0, s>>>(op, per_tensor, n_tensors, out, a0, a1, a2);
}

}  // namespace sg
