// SuperGrok v2 optimizer step on sm_100a: prep, gather, bidirectional Mamba-3 scan, element step.
//
// What the reference does with ~450 launches and ~110 host syncs per step
// (csrc/supergrok2_mamba_peer_kernels.cu:1754-2117, grokking_optimizers/supergrok2.py:310-345)
// is one fixed sequence of launches here, independent of the number of tensors:
//
//   prep      per-tensor clip + NaN scrub, packed fp32 gradient / sharpness, sort keys
//   sort      sg2_sort.cu
//   gather    sorted (g, s) pairs
//   scan 1    per-chunk aggregate 2x2 affine maps        (only tensors split into several chunks)
//   scan 2    carry-in state of every chunk              (tiny)
//   scan 3    re-run every chunk from its carry-in, apply SiLU gate / D skip / out_proj and write the
//             8-float context straight to the element's ORIGINAL index (no un-sort gathers)
//   elem      GRU + 4-head product-key routing + expert MLPs (shared memory) + mu EMA + Adam
//
// Scan decomposition: the sequence of a tensor is cut into chunks of `chunk_len` timesteps; an item is
// (tensor, direction, chunk).  Sixteen lanes (one per d_inner column) own an item; each lane keeps the
// 16 state values of its column (8 RoPE pairs) in registers, so y is accumulated in registers and
// nothing is read-modify-written in global memory.  Per 16-timestep tile the lanes first act as
// "one lane per timestep" to compute x, z, dt, B, C with warp-uniform weights from constant memory,
// park them in shared memory, then act as "one lane per column" for the recurrence.
// The meta-net weights (11,580 floats) live in __constant__ memory; the 144 experts are staged in
// shared memory by the element kernel because their index is data dependent.
#include "sg_native.h"
#include "optim_math.cuh"
#include "peer_fetch.cuh"

namespace sg {

__constant__ float c_w[SG2Pack::TOTAL];

namespace {

using P = SG2Pack;
constexpr int TILE_T = 16;                 // timesteps per tile
constexpr int ROW = 52;                    // floats per timestep row in shared memory: B[16] C[16] (g,s,-,-) out[16]; 13 float4 (odd) keeps 128-bit stores conflict free
constexpr int SCAN_THREADS = 128;          // 8 items per CTA
#ifndef SG_SCAN_MINB
#define SG_SCAN_MINB 3                     // resident CTAs per SM the scan kernel is compiled for (phase 3 at 18.9 M parameters: 6.07 / 6.00 / 6.39 ms with 2 / 3 / 4)
#endif

constexpr int ITEMS_PER_CTA = SCAN_THREADS / 16;

__device__ __forceinline__ float softplus20(float x) { return x > 20.f ? x : __logf(1.f + __expf(x)); }
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }

// ---------------------------------------------------------------------------------------------------- prep
// roles: 1 = grad (launch dtype), 2 = sharpness (fp32), 6 = packed offset (integer smuggled in the pointer slot)
// PACKED: the gradient is read from g_packed itself (fp32, reduced over the ranks and scrubbed by sg2_pull_sqnorm_kernel)
template <typename T, bool PACKED>
__global__ void __launch_bounds__(MT_THREADS) sg2_prep_kernel(const __grid_constant__ MTArgs a, const float* __restrict__ tclip,
                                                              float* g_packed, float* __restrict__ s_packed,
                                                              uint32_t* __restrict__ keys, uint32_t* __restrict__ vals) {
    int lo = 0, hi = a.n;
    const int b = blockIdx.x;
    while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (a.blk_start[mid] <= b) lo = mid; else hi = mid; }
    const int t = lo;
    const int64_t begin = (int64_t)(b - a.blk_start[t]) * MT_CHUNK;
    const int64_t n = a.numel[t];
    const int64_t end = (begin + MT_CHUNK < n) ? begin + MT_CHUNK : n;
    const int64_t off = (int64_t)reinterpret_cast<intptr_t>(a.ptr[6][t]);
    const T* g = reinterpret_cast<const T*>(a.ptr[1][t]);
    const float* sh = reinterpret_cast<const float*>(a.ptr[2][t]);
    const float clip = tclip[a.t_off + t];
    for (int64_t i = begin + threadIdx.x; i < end; i += MT_THREADS) {
        float gv = PACKED ? g_packed[off + i] : Cvt<T>::to(g[i]);
        float sv = sh[i];
        gv = isfinite(gv) ? gv * clip : 0.f;
        if (!isfinite(gv)) gv = 0.f;
        if (!isfinite(sv)) sv = 0.f;
        g_packed[off + i] = gv;
        s_packed[off + i] = sv;
        keys[off + i] = __float_as_uint(fabsf(gv));
        vals[off + i] = (uint32_t)(off + i);
    }
}

// finite-only sum of squares per CTA (per-tensor clip uses the norm of the scrubbed gradient)
template <typename T>
__global__ void __launch_bounds__(MT_THREADS) sg2_sqnorm_kernel(const __grid_constant__ MTArgs a, float* __restrict__ partials) {
    __shared__ float red[32];
    int lo = 0, hi = a.n;
    const int b = blockIdx.x;
    while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (a.blk_start[mid] <= b) lo = mid; else hi = mid; }
    const int t = lo;
    const int64_t begin = (int64_t)(b - a.blk_start[t]) * MT_CHUNK;
    const int64_t n = a.numel[t];
    const int64_t end = (begin + MT_CHUNK < n) ? begin + MT_CHUNK : n;
    const T* g = reinterpret_cast<const T*>(a.ptr[1][t]);
    float acc = 0.f;
    for (int64_t i = begin + threadIdx.x; i < end; i += MT_THREADS) {
        const float gv = Cvt<T>::to(g[i]);
        if (isfinite(gv)) acc = fmaf(gv, gv, acc);
    }
    const float r = block_sum(acc, red);
    if (threadIdx.x == 0) { float* o = partials + 3 * (int64_t)(a.blk_off + b); o[0] = r; o[1] = 0.f; o[2] = 0.f; }
}

// Reduce-scatter fused into the first kernel of the pipeline (ZeRO engine): every rank's gradient buffer has the same layout and
// is mapped into this process; the owner of a tensor reads the tensor's slice of ALL W buffers with 16-byte peer loads (all W
// loads of a vector are in flight before the first is used), sums in fp32, scales by 1/W, scrubs non-finite values, writes the
// packed fp32 gradient that the rest of the pipeline consumes and accumulates the tensor's sum of squares for the per-tensor
// clip.  No reduced copy of the gradient shard exists anywhere else.  The buffers are padded to 8 elements per tensor, so whole
// vectors are read; only elements below the tensor's length are written or counted.
struct PullParams {
    int world, rank;
    float scale;
    char* local_base;            // base of this rank's gradient buffer (the tensors' role-1 pointers point into it)
    PeerPtrs base;               // base of every rank's buffer in this process's address space (base.p[rank] == local_base)
};

template <typename T, int W>
__global__ void __launch_bounds__(MT_THREADS) sg2_pull_sqnorm_kernel(const __grid_constant__ MTArgs a, const __grid_constant__ PullParams pp,
                                                                     float* __restrict__ g_packed, float* __restrict__ partials) {
    constexpr int N = 16 / sizeof(T);
    __shared__ float red[32];
    int lo = 0, hi = a.n;
    const int b = blockIdx.x;
    while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (a.blk_start[mid] <= b) lo = mid; else hi = mid; }
    const int t = lo;
    const int64_t begin = (int64_t)(b - a.blk_start[t]) * MT_CHUNK;
    const int64_t n = a.numel[t];
    const int64_t end = (begin + MT_CHUNK < n) ? begin + MT_CHUNK : n;
    const int64_t off = (int64_t)reinterpret_cast<intptr_t>(a.ptr[6][t]);
    const int64_t elem0 = (reinterpret_cast<char*>(a.ptr[1][t]) - pp.local_base) / (int64_t)sizeof(T);   // tensor start in the flat buffer
    const int nvec = (int)((end - begin + N - 1) / N);
    float acc = 0.f;
    for (int v0 = threadIdx.x; v0 < nvec; v0 += 2 * MT_THREADS) {
        float g[2][N];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int v = v0 + u * MT_THREADS;
            if (v < nvec) fetch_grad<T, N, false, W>(pp.base, nullptr, pp.world, pp.rank, elem0 + begin + (int64_t)v * N, g[u]);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int v = v0 + u * MT_THREADS;
            if (v >= nvec) break;
            const int64_t i0 = begin + (int64_t)v * N;
#pragma unroll
            for (int k = 0; k < N; ++k) {
                if (i0 + k < end) {
                    float gv = g[u][k] * pp.scale;
                    if (!isfinite(gv)) gv = 0.f;
                    g_packed[off + i0 + k] = gv;
                    acc = fmaf(gv, gv, acc);
                }
            }
        }
    }
    const float r = block_sum(acc, red);
    if (threadIdx.x == 0) { float* o = partials + 3 * (int64_t)(a.blk_off + b); o[0] = r; o[1] = 0.f; o[2] = 0.f; }
}

__global__ void __launch_bounds__(256) sg2_gather_kernel(const uint32_t* __restrict__ vals_sorted, const float* __restrict__ g_packed,
                                                         const float* __restrict__ s_packed, float2* __restrict__ gs_sorted,
                                                         int64_t total) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i < total) {
        const uint32_t v = vals_sorted[i];
        gs_sorted[i] = make_float2(g_packed[v], s_packed[v]);
    }
}

// ---------------------------------------------------------------------------------------------------- scan
struct Item {          // 32 bytes
    int64_t off;       // packed offset of the tensor
    int32_t n;         // tensor length
    int32_t ub, ue;    // scan-order range [ub, ue)
    int32_t tensor;    // -1 = padding
    int32_t td;        // index of the (tensor, direction) record
    int32_t last;      // 1 = last chunk of its (tensor, direction)
};
struct TensorDir {     // 32 bytes
    float* h;          // persistent [16,16] state of this tensor / direction
    int32_t item0;     // first item index
    int32_t nc;        // number of chunks
    int32_t pad[4];
};

// The scan's per-timestep inputs x, z, dt (pre-activation), B, C are all AFFINE functions of the two scalars (g, s) of the
// timestep: input_proj is 2 -> 8 and in_proj / dt_proj / B_proj / C_proj are linear maps applied on top of it.  The host folds
// the chain into five [16][3] tables per direction (SG2Pack::AFF*: coefficient of g, coefficient of s, constant), computed in
// fp64.  Per timestep the precompute is then 160 FMAs instead of 1040, and x / z / dt are evaluated by the column's own lane.
//
// Stage A: lane l = timestep (u0 + l): B[16], C[16] and (g, s) of that timestep go to its shared-memory row.
template <int DIR>
__device__ __forceinline__ void stage_a(float* __restrict__ tile, const float2* __restrict__ gs, int64_t off, int n, int u, bool valid,
                                        int l) {
    constexpr int AF = (DIR == 0) ? P::AFF0 : P::AFF1;
    if (!valid) return;
    float4* row = reinterpret_cast<float4*>(tile + l * ROW);
    const int pos = (DIR == 0) ? u : (n - 1 - u);
    const float2 v = gs[off + pos];
    float bc[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) {                       // k < 16: B_k, k >= 16: C_(k-16)
        const int w = AF + P::A_B + 3 * k;               // A_B and A_C tables are contiguous
        bc[k] = fmaf(c_w[w], v.x, fmaf(c_w[w + 1], v.y, c_w[w + 2]));
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) row[q] = make_float4(bc[4 * q], bc[4 * q + 1], bc[4 * q + 2], bc[4 * q + 3]);
    row[8] = make_float4(v.x, v.y, 0.f, 0.f);
}

__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// per (column, pair) transition: Abar_e, Abar_o, cos, sin from dt.   Abar = (1+a)/(1-a) = 2/(1-a) - 1 with a = dt*A/2 <= 0.
__device__ __forceinline__ void pair_coeffs(float dt, float ah_e, float ah_o, float f, float& abe, float& abo, float& cs, float& sn) {
    // the reference denominator is 1 - dt*A/2 + 1e-8; dt*A/2 <= 0, so the sum is >= 1 and adding 1e-8 (less than
    // half an ulp of 1) does not change the fp32 value: it is dropped
    // One reciprocal serves both states of the pair (1/de = dn/(de*dn)): the scan is bound by the special-function pipe (two
    // reciprocals, a sine and a cosine per pair and step at 16 results per clock per SM), so a reciprocal is traded for three
    // multiplies on the FMA pipe.  Both denominators lie in [1, 1 + 10|A|], their product cannot overflow.
    const float de = fmaf(-dt, ah_e, 1.f), dn = fmaf(-dt, ah_o, 1.f);
    const float r2 = 2.f * rcp_approx(de * dn);
    abe = fmaf(dn, r2, -1.f);
    abo = fmaf(de, r2, -1.f);
    __sincosf(dt * f, &sn, &cs);
}

// column constants of lane j: A/2, rope frequencies, and the affine tables of x_j, z_j, dt_j
template <int DIR>
struct ColConst {
    float ah[16], f[8], ux[3], uz[3], ud[3], Dj;
    __device__ __forceinline__ void load(int j) {
        constexpr int W = (DIR == 0) ? P::DIR0 : P::DIR1;
        constexpr int AF = (DIR == 0) ? P::AFF0 : P::AFF1;
#pragma unroll
        for (int s = 0; s < 16; ++s) ah[s] = -0.5f * __expf(c_w[W + P::D_ALOG + j * 16 + s]);
#pragma unroll
        for (int p = 0; p < 8; ++p) f[p] = c_w[W + P::D_ROPE + j * 8 + p];
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            ux[k] = c_w[AF + P::A_X + 3 * j + k]; uz[k] = c_w[AF + P::A_Z + 3 * j + k]; ud[k] = c_w[AF + P::A_DT + 3 * j + k];
        }
        Dj = c_w[W + P::D_D + j];
    }
};

// PHASE 3: run a chunk forward from its carry-in; apply SiLU gate, D skip and out_proj; write the contexts.
// The recurrence stays scalar with sin.approx / cos.approx on the special-function unit: two rewrites that take the sincos off
// that unit (packed f32x2 arithmetic over pairs of RoPE pairs; degree-5 / degree-6 polynomials for |theta| <= 0.25) were measured
// at 18.9 M parameters and ran this phase in 23.5 ms and 24.2 ms against 6.4 ms for this form; so did a hand-made software
// pipeline that computes the coefficients of step l + 1 during the recurrence of step l (10.5 ms at two CTAs per SM, 34.8 ms at three).
template <int DIR>
__device__ void scan_phase3(const Item& it, const TensorDir* __restrict__ tds, const float2* __restrict__ gs,
                            const uint32_t* __restrict__ vals_sorted, const float* __restrict__ carry, float* __restrict__ ctx,
                            float* __restrict__ tile, int item_idx, int j, unsigned hmask) {
    constexpr int W = (DIR == 0) ? P::DIR0 : P::DIR1;
    ColConst<DIR> cc;
    cc.load(j);
    float h[16];
    {
        const float* cin = carry + ((int64_t)item_idx * 16 + j) * 16;
#pragma unroll
        for (int q = 0; q < 4; ++q) { const float4 t = reinterpret_cast<const float4*>(cin)[q]; h[4 * q] = t.x; h[4 * q + 1] = t.y; h[4 * q + 2] = t.z; h[4 * q + 3] = t.w; }
    }
    for (int u0 = it.ub; u0 < it.ue; u0 += TILE_T) {
        const int cnt = (it.ue - u0 < TILE_T) ? (it.ue - u0) : TILE_T;
        stage_a<DIR>(tile, gs, it.off, it.n, u0 + j, j < cnt, j);
        __syncwarp(hmask);
        for (int l = 0; l < cnt; ++l) {                 // lane j = column (unrolling two timesteps together was measured 4 % slower)
            float* row = tile + l * ROW;
            const float2 v = *reinterpret_cast<const float2*>(row + 32);
            const float x = fmaf(cc.ux[0], v.x, fmaf(cc.ux[1], v.y, cc.ux[2]));
            const float z = fmaf(cc.uz[0], v.x, fmaf(cc.uz[1], v.y, cc.uz[2]));
            const float dt = softplus20(fmaf(cc.ud[0], v.x, fmaf(cc.ud[1], v.y, cc.ud[2])));
            float B[16], C[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 t = reinterpret_cast<const float4*>(row)[q];
                B[4 * q] = t.x; B[4 * q + 1] = t.y; B[4 * q + 2] = t.z; B[4 * q + 3] = t.w;
                const float4 c = reinterpret_cast<const float4*>(row + 16)[q];
                C[4 * q] = c.x; C[4 * q + 1] = c.y; C[4 * q + 2] = c.z; C[4 * q + 3] = c.w;
            }
            const float dtx = dt * x;
            float y = 0.f;
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float abe, abo, cs, sn;
                pair_coeffs(dt, cc.ah[2 * p], cc.ah[2 * p + 1], cc.f[p], abe, abo, cs, sn);
                const float he = h[2 * p], ho = h[2 * p + 1];
                const float ne = fmaf(abe, he * cs - ho * sn, dtx * B[2 * p]);
                const float no = fmaf(abo, ho * cs + he * sn, dtx * B[2 * p + 1]);
                h[2 * p] = ne; h[2 * p + 1] = no;
                y = fmaf(ne, C[2 * p], fmaf(no, C[2 * p + 1], y));
            }
            row[36 + j] = fmaf(y, silu(z), cc.Dj * x);    // out_j of this timestep
        }
        __syncwarp(hmask);
        if (j < cnt) {                                    // lane = timestep again: ctx = out_proj . out at the ORIGINAL index
            const float* row = tile + j * ROW;
            float o[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) { const float4 t = reinterpret_cast<const float4*>(row + 36)[q]; o[4 * q] = t.x; o[4 * q + 1] = t.y; o[4 * q + 2] = t.z; o[4 * q + 3] = t.w; }
            float c8[8];
#pragma unroll
            for (int d = 0; d < 8; ++d) {
                float acc = 0.f;
#pragma unroll
                for (int k = 0; k < 16; ++k) acc = fmaf(c_w[W + P::D_OUT + d * 16 + k], o[k], acc);
                c8[d] = acc;
            }
            const int u = u0 + j;
            const int pos = (DIR == 0) ? u : (it.n - 1 - u);
            const uint32_t orig = vals_sorted[it.off + pos];
            float4* dst = reinterpret_cast<float4*>(ctx + (int64_t)orig * 16 + DIR * 8);
            dst[0] = make_float4(c8[0], c8[1], c8[2], c8[3]);
            dst[1] = make_float4(c8[4], c8[5], c8[6], c8[7]);
        }
        __syncwarp(hmask);
    }
    if (it.last) {
        float* dst = tds[it.td].h + j * 16;
#pragma unroll
        for (int q = 0; q < 4; ++q) reinterpret_cast<float4*>(dst)[q] = make_float4(h[4 * q], h[4 * q + 1], h[4 * q + 2], h[4 * q + 3]);
    }
}

// PHASE 1: aggregate affine map (M, b) of a chunk:  h_end = M h_in + b.
// The chunk is walked BACKWARDS in time with the suffix product S = M_last ... M_{t+1}:  b += S b_t ; S <- S M_t.
// With contracting dynamics every entry of S falls below 2^-48 after a few hundred steps; from then on an earlier
// timestep can change b by at most 2^-48 |b_t|, 2^-24 of an fp32 ulp of a state of the size of its own inputs, so the walk
// stops (all 16 columns of the item agree by ballot).  Exact zero cannot be the test: a denormal times 0.7 rounds
// back to the smallest denormal and never reaches zero.  Without contraction the whole chunk is walked.
template <int DIR>
__device__ void scan_phase1(const Item& it, const float2* __restrict__ gs, float* __restrict__ agg, float* __restrict__ tile,
                            int item_idx, int j, unsigned hmask) {
    ColConst<DIR> cc;
    cc.load(j);
    float b[16], m[32];
#pragma unroll
    for (int s = 0; s < 16; ++s) b[s] = 0.f;
#pragma unroll
    for (int p = 0; p < 8; ++p) { m[4 * p] = 1.f; m[4 * p + 1] = 0.f; m[4 * p + 2] = 0.f; m[4 * p + 3] = 1.f; }
    const int len = it.ue - it.ub;
    const int ntile = (len + TILE_T - 1) / TILE_T;
    for (int tI = ntile - 1; tI >= 0; --tI) {
        const int u0 = it.ub + tI * TILE_T;
        const int cnt = (it.ue - u0 < TILE_T) ? (it.ue - u0) : TILE_T;
        stage_a<DIR>(tile, gs, it.off, it.n, u0 + j, j < cnt, j);
        __syncwarp(hmask);
        for (int l = cnt - 1; l >= 0; --l) {
            const float* row = tile + l * ROW;
            const float2 v = *reinterpret_cast<const float2*>(row + 32);
            const float x = fmaf(cc.ux[0], v.x, fmaf(cc.ux[1], v.y, cc.ux[2]));
            const float dt = softplus20(fmaf(cc.ud[0], v.x, fmaf(cc.ud[1], v.y, cc.ud[2])));
            float B[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 t = reinterpret_cast<const float4*>(row)[q];
                B[4 * q] = t.x; B[4 * q + 1] = t.y; B[4 * q + 2] = t.z; B[4 * q + 3] = t.w;
            }
            const float dtx = dt * x;
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float abe, abo, cs, sn;
                pair_coeffs(dt, cc.ah[2 * p], cc.ah[2 * p + 1], cc.f[p], abe, abo, cs, sn);
                const float a0 = m[4 * p], b0 = m[4 * p + 1], c0 = m[4 * p + 2], d0 = m[4 * p + 3];
                const float be = dtx * B[2 * p], bo = dtx * B[2 * p + 1];
                b[2 * p]     = fmaf(a0, be, fmaf(b0, bo, b[2 * p]));
                b[2 * p + 1] = fmaf(c0, be, fmaf(d0, bo, b[2 * p + 1]));
                const float p1 = abe * cs, p2 = abe * sn, p3 = abo * sn, p4 = abo * cs;   // M_t = [[p1,-p2],[p3,p4]]
                m[4 * p]     = fmaf(a0, p1, b0 * p3);
                m[4 * p + 1] = fmaf(b0, p4, -a0 * p2);
                m[4 * p + 2] = fmaf(c0, p1, d0 * p3);
                m[4 * p + 3] = fmaf(d0, p4, -c0 * p2);
            }
        }
        bool zero = true;
#pragma unroll
        for (int k = 0; k < 32; ++k) zero = zero && (fabsf(m[k]) < 3.5527e-15f);   // 2^-48
        __syncwarp(hmask);
        if (__all_sync(hmask, zero)) break;
    }
    float* dst = agg + ((int64_t)item_idx * 16 + j) * 48;      // [pair][a b c d e o]
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        dst[6 * p] = m[4 * p]; dst[6 * p + 1] = m[4 * p + 1]; dst[6 * p + 2] = m[4 * p + 2]; dst[6 * p + 3] = m[4 * p + 3];
        dst[6 * p + 4] = b[2 * p]; dst[6 * p + 5] = b[2 * p + 1];
    }
}

// items [0, n_items0) are direction 0, [n_items0_padded, ...) direction 1; n_items0_padded is a multiple of 8,
// so one CTA (8 items) never mixes directions.
template <int PHASE>
__global__ void __launch_bounds__(SCAN_THREADS, SG_SCAN_MINB) sg2_scan_kernel(const Item* __restrict__ items, int n_items, int dir1_start,
                                                                   const TensorDir* __restrict__ tds, const float2* __restrict__ gs,
                                                                   const uint32_t* __restrict__ vals_sorted, float* __restrict__ agg,
                                                                   const float* __restrict__ carry, float* __restrict__ ctx,
                                                                   const int* __restrict__ status) {
    __shared__ __align__(16) float tiles[ITEMS_PER_CTA][TILE_T * ROW];
    if (status && (*status & 0xff) != STATUS_OK) return;              // a wait on a peer timed out earlier in this step: the persistent scan states stay
    const int slot = threadIdx.x >> 4, j = threadIdx.x & 15;
    const int item_idx = blockIdx.x * ITEMS_PER_CTA + slot;
    const unsigned hmask = 0xffffu << (16 * ((threadIdx.x >> 4) & 1));
    if (item_idx >= n_items) return;
    const Item it = items[item_idx];
    if (it.tensor < 0) return;
    if (PHASE == 1 && it.last) return;            // nobody consumes the aggregate of a last chunk
    if (PHASE == 1) {
        if (item_idx < dir1_start) scan_phase1<0>(it, gs, agg, tiles[slot], item_idx, j, hmask);
        else                       scan_phase1<1>(it, gs, agg, tiles[slot], item_idx, j, hmask);
    } else {
        if (item_idx < dir1_start) scan_phase3<0>(it, tds, gs, vals_sorted, carry, ctx, tiles[slot], item_idx, j, hmask);
        else                       scan_phase3<1>(it, tds, gs, vals_sorted, carry, ctx, tiles[slot], item_idx, j, hmask);
    }
}

// Phase 2: carry-in of every chunk.  One CTA of 128 threads (column j, pair p) per (tensor, direction).  The recurrence over the
// chunks is serial, but the aggregates do not depend on it: they are loaded eight chunks ahead, so a step of the chain costs four
// dependent FMAs instead of a global-memory round trip (a 1 M-element tensor in 700-step chunks has 1,500 links).
__global__ void __launch_bounds__(128) sg2_carry_kernel(const TensorDir* __restrict__ tds, const float* __restrict__ agg,
                                                        float* __restrict__ carry) {
    constexpr int PF = 8;
    const TensorDir td = tds[blockIdx.x];
    const int j = threadIdx.x >> 3, p = threadIdx.x & 7;
    float he = td.h[j * 16 + 2 * p], ho = td.h[j * 16 + 2 * p + 1];
    for (int c0 = 0; c0 < td.nc; c0 += PF) {
        float a[PF][6];
#pragma unroll
        for (int u = 0; u < PF; ++u) {
            const int c = c0 + u;
            if (c + 1 < td.nc) {
                const float2* src = reinterpret_cast<const float2*>(agg + ((int64_t)(td.item0 + c) * 16 + j) * 48 + 6 * p);
                const float2 q0 = src[0], q1 = src[1], q2 = src[2];
                a[u][0] = q0.x; a[u][1] = q0.y; a[u][2] = q1.x; a[u][3] = q1.y; a[u][4] = q2.x; a[u][5] = q2.y;
            }
        }
#pragma unroll
        for (int u = 0; u < PF; ++u) {
            const int c = c0 + u;
            if (c < td.nc) {
                float* co = carry + ((int64_t)(td.item0 + c) * 16 + j) * 16 + 2 * p;
                *reinterpret_cast<float2*>(co) = make_float2(he, ho);
                if (c + 1 < td.nc) {
                    const float ne = fmaf(a[u][0], he, fmaf(a[u][1], ho, a[u][4]));
                    const float no = fmaf(a[u][2], he, fmaf(a[u][3], ho, a[u][5]));
                    he = ne; ho = no;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------- element step
struct ElemParams {
    float beta2, eps, rescale;
    const float* dyn;                  // device table: lr, effective weight decay, lambda_eff and the per-tensor scalars
    const float* w_global;             // packed meta-net weights in global memory (source of the shared-memory expert tables)
    const int* status;                 // optional status word of the collectives: once a wait on a peer has timed out, nothing is updated
    const float* g_packed; const float* s_packed; const float* ctx;
    int* expert_counts;                // [144] or nullptr
    // optional replication of the updated parameter into the same offset of peer buffers (fused all-gather):
    // a parameter at local address local_base + d is also stored to peer_base[r] + d for r < n_peers
    int n_peers; int n_inline; char* local_base; char* peer_base[8];
};

// roles: 0 = param (launch dtype), 1 = m, 2 = v, 3 = mu, 4 = gru [n,4], 5 = fp32 master (optional), 6 = packed offset.
// Step scalars come from the device table prm.dyn (layout: DYN_* in sg_native.h).
template <typename T>
__global__ void __launch_bounds__(MT_THREADS) sg2_elem_kernel(const __grid_constant__ MTArgs a, const __grid_constant__ ElemParams prm) {
    // Expert rows are padded to 17 floats: lanes pick different experts, and with a row pitch of 16 the word k of every expert
    // falls into one of only two banks (16-way conflicts); with 17 the rows of 32 consecutive experts spread over all banks.
    constexpr int EP = SG2_EH + 1;
    if (prm.status && (*prm.status & 0xff) != STATUS_OK) return;      // gradients of a timed-out step are incomplete: keep every state as it is
    __shared__ float sW1[SG2_NE * EP], sB1[SG2_NE * EP], sW2[SG2_NE * EP], sB2[SG2_NE];
    __shared__ int scount[SG2_NE];
    for (int i = threadIdx.x; i < SG2_NE * SG2_EH; i += MT_THREADS) {
        const int j = (i / SG2_EH) * EP + i % SG2_EH;
        // lanes read consecutive words: from global memory that is one coalesced request, from __constant__ memory 32 serial ones
        sW1[j] = prm.w_global[P::EW1 + i]; sB1[j] = prm.w_global[P::EB1 + i]; sW2[j] = prm.w_global[P::EW2 + i];
    }
    for (int i = threadIdx.x; i < SG2_NE; i += MT_THREADS) { sB2[i] = prm.w_global[P::EB2 + i]; scount[i] = 0; }
    __syncthreads();
    int lo = 0, hi = a.n;
    const int b = blockIdx.x;
    while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (a.blk_start[mid] <= b) lo = mid; else hi = mid; }
    const int t = lo;
    const int64_t begin = (int64_t)(b - a.blk_start[t]) * MT_CHUNK;
    const int64_t n = a.numel[t];
    const int64_t end = (begin + MT_CHUNK < n) ? begin + MT_CHUNK : n;
    const int64_t off = (int64_t)reinterpret_cast<intptr_t>(a.ptr[6][t]);
    T* param = reinterpret_cast<T*>(a.ptr[0][t]);
    float* M = reinterpret_cast<float*>(a.ptr[1][t]);
    float* V = reinterpret_cast<float*>(a.ptr[2][t]);
    float* MU = reinterpret_cast<float*>(a.ptr[3][t]);
    float4* GRU = reinterpret_cast<float4*>(a.ptr[4][t]);
    float* MASTER = reinterpret_cast<float*>(a.ptr[5][t]);       // fp32 master copy of a low-precision parameter (may be null)
    const ptrdiff_t pdelta = reinterpret_cast<char*>(param) - prm.local_base;
    const float* ts = prm.dyn + DYN_TS + 4 * (a.t_off + t);
    const float alpha = ts[0], beta1 = ts[1], bc1 = ts[2], bc2 = ts[3];
    const float lr = prm.dyn[DYN_LR], wd_eff = prm.dyn[DYN_WD], lamb_eff = prm.dyn[DYN_LAMB];

    for (int64_t i = begin + threadIdx.x; i < end; i += MT_THREADS) {
        const float g = prm.g_packed[off + i], s = prm.s_packed[off + i];
        float cx[16];                                  // fwd ctx (8) then bwd ctx (8)
        {
            const float4* src = reinterpret_cast<const float4*>(prm.ctx + (off + i) * 16);
#pragma unroll
            for (int q = 0; q < 4; ++q) { const float4 v = src[q]; cx[4 * q] = v.x; cx[4 * q + 1] = v.y; cx[4 * q + 2] = v.z; cx[4 * q + 3] = v.w; }
        }
        const float4 hv = GRU[i];
        const float hold[4] = {hv.x, hv.y, hv.z, hv.w};
        // GRU: input order [g, s, fwd(8), bwd(8), h(4)]
        float zg[4], rg[4], hn[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            float vz = c_w[P::GRU_BZ + r], vr = c_w[P::GRU_BR + r];
            const int wz = P::GRU_WZ + r * 22, wr = P::GRU_WR + r * 22;
            vz = fmaf(c_w[wz], g, fmaf(c_w[wz + 1], s, vz));
            vr = fmaf(c_w[wr], g, fmaf(c_w[wr + 1], s, vr));
#pragma unroll
            for (int k = 0; k < 16; ++k) { vz = fmaf(c_w[wz + 2 + k], cx[k], vz); vr = fmaf(c_w[wr + 2 + k], cx[k], vr); }
#pragma unroll
            for (int k = 0; k < 4; ++k) { vz = fmaf(c_w[wz + 18 + k], hold[k], vz); vr = fmaf(c_w[wr + 18 + k], hold[k], vr); }
            zg[r] = sigmoidf(vz); rg[r] = sigmoidf(vr);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int wh = P::GRU_WH + r * 22;
            float vh = fmaf(c_w[wh], g, fmaf(c_w[wh + 1], s, c_w[P::GRU_BH + r]));
#pragma unroll
            for (int k = 0; k < 16; ++k) vh = fmaf(c_w[wh + 2 + k], cx[k], vh);
#pragma unroll
            for (int k = 0; k < 4; ++k) vh = fmaf(c_w[wh + 18 + k], rg[k] * hold[k], vh);
            hn[r] = (1.f - zg[r]) * hold[r] + zg[r] * tanhf(vh);
        }
        GRU[i] = make_float4(hn[0], hn[1], hn[2], hn[3]);
        // PEER: input order [h_new(4), fwd(8), bwd(8), g, s]
        float total = 0.f;
#pragma unroll
        for (int hd = 0; hd < SG2_HEADS; ++hd) {
            float q[8];
#pragma unroll
            for (int d = 0; d < 8; ++d) {
                const int w = P::PQ + (hd * 8 + d) * 22;
                float acc = 0.f;
#pragma unroll
                for (int k = 0; k < 4; ++k) acc = fmaf(c_w[w + k], hn[k], acc);
#pragma unroll
                for (int k = 0; k < 16; ++k) acc = fmaf(c_w[w + 4 + k], cx[k], acc);
                acc = fmaf(c_w[w + 20], g, fmaf(c_w[w + 21], s, acc));
                q[d] = acc;
            }
            int ba = 0, bb = 0;
            float sa = -1e30f, sb = -1e30f;
#pragma unroll
            for (int k = 0; k < SG2_PK; ++k) {
                const int wa = P::KA + (hd * SG2_PK + k) * 4, wb = P::KB + (hd * SG2_PK + k) * 4;
                const float da = fmaf(q[0], c_w[wa], fmaf(q[1], c_w[wa + 1], fmaf(q[2], c_w[wa + 2], q[3] * c_w[wa + 3])));
                const float db = fmaf(q[4], c_w[wb], fmaf(q[5], c_w[wb + 1], fmaf(q[6], c_w[wb + 2], q[7] * c_w[wb + 3])));
                if (da > sa) { sa = da; ba = k; }
                if (db > sb) { sb = db; bb = k; }
            }
            const int e = ba * SG2_PK + bb;
            if (prm.expert_counts) atomicAdd(&scount[e], 1);
            float ho = sB2[e];
#pragma unroll
            for (int k = 0; k < SG2_EH; ++k) ho = fmaf(sW2[e * EP + k], fmaxf(fmaf(sW1[e * EP + k], g, sB1[e * EP + k]), 0.f), ho);
            total += ho;
        }
        const float smart = g + prm.rescale * total * (1.f / SG2_HEADS);
        float mu = MU[i];
        mu = alpha * mu + (1.f - alpha) * g;
        MU[i] = mu;
        const float fg = smart + lamb_eff * mu;
        float mm = M[i], vv = V[i];
        const float pold = MASTER ? MASTER[i] : Cvt<T>::to(param[i]);
        const float pnew = adam_update(pold, fg, mm, vv, lr, beta1, prm.beta2, prm.eps, wd_eff, bc1, bc2);
        M[i] = mm; V[i] = vv;
        if (MASTER) MASTER[i] = pnew;
        const T pt = Cvt<T>::from(pnew);
        param[i] = pt;
        // Element-granular push (n_inline peers, 0 when the buffers are padded to 16 bytes per tensor and the vector push below is
        // used).  The loop also matters to the compiler: with a store loop of unknown trip count here, ptxas keeps one head's
        // working set live at a time (64-79 registers, three CTAs per SM, weights as immediate constant-bank operands); without
        // it the four unrolled heads are interleaved (128-156 registers), and a rolled head loop turns the weights into indexed
        // constant loads that miss the constant cache (measured: 655 us instead of 419 us at 3.2 M elements).
        for (int r = 0; r < prm.n_inline; ++r) reinterpret_cast<T*>(prm.peer_base[r] + pdelta)[i] = pt;
    }
    if (prm.n_peers > prm.n_inline) {
        // All-gather fused into the step: the chunk this CTA just wrote is replicated into every peer's parameter buffer with one
        // 16-byte store per lane and peer (512 contiguous bytes per warp and store; 2-byte stores from the element loop would put
        // 64 bytes per warp on the link).  The chunk is re-read from this GPU's own memory (L1 / L2 hits).  Tensors are padded to
        // 8 elements in every rank's buffer, so whole vectors are copied.
        __syncthreads();
        constexpr int N = 16 / sizeof(T);
        const int nvec = (int)((end - begin + N - 1) / N);
        const uint4* src = reinterpret_cast<const uint4*>(param + begin);
        for (int v = threadIdx.x; v < nvec; v += MT_THREADS) {
            const uint4 val = src[v];
            for (int r = prm.n_inline; r < prm.n_peers; ++r)
                reinterpret_cast<uint4*>(reinterpret_cast<T*>(prm.peer_base[r] + pdelta) + begin)[v] = val;
        }
    }
    if (prm.expert_counts) {
        __syncthreads();
        for (int i = threadIdx.x; i < SG2_NE; i += MT_THREADS)
            if (scount[i]) atomicAdd(&prm.expert_counts[i], scount[i]);      // integer atomics: order independent
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------------------- host API
void sg2_upload_weights(const float* packed_dev, cudaStream_t s) {
    cudaMemcpyToSymbolAsync(c_w, packed_dev, sizeof(float) * SG2Pack::TOTAL, 0, cudaMemcpyDeviceToDevice, s);
}

void sg2_sqnorm(int dtype, const MTArgs& a, float* partials, cudaStream_t s) {
    const int blocks = a.blk_start[a.n];
    if (blocks <= 0) return;
    count_launch();
    switch (dtype) {
        case F32:  sg2_sqnorm_kernel<float><<<blocks, MT_THREADS, 0, s>>>(a, partials); break;
        case BF16: sg2_sqnorm_kernel<__nv_bfloat16><<<blocks, MT_THREADS, 0, s>>>(a, partials); break;
        default:   sg2_sqnorm_kernel<__half><<<blocks, MT_THREADS, 0, s>>>(a, partials); break;
    }
}

void sg2_prep(int dtype, bool packed_src, const MTArgs& a, const float* tclip, float* g_packed, float* s_packed, uint32_t* keys,
              uint32_t* vals, cudaStream_t s) {
    const int blocks = a.blk_start[a.n];
    if (blocks <= 0) return;
    count_launch();
    if (packed_src) { sg2_prep_kernel<float, true><<<blocks, MT_THREADS, 0, s>>>(a, tclip, g_packed, s_packed, keys, vals); return; }
    switch (dtype) {
        case F32:  sg2_prep_kernel<float, false><<<blocks, MT_THREADS, 0, s>>>(a, tclip, g_packed, s_packed, keys, vals); break;
        case BF16: sg2_prep_kernel<__nv_bfloat16, false><<<blocks, MT_THREADS, 0, s>>>(a, tclip, g_packed, s_packed, keys, vals); break;
        default:   sg2_prep_kernel<__half, false><<<blocks, MT_THREADS, 0, s>>>(a, tclip, g_packed, s_packed, keys, vals); break;
    }
}

// Gradient reduce-scatter + NaN scrub + per-tensor sum of squares in one kernel (role 1 = the tensors' slices of the LOCAL gradient
// buffer, whose base is local_base; bases = every rank's buffer, same layout).
void sg2_pull_sqnorm(int dtype, const MTArgs& a, const PeerPtrs& bases, int world, int rank, void* local_base, float scale,
                     float* g_packed, float* partials, cudaStream_t s) {
    const int blocks = a.blk_start[a.n];
    if (blocks <= 0) return;
    count_launch();
    PullParams pp{};
    pp.world = world; pp.rank = rank; pp.scale = scale; pp.local_base = reinterpret_cast<char*>(local_base); pp.base = bases;
#define PULL(T) \
    if (world == 8) sg2_pull_sqnorm_kernel<T, 8><<<blocks, MT_THREADS, 0, s>>>(a, pp, g_packed, partials); \
    else if (world == 4) sg2_pull_sqnorm_kernel<T, 4><<<blocks, MT_THREADS, 0, s>>>(a, pp, g_packed, partials); \
    else if (world == 2) sg2_pull_sqnorm_kernel<T, 2><<<blocks, MT_THREADS, 0, s>>>(a, pp, g_packed, partials); \
    else sg2_pull_sqnorm_kernel<T, 0><<<blocks, MT_THREADS, 0, s>>>(a, pp, g_packed, partials);
    switch (dtype) { case F32: PULL(float) break; case BF16: PULL(__nv_bfloat16) break; default: PULL(__half) break; }
#undef PULL
}

void sg2_gather(const uint32_t* vals_sorted, const float* g_packed, const float* s_packed, float* gs_sorted, int64_t total,
                cudaStream_t s) {
    if (total <= 0) return;
    count_launch();
    sg2_gather_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(vals_sorted, g_packed, s_packed,
                                                                       reinterpret_cast<float2*>(gs_sorted), total);
}

void sg2_scan(const void* items_dev, int n_items, int dir1_start, const void* tds_dev, int n_td, bool any_multi,
              const float* gs_sorted, const uint32_t* vals_sorted, float* agg, float* carry, float* ctx, const int* status, cudaStream_t s) {
    if (n_items <= 0) return;
    const int blocks = (n_items + ITEMS_PER_CTA - 1) / ITEMS_PER_CTA;
    const Item* items = reinterpret_cast<const Item*>(items_dev);
    const TensorDir* tds = reinterpret_cast<const TensorDir*>(tds_dev);
    const float2* gs = reinterpret_cast<const float2*>(gs_sorted);
    count_launch(any_multi ? 3 : 2);
    if (any_multi) sg2_scan_kernel<1><<<blocks, SCAN_THREADS, 0, s>>>(items, n_items, dir1_start, tds, gs, vals_sorted, agg, carry, ctx, status);
    sg2_carry_kernel<<<n_td, 128, 0, s>>>(tds, agg, carry);
    sg2_scan_kernel<3><<<blocks, SCAN_THREADS, 0, s>>>(items, n_items, dir1_start, tds, gs, vals_sorted, agg, carry, ctx, status);
}

int sg2_scan_ctas_per_sm() { return SG_SCAN_MINB; }

void sg2_elem(int dtype, const MTArgs& a, float beta2, float eps, float rescale, const float* dyn, const float* w_global, const int* status,
              const float* g_packed, const float* s_packed, const float* ctx, int* expert_counts, int n_peers, void* local_base,
              void* const* peer_base, cudaStream_t s) {
    const int blocks = a.blk_start[a.n];
    if (blocks <= 0) return;
    count_launch();
    ElemParams p{};
    p.beta2 = beta2; p.eps = eps; p.rescale = rescale; p.dyn = dyn; p.w_global = w_global; p.status = status;
    p.g_packed = g_packed; p.s_packed = s_packed; p.ctx = ctx; p.expert_counts = expert_counts;
    p.n_peers = n_peers; p.n_inline = 0; p.local_base = reinterpret_cast<char*>(local_base);
    for (int r = 0; r < n_peers && r < 8; ++r) p.peer_base[r] = reinterpret_cast<char*>(peer_base[r]);
    switch (dtype) {
        case F32:  sg2_elem_kernel<float><<<blocks, MT_THREADS, 0, s>>>(a, p); break;
        case BF16: sg2_elem_kernel<__nv_bfloat16><<<blocks, MT_THREADS, 0, s>>>(a, p); break;
        default:   sg2_elem_kernel<__half><<<blocks, MT_THREADS, 0, s>>>(a, p); break;
    }
}

// Writes up to WORDS_MAX 32-bit words, passed as kernel arguments, to device memory: the per-step scalars reach the device
// without a host buffer whose lifetime would have to outlast the copy.
namespace {
constexpr int WORDS_MAX = 960;
struct Words { uint32_t w[WORDS_MAX]; int n; };
__global__ void __launch_bounds__(256) write_words_kernel(const __grid_constant__ Words v, uint32_t* __restrict__ dst) {
    for (int i = threadIdx.x; i < v.n; i += 256) dst[i] = v.w[i];
}
}  // namespace
void write_words(uint32_t* dst, const uint32_t* host_words, int n, cudaStream_t s) {
    for (int o = 0; o < n; o += WORDS_MAX) {
        Words v;
        v.n = (n - o < WORDS_MAX) ? n - o : WORDS_MAX;
        for (int i = 0; i < v.n; ++i) v.w[i] = host_words[o + i];
        count_launch();
        write_words_kernel<<<1, 256, 0, s>>>(v, dst + o);
    }
}

size_t sg2_item_bytes() { return sizeof(Item); }
size_t sg2_td_bytes() { return sizeof(TensorDir); }

}  // namespace sg

#include "sg2_bilevel.cuh"
