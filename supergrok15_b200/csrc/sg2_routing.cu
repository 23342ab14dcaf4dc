// Product-key routing of the SuperGrok v2 bilevel path as two kernels (sm_100a); the arithmetic is csrc/sg2_routing_math.h.
//
// Forward: one thread per (element, head): query, 2 x pk scores, top-4 and softmax per sub-key; writes ia, ib, wa, wb [n, heads, 4]
// (the inputs of the routed expert kernels, csrc/sg2_experts.cu).  Backward: the same thread recomputes its query, turns d wa / d wb
// into score and query gradients, and the tile's query gradients are folded back through Wq into d pin [n, P]; the parameter
// gradients (Wq, both key tables) are summed without atomics: every thread owns fixed outputs, walks the tile's elements in
// shared memory, keeps its sums in registers across tiles and writes them once per CTA; a second kernel adds the CTAs in order.
// It replaces two matrix products, a block-diagonal assembly, a top-k and a softmax over [n, 2 * heads * pk] tensors (and their
// autograd graph) of the PyTorch statement in optim/metanet.py: soft_head.
#include "sg_native.h"
#include "sg2_routing_math.h"

namespace sg {
namespace {
using namespace routing;

constexpr int RT = 256;                   // threads per CTA
constexpr int RMAXW = 4;                  // Wq outputs per thread (heads * 8 * P <= 1024)
constexpr int RMAXK = 2;                  // key-table outputs per thread (2 * heads * pk * 4 <= 512)

struct RWeights { const float* wq; const float* ka; const float* kb; };

__device__ __forceinline__ RWeights stage_weights(float* sm, const float* __restrict__ Wq, const float* __restrict__ KA,
                                                  const float* __restrict__ KB, int heads, int P, int pk) {
    float* wq = sm;
    float* ka = wq + heads * RD * P;
    float* kb = ka + heads * pk * RH;
    for (int i = threadIdx.x; i < heads * RD * P; i += RT) wq[i] = Wq[i];
    for (int i = threadIdx.x; i < heads * pk * RH; i += RT) { ka[i] = KA[i]; kb[i] = KB[i]; }
    return RWeights{wq, ka, kb};
}
__host__ __device__ inline int weights_floats(int heads, int P, int pk) { return heads * RD * P + 2 * heads * pk * RH; }

// CP / CPK > 0: input width and key rows are compile-time constants (loops unroll, the per-element arrays stay in registers)
template <int CP, int CPK>
__global__ void __launch_bounds__(RT) routing_fwd_kernel(const float* __restrict__ pin, const float* __restrict__ Wq, const float* __restrict__ KA,
                                                         const float* __restrict__ KB, int64_t n, int heads, int P_rt, int pk_rt,
                                                         int4* __restrict__ ia, int4* __restrict__ ib, float4* __restrict__ wa,
                                                         float4* __restrict__ wb) {
    const int P = CP > 0 ? CP : P_rt, pk = CPK > 0 ? CPK : pk_rt;
    extern __shared__ float sm[];
    const RWeights w = stage_weights(sm, Wq, KA, KB, heads, P, pk);
    __syncthreads();
    const int epc = RT / heads;
    const int le = threadIdx.x / heads, h = threadIdx.x % heads;
    const int64_t elem = (int64_t)blockIdx.x * epc + le;
    if (le >= epc || elem >= n) return;
    float x[CP > 0 ? CP : RP_MAX], q[RD], a_w[RK], b_w[RK];
    int a_i[RK], b_i[RK];
#pragma unroll
    for (int j = 0; j < P; ++j) x[j] = pin[elem * P + j];
    route_fwd(x, P, w.wq + h * RD * P, w.ka + h * pk * RH, w.kb + h * pk * RH, pk, q, a_i, b_i, a_w, b_w);
    const int64_t r = elem * heads + h;
    ia[r] = make_int4(a_i[0], a_i[1], a_i[2], a_i[3]);
    ib[r] = make_int4(b_i[0], b_i[1], b_i[2], b_i[3]);
    wa[r] = make_float4(a_w[0], a_w[1], a_w[2], a_w[3]);
    wb[r] = make_float4(b_w[0], b_w[1], b_w[2], b_w[3]);
}

// partial: [gridDim.x, heads*8*P + 2*heads*pk*4]  (d Wq | d KA | d KB)
__global__ void __launch_bounds__(RT) routing_bwd_kernel(const float* __restrict__ pin, const float* __restrict__ Wq, const float* __restrict__ KA,
                                                         const float* __restrict__ KB, const int4* __restrict__ ia, const int4* __restrict__ ib,
                                                         const float4* __restrict__ wa, const float4* __restrict__ wb,
                                                         const float4* __restrict__ dwa, const float4* __restrict__ dwb, int64_t n, int heads,
                                                         int P, int pk, float* __restrict__ dpin, float* __restrict__ partial) {
    extern __shared__ float sm[];
    const RWeights w = stage_weights(sm, Wq, KA, KB, heads, P, pk);
    const int epc = RT / heads;
    float* s_pin = sm + weights_floats(heads, P, pk);              // [epc][P]
    float* s_q = s_pin + epc * P;                                  // [epc][heads][8]
    float* s_dq = s_q + epc * heads * RD;                          // [epc][heads][8]
    float* s_dt = s_dq + epc * heads * RD;                         // [epc][heads][8]   (A scores 0..3, B scores 4..7)
    int* s_ix = reinterpret_cast<int*>(s_dt + epc * heads * RD);   // [epc][heads][8]
    const int le = threadIdx.x / heads, h = threadIdx.x % heads;
    const int n_wq = heads * RD * P, n_k = heads * pk * RH;
    float acc_w[RMAXW], acc_k[RMAXK];
#pragma unroll
    for (int u = 0; u < RMAXW; ++u) acc_w[u] = 0.f;
#pragma unroll
    for (int u = 0; u < RMAXK; ++u) acc_k[u] = 0.f;
    __syncthreads();
    const int64_t tiles = (n + epc - 1) / epc;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t left = n - tile * epc;
        const int cnt = left < epc ? (int)left : epc;
        for (int i = threadIdx.x; i < cnt * P; i += RT) s_pin[i] = pin[tile * epc * P + i];
        __syncthreads();
        const bool live = le < cnt;
        if (live) {
            const int64_t r = (tile * epc + le) * heads + h;
            const int4 a4 = ia[r], b4 = ib[r];
            const float4 wa4 = wa[r], wb4 = wb[r], da4 = dwa[r], db4 = dwb[r];
            const int a_i[RK] = {a4.x, a4.y, a4.z, a4.w}, b_i[RK] = {b4.x, b4.y, b4.z, b4.w};
            const float a_w[RK] = {wa4.x, wa4.y, wa4.z, wa4.w}, b_w[RK] = {wb4.x, wb4.y, wb4.z, wb4.w};
            const float a_d[RK] = {da4.x, da4.y, da4.z, da4.w}, b_d[RK] = {db4.x, db4.y, db4.z, db4.w};
            float q[RD], dt[2 * RK], dq[RD];
            query(s_pin + le * P, P, w.wq + h * RD * P, q);
            route_bwd(a_i, b_i, a_w, b_w, a_d, b_d, w.ka + h * pk * RH, w.kb + h * pk * RH, dt, dq);
            const int o = (le * heads + h) * RD;
#pragma unroll
            for (int k = 0; k < RD; ++k) { s_q[o + k] = q[k]; s_dq[o + k] = dq[k]; s_dt[o + k] = dt[k]; }
#pragma unroll
            for (int k = 0; k < RK; ++k) { s_ix[o + k] = a_i[k]; s_ix[o + RK + k] = b_i[k]; }
        }
        __syncthreads();
        if (live) {                                               // d pin[j] = sum over heads and query rows of Wq[hh][o][j] * dq[hh][o]
            const float* dqe = s_dq + le * heads * RD;
            for (int j = h; j < P; j += heads) {
                float a = 0.f;
                for (int t = 0; t < heads * RD; ++t) a = fmaf(w.wq[t * P + j], dqe[t], a);
                dpin[(tile * epc + le) * P + j] = a;
            }
        }
        // parameter gradients: fixed outputs per thread, elements of the tile in order
#pragma unroll
        for (int u = 0; u < RMAXW; ++u) {
            const int id = threadIdx.x + u * RT;
            if (id < n_wq) {
                const int row = id / P, j = id % P;               // row = head * 8 + query row
                float a = acc_w[u];
                for (int m = 0; m < cnt; ++m) a = fmaf(s_dq[m * heads * RD + row], s_pin[m * P + j], a);
                acc_w[u] = a;
            }
        }
#pragma unroll
        for (int u = 0; u < RMAXK; ++u) {
            const int id = threadIdx.x + u * RT;
            if (id < 2 * n_k) {
                const int ab = id / n_k, rem = id % n_k;          // ab: 0 = table A, 1 = table B
                const int hh = rem / (pk * RH), row = (rem / RH) % pk, d = rem % RH;
                float a = acc_k[u];
                for (int m = 0; m < cnt; ++m) {
                    const int o = (m * heads + hh) * RD + ab * RK;
#pragma unroll
                    for (int k = 0; k < RK; ++k)
                        if (s_ix[o + k] == row) a = fmaf(s_dt[o + k], s_q[(m * heads + hh) * RD + ab * RH + d], a);
                }
                acc_k[u] = a;
            }
        }
        __syncthreads();                                          // the tile buffers are rewritten next
    }
    float* out = partial + (int64_t)blockIdx.x * (n_wq + 2 * n_k);
#pragma unroll
    for (int u = 0; u < RMAXW; ++u) { const int id = threadIdx.x + u * RT; if (id < n_wq) out[id] = acc_w[u]; }
#pragma unroll
    for (int u = 0; u < RMAXK; ++u) { const int id = threadIdx.x + u * RT; if (id < 2 * n_k) out[n_wq + id] = acc_k[u]; }
}

__global__ void __launch_bounds__(256) routing_reduce_kernel(const float* __restrict__ partial, int parts, int ng, float* __restrict__ out) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= ng) return;
    float t = 0.f;
    for (int p = 0; p < parts; ++p) t += partial[(int64_t)p * ng + i];
    out[i] = t;
}

size_t fwd_smem(int heads, int P, int pk) { return (size_t)weights_floats(heads, P, pk) * sizeof(float); }
size_t bwd_smem(int heads, int P, int pk) {
    const int epc = RT / heads;
    return (size_t)(weights_floats(heads, P, pk) + epc * P + 4 * epc * heads * RD) * sizeof(float);
}
}  // namespace

bool routing_supported(int heads, int P, int pk, int d_model, int topk) {
    return d_model == routing::RD && topk == routing::RK && heads >= 1 && heads <= 16 && P >= 1 && P <= routing::RP_MAX && pk >= routing::RK &&
           pk <= routing::RPK_MAX && heads * routing::RD * P <= RMAXW * RT && 2 * heads * pk * routing::RH <= RMAXK * RT &&
           bwd_smem(heads, P, pk) <= 200 * 1024;
}
int routing_bwd_ctas(int64_t n, int heads) {
    const int epc = RT / heads;
    const int64_t tiles = (n + epc - 1) / epc;
    return (int)(tiles < 1 ? 1 : (tiles < 4 * 148 ? tiles : 4 * 148));
}
int routing_ng(int heads, int P, int pk) { return heads * routing::RD * P + 2 * heads * pk * routing::RH; }

int routing_fwd(const float* pin, const float* Wq, const float* KA, const float* KB, int64_t n, int heads, int P, int pk, int* ia, int* ib,
                float* wa, float* wb, cudaStream_t s) {
    if (n <= 0) return 0;
    const size_t smem = fwd_smem(heads, P, pk);
    if (cudaFuncSetAttribute(routing_fwd_kernel<22, 12>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(routing_fwd_kernel<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
    const int epc = RT / heads;
    const unsigned grid = (unsigned)((n + epc - 1) / epc);
    count_launch();
    if (P == 22 && pk == 12)                                          // the default meta-net: gru 4 + 2 * d_model 16 + 2 inputs, 144 experts
        routing_fwd_kernel<22, 12><<<grid, RT, smem, s>>>(pin, Wq, KA, KB, n, heads, P, pk, (int4*)ia, (int4*)ib, (float4*)wa, (float4*)wb);
    else
        routing_fwd_kernel<0, 0><<<grid, RT, smem, s>>>(pin, Wq, KA, KB, n, heads, P, pk, (int4*)ia, (int4*)ib, (float4*)wa, (float4*)wb);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int routing_bwd(const float* pin, const float* Wq, const float* KA, const float* KB, const int* ia, const int* ib, const float* wa, const float* wb,
                const float* dwa, const float* dwb, int64_t n, int heads, int P, int pk, float* dpin, float* partial, float* dparams, cudaStream_t s) {
    const int ng = routing_ng(heads, P, pk);
    if (n <= 0) return cudaMemsetAsync(dparams, 0, (size_t)ng * sizeof(float), s) == cudaSuccess ? 0 : 3;
    const size_t smem = bwd_smem(heads, P, pk);
    if (cudaFuncSetAttribute(routing_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
    const int ctas = routing_bwd_ctas(n, heads);
    count_launch(2);
    routing_bwd_kernel<<<ctas, RT, smem, s>>>(pin, Wq, KA, KB, (const int4*)ia, (const int4*)ib, (const float4*)wa, (const float4*)wb,
                                              (const float4*)dwa, (const float4*)dwb, n, heads, P, pk, dpin, partial);
    routing_reduce_kernel<<<(ng + 255) / 256, 256, 0, s>>>(partial, ctas, ng, dparams);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace sg
