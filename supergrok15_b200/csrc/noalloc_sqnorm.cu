// Allocation-free variant of the global-norm / clip-coefficient reduction (see sg_noalloc.h for the contract).
//
// Same two-stage, fixed-order reduction as the multi-tensor OP_SQNORM path in mt_kernels.cu: stage 1 writes one
// partial sum per 8192-element chunk, stage 2 adds the partials in a fixed order and derives the coefficient.
// The difference is where the partials live: a file-scope device array instead of a tensor from an allocator.
#include "sg_noalloc.h"
#include "sg_native.h"
#include "optim_math.cuh"

namespace {

// Scratch of the allocation-free entry point: one partial sum per chunk.  In HOST code the name `g_scratch` is only a
// stand-in for the symbol; its device address is fetched once per device with cudaGetSymbolAddress (below).
static __device__ __align__(256) float g_scratch[SG_NOALLOC_MAX_BLOCKS * 3];

__global__ void __launch_bounds__(256) noalloc_partial_kernel(const float* __restrict__ g, int64_t n, float* __restrict__ partials) {
    __shared__ float red[32];
    const int64_t begin = (int64_t)blockIdx.x * sg::MT_CHUNK;
    const int64_t end = (begin + sg::MT_CHUNK < n) ? begin + sg::MT_CHUNK : n;
    const bool vec = sg::vec_ok<float>(g);
    float acc = 0.f;
    for (int64_t i = begin + (int64_t)threadIdx.x * 4; i < end; i += 256 * 4) {
        const int cnt = (end - i >= 4) ? 4 : (int)(end - i);
        float v[4];
        sg::ld4<float>(g, i, cnt, vec, v);
#pragma unroll
        for (int k = 0; k < 4; ++k) acc = fmaf(v[k], v[k], acc);
    }
    const float r = sg::block_sum(acc, red);
    if (threadIdx.x == 0) partials[blockIdx.x] = r;      // every slot that stage 2 reads is overwritten by this launch
}

__global__ void __launch_bounds__(32) noalloc_final_kernel(const float* __restrict__ partials, int n_blocks, float max_norm,
                                                           float* __restrict__ out) {
    float s = 0.f;
    for (int b = threadIdx.x; b < n_blocks; b += 32) s += partials[b];
    s = sg::warp_sum(s);
    if (threadIdx.x == 0) {
        const float norm = sqrtf(s);
        out[0] = s;
        out[1] = (norm > max_norm) ? max_norm / (norm + 1e-6f) : 1.f;
        out[2] = norm;
    }
}

constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {nullptr};

}  // namespace

extern "C" int sg_clip_coef_noalloc(const float* grad, int64_t n, float max_norm, float* out, cudaStream_t stream) {
    if (grad == nullptr || out == nullptr) return 2;
    const int64_t max_n = (int64_t)SG_NOALLOC_MAX_BLOCKS * sg::MT_CHUNK;
    if (n < 0 || n > max_n) return 1;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return 100 + (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return 1;
    if (g_scratch_addr[dev] == nullptr) {                 // one-time set-up for this device (current device = dev)
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_scratch);
        if (e != cudaSuccess) return 100 + (int)e;
        g_scratch_addr[dev] = p;
    }
    float* scratch = g_scratch_addr[dev];
    const int blocks = (int)((n + sg::MT_CHUNK - 1) / sg::MT_CHUNK);
    if (blocks > 0) {
        noalloc_partial_kernel<<<blocks, 256, 0, stream>>>(grad, n, scratch);
        sg::count_launch();
    }
    noalloc_final_kernel<<<1, 32, 0, stream>>>(scratch, blocks, max_norm, out);
    sg::count_launch();
    e = cudaGetLastError();
    return e == cudaSuccess ? 0 : 100 + (int)e;
}
