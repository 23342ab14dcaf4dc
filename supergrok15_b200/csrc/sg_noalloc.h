// Allocation-free C entry point (no counterpart in the reference, which allocates temporaries through
// PyTorch on every call).
//
// Who needs it: code that may not allocate device memory at the point of the call - a training loop that has
// handed the whole GPU to a fixed-size arena, a plugin running inside another framework's stream callback,
// a real-time control process - but still wants the global gradient norm and clip coefficient that the
// optimizers of this library compute.  The regular path (`ops/elementwise.py: clip_coef_device`) takes its
// two scratch buffers from PyTorch's allocator; this one keeps them in a fixed device array inside the library.
#pragma once
#include <cstdint>
#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest supported input: SG_NOALLOC_MAX_BLOCKS chunks of 8192 elements (134,217,728 fp32 values).
#define SG_NOALLOC_MAX_BLOCKS 16384

// out[0] = sum of squares of grad[0..n), out[1] = clip coefficient (max_norm/(norm+1e-6) if norm > max_norm else 1),
// out[2] = norm.  `grad` and `out` are device pointers supplied by the caller (out: 3 floats); the work is enqueued
// on `stream` and the call does not synchronise.
//
// Returns 0 on success; 1 if n is negative or exceeds the maximum above (nothing is launched); 2 if a pointer is
// null; a cudaError_t value + 100 if the one-time set-up or a launch failed.
//
// * No cudaMalloc / cudaFree / allocating library routine is called, ever.  The scratch (196,608 bytes) is a
//   file-scope device array that every GPU holding this library keeps for the life of the process.
// * The first call on each device resolves the device address of that array (cudaGetSymbolAddress with that device
//   current).  Make this first call outside any stream capture.
// * All calls on a device share the one scratch array: two calls whose kernels can overlap on the GPU (different
//   streams, no dependency between them) race on it.  Serialise them, e.g. by using one stream.
int sg_clip_coef_noalloc(const float* grad, int64_t n, float max_norm, float* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
