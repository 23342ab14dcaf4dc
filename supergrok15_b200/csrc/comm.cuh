// Device-side communication primitives over NVLink 5 / NVSwitch peer mappings.
//
//  * system-scope release/acquire flag access for cross-GPU hand-offs,
//  * NVLS multimem loads (in-switch reduction) and stores (in-switch replication),
//  * BOUNDED waits: every spin carries a deadline (globaltimer); when it passes, the waiter records
//    STATUS_TIMEOUT together with the peer it was waiting for and returns.  Nothing traps and nothing
//    spins forever, so a missing peer leaves the CUDA context usable and the host can raise.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include "sg_native.h"

namespace sg {

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// wait until *flag >= want (monotone epochs) or the deadline passes; returns false on timeout
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want, unsigned long long timeout_ns) {
    const unsigned long long t0 = global_ns();
    int backoff = 32;
    while ((int32_t)(ld_acquire_sys(flag) - want) < 0) {
        if (global_ns() - t0 > timeout_ns) return false;
        __nanosleep(backoff);
        if (backoff < 1024) backoff <<= 1;
    }
    return true;
}

// 16-byte in-switch reductions / replication on a multicast address (NVLS)
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc_addr) : "memory");
    return r;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc_addr) {
    float4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(mc_addr) : "memory");
    return r;
}
__device__ __forceinline__ void multimem_st_u32x4(void* mc_addr, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

}  // namespace sg
