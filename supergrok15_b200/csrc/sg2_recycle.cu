// Device-side recycling of dead PEER experts for the SuperGrok v2 meta-net (sm_100a).
//
// Semantics of the reference's host routine (mamba3_peer_metanet.py:437-491): experts whose share of the activation counts is
// below a threshold are replaced by noisy clones of ONE donor drawn in proportion to the counts; a product sub-key whose whole
// row (or column) of experts died is re-initialised; the counts are cleared.  Here the whole decision runs in one CTA on the
// device - no count is read back by the host, so the step stays free of host synchronisation - and every random number comes
// from Philox4x32-10 keyed by (seed, call index) with the element id as counter, so all data-parallel ranks that hold the same
// counts make bit-identical replacements whatever their thread mapping.
#include "sg_native.h"
#include <cuda_runtime.h>

namespace sg {
namespace {

struct Philox { uint32_t v[4]; };

__device__ __forceinline__ Philox philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
    constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0, hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += W0; k1 += W1;
    }
    return Philox{{c0, c1, c2, c3}};
}
__device__ __forceinline__ float u01(uint32_t x) { return ((float)(x >> 8) + 0.5f) * (1.0f / 16777216.0f); }   // (0, 1)
// one standard normal per (stream, index): Box-Muller on two words of the Philox block
__device__ __forceinline__ float normal_at(uint32_t stream, uint32_t index, uint32_t seed, uint32_t call) {
    const Philox p = philox4x32_10(index, stream, 0u, 0u, seed, call);
    return sqrtf(-2.f * __logf(u01(p.v[0]))) * __cosf(6.283185307179586f * u01(p.v[1]));
}

constexpr int NE = SG2_NE, PK = SG2_PK, EH = SG2_EH, HEADS = SG2_HEADS, KD = 4;    // 144 experts = 12 x 12 sub-keys of width 4

struct RecycleArgs {
    int* counts;                // [144] activation counts (cleared on exit unless their sum is zero)
    float* W1; float* b1; float* W2; float* b2;     // [144,16] [144,16] [144,16] [144]
    float* keyA[HEADS]; float* keyB[HEADS];         // [12,4] each
    float threshold;
    uint32_t seed, call;
    int* info;                  // [2]: number of experts replaced, donor index (-1 if nothing happened); may be null
};

__global__ void __launch_bounds__(256) recycle_kernel(RecycleArgs a) {
    __shared__ float cnt[NE];
    __shared__ int dead[NE];
    __shared__ int donor_s, n_dead_s;
    __shared__ float total_s;
    const int t = threadIdx.x;
    if (t < NE) cnt[t] = (float)a.counts[t];
    __syncthreads();
    if (t == 0) {
        float tot = 0.f;
        for (int i = 0; i < NE; ++i) tot += cnt[i];                  // fixed order
        total_s = tot;
        int nd = 0;
        if (tot > 0.f) for (int i = 0; i < NE; ++i) { dead[i] = (cnt[i] / tot) < a.threshold; nd += dead[i]; }
        n_dead_s = nd;
        int donor = -1;
        if (tot > 0.f && nd > 0) {                                   // inverse-CDF draw proportional to the counts
            const float u = u01(philox4x32_10(0u, 0xD0u, 0u, 0u, a.seed, a.call).v[0]) * tot;
            float run = 0.f;
            for (int i = 0; i < NE; ++i) { run += cnt[i]; if (cnt[i] > 0.f) { donor = i; if (u < run) break; } }
        }
        donor_s = donor;
        if (a.info) { a.info[0] = nd; a.info[1] = donor; }
    }
    __syncthreads();
    if (total_s <= 0.f) return;                                      // nothing was routed yet: keep the counts
    const int donor = donor_s;
    __shared__ float dW1[EH], db1[EH], dW2[EH], db2;
    if (n_dead_s > 0 && donor >= 0) {
        if (t < EH) { dW1[t] = a.W1[donor * EH + t]; db1[t] = a.b1[donor * EH + t]; dW2[t] = a.W2[donor * EH + t]; }
        if (t == 0) db2 = a.b2[donor];
    }
    __syncthreads();                                                 // the donor may itself be below the threshold: clone from the staged copy
    if (n_dead_s > 0 && donor >= 0) {
        // expert weights: stream 1..4 = W1, b1, W2, b2; index = expert * 16 + column
        for (int e = t; e < NE * EH; e += blockDim.x) {
            const int i = e / EH, c = e % EH;
            if (!dead[i]) continue;
            a.W1[e] = dW1[c] + 0.01f * normal_at(1u, (uint32_t)e, a.seed, a.call);
            a.b1[e] = db1[c] + 0.01f * normal_at(2u, (uint32_t)e, a.seed, a.call);
            a.W2[e] = dW2[c] + 0.01f * normal_at(3u, (uint32_t)e, a.seed, a.call);
            if (c == 0) a.b2[i] = db2 + 0.01f * normal_at(4u, (uint32_t)i, a.seed, a.call);
        }
        // sub-keys: row r of A is re-drawn when experts r*12 .. r*12+11 all died, column c of B when experts c, c+12, ... all died
        for (int e = t; e < 2 * PK * HEADS * KD; e += blockDim.x) {
            const int which = e / (PK * HEADS * KD), rem = e % (PK * HEADS * KD);
            const int hd = rem / (PK * KD), r = (rem / KD) % PK, d = rem % KD;
            bool all = true;
            for (int j = 0; j < PK; ++j) all = all && dead[which == 0 ? r * PK + j : j * PK + r];
            if (!all) continue;
            float* key = which == 0 ? a.keyA[hd] : a.keyB[hd];
            key[r * KD + d] = 0.02f * normal_at(5u + (uint32_t)which, (uint32_t)rem, a.seed, a.call);
        }
    }
    __syncthreads();
    if (t < NE) a.counts[t] = 0;
}

}  // namespace

void sg2_recycle(int* counts, float* W1, float* b1, float* W2, float* b2, float* const* keyA, float* const* keyB, float threshold,
                 uint32_t seed, uint32_t call, int* info, cudaStream_t s) {
    RecycleArgs a;
    a.counts = counts; a.W1 = W1; a.b1 = b1; a.W2 = W2; a.b2 = b2;
    for (int h = 0; h < HEADS; ++h) { a.keyA[h] = keyA[h]; a.keyB[h] = keyB[h]; }
    a.threshold = threshold; a.seed = seed; a.call = call; a.info = info;
    count_launch();
    recycle_kernel<<<1, 256, 0, s>>>(a);
}

}  // namespace sg
