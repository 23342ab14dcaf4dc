// Flash attention on the 5th-generation tensor cores (tcgen05 / TMEM / TMA), sm_100a only.  bf16 in, fp32 accumulate.
//
//   O[b, s, h, :] = softmax(Q[b, s, h, :] . K[b, :, h, :]^T / sqrt(hd), causal) . V[b, :, h, :]
//
// q, k, v, o are [B, S, H, hd] views (hd contiguous, heads adjacent: exactly what the projections produce - no transposes).
// One CTA owns 128 query rows of one (batch, head) and walks the key blocks of 128:
//   warp 0      producer: TMA loads Q once, then K_j and V_j into two-deep rings (separate rings: a K slot is free as soon as
//               S_j = Q K_j^T has been issued and completed, a V slot after P_j V_j)
//   warp 1      MMA issuer: S_{j+1} = Q K_{j+1}^T into the other S buffer in TMEM (so it runs under the softmax of block j), then
//               O_blk = P_j V_j.  V is consumed as an MN-major B operand straight from its [keys, hd] TMA tile.
//   warps 2-5   one query row per thread (TMEM lane = row): running max / sum, P_j written as bf16 into the swizzled K-major
//               A-operand tile in shared memory, O accumulated in registers (O = O*alpha + O_blk from TMEM)
// Everything is ordered by mbarriers with bounded waits; a wait that runs out raises the error word and the CTA drains.
// The log-sum-exp of every row is saved for the backward pass.
//
// Replaces nn.MultiheadAttention / F.scaled_dot_product_attention of the model code (the reference model builds its attention
// from nn.MultiheadAttention, grokking_race_v2.py:313-318) for the long-sequence decoder.
#include "sg_native.h"
#include "tc_sm100.cuh"
#include <cfloat>

namespace sg {
namespace {
using namespace tc;

constexpr int FA_THREADS = 192;
constexpr uint32_t TILE_HALF_BYTES = 128 * 128;          // [128 rows x 64 bf16] = 16 KB

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// two fused multiply-adds in one instruction (packed fp32 pair): y = x * a + b
__device__ __forceinline__ void fma2(float x0, float x1, float a, float b, float& y0, float& y1) {
    asm("{\n\t.reg .b64 vx, va, vb, vy;\n\tmov.b64 vx, {%2, %3};\n\tmov.b64 va, {%4, %4};\n\tmov.b64 vb, {%5, %5};\n\t"
        "fma.rn.f32x2 vy, vx, va, vb;\n\tmov.b64 {%0, %1}, vy;\n\t}"
        : "=f"(y0), "=f"(y1) : "f"(x0), "f"(x1), "f"(a), "f"(b));
}
// general packed pair: y = x * a + b with every operand a pair
__device__ __forceinline__ void fma2g(float x0, float x1, float a0, float a1, float b0, float b1, float& y0, float& y1) {
    asm("{\n\t.reg .b64 vx, va, vb, vy;\n\tmov.b64 vx, {%2, %3};\n\tmov.b64 va, {%4, %5};\n\tmov.b64 vb, {%6, %7};\n\t"
        "fma.rn.f32x2 vy, vx, va, vb;\n\tmov.b64 {%0, %1}, vy;\n\t}"
        : "=f"(y0), "=f"(y1) : "f"(x0), "f"(x1), "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ float max3f(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// Row maximum of 128 scores held in registers (three-input max: 64 instructions instead of 128); on the diagonal block the
// entries right of the diagonal are first replaced by -FLT_MAX.
__device__ __forceinline__ float row_max_128(uint32_t (&r)[4][32], bool diag, int row) {
    if (diag) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) if (c * 32 + i > row) r[c][i] = __float_as_uint(-FLT_MAX);
    }
    float mx = -FLT_MAX;
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2) mx = max3f(mx, __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
    return mx;
}
__device__ __forceinline__ void mbar_arrive_(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

struct FaBars {
    uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_full, o_full, o_empty;
    uint32_t tmem_slot, pad;
};

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1) flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                  const __grid_constant__ CUtensorMap map_k,
                                                                  const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                                                                  float* __restrict__ lse, int S, int H, int64_t ld_o, float scale,
                                                                  int causal, int* __restrict__ err) {
    constexpr int HALVES = HD / 64;
    constexpr uint32_t QKV_BYTES = HALVES * TILE_HALF_BYTES;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + QKV_BYTES;                        // [2][QKV_BYTES]
    uint8_t* sV = sK + 2 * QKV_BYTES;                    // [2][QKV_BYTES]
    uint8_t* sP = sV + 2 * QKV_BYTES;                    // [2 halves][16 KB]
    FaBars* bars = reinterpret_cast<FaBars*>(sP + 2 * TILE_HALF_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;                 // long (late) query tiles start first
    const int h = blockIdx.y, b = blockIdx.z;
    const int n_blk = causal ? qt + 1 : S / 128;
    const int row_q = b * S + qt * 128, col0 = h * HD;

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->k_full[i], 1); mbar_init(&bars->k_empty[i], 1); mbar_init(&bars->v_full[i], 1); mbar_init(&bars->v_empty[i], 1);
            mbar_init(&bars->s_full[i], 1); mbar_init(&bars->s_empty[i], 128);
        }
        mbar_init(&bars->p_full, 128); mbar_init(&bars->o_full, 1); mbar_init(&bars->o_empty, 128);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_slot;
    const uint32_t tmem_o = tmem_base + 256;                             // S0 [0,128), S1 [128,256), O_blk [256, 256+HD)

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&bars->q_full, QKV_BYTES);
            for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(sQ + hf * TILE_HALF_BYTES, &map_q, col0 + hf * 64, row_q, &bars->q_full);
            for (int j = 0; j < n_blk; ++j) {
                const int s = j & 1, row_k = b * S + j * 128;
                if (j >= 2 && !mbar_wait(&bars->k_empty[s], ((j >> 1) & 1) ^ 1)) { atomicExch(err, 11); break; }
                mbar_expect_tx(&bars->k_full[s], QKV_BYTES);
                for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(sK + s * QKV_BYTES + hf * TILE_HALF_BYTES, &map_k, col0 + hf * 64, row_k, &bars->k_full[s]);
                if (j >= 2 && !mbar_wait(&bars->v_empty[s], ((j >> 1) & 1) ^ 1)) { atomicExch(err, 12); break; }
                mbar_expect_tx(&bars->v_full[s], QKV_BYTES);
                for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(sV + s * QKV_BYTES + hf * TILE_HALF_BYTES, &map_v, col0 + hf * 64, row_k, &bars->v_full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_bf16(128, HD, 0, 1);     // B = V is MN-major (hd contiguous)
            bool ok = mbar_wait(&bars->q_full, 0);
            if (!ok) atomicExch(err, 13);
            tc_fence_after();
            auto issue_qk = [&](int j) -> bool {
                const int s = j & 1;
                if (!mbar_wait(&bars->k_full[s], (j >> 1) & 1)) { atomicExch(err, 14); return false; }
                if (j >= 2 && !mbar_wait(&bars->s_empty[s], ((j >> 1) & 1) ^ 1)) { atomicExch(err, 15); return false; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint64_t da = make_desc_sw128(smem_u32(sQ + (kk / 4) * TILE_HALF_BYTES)) + 2 * (kk % 4);
                    const uint64_t db = make_desc_sw128(smem_u32(sK + s * QKV_BYTES + (kk / 4) * TILE_HALF_BYTES)) + 2 * (kk % 4);
                    tc_mma_bf16(tmem_base + s * 128, da, db, idesc_qk, kk > 0 ? 1u : 0u);
                }
                tc_commit(&bars->k_empty[s]);
                tc_commit(&bars->s_full[s]);
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < n_blk && ok; ++j) {
                if (j + 1 < n_blk) { ok = issue_qk(j + 1); if (!ok) break; }
                const int s = j & 1;
                if (!mbar_wait(&bars->v_full[s], (j >> 1) & 1)) { atomicExch(err, 16); ok = false; break; }
                if (!mbar_wait(&bars->p_full, j & 1)) { atomicExch(err, 17); ok = false; break; }
                if (j >= 1 && !mbar_wait(&bars->o_empty, (j - 1) & 1)) { atomicExch(err, 18); ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {                         // 128 keys = 8 MMAs of K = 16
                    const uint64_t da = make_desc_sw128(smem_u32(sP + (kk / 4) * TILE_HALF_BYTES)) + 2 * (kk % 4);
                    const uint64_t db = make_desc_sw128_mn(smem_u32(sV + s * QKV_BYTES + kk * 2048), TILE_HALF_BYTES, 1024);
                    tc_mma_bf16(tmem_o, da, db, idesc_pv, kk > 0 ? 1u : 0u);
                }
                tc_commit(&bars->v_empty[s]);
                tc_commit(&bars->o_full);
            }
        }
    } else {
        const int q = warp & 3, row = q * 32 + lane;                     // TMEM lane quarter of this warp; one query row per thread
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const float c2 = scale * 1.4426950408889634f;
        float o[HD];
#pragma unroll
        for (int i = 0; i < HD; ++i) o[i] = 0.f;
        float m = -FLT_MAX, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_blk && ok; ++j) {
            const int s = j & 1;
            if (!mbar_wait(&bars->s_full[s], (j >> 1) & 1)) { atomicExch(err, 19); ok = false; break; }
            tc_fence_after();
            const bool diag = causal && j == qt;
            const uint32_t ts = tmem_base + s * 128 + lane_addr;
            float mx = -FLT_MAX;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tc_ld32(ts + c * 32, r);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float v = (diag && c * 32 + i > row) ? -FLT_MAX : __uint_as_float(r[i]);
                    mx = fmaxf(mx, v);
                }
            }
            const float m_new = fmaxf(m, mx);
            const float alpha = ex2f((m - m_new) * c2);
            const float mc = m_new * c2;
            float rowsum = 0.f;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tc_ld32(ts + c * 32, r);
                tc_wait_ld();
                uint8_t* prow = sP + (c >> 1) * TILE_HALF_BYTES + row * 128;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    uint4 pk;
                    __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int i0 = 8 * k + 2 * u;
                        float p0 = ex2f(fmaf(__uint_as_float(r[i0]), c2, -mc)), p1 = ex2f(fmaf(__uint_as_float(r[i0 + 1]), c2, -mc));
                        if (diag) { if (c * 32 + i0 > row) p0 = 0.f; if (c * 32 + i0 + 1 > row) p1 = 0.f; }
                        hh[u] = __floats2bfloat162_rn(p0, p1);
                        const float2 back = __bfloat1622float2(hh[u]);   // the sum uses the rounded probabilities that the MMA sees
                        rowsum += back.x + back.y;
                    }
                    const int chunk = (c & 1) * 4 + k;
                    *reinterpret_cast<uint4*>(prow + ((chunk ^ (row & 7)) << 4)) = pk;
                }
            }
            tc_fence_before();
            mbar_arrive_(&bars->s_empty[s]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive_(&bars->p_full);
            l = l * alpha + rowsum;
            m = m_new;
            if (!mbar_wait(&bars->o_full, j & 1)) { atomicExch(err, 20); ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t r[32];
                tc_ld32(tmem_o + lane_addr + c * 32, r);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha, __uint_as_float(r[i]));
            }
            tc_fence_before();
            mbar_arrive_(&bars->o_empty);
        }
        if (ok) {
            const float inv = 1.f / l;
            const int64_t grow = (int64_t)row_q + row;
            __nv_bfloat16* orow = out + grow * ld_o + col0;
#pragma unroll
            for (int k = 0; k < HD / 8; ++k) {
                uint4 pk;
                __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                for (int u = 0; u < 4; ++u) hh[u] = __floats2bfloat162_rn(o[8 * k + 2 * u] * inv, o[8 * k + 2 * u + 1] * inv);
                reinterpret_cast<uint4*>(orow)[k] = pk;
            }
            lse[((int64_t)b * H + h) * S + qt * 128 + row] = m * scale + logf(l);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}


// ---------------------------------------------------------------------------------------------------------------------------
// Second forward kernel: nothing of the softmax sits between two MMAs any more.
//   * P_j never leaves the tensor memory: the softmax threads overwrite the first 64 columns of the S_j buffer with the bf16
//     probabilities (tcgen05.st) and O += P_j V_j takes its A operand from TMEM;
//   * O accumulates in TMEM across the key blocks (no per-block read-back).  Each row keeps a reference maximum that is only
//     moved when the true maximum has grown by more than 8 in the exponent (probabilities then stay below 2^8); only then does
//     the row rescale O in TMEM, after waiting for the previous P V to finish.  The final division by the row sum uses the same
//     reference, so the result is exact;
//   * the MMA warp issues S_{j+1} = Q K_{j+1}^T before it waits for P_j: tcgen05.mma executes in issue order, so S_{j+1} lands in
//     the buffer whose P_{j-1} has just been consumed, and the tensor pipe alternates QK / PV while the softmax of the next block
//     runs.
struct Fa2Bars {
    uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full, o_done[2];
    uint32_t tmem_slot, pad;
};

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1) flash_fwd2_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                   const __grid_constant__ CUtensorMap map_k,
                                                                   const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                                                                   float* __restrict__ lse, int S, int H, int64_t ld_o, float scale,
                                                                   int causal, int* __restrict__ err) {
    constexpr int HALVES = HD / 64;
    constexpr uint32_t QKV_BYTES = HALVES * TILE_HALF_BYTES;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + QKV_BYTES;                        // [2][QKV_BYTES]
    uint8_t* sV = sK + 2 * QKV_BYTES;                    // [2][QKV_BYTES]
    Fa2Bars* bars = reinterpret_cast<Fa2Bars*>(sV + 2 * QKV_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int n_blk = causal ? qt + 1 : S / 128;
    const int row_q = b * S + qt * 128, col0 = h * HD;

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->k_full[i], 1); mbar_init(&bars->k_empty[i], 1); mbar_init(&bars->v_full[i], 1); mbar_init(&bars->v_empty[i], 1);
            mbar_init(&bars->s_full[i], 1); mbar_init(&bars->o_done[i], 1);
        }
        mbar_init(&bars->p_full, 128);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_slot;
    const uint32_t tmem_o = tmem_base + 256;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&bars->q_full, QKV_BYTES);
            for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(sQ + hf * TILE_HALF_BYTES, &map_q, col0 + hf * 64, row_q, &bars->q_full);
            for (int j = 0; j < n_blk; ++j) {
                const int s = j & 1, row_k = b * S + j * 128;
                if (j >= 2 && !mbar_wait(&bars->k_empty[s], ((j >> 1) & 1) ^ 1)) { atomicExch(err, 21); break; }
                mbar_expect_tx(&bars->k_full[s], QKV_BYTES);
                for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(sK + s * QKV_BYTES + hf * TILE_HALF_BYTES, &map_k, col0 + hf * 64, row_k, &bars->k_full[s]);
                if (j >= 2 && !mbar_wait(&bars->v_empty[s], ((j >> 1) & 1) ^ 1)) { atomicExch(err, 22); break; }
                mbar_expect_tx(&bars->v_full[s], QKV_BYTES);
                for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(sV + s * QKV_BYTES + hf * TILE_HALF_BYTES, &map_v, col0 + hf * 64, row_k, &bars->v_full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_bf16(128, HD, 0, 1);
            bool ok = mbar_wait(&bars->q_full, 0);
            if (!ok) atomicExch(err, 23);
            tc_fence_after();
            auto issue_qk = [&](int j) -> bool {
                const int s = j & 1;
                if (!mbar_wait(&bars->k_full[s], (j >> 1) & 1)) { atomicExch(err, 24); return false; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint64_t da = make_desc_sw128(smem_u32(sQ + (kk / 4) * TILE_HALF_BYTES)) + 2 * (kk % 4);
                    const uint64_t db = make_desc_sw128(smem_u32(sK + s * QKV_BYTES + (kk / 4) * TILE_HALF_BYTES)) + 2 * (kk % 4);
                    tc_mma_bf16(tmem_base + s * 128, da, db, idesc_qk, kk > 0 ? 1u : 0u);
                }
                tc_commit(&bars->k_empty[s]);
                tc_commit(&bars->s_full[s]);
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < n_blk && ok; ++j) {
                if (j + 1 < n_blk) { ok = issue_qk(j + 1); if (!ok) break; }
                const int s = j & 1;
                if (!mbar_wait(&bars->v_full[s], (j >> 1) & 1)) { atomicExch(err, 26); ok = false; break; }
                if (!mbar_wait(&bars->p_full, j & 1)) { atomicExch(err, 27); ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint64_t db = make_desc_sw128_mn(smem_u32(sV + s * QKV_BYTES + kk * 2048), TILE_HALF_BYTES, 1024);
                    tc_mma_bf16_ta(tmem_o, tmem_base + s * 128 + kk * 8, db, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                }
                tc_commit(&bars->v_empty[s]);
                tc_commit(&bars->o_done[s]);
            }
        }
    } else {
        const int q = warp & 3, row = q * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const float c2 = scale * 1.4426950408889634f;
        float m_ref = -FLT_MAX, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_blk && ok; ++j) {
            const int s = j & 1;
            if (!mbar_wait(&bars->s_full[s], (j >> 1) & 1)) { atomicExch(err, 28); ok = false; break; }
            tc_fence_after();
            const bool diag = causal && j == qt;
            const uint32_t ts = tmem_base + s * 128 + lane_addr;
            uint32_t r[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tc_ld32(ts + c * 32, r[c]);
            tc_wait_ld();
            const float mx = row_max_128(r, diag, row);
            float alpha = 1.f;
            bool move = false;
            if (j == 0) m_ref = mx;
            else if ((mx - m_ref) * c2 > 8.f) { alpha = ex2f((m_ref - mx) * c2); m_ref = mx; move = true; }
            if (j > 0 && __any_sync(0xffffffffu, move)) {
                // O holds the sum up to block j-1 relative to the old reference: wait for P_{j-1} V_{j-1}, then rescale this row in place
                if (!mbar_wait(&bars->o_done[(j - 1) & 1], ((j - 1) >> 1) & 1)) { atomicExch(err, 29); ok = false; break; }
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t t[32];
                    tc_ld32(tmem_o + lane_addr + c * 32, t);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
                    tc_st32(tmem_o + lane_addr + c * 32, t);
                }
            }
            const float mc = m_ref * c2;
            float rowsum = 0.f;
#pragma unroll
            for (int c = 0; c < 2; ++c) {                                // 64 keys -> 32 packed columns per store
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int k0 = c * 64 + 2 * i;
                    float e0, e1;
                    fma2(__uint_as_float(r[k0 >> 5][k0 & 31]), __uint_as_float(r[(k0 + 1) >> 5][(k0 + 1) & 31]), c2, -mc, e0, e1);
                    const float p0 = ex2f(e0), p1 = ex2f(e1);
                    const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
                    rowsum += p0 + p1;
                    pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
                }
                tc_st32(ts + c * 32, pk);
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive_(&bars->p_full);
            l = l * alpha + rowsum;
        }
        if (ok && !mbar_wait(&bars->o_done[(n_blk - 1) & 1], ((n_blk - 1) >> 1) & 1)) { atomicExch(err, 30); ok = false; }
        if (ok) {
            tc_fence_after();
            const float inv = 1.f / l;
            const int64_t grow = (int64_t)row_q + row;
            __nv_bfloat16* orow = out + grow * ld_o + col0;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t t[32];
                tc_ld32(tmem_o + lane_addr + c * 32, t);
                tc_wait_ld();
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    uint4 pk;
                    __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                    for (int u = 0; u < 4; ++u) hh[u] = __floats2bfloat162_rn(__uint_as_float(t[8 * k + 2 * u]) * inv, __uint_as_float(t[8 * k + 2 * u + 1]) * inv);
                    reinterpret_cast<uint4*>(orow)[c * 4 + k] = pk;
                }
            }
            lse[((int64_t)b * H + h) * S + qt * 128 + row] = m_ref * scale + logf(l);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Third forward kernel: two query tiles (A: rows [0,128), B: rows [128,256) of a 256-row block) per CTA in ping-pong, sharing
// every K_j / V_j tile.  Each tile has its own S/P buffer and O accumulator in TMEM (4 x 128 columns) and its own group of 128
// softmax threads.  The MMA warp issues
//     S_A(0), S_B(0), then for j:  O_A += P_A(j) V_j,  S_A(j+1),  O_B += P_B(j) V_j,  S_B(j+1)
// so while one group works on its scores the tensor pipe runs the other tile's two products: each softmax has two MMA slots to
// finish in.  P overlays S in TMEM, O is rescaled lazily (as in the second kernel).  With the causal mask tile A stops one key
// block before tile B.  S must be a multiple of 256.
constexpr int FA3_THREADS = 320;
struct Fa3Bars {
    uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], o_done[2][2];
    uint32_t tmem_slot, pad;
};

template <int HD>
__global__ void __launch_bounds__(FA3_THREADS, 1) flash_fwd3_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                    const __grid_constant__ CUtensorMap map_k,
                                                                    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                                                                    float* __restrict__ lse, int S, int H, int64_t ld_o, float scale,
                                                                    int causal, int* __restrict__ err) {
    constexpr int HALVES = HD / 64;
    constexpr uint32_t QKV_BYTES = HALVES * TILE_HALF_BYTES;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;                                  // [2 tiles][QKV_BYTES]
    uint8_t* sK = sQ + 2 * QKV_BYTES;                    // [2][QKV_BYTES]
    uint8_t* sV = sK + 2 * QKV_BYTES;                    // [2][QKV_BYTES]
    Fa3Bars* bars = reinterpret_cast<Fa3Bars*>(sV + 2 * QKV_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // 1-D grid ordered by decreasing work: all (batch, head) pairs of the last 256-row block first, those of block 0 last
    const int nqb = S / 256, n_hb = (int)gridDim.x / nqb, hb = (int)blockIdx.x % n_hb, qb = nqb - 1 - (int)blockIdx.x / n_hb;
    const int h = hb % H, b = hb / H;
    // key blocks per tile: tile t covers rows of 128-tile index 2*qb + t
    const int nA = causal ? 2 * qb + 1 : S / 128, nB = causal ? 2 * qb + 2 : S / 128;
    const int row_q = b * S + qb * 256, col0 = h * HD;

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->k_full[i], 1); mbar_init(&bars->k_empty[i], 1); mbar_init(&bars->v_full[i], 1); mbar_init(&bars->v_empty[i], 1);
            mbar_init(&bars->s_full[i], 1); mbar_init(&bars->p_full[i], 128);
            mbar_init(&bars->o_done[i][0], 1); mbar_init(&bars->o_done[i][1], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_slot;          // tile t: S/P at t*128, O at 256 + t*128

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&bars->q_full, 2 * QKV_BYTES);
            for (int t = 0; t < 2; ++t)
                for (int hf = 0; hf < HALVES; ++hf)
                    tma_load_2d(sQ + t * QKV_BYTES + hf * TILE_HALF_BYTES, &map_q, col0 + hf * 64, row_q + t * 128, &bars->q_full);
            for (int j = 0; j < nB; ++j) {
                const int s = j & 1, row_k = b * S + j * 128;
                if (j >= 2 && !mbar_wait(&bars->k_empty[s], ((j >> 1) & 1) ^ 1)) { atomicExch(err, 41); break; }
                mbar_expect_tx(&bars->k_full[s], QKV_BYTES);
                for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(sK + s * QKV_BYTES + hf * TILE_HALF_BYTES, &map_k, col0 + hf * 64, row_k, &bars->k_full[s]);
                if (j >= 2 && !mbar_wait(&bars->v_empty[s], ((j >> 1) & 1) ^ 1)) { atomicExch(err, 42); break; }
                mbar_expect_tx(&bars->v_full[s], QKV_BYTES);
                for (int hf = 0; hf < HALVES; ++hf) tma_load_2d(sV + s * QKV_BYTES + hf * TILE_HALF_BYTES, &map_v, col0 + hf * 64, row_k, &bars->v_full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_bf16(128, HD, 0, 1);
            bool ok = mbar_wait(&bars->q_full, 0);
            if (!ok) atomicExch(err, 43);
            tc_fence_after();
            // S_t(j) = Q_t K_j^T ; the K slot is released after tile B (or after tile A when B does not exist - never: nB >= nA)
            auto issue_qk = [&](int t, int j) {
                const int s = j & 1;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint64_t da = make_desc_sw128(smem_u32(sQ + t * QKV_BYTES + (kk / 4) * TILE_HALF_BYTES)) + 2 * (kk % 4);
                    const uint64_t db = make_desc_sw128(smem_u32(sK + s * QKV_BYTES + (kk / 4) * TILE_HALF_BYTES)) + 2 * (kk % 4);
                    tc_mma_bf16(tmem_base + t * 128, da, db, idesc_qk, kk > 0 ? 1u : 0u);
                }
                if (t == 1) tc_commit(&bars->k_empty[s]);
                tc_commit(&bars->s_full[t]);
            };
            auto issue_pv = [&](int t, int j) {
                const int s = j & 1;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint64_t db = make_desc_sw128_mn(smem_u32(sV + s * QKV_BYTES + kk * 2048), TILE_HALF_BYTES, 1024);
                    tc_mma_bf16_ta(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8, db, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                }
                if (t == 1) tc_commit(&bars->v_empty[s]);
                tc_commit(&bars->o_done[t][j & 1]);
            };
            if (ok) {
                if (!mbar_wait(&bars->k_full[0], 0)) { atomicExch(err, 44); ok = false; }
                else { tc_fence_after(); issue_qk(0, 0); issue_qk(1, 0); }
            }
            for (int j = 0; j < nB && ok; ++j) {
                const int s = j & 1;
                if (!mbar_wait(&bars->v_full[s], (j >> 1) & 1)) { atomicExch(err, 45); ok = false; break; }
                const bool next = j + 1 < nB;
                if (next && !mbar_wait(&bars->k_full[(j + 1) & 1], ((j + 1) >> 1) & 1)) { atomicExch(err, 46); ok = false; break; }
                if (j < nA) {
                    if (!mbar_wait(&bars->p_full[0], j & 1)) { atomicExch(err, 47); ok = false; break; }
                    tc_fence_after();
                    issue_pv(0, j);
                    if (j + 1 < nA) issue_qk(0, j + 1);
                }
                if (!mbar_wait(&bars->p_full[1], j & 1)) { atomicExch(err, 48); ok = false; break; }
                tc_fence_after();
                issue_pv(1, j);
                if (next) issue_qk(1, j + 1);
            }
        }
    } else {
        const int t = (warp - 2) >> 2;                                   // tile of this softmax group
        const int q = warp & 3, row = q * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const uint32_t ts = tmem_base + t * 128 + lane_addr, to = tmem_base + 256 + t * 128 + lane_addr;
        const float c2 = scale * 1.4426950408889634f;
        const int n_blk = t == 0 ? nA : nB, diag_j = 2 * qb + t;
        float m_ref = -FLT_MAX, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_blk && ok; ++j) {
            if (!mbar_wait(&bars->s_full[t], j & 1)) { atomicExch(err, 49); ok = false; break; }
            tc_fence_after();
            const bool diag = causal && j == diag_j;
            uint32_t r[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tc_ld32(ts + c * 32, r[c]);
            tc_wait_ld();
            const float mx = row_max_128(r, diag, row);
            float alpha = 1.f;
            bool move = false;
            if (j == 0) m_ref = mx;
            else if ((mx - m_ref) * c2 > 8.f) { alpha = ex2f((m_ref - mx) * c2); m_ref = mx; move = true; }
            if (j > 0 && __any_sync(0xffffffffu, move)) {
                if (!mbar_wait(&bars->o_done[t][(j - 1) & 1], ((j - 1) >> 1) & 1)) { atomicExch(err, 50); ok = false; break; }
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t u[32];
                    tc_ld32(to + c * 32, u);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) u[i] = __float_as_uint(__uint_as_float(u[i]) * alpha);
                    tc_st32(to + c * 32, u);
                }
            }
            const float mc = m_ref * c2;
            float rowsum = 0.f, rowsum1 = 0.f;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int k0 = c * 64 + 2 * i;
                    float e0, e1;
                    fma2(__uint_as_float(r[k0 >> 5][k0 & 31]), __uint_as_float(r[(k0 + 1) >> 5][(k0 + 1) & 31]), c2, -mc, e0, e1);
                    const float p0 = ex2f(e0), p1 = ex2f(e1);
                    const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
                    rowsum += p0; rowsum1 += p1;                  // two independent chains (the compiler may pair them)
                    pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
                }
                tc_st32(ts + c * 32, pk);
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive_(&bars->p_full[t]);
            l = l * alpha + (rowsum + rowsum1);
        }
        if (ok && !mbar_wait(&bars->o_done[t][(n_blk - 1) & 1], ((n_blk - 1) >> 1) & 1)) { atomicExch(err, 51); ok = false; }
        if (ok) {
            tc_fence_after();
            const float inv = 1.f / l;
            const int64_t grow = (int64_t)row_q + t * 128 + row;
            __nv_bfloat16* orow = out + grow * ld_o + col0;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t u[32];
                tc_ld32(to + c * 32, u);
                tc_wait_ld();
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    uint4 pk;
                    __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                    for (int v = 0; v < 4; ++v) hh[v] = __floats2bfloat162_rn(__uint_as_float(u[8 * k + 2 * v]) * inv, __uint_as_float(u[8 * k + 2 * v + 1]) * inv);
                    reinterpret_cast<uint4*>(orow)[c * 4 + k] = pk;
                }
            }
            lse[((int64_t)b * H + h) * S + qb * 256 + t * 128 + row] = m_ref * scale + logf(l);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

template <int HD>
int launch_fwd(const void* q, const void* k, const void* v, int64_t ld, void* out, int64_t ld_o, float* lse, int B, int S, int H, float scale,
               bool causal, int variant, int* err, cudaStream_t st) {
    CUtensorMap mq, mk, mv;
    const int64_t rows = (int64_t)B * S;
    if (!make_map(&mq, q, rows, (int64_t)H * HD, ld, 128, 64, true) || !make_map(&mk, k, rows, (int64_t)H * HD, ld, 128, 64, true) ||
        !make_map(&mv, v, rows, (int64_t)H * HD, ld, 128, 64, true)) return 1;
    constexpr size_t smem = (size_t)(5 * (HD / 64) + 2) * TILE_HALF_BYTES + sizeof(FaBars) + 1024;
    constexpr size_t smem2 = (size_t)(5 * (HD / 64)) * TILE_HALF_BYTES + sizeof(Fa2Bars) + 1024;
    constexpr size_t smem3 = (size_t)(6 * (HD / 64)) * TILE_HALF_BYTES + sizeof(Fa3Bars) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(flash_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
        if (cudaFuncSetAttribute(flash_fwd2_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2) != cudaSuccess) return 2;
        if (cudaFuncSetAttribute(flash_fwd3_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3) != cudaSuccess) return 2;
        configured = true;
    }
    count_launch();
    if (variant == 3 && S % 256 == 0)
        flash_fwd3_kernel<HD><<<dim3((S / 256) * H * B), FA3_THREADS, smem3, st>>>(mq, mk, mv, (__nv_bfloat16*)out, lse, S, H, ld_o, scale, causal ? 1 : 0, err);
    else if (variant >= 2)
        flash_fwd2_kernel<HD><<<dim3(S / 128, H, B), FA_THREADS, smem2, st>>>(mq, mk, mv, (__nv_bfloat16*)out, lse, S, H, ld_o, scale, causal ? 1 : 0, err);
    else
        flash_fwd_kernel<HD><<<dim3(S / 128, H, B), FA_THREADS, smem, st>>>(mq, mk, mv, (__nv_bfloat16*)out, lse, S, H, ld_o, scale, causal ? 1 : 0, err);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}


// ---------------------------------------------------------------------------------------------------------------------------
// Backward pass: two tcgen05 kernels and one small reduction, no atomics, deterministic.
//   delta[b,h,s] = sum_d dO * O                                                       (flash_delta_kernel)
//   kernel A, one CTA per 128 keys:   S^T = K Q_i^T, dP^T = V dO_i^T  ->  P^T, dS^T (threads, one key row each, written as bf16
//                                     into TMEM)  ->  dV += P^T dO_i, dK += dS^T Q_i   over the query tiles i
//   kernel B, one CTA per 128 queries: S = Q K_j^T, dP = dO V_j^T -> dS (threads) -> dQ += dS K_j   over the key tiles j
// with P = exp(S*scale - lse), dS = P * (dP - delta); the factor `scale` of dS is applied once in the epilogues.  The second
// operand of every accumulating product (dO_i, Q_i, K_j) is the SAME shared-memory tile that served as K-major operand of the
// first product, read again through an MN-major descriptor - nothing is transposed or loaded twice.
__global__ void __launch_bounds__(256) flash_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                                          float* __restrict__ delta, int64_t rows, int S, int H, int HD, int64_t ld_o,
                                                          int64_t ld_do) {
    // HD / 8 lanes per (position, head) row, 16 bytes of O and of dO per lane; the lanes of a row sit in one warp
    const int lpr = HD / 8;                                              // 8 or 16
    const int64_t gid = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int64_t item = gid / lpr;                                      // (b*S + s) * H + h
    const int part = (int)(gid % lpr);
    float acc = 0.f;
    const bool live = item < rows * H;
    int64_t bs = 0;
    int h = 0;
    if (live) {
        bs = item / H;
        h = (int)(item % H);
        const uint4 a = *reinterpret_cast<const uint4*>(o + bs * ld_o + (int64_t)h * HD + part * 8);
        const uint4 d = *reinterpret_cast<const uint4*>(dout + bs * ld_do + (int64_t)h * HD + part * 8);
        const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* dh = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 x = __bfloat1622float2(ah[k]), y = __bfloat1622float2(dh[k]);
            acc = fmaf(x.x, y.x, fmaf(x.y, y.y, acc));
        }
    }
    for (int off = lpr >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (live && part == 0) delta[((bs / S) * H + h) * S + bs % S] = acc;
}

struct FbBars {
    uint64_t res_full, ring_full[2], ring_empty[2], a_full, b_full, pa_full, pb_full, done;
    uint32_t tmem_slot, pad;
};

// KV = true: kernel A (resident K, V; ring of Q_i, dO_i; outputs dK, dV).  KV = false: kernel B (resident Q, dO; ring of K_j, V_j;
// output dQ).  In both, "first" products X = R0 . T0^T and Y = R1 . T1^T (R resident, T ring) land in TMEM columns [0,128) and
// [128,256); the threads turn them into bf16 operands in place; the accumulating products read them from TMEM.
template <int HD, bool KV>
__global__ void __launch_bounds__(FA_THREADS, 1) flash_bwd_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                  const __grid_constant__ CUtensorMap map_k,
                                                                  const __grid_constant__ CUtensorMap map_v,
                                                                  const __grid_constant__ CUtensorMap map_do, const float* __restrict__ lse,
                                                                  const float* __restrict__ delta, __nv_bfloat16* __restrict__ out0,
                                                                  __nv_bfloat16* __restrict__ out1, int S, int H, int64_t ld_out, float scale,
                                                                  int causal, int* __restrict__ err) {
    constexpr int HALVES = HD / 64;
    constexpr uint32_t QKV_BYTES = HALVES * TILE_HALF_BYTES;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sR0 = smem;                                 // resident: K (A) or Q (B)
    uint8_t* sR1 = sR0 + QKV_BYTES;                      // resident: V (A) or dO (B)
    uint8_t* sT0 = sR1 + QKV_BYTES;                      // ring [2]: Q_i (A) or K_j (B)
    uint8_t* sT1 = sT0 + 2 * QKV_BYTES;                  // ring [2]: dO_i (A) or V_j (B)
    float* s_lse = reinterpret_cast<float*>(sT1 + 2 * QKV_BYTES);       // [2][128] (kernel A: per-query vectors of the current tile)
    float* s_del = s_lse + 256;                                          // [2][128]
    FbBars* bars = reinterpret_cast<FbBars*>(s_del + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nt = S / 128;
    // 1-D grid ordered by decreasing work: kernel A starts with key tile 0 (visited by every query tile), kernel B with the last
    // query tile; all (batch, head) pairs of one tile index are adjacent
    const int n_hb = (int)gridDim.x / nt, hb = (int)blockIdx.x % n_hb, ord = (int)blockIdx.x / n_hb;
    const int tile = KV ? ord : nt - 1 - ord;
    const int h = hb % H, b = hb / H;
    // tiles of the other sequence axis that interact with this one
    const int first = KV ? (causal ? tile : 0) : 0;
    const int n_it = KV ? nt - first : (causal ? tile + 1 : nt);
    const int row_res = b * S + tile * 128, col0 = h * HD;

    if (threadIdx.x == 0) {
        mbar_init(&bars->res_full, 1);
        for (int i = 0; i < 2; ++i) { mbar_init(&bars->ring_full[i], 1); mbar_init(&bars->ring_empty[i], 1); }
        mbar_init(&bars->a_full, 1); mbar_init(&bars->b_full, 1); mbar_init(&bars->pa_full, 128); mbar_init(&bars->pb_full, 128);
        mbar_init(&bars->done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_slot;
    const uint32_t tm_x = tmem_base, tm_y = tmem_base + 128, tm_acc0 = tmem_base + 256, tm_acc1 = tmem_base + 384;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&bars->res_full, 2 * QKV_BYTES);
            for (int hf = 0; hf < HALVES; ++hf) {
                tma_load_2d(sR0 + hf * TILE_HALF_BYTES, KV ? &map_k : &map_q, col0 + hf * 64, row_res, &bars->res_full);
                tma_load_2d(sR1 + hf * TILE_HALF_BYTES, KV ? &map_v : &map_do, col0 + hf * 64, row_res, &bars->res_full);
            }
            for (int it = 0; it < n_it; ++it) {
                const int s = it & 1, row_t = b * S + (first + it) * 128;
                if (it >= 2 && !mbar_wait(&bars->ring_empty[s], ((it >> 1) & 1) ^ 1)) { atomicExch(err, 31); break; }
                mbar_expect_tx(&bars->ring_full[s], 2 * QKV_BYTES);
                for (int hf = 0; hf < HALVES; ++hf) {
                    tma_load_2d(sT0 + s * QKV_BYTES + hf * TILE_HALF_BYTES, KV ? &map_q : &map_k, col0 + hf * 64, row_t, &bars->ring_full[s]);
                    tma_load_2d(sT1 + s * QKV_BYTES + hf * TILE_HALF_BYTES, KV ? &map_do : &map_v, col0 + hf * 64, row_t, &bars->ring_full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_first = make_idesc_bf16(128, 128, 0, 0);
            constexpr uint32_t idesc_acc = make_idesc_bf16(128, HD, 0, 1);
            bool ok = mbar_wait(&bars->res_full, 0);
            if (!ok) atomicExch(err, 32);
            for (int it = 0; it < n_it && ok; ++it) {
                const int s = it & 1;
                if (!mbar_wait(&bars->ring_full[s], (it >> 1) & 1)) { atomicExch(err, 33); ok = false; break; }
                tc_fence_after();
                const uint32_t t0 = smem_u32(sT0 + s * QKV_BYTES), t1 = smem_u32(sT1 + s * QKV_BYTES);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    tc_mma_bf16(tm_x, make_desc_sw128(smem_u32(sR0 + (kk / 4) * TILE_HALF_BYTES)) + 2 * (kk % 4),
                                make_desc_sw128(t0 + (kk / 4) * TILE_HALF_BYTES) + 2 * (kk % 4), idesc_first, kk > 0 ? 1u : 0u);
                tc_commit(&bars->a_full);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    tc_mma_bf16(tm_y, make_desc_sw128(smem_u32(sR1 + (kk / 4) * TILE_HALF_BYTES)) + 2 * (kk % 4),
                                make_desc_sw128(t1 + (kk / 4) * TILE_HALF_BYTES) + 2 * (kk % 4), idesc_first, kk > 0 ? 1u : 0u);
                tc_commit(&bars->b_full);
                if (KV) {                                                // dV += P^T . dO_i   (A = P^T in the X columns, B = dO_i MN-major)
                    if (!mbar_wait(&bars->pa_full, it & 1)) { atomicExch(err, 34); ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)
                        tc_mma_bf16_ta(tm_acc0, tm_x + kk * 8, make_desc_sw128_mn(t1 + kk * 2048, TILE_HALF_BYTES, 1024), idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
                }
                // dK += dS^T . Q_i  (kernel A)   /   dQ += dS . K_j  (kernel B):  A = dS in the Y columns, B = ring tile 0 MN-major
                if (!mbar_wait(&bars->pb_full, it & 1)) { atomicExch(err, 35); ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)
                    tc_mma_bf16_ta(KV ? tm_acc1 : tm_acc0, tm_y + kk * 8, make_desc_sw128_mn(t0 + kk * 2048, TILE_HALF_BYTES, 1024), idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
                tc_commit(&bars->ring_empty[s]);
            }
            tc_commit(&bars->done);
        }
    } else {
        const int q = warp & 3, row = q * 32 + lane, tl = (int)threadIdx.x - 64;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const float c2 = scale * 1.4426950408889634f;
        const int64_t vec0 = ((int64_t)b * H + h) * S;
        float lse_row = 0.f, del_row = 0.f;
        if (!KV) { lse_row = lse[vec0 + tile * 128 + row] * 1.4426950408889634f; del_row = delta[vec0 + tile * 128 + row]; }
        bool ok = true;
        if (KV) {                                                        // per-query vectors of the first query tile
            s_lse[tl] = -lse[vec0 + first * 128 + tl] * 1.4426950408889634f;
            s_del[tl] = delta[vec0 + first * 128 + tl];
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        for (int it = 0; it < n_it && ok; ++it) {
            const int other = first + it, bs = it & 1;
            // kernel A: the per-query vectors of the NEXT tile are fetched now and parked in the other buffer at the end of this
            // iteration, so their global-memory latency hides behind the work on this tile
            float nx_lse = 0.f, nx_del = 0.f;
            if (KV && it + 1 < n_it) { nx_lse = lse[vec0 + (other + 1) * 128 + tl]; nx_del = delta[vec0 + (other + 1) * 128 + tl]; }
            if (!mbar_wait(&bars->a_full, it & 1)) { atomicExch(err, 36); ok = false; break; }
            tc_fence_after();
            const bool diag = causal && other == tile;
            uint32_t r[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tc_ld32(tm_x + lane_addr + c * 32, r[c]);
            tc_wait_ld();
            // P (kernel B: row = query, column = key) or P^T (kernel A: row = key, column = query), kept in fp32 for dS.
            // s_lse holds -lse*log2(e), read four columns per shared-memory load; two scores per packed fma.
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float4 nl = make_float4(-lse_row, -lse_row, -lse_row, -lse_row);
                    if (KV) nl = *reinterpret_cast<const float4*>(s_lse + bs * 128 + c * 32 + i);
                    float e0, e1, e2, e3;
                    fma2g(__uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]), c2, c2, nl.x, nl.y, e0, e1);
                    fma2g(__uint_as_float(r[c][i + 2]), __uint_as_float(r[c][i + 3]), c2, c2, nl.z, nl.w, e2, e3);
                    r[c][i] = __float_as_uint(ex2f(e0)); r[c][i + 1] = __float_as_uint(ex2f(e1));
                    r[c][i + 2] = __float_as_uint(ex2f(e2)); r[c][i + 3] = __float_as_uint(ex2f(e3));
                }
            if (diag) {                                                  // key index must not exceed the query index
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) if (KV ? c * 32 + i < row : c * 32 + i > row) r[c][i] = 0u;
            }
            if (KV) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t pk[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int k0 = c * 64 + 2 * i;
                        const __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(r[k0 >> 5][k0 & 31]), __uint_as_float(r[(k0 + 1) >> 5][(k0 + 1) & 31]));
                        pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
                    }
                    tc_st32(tm_x + lane_addr + c * 32, pk);
                }
                tc_wait_st();
                tc_fence_before();
                mbar_arrive_(&bars->pa_full);
            }
            if (!mbar_wait(&bars->b_full, it & 1)) { atomicExch(err, 37); ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t d0[32], d1[32], pk[32];
                tc_ld32(tm_y + lane_addr + c * 64, d0);
                tc_ld32(tm_y + lane_addr + c * 64 + 32, d1);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int k0 = c * 64 + 2 * i;                        // columns k0, k0+1
                    const float dp0 = __uint_as_float(i < 16 ? d0[2 * i] : d1[2 * i - 32]);
                    const float dp1 = __uint_as_float(i < 16 ? d0[2 * i + 1] : d1[2 * i - 31]);
                    float2 de = make_float2(del_row, del_row);
                    if (KV) de = *reinterpret_cast<const float2*>(s_del + bs * 128 + k0);
                    float t0, t1, ds0, ds1;
                    fma2g(de.x, de.y, -1.f, -1.f, dp0, dp1, t0, t1);                                  // dP - delta
                    fma2g(__uint_as_float(r[k0 >> 5][k0 & 31]), __uint_as_float(r[(k0 + 1) >> 5][(k0 + 1) & 31]), t0, t1, 0.f, 0.f, ds0, ds1);
                    const __nv_bfloat162 hh = __floats2bfloat162_rn(ds0, ds1);
                    pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
                }
                // all four loads of this row precede the stores that overwrite the first 64 columns: c = 0 writes columns [0,32)
                // after reading [0,64); c = 1 writes [32,64) after reading [64,128)
                tc_st32(tm_y + lane_addr + c * 32, pk);
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive_(&bars->pb_full);
            if (KV) {                                                    // buffer (it+1)&1 was last read in iteration it-1
                if (it + 1 < n_it) { s_lse[(bs ^ 1) * 128 + tl] = -nx_lse * 1.4426950408889634f; s_del[(bs ^ 1) * 128 + tl] = nx_del; }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
        }
        if (ok && !mbar_wait(&bars->done, 0)) { atomicExch(err, 38); ok = false; }
        if (ok) {
            tc_fence_after();
            const int64_t grow = (int64_t)row_res + row;
#pragma unroll 1
            for (int which = 0; which < (KV ? 2 : 1); ++which) {
                __nv_bfloat16* orow = (which == 0 ? out0 : out1) + grow * ld_out + col0;
                const float f = (KV && which == 0) ? 1.f : scale;         // dV needs no scale; dK and dQ carry the softmax scale
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t t[32];
                    tc_ld32((which == 0 ? tm_acc0 : tm_acc1) + lane_addr + c * 32, t);
                    tc_wait_ld();
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        uint4 pk;
                        __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                        for (int u = 0; u < 4; ++u) hh[u] = __floats2bfloat162_rn(__uint_as_float(t[8 * k + 2 * u]) * f, __uint_as_float(t[8 * k + 2 * u + 1]) * f);
                        reinterpret_cast<uint4*>(orow)[c * 4 + k] = pk;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

template <int HD>
int launch_bwd(const void* q, const void* k, const void* v, int64_t ld, const void* o, const void* dout, int64_t ld_o, const float* lse, float* delta,
               void* dq, void* dk, void* dv, int B, int S, int H, float scale, bool causal, int* err, cudaStream_t st) {
    CUtensorMap mq, mk, mv, md;
    const int64_t rows = (int64_t)B * S;
    if (!make_map(&mq, q, rows, (int64_t)H * HD, ld, 128, 64, true)) return 1100 + last_map_error();
    if (!make_map(&mk, k, rows, (int64_t)H * HD, ld, 128, 64, true)) return 12;
    if (!make_map(&mv, v, rows, (int64_t)H * HD, ld, 128, 64, true)) return 13;
    if (!make_map(&md, dout, rows, (int64_t)H * HD, ld_o, 128, 64, true)) return 14;
    constexpr size_t smem = (size_t)(6 * (HD / 64)) * TILE_HALF_BYTES + 2048 + sizeof(FbBars) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(flash_bwd_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
        if (cudaFuncSetAttribute(flash_bwd_kernel<HD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
        configured = true;
    }
    count_launch(3);
    flash_delta_kernel<<<(unsigned)((rows * H * (HD / 8) + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, rows, S, H, HD, ld_o, ld_o);
    const int64_t ld_out = (int64_t)H * HD;
    flash_bwd_kernel<HD, true><<<dim3((S / 128) * H * B), FA_THREADS, smem, st>>>(mq, mk, mv, md, lse, delta, (__nv_bfloat16*)dv, (__nv_bfloat16*)dk, S, H,
                                                                             ld_out, scale, causal ? 1 : 0, err);
    flash_bwd_kernel<HD, false><<<dim3((S / 128) * H * B), FA_THREADS, smem, st>>>(mq, mk, mv, md, lse, delta, (__nv_bfloat16*)dq, nullptr, S, H, ld_out,
                                                                              scale, causal ? 1 : 0, err);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace

bool flash_attn_supported(int S, int HD) { return S % 128 == 0 && (HD == 64 || HD == 128); }

// q, k, v: bf16 [B, S, H, HD] with a common row pitch `ld` (elements between consecutive positions; >= H*HD); out: [B, S, H, HD] with
// row pitch ld_o; lse: fp32 [B, H, S].  variant 1: P through shared memory, O in registers; variant 2: P and O stay in TMEM; variant 3: two query tiles per CTA in
// ping-pong (falls back to 2 when S is not a multiple of 256).
// Returns 0 on success.
int flash_attn_fwd(const void* q, const void* k, const void* v, int64_t ld, void* out, int64_t ld_o, float* lse, int B, int S, int H, int HD,
                   float scale, bool causal, int variant, int* err, cudaStream_t st) {
    if (!flash_attn_supported(S, HD)) return 6;
    if (HD == 128) return launch_fwd<128>(q, k, v, ld, out, ld_o, lse, B, S, H, scale, causal, variant, err, st);
    return launch_fwd<64>(q, k, v, ld, out, ld_o, lse, B, S, H, scale, causal, variant, err, st);
}

// Gradients of flash_attn_fwd.  o and dout: [B, S, H, HD] with row pitch ld_o; dq, dk, dv: contiguous [B, S, H, HD]; delta: fp32
// scratch [B, H, S].
int flash_attn_bwd(const void* q, const void* k, const void* v, int64_t ld, const void* o, const void* dout, int64_t ld_o, const float* lse,
                   float* delta, void* dq, void* dk, void* dv, int B, int S, int H, int HD, float scale, bool causal, int* err, cudaStream_t st) {
    if (!flash_attn_supported(S, HD)) return 6;
    if (HD == 128) return launch_bwd<128>(q, k, v, ld, o, dout, ld_o, lse, delta, dq, dk, dv, B, S, H, scale, causal, err, st);
    return launch_bwd<64>(q, k, v, ld, o, dout, ld_o, lse, delta, dq, dk, dv, B, S, H, scale, causal, err, st);
}

}  // namespace sg
