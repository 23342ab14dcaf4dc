// bf16 x bf16 -> fp32 GEMM on the 5th-generation tensor cores (tcgen05 / TMEM / TMA), sm_100a only.
//
//   C[M,N] = epilogue( A[M,K] . B[N,K]^T )        A and B row-major with K contiguous ("TN": x . W^T of nn.Linear)
//
// One CTA computes a 128 x BN output tile.  Warp-specialised:
//   warp 0   producer   one lane issues TMA 2-D tile loads (128-byte swizzle, no multicast) into a STAGES-deep ring
//   warp 1   MMA        allocates TMEM, one lane issues tcgen05.mma (M=128, N=BN, K=16) four times per 64-wide K block,
//                       tcgen05.commit releases the ring slot / signals the epilogue
//   warps 2-5 epilogue  tcgen05.ld 32 lanes x 32 columns at a time -> alpha*acc + beta*D + bias + diag, activation -> global
// Synchronisation is by mbarriers (full / empty per stage, one accumulator-ready barrier).  Every wait is bounded: when a
// wait runs out the waiter raises an error word in global memory, the CTA drains, frees its TMEM and returns.
//
// This kernel family replaces cuBLAS (torch::mm) on the named paths of the reference: the Newton-Schulz chain of Muon
// (csrc/ops.cpp:713-727) and the model's Linear layers.
#include "sg_native.h"
#include "tc_sm100.cuh"

namespace sg {
namespace {
using namespace tc;

constexpr int BM = 128, BK = 64;                 // BK bf16 = 128 bytes = one swizzle row
constexpr int GEMM_THREADS = 192;
struct Epilogue {
    float alpha, beta, diag;       // C = act(alpha*acc + beta*D[m,n] + bias[n] + (m==n ? diag : 0))
    const void* D; int ldd; int d_is_bf16;
    const void* bias; int bias_is_bf16;
    int act;                       // 0 none, 1 gelu (erf), 2 silu
    int c_is_bf16;
    void* C2; int ldc2;            // optional second output: C2[n, m] = C[m, n] (transposed copy, same dtype)
    int diag_off;                  // the identity is added where m + diag_off == n (a row block of a larger square matrix)
};

// All-gather fused into the GEMM (AG = true).  B (the weight, [N, K] row-major, K contiguous, ld == K) is sharded by rows over
// `world` ranks: every rank's buffer has the full [N, K] layout, rank r's rows [r*N/world, (r+1)*N/world) are valid there.
// The first `n_copy` CTAs of the launch are copiers: they pull the remote shards with plain peer loads (16 bytes per lane, eight
// loads in flight per thread) into this rank's buffer, 32 rows at a time, and bump a counter per 32-row group with a release.
// The GEMM CTAs visit the n tiles starting at this rank's own shard and continuing in the order the copiers fetch; before the
// first TMA load of a tile's B operand the producer waits (bounded) until the tile's counter shows all its remote groups, so the
// transfer of shard k+1 hides behind the MMAs of shard k and every remote byte crosses NVLink once.  Copiers never wait on
// anything, so the kernel cannot deadlock; a wait that runs out raises the error word.
struct AgArgs {
    PeerPtrs w;                 // every rank's [N, K] bf16 buffer (w.p[rank] is the local one that the B tensor map covers)
    int rank, world, n_copy;
    int* counters;              // [n tiles of BN rows] monotone counters in local memory
    int epoch;                  // call number (1, 2, ...): a tile is ready when counter >= epoch * remote_groups(tile)
    const int* epoch_ptr;       // optional: the call number is read from device memory (a launch replayed from a CUDA graph sees
                                // the value a preceding kernel of the same graph has bumped)
    PeerPtrs aux;               // RS mode: every rank's flag array
    int m_tiles_loc;            // RS mode: 128-row tiles per rank
    unsigned long long timeout_ns;
    void* c_local; int ldc;     // RS mode: this rank's reduced rows [M / world, N] (bf16)
    unsigned long long* sched;  // monotone tile ticket counter (local memory): GEMM CTAs draw tiles dynamically, because the SMs
                                // that ran a copier CTA first join the GEMM late and must take fewer tiles
};
constexpr int AG_ROWS = 32;     // rows per copy group

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

template <int BN>
__device__ void ag_copier(const AgArgs& ag, int N, int K) {
    const int rows_per_shard = N / ag.world, groups_per_shard = rows_per_shard / AG_ROWS;
    const int total = (ag.world - 1) * groups_per_shard;
    const int64_t vec_per_group = (int64_t)AG_ROWS * K * 2 / 16;
    uint4* dst_base = reinterpret_cast<uint4*>(ag.w.p[ag.rank]);
    for (int idx = blockIdx.x; idx < total; idx += ag.n_copy) {
        const int src = (ag.rank + 1 + idx / groups_per_shard) % ag.world;
        const int row0 = src * rows_per_shard + (idx % groups_per_shard) * AG_ROWS;
        const int64_t v0 = (int64_t)row0 * K * 2 / 16;
        const uint4* sp = reinterpret_cast<const uint4*>(ag.w.p[src]) + v0;
        uint4* dp = dst_base + v0;
        for (int64_t v = threadIdx.x; v < vec_per_group; v += (int64_t)blockDim.x * 8) {
            uint4 t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) if (v + (int64_t)u * blockDim.x < vec_per_group) t[u] = sp[v + (int64_t)u * blockDim.x];
#pragma unroll
            for (int u = 0; u < 8; ++u) if (v + (int64_t)u * blockDim.x < vec_per_group) dp[v + (int64_t)u * blockDim.x] = t[u];
        }
        __syncthreads();
        if (threadIdx.x == 0) { __threadfence(); red_release_gpu_add(ag.counters + row0 / BN, 1); }
    }
}

// number of 32-row groups of n tile `nt` that live on other ranks
template <int BN>
__device__ __forceinline__ int ag_remote_groups(const AgArgs& ag, int N, int nt) {
    const int rows_per_shard = N / ag.world;
    const int lo = nt * BN, hi = (lo + BN < N) ? lo + BN : N;
    const int own_lo = ag.rank * rows_per_shard, own_hi = own_lo + rows_per_shard;
    const int olo = lo > own_lo ? lo : own_lo, ohi = hi < own_hi ? hi : own_hi;
    const int own = ohi > olo ? ohi - olo : 0;
    return (hi - lo - own) / AG_ROWS;
}

// Reduce-scatter fused into the GEMM (MODE 2).  Every rank computes the full [M, N] partial product of its K slice; rows
// [o*M/world, (o+1)*M/world) belong to rank o.  The epilogue sends each finished tile straight to its owner with plain peer
// stores (bf16, 128-byte row segments) into the slot the owner keeps for this sender, then bumps the owner's arrival counter for that
// 128-row block with a system-scope release.  Tiles are visited owner by owner starting at rank+1 and ending with this rank's
// own rows, so the remote traffic leaves first and overlaps the remaining MMAs.  The epilogue of an own tile waits (bounded) until
// that 128-row block has arrived from every other sender, adds their slots to the fp32 accumulator in rank order (deterministic)
// and writes the finished rows with TMA: the reduction costs no extra pass and the own partial never touches memory.  Slots and
// counters are double-buffered by call parity: a sender may already be one call ahead of a receiver that is still reducing.
//   slots (w.p[o]):   bf16 [2 parities][world senders][M / world][N]
//   flags (aux.p[o]): int  [2 parities][world senders][m_tiles_loc]
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
    asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Tile order of the plain GEMM: groups of RASTER_GM tile rows; inside a group m varies fastest, then n.  The ~148 tiles in flight
// then cover a near-square patch (16 A panels x ~9 B panels instead of ~5 x all n panels), and B is streamed from DRAM once per
// group of 16 tile rows instead of once per tile row (n fastest re-read the operands ~7x at 8192 x 8192 x 4096).
constexpr int RASTER_GM = 16;
__host__ __device__ __forceinline__ void plain_tile_coords(int tl, int n_tiles_m, int n_tiles_n, int& mt, int& nt) {
    const int per_group = RASTER_GM * n_tiles_n;
    const int first_m = (tl / per_group) * RASTER_GM;
    const int gsz = (n_tiles_m - first_m < RASTER_GM) ? n_tiles_m - first_m : RASTER_GM;
    const int r = tl % per_group;
    mt = first_m + r % gsz;
    nt = r / gsz;
}

// Tile order of the fused all-gather GEMM: shard by shard, starting at this rank's own and continuing in the order the copiers
// fetch; inside a shard the n tiles vary fastest (a wave of CTAs then spreads over the shard's B tiles instead of all reading the
// same one).  When a shard is not a whole number of n tiles the order is m fastest over the rotated n tiles.
template <int BN>
__device__ __forceinline__ void ag_tile_coords(const AgArgs& ag, int N, int n_tiles_m, int n_tiles_n, int tl, int& m0, int& nt) {
    const int rows_per_shard = N / ag.world;
    if (rows_per_shard % BN == 0) {
        const int tps = rows_per_shard / BN, per_shard = tps * n_tiles_m;
        const int sh = (tl / per_shard + ag.rank) % ag.world, rem = tl % per_shard;
        m0 = (rem / tps) * BM;
        nt = sh * tps + rem % tps;
    } else {
        nt = ((tl / n_tiles_m) + (ag.rank * rows_per_shard) / BN) % n_tiles_n;
        m0 = (tl % n_tiles_m) * BM;
    }
}

// Persistent kernel: CTA b computes tiles b, b + gridDim.x, ...  The accumulator is double-buffered in TMEM (2 x BN columns) so
// the epilogue of tile i overlaps the MMAs of tile i+1.  The epilogue converts 32 rows x 128 bytes at a time, parks them in
// shared memory in the 128-byte-swizzled layout and lets TMA store them (coalesced, clipped at the matrix edge).
// A_MN / B_MN: the operand is stored transposed, [K, M] resp. [K, N] row-major (its M / N index contiguous).  Its stage is then
// loaded as 64-column boxes of BK rows (chunk c = columns [64c, 64c+64) at c * 8 KB) and read through an MN-major descriptor, so
// dgrad (dX = dY . W) and wgrad (dW = dY^T . X) take their operands where the forward pass left them - no transposed copies.
template <int BN, int STAGES, int MODE, bool A_MN = false, bool B_MN = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                  const __grid_constant__ CUtensorMap map_b,
                                                                  const __grid_constant__ CUtensorMap map_c, int M, int N, int K,
                                                                  int splits, Epilogue ep, int* __restrict__ err, AgArgs ag) {
    constexpr bool AG = MODE == 1, RS = MODE == 2;
    if constexpr (MODE != 0) {
        if (ag.epoch_ptr) ag.epoch = *ag.epoch_ptr;
    }
    if constexpr (AG) {
        if ((int)blockIdx.x < ag.n_copy) { ag_copier<BN>(ag, N, K); return; }
    }
    const int cta = AG ? (int)blockIdx.x - ag.n_copy : (int)blockIdx.x;          // index among the GEMM CTAs
    const int n_cta = AG ? (int)gridDim.x - ag.n_copy : (int)gridDim.x;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t STG_BYTES = 32 * 128;                       // one staging buffer: 32 rows x 128 bytes
    uint8_t* staging = smem + STAGES * STAGE_BYTES;                 // [4 warps][2][STG_BYTES]
    uint64_t* full = reinterpret_cast<uint64_t*>(staging + 4 * 2 * STG_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;                            // [2]
    uint64_t* acc_empty = acc_full + 2;                             // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    uint64_t* sched_full = reinterpret_cast<uint64_t*>(tmem_slot + 2);      // [2]  (AG only) tile ticket hand-off producer -> MMA / epilogue
    uint64_t* sched_empty = sched_full + 2;                                 // [2]
    int* sched_tile = reinterpret_cast<int*>(sched_empty + 2);             // [2]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // split-K: work item = (split, m tile, n tile); split s covers k blocks [s*KB, (s+1)*KB) and writes an fp32 partial tile into
    // rows [s*Mpad, s*Mpad + M) of the workspace that map_c describes (summed by gemm_splitk_reduce_kernel)
    const int KB_all = (K + BK - 1) / BK;
    const int KB = (KB_all + splits - 1) / splits;
    const int n_tiles_n = (N + BN - 1) / BN, n_tiles_m = (M + BM - 1) / BM;
    const int tiles_per_split = n_tiles_n * n_tiles_m, n_tiles = tiles_per_split * splits;
    const int Mpad = n_tiles_m * BM;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        if constexpr (AG) { for (int b = 0; b < 2; ++b) { mbar_init(&sched_full[b], 1); mbar_init(&sched_empty[b], 5); } }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)(2 * BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            // AG: tiles are drawn from a ticket counter (one terminating draw per CTA, so call e starts at (e-1)*(n_tiles+n_cta));
            // the ticket goes to the MMA and epilogue warps through a two-slot mailbox in shared memory.
            const unsigned long long sched_base = AG ? (unsigned long long)(ag.epoch - 1) * (unsigned long long)(n_tiles + n_cta) : 0ull;
            uint32_t tcount = 0;
            for (int tile = cta; ok; tile += n_cta, ++tcount) {
                if constexpr (AG) {
                    const uint32_t slot = tcount & 1;
                    if (tcount >= 2 && !mbar_wait(&sched_empty[slot], ((tcount >> 1) & 1) ^ 1)) { atomicExch(err, 6); ok = false; break; }
                    const unsigned long long ticket = atomicAdd(ag.sched, 1ull) - sched_base;
                    tile = ticket < (unsigned long long)n_tiles ? (int)ticket : -1;
                    sched_tile[slot] = tile;
                    mbar_arrive(&sched_full[slot]);
                    if (tile < 0) break;
                } else if (tile >= n_tiles) break;
                const int sp = tile / tiles_per_split, tl = tile % tiles_per_split;
                int m0, n0;
                { int mt_, nt_; plain_tile_coords(tl, n_tiles_m, n_tiles_n, mt_, nt_); m0 = mt_ * BM; n0 = nt_ * BN; }
                const int kb0 = sp * KB;
                if constexpr (RS) {                                // owner by owner from rank+1, own rows last; n fastest
                    const int per_owner = ag.m_tiles_loc * n_tiles_n, owner = (ag.rank + 1 + tl / per_owner) % ag.world;
                    m0 = (owner * ag.m_tiles_loc + (tl % per_owner) / n_tiles_n) * BM; n0 = ((tl % per_owner) % n_tiles_n) * BN;
                }
                if constexpr (AG) {
                    int nt;
                    ag_tile_coords<BN>(ag, N, n_tiles_m, n_tiles_n, tl, m0, nt);
                    n0 = nt * BN;
                    const int need = ag.epoch * ag_remote_groups<BN>(ag, N, nt);
                    if (need > 0) {
                        const unsigned long long t0 = globaltimer_ns();
                        while (ld_acquire_gpu(ag.counters + nt) < need) {
                            if (globaltimer_ns() - t0 > 2000000000ull) { atomicExch(err, 5); ok = false; break; }
                            __nanosleep(200);
                        }
                        if (!ok) break;
                        asm volatile("fence.proxy.async.global;" ::: "memory");     // peer data was written by generic-proxy stores
                    }
                }
                for (int kb = 0; kb < KB; ++kb, ++it) {           // k blocks past the end of K are zero-filled by TMA
                    const int s = it % STAGES;
                    if (it >= (uint32_t)STAGES && !mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1)) { atomicExch(err, 1); ok = false; break; }
                    uint8_t* a_dst = smem + s * STAGE_BYTES;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    if constexpr (A_MN) {
#pragma unroll
                        for (int c = 0; c < BM / 64; ++c) tma_load_2d(a_dst + c * (BK * 128), &map_a, m0 + 64 * c, (kb0 + kb) * BK, &full[s]);
                    } else tma_load_2d(a_dst, &map_a, (kb0 + kb) * BK, m0, &full[s]);
                    if constexpr (B_MN) {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c) tma_load_2d(a_dst + A_BYTES + c * (BK * 128), &map_b, n0 + 64 * c, (kb0 + kb) * BK, &full[s]);
                    } else tma_load_2d(a_dst + A_BYTES, &map_b, (kb0 + kb) * BK, n0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D fp32, A/B bf16, both K-major, N>>3 at bit 17, M>>4 at bit 24
            constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
            uint32_t it = 0, t = 0;
            bool ok = true;
            for (int tile = cta; ok; tile += n_cta, ++t) {
                if constexpr (AG) {
                    if (!mbar_wait(&sched_full[t & 1], (t >> 1) & 1)) { atomicExch(err, 7); break; }
                    tile = sched_tile[t & 1];
                    mbar_arrive(&sched_empty[t & 1]);
                }
                if (tile < 0 || tile >= n_tiles) break;
                const uint32_t buf = t & 1;
                if (t >= 2 && !mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1)) { atomicExch(err, 4); ok = false; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < KB && ok; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full[s], (it / STAGES) & 1)) { atomicExch(err, 2); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
                    // K-major: 16 bf16 = 32 bytes per MMA, the start address advances by 2 (16-byte units); MN-major: 16 K rows of
                    // 128 bytes = 2048 bytes per MMA, 64-column chunks BK * 128 bytes apart
                    const uint64_t da = A_MN ? make_desc_sw128_mn(a_addr, BK * 128, 1024) : make_desc_sw128(a_addr);
                    const uint64_t db = B_MN ? make_desc_sw128_mn(a_addr + A_BYTES, BK * 128, 1024) : make_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (int k4 = 0; k4 < BK / 16; ++k4)
                        tc_mma_bf16(tmem_d, da + (A_MN ? 128 : 2) * k4, db + (B_MN ? 128 : 2) * k4, idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
                    tc_commit(&empty[s]);                         // slot reusable once these MMAs have read it
                }
                tc_commit(&acc_full[buf]);                        // accumulator of this tile complete (also arrives when bailing out)
            }
        }
    } else {
        const int q = warp & 3;                                   // TMEM lane quarter this warp may access
        uint8_t* stg = staging + (warp - 2) * 2 * STG_BYTES;
        uint32_t t = 0, sbuf = 0;
        bool ok = true;
        for (int tile = cta; ok; tile += n_cta, ++t) {
            if constexpr (AG) {
                int tk = 0;
                bool got = true;
                if (lane == 0) {
                    got = mbar_wait(&sched_full[t & 1], (t >> 1) & 1);
                    if (got) { tk = sched_tile[t & 1]; mbar_arrive(&sched_empty[t & 1]); } else atomicExch(err, 8);
                }
                got = __shfl_sync(0xffffffffu, (int)got, 0) != 0;
                tile = __shfl_sync(0xffffffffu, tk, 0);
                if (!got) break;
            }
            if (tile < 0 || tile >= n_tiles) break;
            const int sp = tile / tiles_per_split, tl = tile % tiles_per_split;
            int m0, n0;
            { int mt_, nt_; plain_tile_coords(tl, n_tiles_m, n_tiles_n, mt_, nt_); m0 = mt_ * BM; n0 = nt_ * BN; }
            if constexpr (AG) {
                int nt;
                ag_tile_coords<BN>(ag, N, n_tiles_m, n_tiles_n, tl, m0, nt);
                n0 = nt * BN;
            }
            int rs_owner = 0, rs_mloc = 0;
            if constexpr (RS) {
                const int per_owner = ag.m_tiles_loc * n_tiles_n;
                rs_owner = (ag.rank + 1 + tl / per_owner) % ag.world;
                rs_mloc = (tl % per_owner) / n_tiles_n;
                m0 = (rs_owner * ag.m_tiles_loc + rs_mloc) * BM; n0 = ((tl % per_owner) % n_tiles_n) * BN;
            }
            const uint32_t buf = t & 1;
            if (!mbar_wait(&acc_full[buf], (t >> 1) & 1)) { if (lane == 0) atomicExch(err, 3); ok = false; break; }
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            bool rs_own = false;
            if constexpr (RS) {
                rs_own = rs_owner == ag.rank;
                if (!rs_own) sbuf = 0;                            // remote tiles pair the buffers (they all precede the TMA-stored own tiles)
                if (rs_own && ag.world > 1) {                     // every other sender's part of this 128-row block must have arrived
                    int good = 1;
                    if (lane == 0) {
                        const int parity = (ag.epoch - 1) & 1, target = ((ag.epoch - 1) / 2 + 1) * 4 * n_tiles_n;
                        const int* fl = reinterpret_cast<const int*>(ag.aux.p[ag.rank]) + parity * ag.world * ag.m_tiles_loc + rs_mloc;
                        const unsigned long long t0 = globaltimer_ns();
                        for (int src = 0; src < ag.world && good; ++src) {
                            if (src == ag.rank) continue;
                            while (ld_acquire_sys(fl + src * ag.m_tiles_loc) < target) {
                                if (globaltimer_ns() - t0 > ag.timeout_ns) { atomicExch(err, 9); good = 0; break; }
                                __nanosleep(200);
                            }
                        }
                    }
                    good = __shfl_sync(0xffffffffu, good, 0);
                    if (!good) { ok = false; break; }
                }
            }
            constexpr int CPC = 32;                               // accumulator columns per tcgen05.ld
            const int cols_per_box = ep.c_is_bf16 ? 64 : 32;      // 128 bytes of output per row
#pragma unroll 1
            for (int c = 0; c < BN; c += cols_per_box) {
                if (n0 + c >= N) break;
                // wait until the TMA store that last used this staging buffer has read it
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                __syncwarp();
                uint8_t* sb = stg + sbuf * STG_BYTES;
                for (int h = 0; h < cols_per_box; h += CPC) {
                    uint32_t r[32];
                    tc_ld32(tmem_base + buf * BN + ((uint32_t)(q * 32) << 16) + (uint32_t)(c + h), r);
                    tc_wait_ld();
                    if constexpr (RS) {
                        if (rs_own) {                             // add the other ranks' partial rows (bf16 slots) in rank order
                            const int Mloc = M / ag.world, parity = (ag.epoch - 1) & 1;
                            for (int src = 0; src < ag.world; ++src) {
                                if (src == ag.rank) continue;
                                const uint4* sp4 = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(ag.w.p[ag.rank]) +
                                    ((int64_t)(parity * ag.world + src) * Mloc + rs_mloc * BM + q * 32 + lane) * N + n0 + c + h);
                                uint4 t4[4];
#pragma unroll
                                for (int k = 0; k < 4; ++k) t4[k] = __ldcg(sp4 + k);
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&t4[k]);
#pragma unroll
                                    for (int u = 0; u < 4; ++u) {
                                        const float2 f = __bfloat1622float2(hh[u]);
                                        r[8 * k + 2 * u] = __float_as_uint(__uint_as_float(r[8 * k + 2 * u]) + f.x);
                                        r[8 * k + 2 * u + 1] = __float_as_uint(__uint_as_float(r[8 * k + 2 * u + 1]) + f.y);
                                    }
                                }
                            }
                        }
                    }
                    const bool plain = (ep.D == nullptr) && (ep.bias == nullptr) && ep.diag == 0.f && ep.act == 0 && ep.alpha == 1.f;
                    if (!plain) {
                        // bias of these 32 columns: one load per lane, handed round by shuffles (a load per element made the
                        // epilogue wait on memory 32 times per chunk)
                        float bias_l = 0.f;
                        if (ep.bias && n0 + c + h + lane < N)
                            bias_l = ep.bias_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ep.bias)[n0 + c + h + lane])
                                                     : reinterpret_cast<const float*>(ep.bias)[n0 + c + h + lane];
                        // alpha and bias only (a Linear forward): one FMA per element, no per-element branches.  The general loop
                        // below took 360 us for a 32768 x 1536 x 512 product with a bias against 50 us without one.
                        const bool simple = (ep.D == nullptr) && ep.diag == 0.f && ep.act == 0;
                        if (simple) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                r[j] = __float_as_uint(fmaf(ep.alpha, __uint_as_float(r[j]), __shfl_sync(0xffffffffu, bias_l, j)));
                        } else
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int col = n0 + c + h + j;
                            float v = ep.alpha * __uint_as_float(r[j]);
                            const float bias_j = __shfl_sync(0xffffffffu, bias_l, j);
                            if (row < M && col < N) {
                                if (ep.D) v += ep.beta * (ep.d_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ep.D)[(int64_t)row * ep.ldd + col])
                                                                       : reinterpret_cast<const float*>(ep.D)[(int64_t)row * ep.ldd + col]);
                                v += bias_j;
                            }
                            if (row + ep.diag_off == col) v += ep.diag;
                            if (ep.act == 1) v = 0.5f * v * (1.f + erff(v * 0.70710678f));
                            else if (ep.act == 2) v = v / (1.f + __expf(-v));
                            r[j] = __float_as_uint(v);
                        }
                    }
                    if (ep.C2 && row < M) {
                        if (ep.c_is_bf16) { __nv_bfloat16* d2 = reinterpret_cast<__nv_bfloat16*>(ep.C2);
#pragma unroll                                                    // full unroll: r[] must stay in registers (no dynamic index)
                            for (int j = 0; j < 32; ++j) if (n0 + c + h + j < N) d2[(int64_t)(n0 + c + h + j) * ep.ldc2 + row] = __float2bfloat16_rn(__uint_as_float(r[j]));
                        } else { float* d2 = reinterpret_cast<float*>(ep.C2);
#pragma unroll
                            for (int j = 0; j < 32; ++j) if (n0 + c + h + j < N) d2[(int64_t)(n0 + c + h + j) * ep.ldc2 + row] = __uint_as_float(r[j]);
                        }
                    }
                    // park this lane's row segment in the swizzled staging tile: 16-byte chunk k of row `lane` lives at chunk k ^ (lane & 7)
                    uint8_t* rowp = sb + lane * 128;
                    if (ep.c_is_bf16) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {             // 32 columns -> 64 bytes -> 4 chunks
                            uint4 o;
                            __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                            for (int u = 0; u < 4; ++u) hh[u] = __floats2bfloat162_rn(__uint_as_float(r[8 * k + 2 * u]), __uint_as_float(r[8 * k + 2 * u + 1]));
                            const int chunk = (h / 8) + k;        // h is 0 or 32 -> chunks 0..3 or 4..7
                            *reinterpret_cast<uint4*>(rowp + ((chunk ^ (lane & 7)) << 4)) = o;
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 8; ++k)
                            *reinterpret_cast<uint4*>(rowp + ((k ^ (lane & 7)) << 4)) = make_uint4(r[4 * k], r[4 * k + 1], r[4 * k + 2], r[4 * k + 3]);
                    }
                }
                if (RS && !rs_own) {
                    // Two adjacent 64-column chunks are parked in the two staging buffers and leave together, so that every row
                    // segment that crosses NVLink is 256 contiguous bytes (2 rows of 16 lanes per store instruction).
                    const bool last = (c + cols_per_box >= BN) || (n0 + c + cols_per_box >= N);
                    if (sbuf == 1 || last) {
                        __syncwarp();
                        const int nb = (int)sbuf + 1, c_base = c - (int)sbuf * cols_per_box;
                        const int Mloc = M / ag.world, parity = (ag.epoch - 1) & 1;
                        __nv_bfloat16* slot = reinterpret_cast<__nv_bfloat16*>(ag.w.p[rs_owner]) + ((int64_t)(parity * ag.world + ag.rank) * Mloc) * N;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int rr = i * 2 + (lane >> 4), j = lane & 15, b = j >> 3, ch = j & 7;
                            if (b < nb) {
                                const uint4 val = *reinterpret_cast<const uint4*>(stg + b * STG_BYTES + rr * 128 + ((ch ^ (rr & 7)) << 4));
                                const int lrow = rs_mloc * BM + q * 32 + rr;
                                *(reinterpret_cast<uint4*>(slot + (int64_t)lrow * N + n0 + c_base) + j) = val;
                            }
                        }
                        __syncwarp();
                        sbuf = 1;                                 // toggled to 0 below: the next pair starts in buffer 0
                    }
                } else {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {                           // RS: map_c covers this rank's [M / world, N] rows
                        tma_store_2d(&map_c, sb, n0 + c, RS ? rs_mloc * BM + q * 32 : sp * Mpad + m0 + q * 32);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
                sbuf ^= 1;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);          // this warp no longer reads the TMEM buffer
            if constexpr (RS) {                                   // this warp's part of the tile has left: tell the owner
                if (lane == 0 && !rs_own) {
                    __threadfence_system();
                    const int parity = (ag.epoch - 1) & 1;
                    red_release_sys_add(reinterpret_cast<int*>(ag.aux.p[rs_owner]) + (parity * ag.world + ag.rank) * ag.m_tiles_loc + rs_mloc, 1);
                }
            }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * BN)) : "memory");
    }
}

// sums the split-K partial tiles (fixed order) and applies the epilogue
__global__ void __launch_bounds__(256) gemm_splitk_reduce_kernel(const float* __restrict__ ws, int splits, int Mpad, int ldw, int M, int N,
                                                                 Epilogue ep, void* __restrict__ C, int ldc) {
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= (int64_t)M * N) return;
    const int row = (int)(idx / N), col = (int)(idx % N);
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += ws[((int64_t)s * Mpad + row) * ldw + col];
    float v = ep.alpha * acc;
    if (ep.D) v += ep.beta * (ep.d_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ep.D)[(int64_t)row * ep.ldd + col])
                                           : reinterpret_cast<const float*>(ep.D)[(int64_t)row * ep.ldd + col]);
    if (ep.bias) v += ep.bias_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ep.bias)[col]) : reinterpret_cast<const float*>(ep.bias)[col];
    if (row + ep.diag_off == col) v += ep.diag;
    if (ep.act == 1) v = 0.5f * v * (1.f + erff(v * 0.70710678f));
    else if (ep.act == 2) v = v / (1.f + __expf(-v));
    if (ep.c_is_bf16) reinterpret_cast<__nv_bfloat16*>(C)[(int64_t)row * ldc + col] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(C)[(int64_t)row * ldc + col] = v;
    if (ep.C2) {
        if (ep.c_is_bf16) reinterpret_cast<__nv_bfloat16*>(ep.C2)[(int64_t)col * ep.ldc2 + row] = __float2bfloat16_rn(v);
        else reinterpret_cast<float*>(ep.C2)[(int64_t)col * ep.ldc2 + row] = v;
    }
}

// ---- host side -------------------------------------------------------------------------------------------------
}  // namespace
static int g_map_error = 0;                      // CUresult of the most recent encode (diagnostics only)
bool tc::make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld_elems, int box_rows, int box_cols, bool bf16) {
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld_elems * (bf16 ? 2 : 4)};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    // The driver entry point is looked up through the runtime, so that the module links against cudart only and loads on a host
    // that has no driver library (a build-only machine).
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) fn = nullptr;
        return reinterpret_cast<EncodeFn>(fn);
    }();
    if (!encode) { g_map_error = -1; return false; }
    CUresult r = encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                                              const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_ERROR_INVALID_CONTEXT) {
        // A host thread that has made no runtime call yet (an autograd worker thread, for one) has no current context for the
        // driver API: bind the primary context of the current device and try once more.
        cudaFree(nullptr);
        r = encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    g_map_error = (int)r;
    return r == CUDA_SUCCESS;
}
int tc::last_map_error() { return g_map_error; }
namespace {

int num_sms() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

template <int BN, int STAGES, int MODE = 0, bool A_MN = false, bool B_MN = false>
int launch(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const Epilogue& ep_in, void* C, int ldc, float* ws,
           int64_t ws_floats, int* err, cudaStream_t s, const AgArgs& ag = AgArgs{}) {
    CUtensorMap ma, mb, mc;
    // K-major operand: [rows = M or N, cols = K], box BM (BN) x 64; transposed operand: [rows = K, cols = M or N], box 64 x 64
    if (!(A_MN ? make_map(&ma, A, K, M, lda, BK, 64, true) : make_map(&ma, A, M, K, lda, BM, BK, true))) return 1;
    if (!(B_MN ? make_map(&mb, B, K, N, ldb, BK, 64, true) : make_map(&mb, B, N, K, ldb, BN, BK, true))) return 1;
    // split-K when the output has too few tiles to fill the GPU and K is long
    const int tiles_mn = ((N + BN - 1) / BN) * ((M + BM - 1) / BM);
    const int KB_all = (K + BK - 1) / BK;
    const int Mpad = ((M + BM - 1) / BM) * BM, ldw = ((N + 3) / 4) * 4;
    int splits = 1;
    if (ws != nullptr && tiles_mn * 2 <= num_sms() && KB_all >= 16) {
        splits = num_sms() / tiles_mn;
        if (splits > KB_all / 4) splits = KB_all / 4;
        while (splits > 1 && (int64_t)splits * Mpad * ldw > ws_floats) --splits;
        if (splits < 1) splits = 1;
    }
    Epilogue ep = ep_in;
    if (splits > 1) {
        ep = Epilogue{1.f, 0.f, 0.f, nullptr, 0, 0, nullptr, 0, 0, 0, nullptr, 0, 0};   // plain fp32 partial sums
        if (!make_map(&mc, ws, (int64_t)splits * Mpad, N, ldw, 32, 32, false)) return 4;
    } else if (!make_map(&mc, C, MODE == 2 ? M / ag.world : M, N, ldc, 32, ep.c_is_bf16 ? 64 : 32, ep.c_is_bf16 != 0)) return 4;
    constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 4 * 2 * 4096 + 1024 + 256;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tn_kernel<BN, STAGES, MODE, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 2;
        configured = true;
    }
    const int tiles = tiles_mn * splits;
    // copier CTAs (all-gather mode) come first in the grid; an SM that ran one takes a GEMM CTA afterwards
    const int grid = (tiles < num_sms() ? tiles : num_sms()) + (MODE == 1 ? ag.n_copy : 0);
    count_launch();
    gemm_tn_kernel<BN, STAGES, MODE, A_MN, B_MN><<<grid, GEMM_THREADS, smem, s>>>(ma, mb, mc, M, N, K, splits, ep, err, ag);
    if (splits > 1) {
        count_launch();
        gemm_splitk_reduce_kernel<<<(unsigned)(((int64_t)M * N + 255) / 256), 256, 0, s>>>(ws, splits, Mpad, ldw, M, N, ep_in, C, ldc);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace

// (tile row, tile column) of work item `tile` of the plain GEMM, as the kernel computes it: lets the host check that the order
// visits every tile exactly once.
void gemm_plain_tile_coords(int tile, int n_tiles_m, int n_tiles_n, int* mt, int* nt) { plain_tile_coords(tile, n_tiles_m, n_tiles_n, *mt, *nt); }

// C = act(alpha * A[M,K] . B[N,K]^T + beta * D + bias + diag*I); A, B bf16 with leading dimensions lda / ldb (elements, multiples of 8).
// a_t / b_t: the operand is passed transposed, as a [K, M] resp. [K, N] row-major matrix (supported: none, b_t, a_t && b_t).
// Returns 0 on success.  `err` (device int, zeroed by the caller) becomes non-zero if a pipeline wait timed out.
int gemm_bf16_tn(const void* A, int lda, const void* B, int ldb, int M, int N, int K, float alpha, float beta, const void* D, int ldd,
                 bool d_bf16, const void* bias, bool bias_bf16, float diag, int act, void* C, int ldc, bool c_bf16, void* C2, int ldc2,
                 float* splitk_ws, int64_t splitk_ws_floats, int* err, cudaStream_t s, bool a_t, bool b_t) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    Epilogue ep{alpha, beta, diag, D, ldd, d_bf16 ? 1 : 0, bias, bias_bf16 ? 1 : 0, act, c_bf16 ? 1 : 0, C2, ldc2, 0};
    // the output goes through TMA: its base must be 16-byte aligned and its row pitch a multiple of 16 bytes
    if ((reinterpret_cast<uintptr_t>(C) & 15) != 0 || (ldc * (c_bf16 ? 2 : 4)) % 16 != 0) return 5;
    if (a_t && !b_t) return 7;                               // not instantiated (no caller needs A^T . B^T-free form)
#define SG_GEMM_GO(AT, BT) \
    { if (N > 128) return launch<256, 4, 0, AT, BT>(A, lda, B, ldb, M, N, K, ep, C, ldc, splitk_ws, splitk_ws_floats, err, s); \
      return launch<128, 6, 0, AT, BT>(A, lda, B, ldb, M, N, K, ep, C, ldc, splitk_ws, splitk_ws_floats, err, s); }
    if (a_t) SG_GEMM_GO(true, true)
    if (b_t) SG_GEMM_GO(false, true)
    SG_GEMM_GO(false, false)
#undef SG_GEMM_GO
}

// C[M, N] = A[M, K] . Wfull[N, K]^T where Wfull is assembled inside the kernel from the row shards of `world` ranks (see AgArgs).
// w_peers[r] is rank r's [N, K] bf16 buffer (contiguous rows); counters: int[ceil(N / 256)] in local memory, zeroed once by the
// caller; sched: one 64-bit ticket counter, zeroed once by the caller; epoch counts the calls that used these counters (1, 2, ...)
// and every call with the same counters must have the same M, N and grid.  N must be a multiple of world * 32.
// Epilogue: C = alpha * acc + beta * D + diag * [m + diag_off == n], optional transposed copy C2 (the row-sharded Newton-Schulz
// iteration of Muon builds its polynomial a I + b G + c G G and hands X on in both layouts from here).
int gemm_bf16_tn_allgather(const void* A, int lda, const PeerPtrs& w_peers, int rank, int world, int M, int N, int K, void* C, int ldc,
                           bool c_bf16, int* counters, void* sched, int epoch, int n_copy, int* err, cudaStream_t s, float alpha,
                           float beta, const void* D, int ldd, bool d_bf16, float diag, int diag_off, void* C2, int ldc2, const int* epoch_ptr) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (world < 1 || world > MAX_RANKS || N % (world * AG_ROWS) != 0 || K % 8 != 0) return 6;
    if ((reinterpret_cast<uintptr_t>(C) & 15) != 0 || (ldc * (c_bf16 ? 2 : 4)) % 16 != 0) return 5;
    Epilogue ep{alpha, beta, diag, D, ldd, d_bf16 ? 1 : 0, nullptr, 0, 0, c_bf16 ? 1 : 0, C2, ldc2, diag_off};
    AgArgs ag{};
    ag.w = w_peers; ag.rank = rank; ag.world = world; ag.n_copy = world > 1 ? n_copy : 0; ag.counters = counters; ag.epoch = epoch; ag.epoch_ptr = epoch_ptr;
    ag.sched = reinterpret_cast<unsigned long long*>(sched);
    // one tile width (256 rows) for every shape, so the counters have a fixed meaning; a tile that straddles two shards simply
    // waits for the remote groups of both
    return launch<256, 4, 1>(A, lda, w_peers.p[rank], K, M, N, K, ep, C, ldc, nullptr, 0, err, s, ag);
}

// Reduce-scatter fused into the GEMM: every rank passes its K slice A[M, Kloc], B[N, Kloc]; rank r receives
// C_local[M / world, N] = sum over ranks of (A . B^T)[r*M/world : (r+1)*M/world] in bf16 (fp32 accumulation, rank order).
// slots[o] / flags[o]: rank o's slot and flag buffers (layouts above the kernel); flags are zeroed once by the caller and epoch
// counts the calls (1, 2, ...).  M must be a multiple of world * 128 and N of 64.
int gemm_bf16_tn_reducescatter(const void* A, int lda, const void* B, int ldb, int M, int N, int K, const PeerPtrs& slots, const PeerPtrs& flags,
                               int rank, int world, void* c_local, int ldc, int epoch, unsigned long long timeout_ns, int* err, cudaStream_t s,
                               const int* epoch_ptr) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (world < 1 || world > MAX_RANKS || M % (world * BM) != 0 || N % 64 != 0 || ldc % 8 != 0) return 6;
    Epilogue ep{1.f, 0.f, 0.f, nullptr, 0, 0, nullptr, 0, 0, 1, nullptr, 0, 0};
    AgArgs ag{};
    ag.w = slots; ag.aux = flags; ag.rank = rank; ag.world = world; ag.epoch = epoch; ag.epoch_ptr = epoch_ptr; ag.m_tiles_loc = M / world / BM;
    ag.timeout_ns = timeout_ns; ag.c_local = c_local; ag.ldc = ldc;
    if (N > 128) return launch<256, 4, 2>(A, lda, B, ldb, M, N, K, ep, c_local, ldc, nullptr, 0, err, s, ag);
    return launch<128, 6, 2>(A, lda, B, ldb, M, N, K, ep, c_local, ldc, nullptr, 0, err, s, ag);
}

}  // namespace sg
