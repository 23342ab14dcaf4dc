// Segmented stable radix sort of |g| keys for the SuperGrok v2 step (sm_100a).
//
// Replaces thrust::sort_by_key / cub::DeviceSegmentedRadixSort / argsort in the reference
// (csrc/supergrok2_mamba_peer_kernels.cu:1540, :1865; backward_kernels.cu:2586, :3182).
//
// All tensors of a step are sorted in ONE batched sort over the packed key array: keys are the
// bit patterns of non-negative floats (monotone as unsigned integers), the payload is the global
// element index.  Four stable LSD passes over the key bytes are followed by stable passes over the
// bytes of the segment id (derived from the payload by binary search), which regroups the elements
// by tensor without disturbing the key order inside a tensor.  Work is spread evenly over the GPU
// whatever the segment sizes are.  Each pass = per-CTA digit histogram, a scan of the
// [digit][cta] table, and a stable scatter with warp-private ranking (match_any).  No atomics on
// global memory: the result is deterministic and equals a stable argsort.
#include "sg_native.h"
#include <cuda_runtime.h>

namespace sg {
namespace {

constexpr int SORT_THREADS = 256;
constexpr int SORT_WARPS = SORT_THREADS / 32;
#ifndef SG_SORT_IPT
#define SG_SORT_IPT 16
#endif
#ifndef SG_SORT_MINB
#define SG_SORT_MINB 3                  // resident CTAs per SM of the scatter (80 registers): 1,014 -> 839 us per step at 18.9 M keys
#endif
constexpr int SORT_IPT = SG_SORT_IPT;                  // items per thread
constexpr int SORT_TILE = SORT_THREADS * SORT_IPT;    // 4096 keys per CTA
constexpr int MAX_SEG = 4096;

__device__ __forceinline__ int seg_of(uint32_t gidx, const int64_t* __restrict__ seg_off, int n_seg) {
    int lo = 0, hi = n_seg;                           // seg_off[lo] <= gidx < seg_off[lo+1]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (seg_off[mid] <= (int64_t)gidx) lo = mid; else hi = mid;
    }
    return lo;
}

// digit of element for this pass: key byte (pass < 4) or segment-id byte (pass >= 4)
__device__ __forceinline__ uint32_t digit_of(uint32_t key, uint32_t val, int pass, const int64_t* seg_off, int n_seg) {
    if (pass < 4) return (key >> (8 * pass)) & 0xffu;
    return ((uint32_t)seg_of(val, seg_off, n_seg) >> (8 * (pass - 4))) & 0xffu;
}

// warp w of the CTA owns the contiguous range [tile + w*32*IPT, tile + (w+1)*32*IPT); item r of lane l is
// tile + w*32*IPT + r*32 + l, so (warp, round, lane) order equals index order: ranking in that order is stable.
__global__ void __launch_bounds__(SORT_THREADS) sort_hist_kernel(const uint32_t* __restrict__ keys,
                                                                 const uint32_t* __restrict__ vals, uint32_t* __restrict__ hist,
                                                                 const int64_t* __restrict__ seg_off, int n_seg, int64_t total,
                                                                 int pass, int n_blocks) {
    __shared__ uint32_t cnt[256];
    cnt[threadIdx.x] = 0;
    __syncthreads();
    const int64_t base = (int64_t)blockIdx.x * SORT_TILE;
    for (int r = 0; r < SORT_IPT; ++r) {
        const int64_t i = base + (int64_t)r * SORT_THREADS + threadIdx.x;
        if (i < total) atomicAdd(&cnt[digit_of(keys[i], vals[i], pass, seg_off, n_seg)], 1u);   // integer smem atomics: exact
    }
    __syncthreads();
    hist[(int64_t)threadIdx.x * n_blocks + blockIdx.x] = cnt[threadIdx.x];
}

// Row d of the [256][n_blocks] table: exclusive scan in place over the CTAs, row total to tot[d].  One CTA per digit.
__global__ void __launch_bounds__(256) sort_scan_rows_kernel(uint32_t* __restrict__ hist, uint32_t* __restrict__ tot, int n_blocks) {
    __shared__ uint32_t wsum[8];
    __shared__ uint32_t carry_s;
    uint32_t* row = hist + (int64_t)blockIdx.x * n_blocks;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int base = 0; base < n_blocks; base += 256 * 4) {
        const int i0 = base + threadIdx.x * 4;
        uint32_t v[4], s = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) { v[k] = (i0 + k < n_blocks) ? row[i0 + k] : 0u; s += v[k]; }
        uint32_t inc = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += t; }
        if (lane == 31) wsum[w] = inc;
        __syncthreads();
        uint32_t woff = 0;
#pragma unroll
        for (int ww = 0; ww < 8; ++ww) if (ww < w) woff += wsum[ww];
        uint32_t ex = carry_s + woff + (inc - s);
#pragma unroll
        for (int k = 0; k < 4; ++k) { if (i0 + k < n_blocks) row[i0 + k] = ex; ex += v[k]; }
        __syncthreads();
        if (threadIdx.x == 255) carry_s = ex;
        __syncthreads();
    }
    if (threadIdx.x == 0) tot[blockIdx.x] = carry_s;
}

// Stable scatter of one tile.  The keys are first ranked (warp-private match_any ranking, then a scan over the warps) and parked in
// shared memory in their digit order inside the tile; the tile is then written out entry by entry, so that the entries of one
// digit - which go to consecutive global positions - are stored by consecutive lanes (runs of ~16 keys = 64 bytes instead of
// isolated 4-byte writes).
__global__ void __launch_bounds__(SORT_THREADS, SG_SORT_MINB) sort_scatter_kernel(const uint32_t* __restrict__ keys_in,
                                                                    const uint32_t* __restrict__ vals_in,
                                                                    uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out,
                                                                    const uint32_t* __restrict__ hist,
                                                                    const uint32_t* __restrict__ tot,
                                                                    const int64_t* __restrict__ seg_off, int n_seg, int64_t total,
                                                                    int pass, int n_blocks) {
    __shared__ uint32_t wcnt[SORT_WARPS][256];        // per-warp running digit counts -> warp bases inside the tile's digit run
    __shared__ uint32_t gbase[256];                   // global position of this tile's first key of digit d
    __shared__ uint32_t tstart[256];                  // position of digit d inside the tile (exclusive scan of the tile's digit counts)
    __shared__ uint32_t wtot[SORT_WARPS];
    __shared__ uint32_t s_key[SORT_TILE], s_val[SORT_TILE];
    __shared__ uint8_t s_dig[SORT_TILE];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < SORT_WARPS * 256; i += SORT_THREADS) (&wcnt[0][0])[i] = 0;
    {   // digit base = exclusive scan of the 256 digit totals (thread d owns digit d)
        const uint32_t t = tot[threadIdx.x];
        uint32_t inc = t;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const uint32_t u = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += u; }
        if (lane == 31) wtot[w] = inc;
        __syncthreads();
        uint32_t woff = 0;
#pragma unroll
        for (int ww = 0; ww < SORT_WARPS; ++ww) if (ww < w) woff += wtot[ww];
        gbase[threadIdx.x] = woff + (inc - t) + hist[(int64_t)threadIdx.x * n_blocks + blockIdx.x];
    }
    __syncthreads();
    const int64_t tile0 = (int64_t)blockIdx.x * SORT_TILE;
    const int64_t wbase = tile0 + (int64_t)w * (32 * SORT_IPT);
    const int n_tile = (int)((total - tile0 < SORT_TILE) ? total - tile0 : SORT_TILE);
    uint32_t k[SORT_IPT], v[SORT_IPT], d[SORT_IPT], rk[SORT_IPT];
    // all 32 loads of the thread are issued before the ranking starts: the warp votes below are scheduling barriers, and with the
    // loads inside that loop every round waited for its own pair (ncu: 10 cycles of long-scoreboard stall per issued instruction)
#pragma unroll
    for (int r = 0; r < SORT_IPT; ++r) {
        const int64_t i = wbase + r * 32 + lane;
        const bool ok = i < total;
        k[r] = ok ? keys_in[i] : 0u;
        v[r] = ok ? vals_in[i] : 0u;
    }
#pragma unroll
    for (int r = 0; r < SORT_IPT; ++r) {
        const bool ok = wbase + r * 32 + lane < total;
        d[r] = ok ? digit_of(k[r], v[r], pass, seg_off, n_seg) : 0xffffffffu;
        const uint32_t peers = __match_any_sync(0xffffffffu, d[r]);
        const int leader = __ffs(peers) - 1;
        uint32_t prior = 0;
        if (ok && lane == leader) { prior = wcnt[w][d[r]]; wcnt[w][d[r]] = prior + __popc(peers); }
        prior = __shfl_sync(0xffffffffu, prior, leader);
        rk[r] = prior + __popc(peers & ((1u << lane) - 1u));
        __syncwarp();
    }
    __syncthreads();
    uint32_t my_cnt;
    {   // exclusive scan over warps for digit = threadIdx.x; the total is the tile's count of that digit
        uint32_t run = 0;
#pragma unroll
        for (int ww = 0; ww < SORT_WARPS; ++ww) { const uint32_t c = wcnt[ww][threadIdx.x]; wcnt[ww][threadIdx.x] = run; run += c; }
        my_cnt = run;
    }
    {   // exclusive scan of the tile's digit counts over the 256 digits
        uint32_t inc = my_cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const uint32_t u = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += u; }
        __syncthreads();                              // wtot is reused
        if (lane == 31) wtot[w] = inc;
        __syncthreads();
        uint32_t woff = 0;
#pragma unroll
        for (int ww = 0; ww < SORT_WARPS; ++ww) if (ww < w) woff += wtot[ww];
        tstart[threadIdx.x] = woff + (inc - my_cnt);
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < SORT_IPT; ++r) {
        const int64_t i = wbase + r * 32 + lane;
        if (i < total) {
            const uint32_t lp = tstart[d[r]] + wcnt[w][d[r]] + rk[r];
            s_key[lp] = k[r]; s_val[lp] = v[r]; s_dig[lp] = (uint8_t)d[r];
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_tile; e += SORT_THREADS) {
        const uint32_t dg = s_dig[e];
        const int64_t pos = (int64_t)gbase[dg] + ((uint32_t)e - tstart[dg]);
        keys_out[pos] = s_key[e];
        vals_out[pos] = s_val[e];
    }
}

}  // namespace

size_t sg2_sort_blocks(int64_t total) { return (size_t)((total + SORT_TILE - 1) / SORT_TILE); }

void sg2_segmented_sort(uint32_t* keys0, uint32_t* keys1, uint32_t* vals0, uint32_t* vals1, uint32_t* hist,
                        uint32_t* tot, const int64_t* seg_offsets_dev, int n_seg, int64_t total, int* out_buf_index, cudaStream_t s) {
    uint32_t* k[2] = {keys0, keys1};
    uint32_t* v[2] = {vals0, vals1};
    int cur = 0;
    if (total > 0) {
        const int nb = (int)sg2_sort_blocks(total);
        int seg_passes = 0;
        for (int x = n_seg - 1; x > 0; x >>= 8) ++seg_passes;     // bytes needed for the largest segment id
        for (int pass = 0; pass < 4 + seg_passes; ++pass) {
            count_launch(3);
            sort_hist_kernel<<<nb, SORT_THREADS, 0, s>>>(k[cur], v[cur], hist, seg_offsets_dev, n_seg, total, pass, nb);
            sort_scan_rows_kernel<<<256, 256, 0, s>>>(hist, tot, nb);
            sort_scatter_kernel<<<nb, SORT_THREADS, 0, s>>>(k[cur], v[cur], k[cur ^ 1], v[cur ^ 1], hist, tot, seg_offsets_dev,
                                                            n_seg, total, pass, nb);
            cur ^= 1;
        }
    }
    *out_buf_index = cur;
}

}  // namespace sg
