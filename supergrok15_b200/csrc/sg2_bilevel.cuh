// Adjoint of the bidirectional Mamba-3 scan (bilevel meta-learning path), included at the end of sg2_kernels.cu so it
// shares the __constant__ weight block of that translation unit.
//
// The reference runs this adjoint serially: one 16-thread CTA per parameter tensor walks N timesteps backwards
// (csrc/supergrok2_mamba_peer_backward_kernels.cu:1043, :1506) and drops the cross-column terms of d_x.  Here the adjoint
// uses the same chunk decomposition as the forward scan, so every SM works on it:
//
//   adj 1   per chunk: aggregate of the reverse recurrence  dh[t-1] = M_t^T (dh[t] + dy_t C_t)   (prefix product walked
//           forwards from the chunk start, with the same 2^-100 early exit as the forward aggregates)
//   adj 2   carry: dh arriving at the end of every chunk (chunks in reverse order; the last chunk receives zero)
//   adj 3   per chunk: re-run the chunk forwards storing the state at every 16-step tile boundary (global scratch), then
//           walk the tiles backwards: recompute the 16 states of the tile into shared memory, run the exact adjoint of
//           each timestep, accumulate parameter gradients privately per lane
//   adj 4   fixed-order reduction of the per-item partial gradients
//
// Because x, z, dt, B and C are affine in (g, s) (SG2Pack::AFF* tables), their weight gradients are gradients of the
// TABLES:  dU[j][k] += d value_j[t] * (g_t, s_t, 1)[k].  The chain rule from the tables to input_proj / in_proj / dt_proj /
// B_proj / C_proj is a handful of tiny matrix products done by autograd on the host.  This formulation contains the
// cross-column terms exactly (every column's dependence on B_s and C_s goes through the shared tables).
// Per direction the kernel produces NG = 138 + 128 gradient values:
//   [0,256)    d A_log [16][16]          [256,384)  d rope_freq [16][8]      [384,400)  d D [16]
//   [400,448)  d U_x [16][3]   [448,496) d U_z   [496,544) d U_dt   [544,592) d U_B [16][3]   [592,640) d U_C [16][3]
//   [640,768)  d out_proj [8][16]
#pragma once

namespace sg {
namespace {

constexpr int BL_TILE = 16;                    // timesteps per backward tile
constexpr int BL_ITEMS = 4;                    // items per CTA (64 threads)
constexpr int BL_THREADS = BL_ITEMS * 16;
constexpr int BL_NG = 768;                     // gradient values per direction (layout above)
constexpr int BL_LANE_ACC = 16 + 8 + 1 + 9 + 8;   // register-resident accumulators per lane: dah, df, dD, dUx/Uz/Udt, dWout column
constexpr int BL_ROW = 60;                     // floats per timestep row in shared memory: B16 C16 (g,s,-,-) gout16 dctx8

// g_out_j[t] = sum_d dctx[t][d] * Wout[d][j]  and  B, C of the timestep: lane l = timestep
template <int DIR>
__device__ __forceinline__ void bl_stage_a(float* __restrict__ tile, const float2* __restrict__ gs, const uint32_t* __restrict__ vals_sorted,
                                           const float* __restrict__ dctx, int64_t off, int n, int u, bool valid, int l) {
    constexpr int W = (DIR == 0) ? P::DIR0 : P::DIR1;
    constexpr int AF = (DIR == 0) ? P::AFF0 : P::AFF1;
    if (!valid) return;
    float4* row = reinterpret_cast<float4*>(tile + l * BL_ROW);
    const int pos = (DIR == 0) ? u : (n - 1 - u);
    const float2 v = gs[off + pos];
    float bc[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        const int w = AF + P::A_B + 3 * k;
        bc[k] = fmaf(c_w[w], v.x, fmaf(c_w[w + 1], v.y, c_w[w + 2]));
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) row[q] = make_float4(bc[4 * q], bc[4 * q + 1], bc[4 * q + 2], bc[4 * q + 3]);
    row[8] = make_float4(v.x, v.y, 0.f, 0.f);
    const uint32_t orig = vals_sorted[off + pos];
    const float4* dc = reinterpret_cast<const float4*>(dctx + (int64_t)orig * 16 + DIR * 8);
    const float4 d0 = dc[0], d1 = dc[1];
    const float d8[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
    float go[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        float acc = 0.f;
#pragma unroll
        for (int d = 0; d < 8; ++d) acc = fmaf(d8[d], c_w[W + P::D_OUT + d * 16 + j], acc);
        go[j] = acc;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) row[9 + q] = make_float4(go[4 * q], go[4 * q + 1], go[4 * q + 2], go[4 * q + 3]);
    row[13] = d0; row[14] = d1;
}

// ---- adj 1: aggregate of the reverse recurrence over a chunk (walked forwards from the chunk start) ----
template <int DIR>
__device__ void bl_adj1(const Item& it, const float2* __restrict__ gs, const uint32_t* __restrict__ vals_sorted, const float* __restrict__ dctx,
                        float* __restrict__ agg, float* __restrict__ tile, int item_idx, int j, unsigned hmask) {
    ColConst<DIR> cc;
    cc.load(j);
    float acc[16], m[32];                         // P (2x2 per pair) and accumulated injection
#pragma unroll
    for (int s = 0; s < 16; ++s) acc[s] = 0.f;
#pragma unroll
    for (int p = 0; p < 8; ++p) { m[4 * p] = 1.f; m[4 * p + 1] = 0.f; m[4 * p + 2] = 0.f; m[4 * p + 3] = 1.f; }
    for (int u0 = it.ub; u0 < it.ue; u0 += BL_TILE) {
        const int cnt = (it.ue - u0 < BL_TILE) ? (it.ue - u0) : BL_TILE;
        bl_stage_a<DIR>(tile, gs, vals_sorted, dctx, it.off, it.n, u0 + j, j < cnt, j);
        __syncwarp(hmask);
        for (int l = 0; l < cnt; ++l) {
            const float* row = tile + l * BL_ROW;
            const float2 v = *reinterpret_cast<const float2*>(row + 32);
            const float z = fmaf(cc.uz[0], v.x, fmaf(cc.uz[1], v.y, cc.uz[2]));
            const float dt = softplus20(fmaf(cc.ud[0], v.x, fmaf(cc.ud[1], v.y, cc.ud[2])));
            const float dy = row[36 + j] * silu(z);
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float abe, abo, cs, sn;
                pair_coeffs(dt, cc.ah[2 * p], cc.ah[2 * p + 1], cc.f[p], abe, abo, cs, sn);
                // M_t^T = [[abe*cs, abo*sn], [-abe*sn, abo*cs]];  P <- P * M_t^T ;  acc += P * (dy*C)
                const float a0 = m[4 * p], b0 = m[4 * p + 1], c0 = m[4 * p + 2], d0 = m[4 * p + 3];
                const float t1 = abe * cs, t2 = abo * sn, t3 = -abe * sn, t4 = abo * cs;
                const float na = fmaf(a0, t1, b0 * t3), nb = fmaf(a0, t2, b0 * t4), nc = fmaf(c0, t1, d0 * t3), nd = fmaf(c0, t2, d0 * t4);
                m[4 * p] = na; m[4 * p + 1] = nb; m[4 * p + 2] = nc; m[4 * p + 3] = nd;
                const float ie = dy * row[16 + 2 * p], io = dy * row[16 + 2 * p + 1];
                acc[2 * p] = fmaf(na, ie, fmaf(nb, io, acc[2 * p]));
                acc[2 * p + 1] = fmaf(nc, ie, fmaf(nd, io, acc[2 * p + 1]));
            }
        }
        bool zero = true;
#pragma unroll
        for (int k = 0; k < 32; ++k) zero = zero && (fabsf(m[k]) < 7.8886e-31f);
        __syncwarp(hmask);
        if (__all_sync(hmask, zero)) break;
    }
    float* dst = agg + ((int64_t)item_idx * 16 + j) * 48;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        dst[6 * p] = m[4 * p]; dst[6 * p + 1] = m[4 * p + 1]; dst[6 * p + 2] = m[4 * p + 2]; dst[6 * p + 3] = m[4 * p + 3];
        dst[6 * p + 4] = acc[2 * p]; dst[6 * p + 5] = acc[2 * p + 1];
    }
}

__global__ void __launch_bounds__(BL_THREADS) sg2_adj1_kernel(const Item* __restrict__ items, int n_items, int dir1_start,
                                                              const float2* __restrict__ gs, const uint32_t* __restrict__ vals_sorted,
                                                              const float* __restrict__ dctx, float* __restrict__ agg) {
    __shared__ __align__(16) float tiles[BL_ITEMS][BL_TILE * BL_ROW];
    const int slot = threadIdx.x >> 4, j = threadIdx.x & 15;
    const int item_idx = blockIdx.x * BL_ITEMS + slot;
    const unsigned hmask = 0xffffu << (16 * ((threadIdx.x >> 4) & 1));
    if (item_idx >= n_items) return;
    const Item it = items[item_idx];
    if (it.tensor < 0 || it.ub == 0) return;            // the first chunk's aggregate has no consumer
    if (item_idx < dir1_start) bl_adj1<0>(it, gs, vals_sorted, dctx, agg, tiles[slot], item_idx, j, hmask);
    else                       bl_adj1<1>(it, gs, vals_sorted, dctx, agg, tiles[slot], item_idx, j, hmask);
}

// ---- adj 2: dh arriving at the end of every chunk ----
__global__ void __launch_bounds__(128) sg2_adj2_kernel(const TensorDir* __restrict__ tds, const float* __restrict__ agg, float* __restrict__ dcarry) {
    const TensorDir td = tds[blockIdx.x];
    const int j = threadIdx.x >> 3, p = threadIdx.x & 7;
    float de = 0.f, dd = 0.f;                             // nothing flows into the final state
    for (int c = td.nc - 1; c >= 0; --c) {
        const int64_t idx = (int64_t)(td.item0 + c);
        float* co = dcarry + (idx * 16 + j) * 16 + 2 * p;
        co[0] = de; co[1] = dd;
        if (c > 0) {
            const float* a = agg + (idx * 16 + j) * 48 + 6 * p;
            const float ne = fmaf(a[0], de, fmaf(a[1], dd, a[4]));
            const float no = fmaf(a[2], de, fmaf(a[3], dd, a[5]));
            de = ne; dd = no;
        }
    }
}

// forward recurrence through the cnt timesteps of one tile whose rows stage_a has parked in `tile` (state only: no outputs)
template <int DIR>
__device__ __forceinline__ void bl_advance_tile(const ColConst<DIR>& cc, const float* __restrict__ tile, int cnt, float (&h)[16]) {
    for (int l = 0; l < cnt; ++l) {
        const float* row = tile + l * ROW;
        const float2 v = *reinterpret_cast<const float2*>(row + 32);
        const float x = fmaf(cc.ux[0], v.x, fmaf(cc.ux[1], v.y, cc.ux[2]));
        const float dt = softplus20(fmaf(cc.ud[0], v.x, fmaf(cc.ud[1], v.y, cc.ud[2])));
        const float dtx = dt * x;
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            float abe, abo, cs, sn;
            pair_coeffs(dt, cc.ah[2 * p], cc.ah[2 * p + 1], cc.f[p], abe, abo, cs, sn);
            const float he = h[2 * p], ho = h[2 * p + 1];
            h[2 * p] = fmaf(abe, he * cs - ho * sn, dtx * row[2 * p]);
            h[2 * p + 1] = fmaf(abo, ho * cs + he * sn, dtx * row[2 * p + 1]);
        }
    }
}

// ---- adj 3: the adjoint proper ----
// State snapshots are kept at the start of every `snap_every`-th tile (checkpoint interval = snap_every * BL_TILE timesteps); a tile
// that does not start at a snapshot is reached by re-running the forward recurrence from the snapshot before it, which trades
// (snap_every - 1) / 2 extra tile passes on average for 1 / snap_every of the snapshot memory.  The gradients do not depend on it.
template <int DIR>
__device__ void bl_adj3(const Item& it, const float2* __restrict__ gs, const uint32_t* __restrict__ vals_sorted, const float* __restrict__ dctx,
                        const float* __restrict__ carry, const float* __restrict__ dcarry, float* __restrict__ snaps, int64_t snap_base,
                        float* __restrict__ partial, float* __restrict__ tile, float* __restrict__ hist, float* __restrict__ sacc,
                        int item_idx, int j, unsigned hmask, int snap_every) {
    ColConst<DIR> cc;
    cc.load(j);
    const int len = it.ue - it.ub;
    const int ntile = (len + BL_TILE - 1) / BL_TILE;
    float h[16];
    // ---- forward re-run of the chunk: state snapshot at every tile start
    {
        const float* cin = carry + ((int64_t)item_idx * 16 + j) * 16;
#pragma unroll
        for (int q = 0; q < 4; ++q) { const float4 t = reinterpret_cast<const float4*>(cin)[q]; h[4 * q] = t.x; h[4 * q + 1] = t.y; h[4 * q + 2] = t.z; h[4 * q + 3] = t.w; }
    }
    for (int tI = 0; tI < ntile; ++tI) {
        const int u0 = it.ub + tI * BL_TILE;
        const int cnt = (it.ue - u0 < BL_TILE) ? (it.ue - u0) : BL_TILE;
        if (tI % snap_every == 0) {
            float* sp = snaps + ((snap_base + tI / snap_every) * 16 + j) * 16;
#pragma unroll
            for (int q = 0; q < 4; ++q) reinterpret_cast<float4*>(sp)[q] = make_float4(h[4 * q], h[4 * q + 1], h[4 * q + 2], h[4 * q + 3]);
        }
        if (tI == ntile - 1) break;                        // the last tile is recomputed by the backward loop anyway
        stage_a<DIR>(tile, gs, it.off, it.n, u0 + j, j < cnt, j);      // rows of the forward layout (ROW floats)
        __syncwarp(hmask);
        bl_advance_tile<DIR>(cc, tile, cnt, h);
        __syncwarp(hmask);
    }
    // ---- backward over the tiles
    float dh[16], dah[16], df[8], dux[3] = {0.f, 0.f, 0.f}, duz[3] = {0.f, 0.f, 0.f}, dud[3] = {0.f, 0.f, 0.f}, dwo[8], dD = 0.f;
    {
        const float* din = dcarry + ((int64_t)item_idx * 16 + j) * 16;
#pragma unroll
        for (int q = 0; q < 4; ++q) { const float4 t = reinterpret_cast<const float4*>(din)[q]; dh[4 * q] = t.x; dh[4 * q + 1] = t.y; dh[4 * q + 2] = t.z; dh[4 * q + 3] = t.w; }
    }
#pragma unroll
    for (int s = 0; s < 16; ++s) dah[s] = 0.f;
#pragma unroll
    for (int p = 0; p < 8; ++p) { df[p] = 0.f; dwo[p] = 0.f; }
    // lane-private accumulators of dU_B / dU_C in shared memory: sacc[a * BL_THREADS + tid], a in [0, 96)
    float* my = sacc + threadIdx.x;
    for (int a = 0; a < 96; ++a) my[a * BL_THREADS] = 0.f;
    for (int tI = ntile - 1; tI >= 0; --tI) {
        const int u0 = it.ub + tI * BL_TILE;
        const int cnt = (it.ue - u0 < BL_TILE) ? (it.ue - u0) : BL_TILE;
        {   // state at the start of this tile: the snapshot, advanced through the tiles between the snapshot and this one
            const int t0 = tI - tI % snap_every;
            const float* sp = snaps + ((snap_base + t0 / snap_every) * 16 + j) * 16;
#pragma unroll
            for (int q = 0; q < 4; ++q) { const float4 t = reinterpret_cast<const float4*>(sp)[q]; h[4 * q] = t.x; h[4 * q + 1] = t.y; h[4 * q + 2] = t.z; h[4 * q + 3] = t.w; }
            for (int t = t0; t < tI; ++t) {                // full tiles (only the last tile of a chunk can be short)
                stage_a<DIR>(tile, gs, it.off, it.n, it.ub + t * BL_TILE + j, true, j);
                __syncwarp(hmask);
                bl_advance_tile<DIR>(cc, tile, BL_TILE, h);
                __syncwarp(hmask);
            }
        }
        bl_stage_a<DIR>(tile, gs, vals_sorted, dctx, it.off, it.n, u0 + j, j < cnt, j);
        __syncwarp(hmask);
        // forward through the tile, keeping h BEFORE each step: hist[(l*16 + s) * 16 + j]
        for (int l = 0; l < cnt; ++l) {
            const float* row = tile + l * BL_ROW;
            const float2 v = *reinterpret_cast<const float2*>(row + 32);
            const float x = fmaf(cc.ux[0], v.x, fmaf(cc.ux[1], v.y, cc.ux[2]));
            const float dt = softplus20(fmaf(cc.ud[0], v.x, fmaf(cc.ud[1], v.y, cc.ud[2])));
            const float dtx = dt * x;
#pragma unroll
            for (int s = 0; s < 16; ++s) hist[(l * 16 + s) * 16 + j] = h[s];
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                float abe, abo, cs, sn;
                pair_coeffs(dt, cc.ah[2 * p], cc.ah[2 * p + 1], cc.f[p], abe, abo, cs, sn);
                const float he = h[2 * p], ho = h[2 * p + 1];
                h[2 * p] = fmaf(abe, he * cs - ho * sn, dtx * row[2 * p]);
                h[2 * p + 1] = fmaf(abo, ho * cs + he * sn, dtx * row[2 * p + 1]);
            }
        }
        // reverse through the tile
        for (int l = cnt - 1; l >= 0; --l) {
            const float* row = tile + l * BL_ROW;
            const float2 v = *reinterpret_cast<const float2*>(row + 32);
            const float in3[3] = {v.x, v.y, 1.f};
            const float x = fmaf(cc.ux[0], v.x, fmaf(cc.ux[1], v.y, cc.ux[2]));
            const float z = fmaf(cc.uz[0], v.x, fmaf(cc.uz[1], v.y, cc.uz[2]));
            const float dtr = fmaf(cc.ud[0], v.x, fmaf(cc.ud[1], v.y, cc.ud[2]));
            const float dt = softplus20(dtr);
            const float dtx = dt * x;
            const float gout = row[36 + j];
            const float sz = sigmoidf(z), sl = z * sz;
            const float dy = gout * sl;
            float y = 0.f, ddt = 0.f, ddtx = 0.f;
#pragma unroll
            for (int p = 0; p < 8; ++p) {
                const int e = 2 * p, o = 2 * p + 1;
                float abe, abo, cs, sn;
                pair_coeffs(dt, cc.ah[e], cc.ah[o], cc.f[p], abe, abo, cs, sn);
                const float he = hist[(l * 16 + e) * 16 + j], ho = hist[(l * 16 + o) * 16 + j];
                const float re = he * cs - ho * sn, ro = ho * cs + he * sn;
                const float Be = row[e], Bo = row[o], Ce = row[16 + e], Co = row[16 + o];
                const float hce = fmaf(abe, re, dtx * Be), hco = fmaf(abo, ro, dtx * Bo);     // state AFTER this step
                y = fmaf(hce, Ce, fmaf(hco, Co, y));
                const float de = fmaf(dy, Ce, dh[e]), dd = fmaf(dy, Co, dh[o]);
                const float dCe = dy * hce, dCo = dy * hco, dBe = de * dtx, dBo = dd * dtx;
#pragma unroll
                for (int k = 0; k < 3; ++k) {
                    my[(e * 3 + k) * BL_THREADS] = fmaf(dBe, in3[k], my[(e * 3 + k) * BL_THREADS]);
                    my[(o * 3 + k) * BL_THREADS] = fmaf(dBo, in3[k], my[(o * 3 + k) * BL_THREADS]);
                    my[(48 + e * 3 + k) * BL_THREADS] = fmaf(dCe, in3[k], my[(48 + e * 3 + k) * BL_THREADS]);
                    my[(48 + o * 3 + k) * BL_THREADS] = fmaf(dCo, in3[k], my[(48 + o * 3 + k) * BL_THREADS]);
                }
                ddtx = fmaf(de, Be, fmaf(dd, Bo, ddtx));
                const float dabe = de * re, dabo = dd * ro, dre = de * abe, dro = dd * abo;
                const float dcs = fmaf(dre, he, dro * ho), dsn = fmaf(dro, he, -dre * ho);
                const float dth = fmaf(cs, dsn, -sn * dcs);
                ddt = fmaf(dth, cc.f[p], ddt);
                df[p] = fmaf(dth, dt, df[p]);
                const float gae = dabe * (abe + 1.f) * (abe + 1.f) * 0.5f, gao = dabo * (abo + 1.f) * (abo + 1.f) * 0.5f;
                ddt = fmaf(gae, cc.ah[e], fmaf(gao, cc.ah[o], ddt));
                dah[e] = fmaf(gae, dt, dah[e]); dah[o] = fmaf(gao, dt, dah[o]);
                dh[e] = fmaf(dre, cs, dro * sn);
                dh[o] = fmaf(dro, cs, -dre * sn);
            }
            const float outj = fmaf(y, sl, cc.Dj * x);
            const float dz = gout * y * sz * (1.f + z * (1.f - sz));
            dD = fmaf(gout, x, dD);
            const float dx = fmaf(gout, cc.Dj, ddtx * dt);
            ddt = fmaf(ddtx, x, ddt);
            const float ddtr = ddt * (dtr > 20.f ? 1.f : sigmoidf(dtr));
#pragma unroll
            for (int k = 0; k < 3; ++k) { dux[k] = fmaf(dx, in3[k], dux[k]); duz[k] = fmaf(dz, in3[k], duz[k]); dud[k] = fmaf(ddtr, in3[k], dud[k]); }
#pragma unroll
            for (int d = 0; d < 8; ++d) dwo[d] = fmaf(row[52 + d], outj, dwo[d]);
        }
        __syncwarp(hmask);
    }
    // ---- per-item partial gradients: [item][BL_NG], written by the 16 lanes
    float* out = partial + (int64_t)item_idx * BL_NG;
#pragma unroll
    for (int s = 0; s < 16; ++s) out[j * 16 + s] = dah[s];              // d(A/2); converted to d A_log by the reduction kernel
#pragma unroll
    for (int p = 0; p < 8; ++p) out[256 + j * 8 + p] = df[p];
    out[384 + j] = dD;
#pragma unroll
    for (int k = 0; k < 3; ++k) { out[400 + j * 3 + k] = dux[k]; out[448 + j * 3 + k] = duz[k]; out[496 + j * 3 + k] = dud[k]; }
#pragma unroll
    for (int d = 0; d < 8; ++d) out[640 + d * 16 + j] = dwo[d];
    // dU_B / dU_C: sum over the 16 lanes of this item (fixed order), lane s writes row s
    __syncwarp(hmask);
    const int base = threadIdx.x & ~15;
    for (int k = 0; k < 3; ++k) {
        float sb = 0.f, sc = 0.f;
        for (int jj = 0; jj < 16; ++jj) {
            sb += sacc[(j * 3 + k) * BL_THREADS + base + jj];
            sc += sacc[(48 + j * 3 + k) * BL_THREADS + base + jj];
        }
        out[544 + j * 3 + k] = sb;
        out[592 + j * 3 + k] = sc;
    }
}

__global__ void __launch_bounds__(BL_THREADS) sg2_adj3_kernel(const Item* __restrict__ items, int n_items, int dir1_start,
                                                              const int64_t* __restrict__ snap_base, const float2* __restrict__ gs,
                                                              const uint32_t* __restrict__ vals_sorted, const float* __restrict__ dctx,
                                                              const float* __restrict__ carry, const float* __restrict__ dcarry,
                                                              float* __restrict__ snaps, float* __restrict__ partial, int snap_every) {
    extern __shared__ __align__(16) float bl_smem[];
    float* tiles = bl_smem;                                             // [BL_ITEMS][BL_TILE*BL_ROW]  (BL_ROW >= ROW)
    float* hist = tiles + BL_ITEMS * BL_TILE * BL_ROW;                  // [BL_ITEMS][BL_TILE*16*16]
    float* sacc = hist + BL_ITEMS * BL_TILE * 256;                      // [96][BL_THREADS]
    const int slot = threadIdx.x >> 4, j = threadIdx.x & 15;
    const int item_idx = blockIdx.x * BL_ITEMS + slot;
    const unsigned hmask = 0xffffu << (16 * ((threadIdx.x >> 4) & 1));
    if (item_idx >= n_items) return;
    const Item it = items[item_idx];
    if (it.tensor < 0) {
        for (int k = j; k < BL_NG; k += 16) partial[(int64_t)item_idx * BL_NG + k] = 0.f;
        return;
    }
    float* tile = tiles + slot * BL_TILE * BL_ROW;
    float* hs = hist + slot * BL_TILE * 256;
    if (item_idx < dir1_start) bl_adj3<0>(it, gs, vals_sorted, dctx, carry, dcarry, snaps, snap_base[item_idx], partial, tile, hs, sacc, item_idx, j, hmask, snap_every);
    else                       bl_adj3<1>(it, gs, vals_sorted, dctx, carry, dcarry, snaps, snap_base[item_idx], partial, tile, hs, sacc, item_idx, j, hmask, snap_every);
}

// ---- adj 4: fixed-order sum over the items of each direction; d(A/2) -> d A_log ----
__global__ void __launch_bounds__(256) sg2_adj4_kernel(const float* __restrict__ partial, int n_items, int dir1_start, float* __restrict__ grads) {
    const int dir = blockIdx.y;
    const int k = blockIdx.x * 256 + threadIdx.x;
    if (k >= BL_NG) return;
    const int i0 = dir == 0 ? 0 : dir1_start, i1 = dir == 0 ? dir1_start : n_items;
    float s = 0.f;
    for (int i = i0; i < i1; ++i) s += partial[(int64_t)i * BL_NG + k];
    if (k < 256) {                                                      // ah = -0.5*exp(A_log)  =>  d A_log = d ah * ah
        const int W = (dir == 0) ? P::DIR0 : P::DIR1;
        s *= -0.5f * __expf(c_w[W + P::D_ALOG + k]);
    }
    grads[dir * BL_NG + k] = s;
}

}  // namespace

size_t sg2_bilevel_smem_bytes() { return (size_t)(BL_ITEMS * BL_TILE * BL_ROW + BL_ITEMS * BL_TILE * 256 + 96 * BL_THREADS) * sizeof(float); }
int sg2_bilevel_ng() { return BL_NG; }
int sg2_bilevel_tile() { return BL_TILE; }

// dctx [total,16] (original order) -> grads [2][BL_NG].  Uses the forward scan's carry (chunk carry-in states of THIS forward),
// agg/dcarry scratch of the same sizes as the forward ones, snaps [sum over items of ceil(tiles / snap_every), 16, 16] and
// partial [n_items, BL_NG].  snap_base[item] = index of the item's first snapshot.
void sg2_scan_backward(const void* items_dev, int n_items, int dir1_start, const void* tds_dev, int n_td, const int64_t* snap_base_dev,
                       const float* gs_sorted, const uint32_t* vals_sorted, const float* dctx, const float* carry, float* agg, float* dcarry,
                       float* snaps, float* partial, float* grads, int snap_every, cudaStream_t s) {
    if (n_items <= 0) return;
    if (snap_every < 1) snap_every = 1;
    const Item* items = reinterpret_cast<const Item*>(items_dev);
    const TensorDir* tds = reinterpret_cast<const TensorDir*>(tds_dev);
    const float2* gs = reinterpret_cast<const float2*>(gs_sorted);
    const int blocks = (n_items + BL_ITEMS - 1) / BL_ITEMS;
    const size_t smem = sg2_bilevel_smem_bytes();
    static bool configured = false;
    if (!configured) { cudaFuncSetAttribute(sg2_adj3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); configured = true; }
    count_launch(4);
    sg2_adj1_kernel<<<blocks, BL_THREADS, 0, s>>>(items, n_items, dir1_start, gs, vals_sorted, dctx, agg);
    sg2_adj2_kernel<<<n_td, 128, 0, s>>>(tds, agg, dcarry);
    sg2_adj3_kernel<<<blocks, BL_THREADS, smem, s>>>(items, n_items, dir1_start, snap_base_dev, gs, vals_sorted, dctx, carry, dcarry, snaps, partial, snap_every);
    sg2_adj4_kernel<<<dim3((BL_NG + 255) / 256, 2), 256, 0, s>>>(partial, n_items, dir1_start, grads);
}

}  // namespace sg
