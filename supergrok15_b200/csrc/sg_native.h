// Host-visible declarations of the sm_100a kernel launchers.
//
// Every launcher takes raw device pointers and a CUDA stream, allocates nothing, and
// never synchronises the host.  The PyTorch binding file (bindings.cpp) converts tensors
// to these arguments; the kernels themselves are plain CUDA translation units that do not
// include any PyTorch header.
#pragma once
#include <cstdint>
#include <cuda_runtime_api.h>

namespace sg {

// ----------------------------------------------------------------------------------------
// Multi-tensor launch descriptor: one launch covers up to MT_MAX tensors.  The struct is a
// kernel parameter (large kernel parameters, <= 32 KB), so no table upload is needed.
// ----------------------------------------------------------------------------------------
constexpr int MT_MAX = 96;          // tensors per launch
constexpr int MT_CHUNK = 8192;      // elements per CTA
constexpr int MT_THREADS = 256;
constexpr int MT_NP = 7;            // pointer roles per tensor
constexpr int MT_NS = 4;            // per-tensor float scalars

struct MTArgs {
    void*   ptr[MT_NP][MT_MAX];
    int64_t numel[MT_MAX];
    int     blk_start[MT_MAX + 1];  // CTA index range of tensor t is [blk_start[t], blk_start[t+1])
    float   ts[MT_MAX][MT_NS];
    int     n;                      // tensors in this launch
    int     t_off;                  // index of tensor 0 of this launch in the caller's full list
    int     blk_off;                // CTA offset of this launch in the caller's partials array
};

enum DType : int { F32 = 0, BF16 = 1, F16 = 2 };

// Bounds-checked build of the multi-tensor kernels (mt_kernels.cu compiled with -DGROK_BOUNDS_CHECK): accesses beyond the driver's
// record of each allocation are skipped and the first one is reported {count, op, role, tensor, index low, index high, is_store, 0}.
// In the regular build these report "disabled" / zeros.
bool bounds_check_enabled();
void bounds_reset();
void bounds_report(int out[8]);
void bounds_cap(long long bytes);               // test hook: treat every allocation as at most this many bytes (-1: off)
long long bounds_extent_of(const void* ptr);    // bytes addressable from ptr according to the driver (0: unknown)

// Number of kernels of this library enqueued so far by this process (every launcher counts its launches).
void count_launch(int n = 1);
long long launch_count();

// Element-wise optimizer ids (pointer roles listed per op; p/g use the launch dtype, the rest fp32).
enum MTOp : int {
    OP_ADAMW = 0,        // p g m v                ts: bc1 bc2
    OP_LION,             // p g m
    OP_GROKFAST_EMA,     // - g e                  (g updated in place)
    OP_GROKFAST_ADAMW,   // p g m v e              ts: bc1 bc2   (EMA + amplify + AdamW, g updated in place)
    OP_GROKADAMW,        // p g m v e              ts: bc1 bc2
    OP_PRODIGY,          // p g m v s              ts: bc1 bc2
    OP_NEURALGROK,       // p g m v                ts: bc1 bc2
    OP_SG15,             // p g m v mu sharp       ts: alpha_i beta1_i bc1 bc2
    OP_SG11_A,           // - g mu sharp smart     ts: alpha_i              -> partials {sg.mu, sg.sg, mu.mu}
    OP_SG11_B,           // p smart m v mu         ts: beta1_i bc1 bc2
    OP_PERTURB,          // p g backup             p += scale*g, backup = p_old
    OP_RESTORE,          // p - backup
    OP_SHARP_RESTORE,    // p g backup gsam sharp  sharp = |gsam-g| ; p = backup
    OP_LOOKSAM_DIR,      // - g v gsam             v = (gsam-g)/norm_t
    OP_LOOKSAM_ADJ,      // - g v                  g += alpha*|g|_t * v
    OP_MUON_MOMENTUM,    // - g buf                buf = mom*buf+g -> partials {buf.buf}
    OP_MUON_UPDATE,      // p x                    p = (p + s*x)*decay   (x fp32)
    OP_SCALE,            // - g                    g *= scale
    OP_SQNORM,           // - g                    -> partials {g.g}
    OP_PRODIGY_REDUCE,   // p g p0 s               -> partials {g.(p-p0), sum s}
    OP_DIFF_SQNORM,      // - g gsam               -> partials {(gsam-g)^2, g.g}
    OP_COUNT
};

struct MTParams {
    float lr, beta1, beta2, eps, wd;
    float alpha, lamb, rescale;       // op-specific (EMA alpha, lambda, meta-net rescale / amplifier beta)
    float extra0, extra1;             // op-specific
    const float* clip;                // device scalar multiplied into g (nullptr -> 1)
    const float* dscal;               // device scalar(s): d_lr (Prodigy), rho/norm (perturb), ...
    const float* tscal;               // device per-tensor scalars (index t_off+t): gates, norms
    const float* W1; const float* b1; const float* W2; const float* b2;   // small MLP weights
    int hidden;
    int write_grad;                   // 1: write the clipped / amplified gradient back
    float* partials;                  // [blocks][3] per-CTA partial sums (reductions only)
};

void mt_launch(int op, int dtype, const MTArgs& a, const MTParams& p, cudaStream_t s);

// Deterministic second stage of the reductions: sums CTA partials per tensor in a fixed order.
// out[(t_off+t)*3 + k] = sum over the tensor's CTAs of partials[.][k].
void mt_finalize_per_tensor(const MTArgs& a, const float* partials, float* out, cudaStream_t s);

enum ScalarOp : int {
    SC_CLIP = 0,        // in: per-tensor {sq} ; out[0]=sumsq out[1]=clip coef (max/(norm+1e-6) if norm>max else 1) out[2]=norm
    SC_PRODIGY,         // in: per-tensor {num, den}; out[0] = d_lr (in/out), monotone update
    SC_SG11_GATES,      // in: per-tensor {dot, sg2, mu2}; out[t] = ramp>0 ? ramp*sigmoid(T*cos)*lamb : 0
    SC_SAM_SCALE,       // in: per-tensor {sq}; out[0] = rho/(sqrt(sum)+1e-12)
    SC_LOOKSAM_NORMS,   // in: per-tensor {dsq, gsq}; out[2t] = dnorm<1e-12 ? 0 : 1/dnorm ; out[2t+1] = sqrt(gsq)
    SC_MUON_NORMS,      // in: per-tensor {sq}; out[t] = 1/(sqrt(sq)+1e-7)
    SC_SG2_CLIP,        // in: per-tensor {sq}; out[t] = norm>max ? max/(norm+1e-12) : 1
    SC_SUM3             // in: per-tensor {a,b,c}; out[0..2] = column sums (fixed order)
};
void scalar_finalize(int op, const float* per_tensor, int n_tensors, float* out, float a0, float a1, float a2,
                     cudaStream_t s);

// ----------------------------------------------------------------------------------------
// SuperGrok v2 step (magnitude sort -> bidirectional scan -> element step)
// ----------------------------------------------------------------------------------------
constexpr int SG2_DM = 8, SG2_DI = 16, SG2_DS = 16, SG2_GRU = 4, SG2_HEADS = 4, SG2_PK = 12, SG2_NE = 144,
              SG2_EH = 16;

// Offsets (floats) into the packed meta-net weight vector.
struct SG2Pack {
    static constexpr int IN_W = 0;                       // [8,2]
    static constexpr int IN_B = IN_W + 16;               // [8]
    static constexpr int DIR0 = IN_B + 8;                // forward-direction block
    // per direction:
    static constexpr int D_INPROJ = 0;                   // [32,8]
    static constexpr int D_DTW = D_INPROJ + 256;         // [16,16]
    static constexpr int D_DTB = D_DTW + 256;            // [16]
    static constexpr int D_BW = D_DTB + 16;              // [16,16]
    static constexpr int D_CW = D_BW + 256;              // [16,16]
    static constexpr int D_ALOG = D_CW + 256;            // [16,16]
    static constexpr int D_D = D_ALOG + 256;             // [16]
    static constexpr int D_ROPE = D_D + 16;              // [16,8]
    static constexpr int D_OUT = D_ROPE + 128;           // [8,16]
    static constexpr int DIR_SIZE = D_OUT + 128;         // 1568
    static constexpr int DIR1 = DIR0 + DIR_SIZE;
    static constexpr int GRU_WZ = DIR1 + DIR_SIZE;       // [4,22]
    static constexpr int GRU_WR = GRU_WZ + 88;
    static constexpr int GRU_WH = GRU_WR + 88;
    static constexpr int GRU_BZ = GRU_WH + 88;           // [4]
    static constexpr int GRU_BR = GRU_BZ + 4;
    static constexpr int GRU_BH = GRU_BR + 4;
    static constexpr int PQ = GRU_BH + 4;                // [4,8,22]
    static constexpr int KA = PQ + 704;                  // [4,12,4]
    static constexpr int KB = KA + 192;                  // [4,12,4]
    static constexpr int EW1 = KB + 192;                 // [144,16]
    static constexpr int EB1 = EW1 + 2304;
    static constexpr int EW2 = EB1 + 2304;
    static constexpr int EB2 = EW2 + 2304;               // [144]
    static constexpr int NET = EB2 + 144;                // 11,580 floats of meta-net weights
    // folded affine tables of the scan inputs, per direction: value = t[0]*g + t[1]*s + t[2]
    static constexpr int A_X = 0;                        // [16][3] x_j
    static constexpr int A_Z = A_X + 48;                 // [16][3] z_j
    static constexpr int A_DT = A_Z + 48;                // [16][3] dt_j before softplus
    static constexpr int A_B = A_DT + 48;                // [16][3] B_s
    static constexpr int A_C = A_B + 48;                 // [16][3] C_s   (must follow A_B)
    static constexpr int AFF_SIZE = A_C + 48;            // 240
    static constexpr int AFF0 = NET;
    static constexpr int AFF1 = AFF0 + AFF_SIZE;
    static constexpr int TOTAL = AFF1 + AFF_SIZE;        // 12,060
};

// Layout of the device table of per-step scalars (32-bit words).  The host rewrites it before every step (one tiny kernel whose
// arguments are the values), so the kernels that read it can sit in a CUDA graph that is replayed unchanged step after step.
constexpr int DYN_EPOCH = 0;             // uint32: barrier epoch base of the step (barrier_kernel, csrc/dist_kernels.cu)
constexpr int DYN_LR = 8, DYN_WD = 9, DYN_LAMB = 10;
constexpr int DYN_TS = 16;               // per tensor t: alpha, beta1, bc1, bc2 at DYN_TS + 4 t

struct SG2Tensor {          // one entry per parameter tensor handled by a v2 step
    int64_t off;            // offset of the tensor in every packed [total_N] array
    int64_t n;              // elements
    float alpha, lamb_eff, beta1, bc1, bc2;   // per-tensor scalars
    float pad;
    void* param;            // parameter storage (launch dtype)
    float* m; float* v; float* mu; float* gru;      // fp32 state ([n], [n], [n], [n,4])
    float* h_fwd; float* h_bwd;                     // persistent scan states [16,16]
    const float* sharp;     // fp32 sharpness [n]
};

struct SG2Work {            // device workspace carved by the host from one arena
    float* g;               // [total] clipped, NaN-scrubbed gradient (original order)
    float* gs_sorted;       // [total,2] sorted (g, s)
    uint32_t* keys[2];      // [total] ping-pong
    uint32_t* vals[2];      // [total] ping-pong (global element index)
    uint32_t* hist;         // [256 * sort_blocks]
    float* ctx;             // [total,16] fwd ctx (8) + bwd ctx (8), original order
    float* agg;             // [items, 16, 8, 6] chunk aggregates
    float* carry;           // [items, 16, 16] chunk carry-in states
    float* partials;        // [blocks*3]
    float* tnorm;           // [n_tensors*3]
    float* tclip;           // [n_tensors]
    int* status;            // device status word (0 = ok)
};

size_t sg2_sort_blocks(int64_t total);
void sg2_segmented_sort(uint32_t* keys0, uint32_t* keys1, uint32_t* vals0, uint32_t* vals1, uint32_t* hist,
                        uint32_t* tot256, const int64_t* seg_offsets_dev, int n_seg, int64_t total, int* out_buf_index,
                        cudaStream_t s);

}  // namespace sg

// ----------------------------------------------------------------------------------------
// In-kernel collectives (dist_kernels.cu)
// ----------------------------------------------------------------------------------------
namespace sg {
constexpr int MAX_RANKS = 8;
constexpr int STATUS_OK = 0;
constexpr int STATUS_TIMEOUT = 1;     // status word = STATUS_TIMEOUT | (peer << 8) | (site << 16)
struct PeerPtrs { void* p[MAX_RANKS]; };
int sg2_scan_ctas_per_sm();          // resident CTAs per SM the scan kernel is compiled for (the host sizes its chunks in whole waves)
void write_words(uint32_t* dst, const uint32_t* host_words, int n, cudaStream_t s);
}  // namespace sg
