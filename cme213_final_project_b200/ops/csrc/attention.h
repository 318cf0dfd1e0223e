// Attention interface shared by the SIMT kernels, the tcgen05 kernels and the engine.
//
// One layout descriptor serves both head layouts of the framework:
//   * "flat": the reference's reinterpretation of the row-major [B*T, D] projection as [B*H, T, HD]
//     (FINAL_CLEAN_CODE_/src/model/transformer.cu:71-75,352-356) -> nb = B*H, nh = 1, batch stride T*HD,
//     row stride HD;
//   * "split": the standard [B, T, H, HD] split -> nb = B, nh = H, batch stride T*D, head stride HD,
//     row stride D.
// Element (b, h, t, d) of Q / K / V / dQ / dK / dV lives at  b*sb + h*sh + t*st + d;  O and dO have their own
// strides (osb, osh, ost), because a fused [B*T, 3D] projection buffer has a different row pitch than O.
#pragma once
#include "common.h"

struct CmeAttn {
    int nb, nh, T, HD;
    long long sb, sh, st;        // strides of Q / K / V / dQ / dK / dV
    long long osb, osh, ost;     // strides of O / dO
    int causal;
    float scale;                 // 1 / sqrt(HD)
    int dtype;                   // CME_BF16 or CME_F32
    const void* q; const void* k; const void* v;
    void* o;                     // forward output / backward input
    float* lse;                  // [nb*nh, T] log-sum-exp of scaled scores (saved by forward)
    // backward only
    const void* d_o; void* dq; void* dk; void* dv;
    float* delta;                // [nb*nh, T] scratch: rowsum(dO * O)
    float* dq_accum;             // fp32 scratch [nb*nh*T*HD] for the tcgen05 backward (may be null)
    void* ws; long long ws_bytes;    // scratch of attention_gemm_ws_bytes() for the batched-GEMM path (may be null)
    int* dq_sem;                 // [nb*nh * ceil(T / 128)] ints, zero before the first launch (the kernel leaves them zero);
                                 // needed by dq_mode 1 and 2
    int dq_mode;                 // how the tcgen05 backward completes dQ from the key blocks' parts:
                                 //   0  the launch clears dq_accum, the parts are added in arrival order, a second kernel
                                 //      scales and casts the sums
                                 //   1  the parts are added in a fixed order (bit-reproducible); key block 0 finishes
                                 //   2  arrival order; the CTA whose part comes last scales, casts and writes zeros back:
                                 //      dq_accum must be zero before the first launch and is zero after every launch
    int dq_accum_clean;          // dq_mode 0: non-zero = the caller has cleared dq_accum itself (e.g. on another stream,
                                 // ahead of time); the launch then skips its own clear
};

constexpr int CME_ATTN_FINISH_MAX_QBLOCKS = 64;      // dq_mode 2: query blocks (of 128 rows) per sequence

int attention_simt_fwd(const CmeAttn* a, cudaStream_t st);
int attention_simt_bwd(const CmeAttn* a, cudaStream_t st);
int attention_gemm_supported(const CmeAttn* a);
int attention_gemm_fwd(const CmeAttn* a, cudaStream_t st);
int attention_gemm_bwd(const CmeAttn* a, cudaStream_t st);
long long attention_gemm_ws_bytes(int nb, int T);
int attention_tc_supported(const CmeAttn* a);
int attention_tc_fwd(const CmeAttn* a, cudaStream_t st);
int attention_tc_bwd(const CmeAttn* a, cudaStream_t st);
