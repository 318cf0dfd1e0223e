// GEMM interface shared by the tcgen05 kernel, the SIMT fallback and the engine.
//
// One descriptor covers every GEMM site of the reference (FINAL_CLEAN_CODE_/include/kernels.h:6-60:
// gemm_tiled / _AT / _BT, their `_acc` twins, split-K, strided-batched NN / TN / NT) and the epilogues it
// runs as separate kernels (bias+ReLU, bias+residual, ReLU-backward; activations.cu:84-199).
#pragma once
#include "common.h"

enum CmeAct : int { CME_ACT_NONE = 0, CME_ACT_RELU = 1, CME_ACT_GELU = 2 };

// C[b] (+)= epilogue(A[b] * B[b]);   row-major storage everywhere.
//   a_trans = 0: A stored [M, K] (lda = row stride);  1: A stored [K, M]
//   b_trans = 0: B stored [K, N] (ldb = row stride);  1: B stored [N, K]
//   batch strides are in elements; 0 means the operand is shared by all batches.
// Epilogue, in this order:  acc += bias[n];  aux_out[m,n] = acc (pre-activation, optional);
//   acc = act(acc);  acc *= act'(aux_in[m,n]) (dact);  acc += residual[m,n];  acc += C_old (accumulate).
struct CmeGemm {
    int M, N, K, batch;
    const void* A; long long lda, strideA; int a_trans;
    const void* B; long long ldb, strideB; int b_trans;
    void* C; long long ldc, strideC; int c_dtype;        // CME_BF16 or CME_F32
    int ab_dtype;                                         // CME_BF16 or CME_F32 (SIMT path only)
    const void* bias;                                     // [N], same dtype as A/B, or null
    const void* residual; long long ldres;                // [M, N] same dtype as C, or null (batch stride = strideC)
    void* aux_out; const void* aux_in; long long ldaux;   // [M, N] same dtype as C
    int act, dact, accumulate;
    void* workspace; long long workspace_bytes;           // fp32 scratch for split-K partial sums (may be null)
    int force_bn, force_splits;                           // 0 = choose automatically
};

int gemm_tcgen05_supported(const CmeGemm* g);
int gemm_tcgen05_launch(const CmeGemm* g, cudaStream_t stream);
int gemm_simt_launch(const CmeGemm* g, cudaStream_t stream);
