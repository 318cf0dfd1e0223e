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
// aux_deriv != 0 changes what the auxiliary tensor holds: the forward product stores act'(pre-activation) in
//   aux_out instead of the pre-activation (one tanh serves GELU and its derivative), and the backward product
//   multiplies by aux_in as it is -- the derivative is evaluated once, in forward, instead of once more per
//   backward element.  (For ReLU the derivative is the sign of the activation; aux_deriv is ignored.)
// colsum != null asks for column sums of the stored C (a bias gradient when C is the gradient of a pre-activation):
//   the kernel writes one fp32 row of partial sums per 32 rows of C, [ceil(M / 32)][N], and *colsum_slabs receives
//   the number of such rows -- or 0 when the kernel that ran cannot produce them (the caller then sums C itself).
//   cme_colsum_slabs_finalize adds the rows up in a fixed order.
struct CmeGemm {
    int M, N, K, batch;
    const void* A; long long lda, strideA; int a_trans;
    const void* B; long long ldb, strideB; int b_trans;
    void* C; long long ldc, strideC; int c_dtype;        // CME_BF16 or CME_F32
    int ab_dtype;                                         // CME_BF16, or CME_F32: exact on the SIMT kernel, tf32 tensor-core
                                                          // math on the tcgen05 kernel when allow_tf32 is set
    const void* bias;                                     // [N], same dtype as A/B, or null
    const void* residual; long long ldres;                // [M, N] same dtype as C, or null (batch stride = strideC)
    void* aux_out; const void* aux_in; long long ldaux;   // [M, N] same dtype as C
    int act, dact, accumulate;
    void* workspace; long long workspace_bytes;           // fp32 scratch for split-K partial sums (may be null)
    int force_bn, force_splits;                           // 0 = choose automatically
    int aux_deriv;                                        // aux tensors hold act'(pre-activation), see above
    float* colsum; int* colsum_slabs;                     // optional column sums of C (device scratch, host count)
    int allow_tf32;                                       // fp32 operands may be multiplied as tf32 (10-bit mantissa
                                                          // inputs, fp32 accumulation): plain products with fp32 output
};

int gemm_tcgen05_supported(const CmeGemm* g);
int gemm_tcgen05_launch(const CmeGemm* g, cudaStream_t stream);
int gemm_simt_launch(const CmeGemm* g, cudaStream_t stream);
