// Attention as strided-batched tensor-core GEMMs around row kernels, for short sequences and head sizes the
// fused kernel does not take (the reference's shapes: T = 64, head size 32 / 64 / 128, flat head view).
//
// This is the reference's production structure (FINAL_CLEAN_CODE_/src/kernels/attention.cu:181-200 forward:
// batched Q K^T, in-place scale+softmax, batched P V; :298-328 backward: four batched GEMMs and compute_ds_kernel)
// on this library's tcgen05 batched GEMM.  Differences: scores stay fp32 between the GEMM and the row kernel,
// probabilities are stored once in bf16, the forward saves only the log-sum-exp, and the backward recomputes P
// from it (so no [B*H, T, T] buffer has to live across the step); dS already carries the 1/sqrt(hd) factor.
#include "attention.h"
#include "gemm.h"

extern "C" int cme_gemm(const CmeGemm*, int, void*);
int attention_delta_launch(const CmeAttn* a, cudaStream_t st);

namespace {

// One warp per score row: P = softmax(scale * S) (bf16), lse = log-sum-exp of the scaled row.
__global__ void softmax_rows_kernel(const float* __restrict__ S, __nv_bfloat16* __restrict__ P, float* __restrict__ lse,
                                    long long rows, int T, float scale, int causal) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31, q = (int)(row % T);
    const float* s = S + row * T;
    const int n = causal ? q + 1 : T;
    float m = -INFINITY;
    for (int j = lane; j < n; j += 32) m = fmaxf(m, s[j] * scale);
    m = warp_max(m);
    float sum = 0.f;
    for (int j = lane; j < n; j += 32) sum += __expf(s[j] * scale - m);
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int j = lane; j < T; j += 32)
        P[row * T + j] = __float2bfloat16_rn(j < n ? __expf(s[j] * scale - m) * inv : 0.f);
    if (lane == 0) lse[row] = m + logf(sum);
}

// One warp per row: P = exp(scale * S - lse) and dS = scale * P * (dP - delta), both bf16.
__global__ void ds_rows_kernel(const float* __restrict__ S, const float* __restrict__ dP, const float* __restrict__ lse,
                               const float* __restrict__ delta, __nv_bfloat16* __restrict__ P,
                               __nv_bfloat16* __restrict__ dS, long long rows, int T, float scale, int causal) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31, q = (int)(row % T);
    const int n = causal ? q + 1 : T;
    const float l = lse[row], d = delta[row];
    for (int j = lane; j < T; j += 32) {
        const long long i = row * T + j;
        const float p = j < n ? __expf(S[i] * scale - l) : 0.f;
        P[i] = __float2bfloat16_rn(p);
        dS[i] = __float2bfloat16_rn(scale * p * (dP[i] - d));
    }
}

int bgemm(int M, int N, int K, int batch, const void* A, long long lda, long long sA, int a_trans, const void* B,
          long long ldb, long long sB, int b_trans, void* C, long long ldc, long long sC, int c_f32, cudaStream_t st) {
    CmeGemm g{};
    g.M = M; g.N = N; g.K = K; g.batch = batch;
    g.A = A; g.lda = lda; g.strideA = sA; g.a_trans = a_trans;
    g.B = B; g.ldb = ldb; g.strideB = sB; g.b_trans = b_trans;
    g.C = C; g.ldc = ldc; g.strideC = sC; g.c_dtype = c_f32 ? CME_F32 : CME_BF16; g.ab_dtype = CME_BF16;
    return cme_gemm(&g, 0, st);
}

struct Carve { float* S; float* dP; __nv_bfloat16* P; __nv_bfloat16* dS; };
Carve carve(const CmeAttn* a) {
    const long long n = (long long)a->nb * a->T * a->T;
    char* w = static_cast<char*>(a->ws);
    Carve c;
    c.S = reinterpret_cast<float*>(w);
    c.dP = c.S + n;
    c.P = reinterpret_cast<__nv_bfloat16*>(c.dP + n);
    c.dS = c.P + n;
    return c;
}

}  // namespace

long long attention_gemm_ws_bytes(int nb, int T) { return (long long)nb * T * T * 12 + 256; }

int attention_gemm_supported(const CmeAttn* a) {
    if (a->dtype != CME_BF16 || a->nh != 1) return 0;                 // flat [B*H, T, HD] views only
    if (a->HD % 8 || a->T % 8 || a->st != a->HD || a->ost != a->HD) return 0;
    if (a->sb != (long long)a->T * a->HD || a->osb != a->sb) return 0;
    if (!a->ws || a->ws_bytes < attention_gemm_ws_bytes(a->nb, a->T)) return 0;
    if ((reinterpret_cast<uintptr_t>(a->ws) & 255) != 0) return 0;
    return a->T <= 512;
}

int attention_gemm_fwd(const CmeAttn* a, cudaStream_t st) {
    CME_REQUIRE(attention_gemm_supported(a), CME_ERR_SHAPE, "attention: shape not supported by the GEMM path");
    const Carve c = carve(a);
    const int T = a->T, HD = a->HD, BH = a->nb;
    const long long hs = (long long)T * HD, ss = (long long)T * T, rows = (long long)BH * T;
    int rc;
    // S = Q K^T
    if ((rc = bgemm(T, T, HD, BH, a->q, HD, hs, 0, a->k, HD, hs, 1, c.S, T, ss, 1, st))) return rc;
    softmax_rows_kernel<<<cme_cdiv(rows, 8), 256, 0, st>>>(c.S, c.P, a->lse, rows, T, a->scale, a->causal);
    CME_LAUNCH_CHECK();
    // O = P V
    return bgemm(T, HD, T, BH, c.P, T, ss, 0, a->v, HD, hs, 0, a->o, HD, hs, 0, st);
}

int attention_gemm_bwd(const CmeAttn* a, cudaStream_t st) {
    CME_REQUIRE(attention_gemm_supported(a), CME_ERR_SHAPE, "attention: shape not supported by the GEMM path");
    CME_REQUIRE(a->delta && a->d_o && a->dq && a->dk && a->dv, CME_ERR_SHAPE, "attention backward: missing buffer");
    const Carve c = carve(a);
    const int T = a->T, HD = a->HD, BH = a->nb;
    const long long hs = (long long)T * HD, ss = (long long)T * T, rows = (long long)BH * T;
    int rc;
    if ((rc = attention_delta_launch(a, st))) return rc;
    if ((rc = bgemm(T, T, HD, BH, a->q, HD, hs, 0, a->k, HD, hs, 1, c.S, T, ss, 1, st))) return rc;       // S = Q K^T
    if ((rc = bgemm(T, T, HD, BH, a->d_o, HD, hs, 0, a->v, HD, hs, 1, c.dP, T, ss, 1, st))) return rc;    // dP = dO V^T
    ds_rows_kernel<<<cme_cdiv(rows, 8), 256, 0, st>>>(c.S, c.dP, a->lse, a->delta, c.P, c.dS, rows, T, a->scale,
                                                      a->causal);
    CME_LAUNCH_CHECK();
    if ((rc = bgemm(T, HD, T, BH, c.P, T, ss, 1, a->d_o, HD, hs, 0, a->dv, HD, hs, 0, st))) return rc;    // dV = P^T dO
    if ((rc = bgemm(T, HD, T, BH, c.dS, T, ss, 0, a->k, HD, hs, 0, a->dq, HD, hs, 0, st))) return rc;     // dQ = dS K
    return bgemm(T, HD, T, BH, c.dS, T, ss, 1, a->q, HD, hs, 0, a->dk, HD, hs, 0, st);                    // dK = dS^T Q
}
