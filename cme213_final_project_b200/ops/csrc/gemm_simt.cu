// Generic CUDA-core GEMM: any shape, any of the four storage combinations, fp32 or bf16 operands, fp32
// accumulation, the full epilogue of gemm.h.  It is the strict-fp32 path of the parity model, the
// fallback for shapes the TMA path cannot address (e.g. the reference's N = vocab = 65 output head,
// which FINAL_CLEAN_CODE_/src/kernels/gemm.cu:742-754 also routes to its scalar kernel), and the
// independent implementation the tcgen05 kernel is checked against.
//
// 64 x 64 output tile, 16-deep K slices in shared memory, 256 threads, 4 x 4 outputs per thread
// (same blocking as the reference's first register-tiled kernel, gemm.cu:510-600, written afresh with
// stride-generic loads so one kernel serves NN / NT / TN and batches).
#include "gemm.h"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

struct SimtParams {
    int M, N, K;
    long long a_rs, a_cs, b_rs, b_cs;      // element strides of A(m,k) and B(k,n)
    long long strideA, strideB, strideC;
    long long ldc, ldres, ldaux;
    const void* A; const void* B; void* C;
    const void* bias; const void* residual; void* aux_out; const void* aux_in;
    int act, dact, accumulate;
};

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtParams p) {
    __shared__ float sA[TK][TM + 1];
    __shared__ float sB[TK][TN + 1];
    const int b = blockIdx.z;
    const TI* A = reinterpret_cast<const TI*>(p.A) + b * p.strideA;
    const TI* B = reinterpret_cast<const TI*>(p.B) + b * p.strideB;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < p.K; k0 += TK) {
        for (int i = threadIdx.x; i < TM * TK; i += 256) {
            // A tile: pick the loop order that follows the contiguous direction of A
            int m, k;
            if (p.a_cs == 1) { k = i % TK; m = i / TK; } else { m = i % TM; k = i / TM; }
            const int gm = m0 + m, gk = k0 + k;
            sA[k][m] = (gm < p.M && gk < p.K) ? to_f32<TI>(A[gm * p.a_rs + gk * p.a_cs]) : 0.f;
        }
        for (int i = threadIdx.x; i < TN * TK; i += 256) {
            int n, k;
            if (p.b_cs == 1) { n = i % TN; k = i / TN; } else { k = i % TK; n = i / TK; }
            const int gn = n0 + n, gk = k0 + k;
            sB[k][n] = (gn < p.N && gk < p.K) ? to_f32<TI>(B[gk * p.b_rs + gn * p.b_cs]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], bb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sA[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bb[j] = sB[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
        }
        __syncthreads();
    }
    TO* C = reinterpret_cast<TO*>(p.C) + b * p.strideC;
    const TO* R = p.residual ? reinterpret_cast<const TO*>(p.residual) + b * p.strideC : nullptr;
    TO* XO = p.aux_out ? reinterpret_cast<TO*>(p.aux_out) + b * p.strideC : nullptr;
    const TO* XI = p.aux_in ? reinterpret_cast<const TO*>(p.aux_in) + b * p.strideC : nullptr;
    const TI* bias = reinterpret_cast<const TI*>(p.bias);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            float v = acc[i][j];
            if (bias) v += to_f32<TI>(bias[n]);
            if (XO) XO[m * p.ldaux + n] = from_f32<TO>(v);
            if (p.act == CME_ACT_RELU) v = fmaxf(v, 0.f);
            else if (p.act == CME_ACT_GELU) v = gelu_f(v);
            if (p.dact) {
                const float x = to_f32<TO>(XI[m * p.ldaux + n]);
                v = (p.dact == CME_ACT_RELU) ? (x > 0.f ? v : 0.f) : v * dgelu_f(x);
            }
            if (R) v += to_f32<TO>(R[m * p.ldres + n]);
            if (p.accumulate) v += to_f32<TO>(C[m * p.ldc + n]);
            C[m * p.ldc + n] = from_f32<TO>(v);
        }
    }
}

}  // namespace

int gemm_simt_launch(const CmeGemm* g, cudaStream_t stream) {
    CME_REQUIRE(g->M > 0 && g->N > 0 && g->K > 0 && g->batch > 0, CME_ERR_SHAPE, "empty gemm");
    SimtParams p{};
    p.M = g->M; p.N = g->N; p.K = g->K;
    if (!g->a_trans) { p.a_rs = g->lda; p.a_cs = 1; } else { p.a_rs = 1; p.a_cs = g->lda; }
    if (!g->b_trans) { p.b_rs = g->ldb; p.b_cs = 1; } else { p.b_rs = 1; p.b_cs = g->ldb; }
    p.strideA = g->strideA; p.strideB = g->strideB; p.strideC = g->strideC;
    p.ldc = g->ldc; p.ldres = g->ldres; p.ldaux = g->ldaux;
    p.A = g->A; p.B = g->B; p.C = g->C;
    p.bias = g->bias; p.residual = g->residual; p.aux_out = g->aux_out; p.aux_in = g->aux_in;
    p.act = g->act; p.dact = g->dact; p.accumulate = g->accumulate;
    dim3 grid(cme_cdiv(g->N, TN), cme_cdiv(g->M, TM), g->batch);
    const bool in_bf = g->ab_dtype == CME_BF16, out_bf = g->c_dtype == CME_BF16;
    if (in_bf && out_bf) gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(p);
    else if (in_bf && !out_bf) gemm_simt_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(p);
    else if (!in_bf && !out_bf) gemm_simt_kernel<float, float><<<grid, 256, 0, stream>>>(p);
    else gemm_simt_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>(p);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

// Dispatch: tcgen05 when the shape allows it, SIMT otherwise.  backend: 0 auto, 1 tcgen05 only, 2 SIMT only.
CME_API int cme_gemm(const CmeGemm* g, int backend, void* stream) {
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (backend == 2) return gemm_simt_launch(g, st);
    if (gemm_tcgen05_supported(g)) return gemm_tcgen05_launch(g, st);
    CME_REQUIRE(backend != 1, CME_ERR_SHAPE, "gemm shape/alignment not supported by the tcgen05 kernel");
    return gemm_simt_launch(g, st);
}
