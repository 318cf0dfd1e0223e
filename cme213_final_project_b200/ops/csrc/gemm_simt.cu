// Generic CUDA-core GEMM: any shape, any of the four storage combinations, fp32 or bf16 operands, fp32
// accumulation, the full epilogue of gemm.h.  It is the strict-fp32 path of the parity model, the
// fallback for shapes the TMA path cannot address (e.g. the reference's N = vocab = 65 output head,
// which FINAL_CLEAN_CODE_/src/kernels/gemm.cu:742-754 also routes to its scalar kernel), and the
// independent implementation the tcgen05 kernel is checked against.
//
// 64 x 64 output tile, 32-deep K slices in shared memory, 256 threads, 4 x 4 outputs per thread, the next
// slice prefetched into registers while the current one is multiplied; skinny products with a long reduction
// (weight gradients of the 65-column head) split K over the grid and are summed in a fixed order.  One
// stride-generic kernel serves NN / NT / TN and batches (the reference keeps a kernel per layout, gemm.cu:483-1998).
#include "gemm.h"

namespace {

constexpr int TM = 64, TN = 64, TK = 32;

struct SimtParams {
    int M, N, K;
    long long a_rs, a_cs, b_rs, b_cs;      // element strides of A(m,k) and B(k,n)
    long long strideA, strideB, strideC;
    long long ldc, ldres, ldaux;
    const void* A; const void* B; void* C;
    const void* bias; const void* residual; void* aux_out; const void* aux_in;
    int act, dact, accumulate, aux_deriv;
    int batch, splits, k_per_split;        // grid.z = batch * splits; split > 0 writes fp32 partials to `partial`
    float* partial;
};

// Global -> register stage of one K slice (8 A values and 8 B values per thread), issued one slice ahead of the
// arithmetic so the global-memory latency of slice i+1 hides behind the FMAs of slice i.
template <typename TI>
__device__ __forceinline__ void fetch_slice(const SimtParams& p, const TI* A, const TI* B, int m0, int n0, int k0,
                                            int kend, float* ra, float* rb) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + j * 256;
        int m, k;
        if (p.a_cs == 1) { k = i % TK; m = i / TK; } else { m = i % TM; k = i / TM; }
        const int gm = m0 + m, gk = k0 + k;
        ra[j] = (gm < p.M && gk < kend) ? to_f32<TI>(A[gm * p.a_rs + gk * p.a_cs]) : 0.f;
        int n, kk;
        if (p.b_cs == 1) { n = i % TN; kk = i / TN; } else { kk = i % TK; n = i / TK; }
        const int gn = n0 + n, gk2 = k0 + kk;
        rb[j] = (gn < p.N && gk2 < kend) ? to_f32<TI>(B[gk2 * p.b_rs + gn * p.b_cs]) : 0.f;
    }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtParams p) {
    __shared__ float sA[TK][TM + 1];
    __shared__ float sB[TK][TN + 1];
    const int b = blockIdx.z % p.batch, split = blockIdx.z / p.batch;
    const TI* A = reinterpret_cast<const TI*>(p.A) + b * p.strideA;
    const TI* B = reinterpret_cast<const TI*>(p.B) + b * p.strideB;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int kbeg = split * p.k_per_split, kend = min(p.K, kbeg + p.k_per_split);
    float acc[4][4] = {};
    float ra[8], rb[8];
    fetch_slice<TI>(p, A, B, m0, n0, kbeg, kend, ra, rb);
    for (int k0 = kbeg; k0 < kend; k0 += TK) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = threadIdx.x + j * 256;
            int m, k;
            if (p.a_cs == 1) { k = i % TK; m = i / TK; } else { m = i % TM; k = i / TM; }
            sA[k][m] = ra[j];
            int n, kk;
            if (p.b_cs == 1) { n = i % TN; kk = i / TN; } else { kk = i % TK; n = i / TK; }
            sB[kk][n] = rb[j];
        }
        __syncthreads();
        if (k0 + TK < kend) fetch_slice<TI>(p, A, B, m0, n0, k0 + TK, kend, ra, rb);
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
    if (p.splits > 1) {          // fp32 partial sums: [split][batch][M][N]
        float* P = p.partial + ((long long)split * p.batch + b) * p.M * p.N;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int m = m0 + ty * 4 + i;
            if (m >= p.M) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + tx * 4 + j;
                if (n < p.N) P[(long long)m * p.N + n] = acc[i][j];
            }
        }
        return;
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
            if (XO) XO[m * p.ldaux + n] = from_f32<TO>((p.aux_deriv && p.act == CME_ACT_GELU) ? dgelu_f(v) : v);
            if (p.act == CME_ACT_RELU) v = fmaxf(v, 0.f);
            else if (p.act == CME_ACT_GELU) v = gelu_f(v);
            if (p.dact) {
                const float x = to_f32<TO>(XI[m * p.ldaux + n]);
                v = (p.dact == CME_ACT_RELU) ? (x > 0.f ? v : 0.f) : p.aux_deriv ? v * x : v * dgelu_f(x);
            }
            if (R) v += to_f32<TO>(R[m * p.ldres + n]);
            if (p.accumulate) v += to_f32<TO>(C[m * p.ldc + n]);
            C[m * p.ldc + n] = from_f32<TO>(v);
        }
    }
}

// C (+)= sum over splits of the fp32 partials, fixed order.
template <typename TO>
__global__ void simt_splitk_reduce_kernel(const float* __restrict__ P, int splits, int batch, int M, int N, TO* C,
                                          long long ldc, long long strideC, int accumulate) {
    const long long per = (long long)batch * M * N;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per; i += (long long)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < splits; ++k) s += P[k * per + i];
        const long long b = i / ((long long)M * N), rem = i % ((long long)M * N);
        TO* dst = C + b * strideC + (rem / N) * ldc + (rem % N);
        *dst = from_f32<TO>(accumulate ? to_f32<TO>(*dst) + s : s);
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
    p.act = g->act; p.dact = g->dact; p.accumulate = g->accumulate; p.aux_deriv = g->aux_deriv;
    p.batch = g->batch;
    if (g->colsum_slabs) *g->colsum_slabs = 0;              // this kernel does not sum columns; the caller does
    // Split K when the output has few tiles and the reduction is long (skinny weight gradients).
    const long long tiles = (long long)cme_cdiv(g->N, TN) * cme_cdiv(g->M, TM) * g->batch;
    const bool plain = !g->bias && !g->residual && !g->aux_out && !g->act && !g->dact;
    int splits = 1;
    if (plain && g->workspace && tiles < 64 && g->K >= 512) {
        splits = (int)(256 / tiles);
        if (splits > g->K / 64) splits = g->K / 64;
        while (splits > 1 && (long long)splits * g->batch * g->M * g->N * 4 > g->workspace_bytes) --splits;
        if (splits < 1) splits = 1;
    }
    p.k_per_split = cme_cdiv(cme_cdiv(g->K, splits), TK) * TK;
    splits = cme_cdiv(g->K, p.k_per_split);
    p.splits = splits;
    p.partial = reinterpret_cast<float*>(g->workspace);
    dim3 grid(cme_cdiv(g->N, TN), cme_cdiv(g->M, TM), g->batch * splits);
    const bool in_bf = g->ab_dtype == CME_BF16, out_bf = g->c_dtype == CME_BF16;
    if (in_bf && out_bf) gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(p);
    else if (in_bf && !out_bf) gemm_simt_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>(p);
    else if (!in_bf && !out_bf) gemm_simt_kernel<float, float><<<grid, 256, 0, stream>>>(p);
    else gemm_simt_kernel<float, __nv_bfloat16><<<grid, 256, 0, stream>>>(p);
    CME_LAUNCH_CHECK();
    if (splits > 1) {
        const long long per = (long long)g->batch * g->M * g->N;
        const int blocks = (int)((per + 255) / 256 < 1024 ? (per + 255) / 256 : 1024);
        if (out_bf)
            simt_splitk_reduce_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
                p.partial, splits, g->batch, g->M, g->N, reinterpret_cast<__nv_bfloat16*>(g->C), g->ldc, g->strideC,
                g->accumulate);
        else
            simt_splitk_reduce_kernel<float><<<blocks, 256, 0, stream>>>(p.partial, splits, g->batch, g->M, g->N,
                                                                       reinterpret_cast<float*>(g->C), g->ldc,
                                                                       g->strideC, g->accumulate);
        CME_LAUNCH_CHECK();
    }
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
