// CUDA-core attention, forward and backward, any head size up to 128, fp32 or bf16 I/O, fp32 math.
//
// This is the strict-precision / any-shape path (parity tests, head sizes the tensor-core kernel does not
// take).  The reference's production attention materialises scores, probabilities and their gradients as
// three [B*H, T, T] buffers around batched GEMMs (FINAL_CLEAN_CODE_/src/kernels/attention.cu:138-200,
// 253-328); its streaming kernel (:56-136) is forward-only and unused.  Here both directions stream
// key / query tiles through shared memory with an online softmax, keep only the log-sum-exp per row,
// and recompute probabilities in the backward pass, so nothing of size T x T touches global memory.
#include "attention.h"

namespace {

constexpr int RT = 16;       // rows owned by a block (queries in fwd / dQ, keys in dK / dV)
constexpr int CT = 32;       // columns streamed per step
constexpr int MAXD = 16;     // HD / 8 per thread -> HD <= 128

__device__ __forceinline__ long long head_base(const CmeAttn& a, int bh) {
    return (long long)(bh / a.nh) * a.sb + (long long)(bh % a.nh) * a.sh;
}
__device__ __forceinline__ long long head_base_o(const CmeAttn& a, int bh) {
    return (long long)(bh / a.nh) * a.osb + (long long)(bh % a.nh) * a.osh;
}

template <typename T>
__device__ __forceinline__ void load_tile(float* dst, const T* src, long long base, long long st, int r0, int rows,
                                          int T_, int HD, float mul) {
    for (int i = threadIdx.x; i < rows * HD; i += blockDim.x) {
        const int r = i / HD, d = i % HD;
        dst[r * (HD + 1) + d] = (r0 + r < T_) ? to_f32<T>(src[base + (long long)(r0 + r) * st + d]) * mul : 0.f;
    }
}

template <typename T>
__global__ void __launch_bounds__(128) attn_fwd_kernel(const CmeAttn a) {
    extern __shared__ float sm[];
    const int HD = a.HD, P = HD + 1;
    float* sQ = sm;                    // [RT][P]
    float* sK = sQ + RT * P;           // [CT][P]
    float* sV = sK + CT * P;           // [CT][P]
    float* sP = sV + CT * P;           // [RT][CT]
    const int bh = blockIdx.y, q0 = blockIdx.x * RT;
    const long long base = head_base(a, bh);
    const int r = threadIdx.x >> 3, s = threadIdx.x & 7;
    const T* q = (const T*)a.q; const T* k = (const T*)a.k; const T* v = (const T*)a.v;
    load_tile<T>(sQ, q, base, a.st, q0, RT, a.T, HD, a.scale);
    float m = -INFINITY, l = 0.f, o[MAXD];
#pragma unroll
    for (int i = 0; i < MAXD; ++i) o[i] = 0.f;
    const int kend = a.causal ? min(a.T, q0 + RT) : a.T;
    for (int k0 = 0; k0 < kend; k0 += CT) {
        __syncthreads();
        load_tile<T>(sK, k, base, a.st, k0, CT, a.T, HD, 1.f);
        load_tile<T>(sV, v, base, a.st, k0, CT, a.T, HD, 1.f);
        __syncthreads();
        float sc[4], tmax = -INFINITY;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int j = s + 8 * jj;
            float d = 0.f;
            for (int x = 0; x < HD; ++x) d += sQ[r * P + x] * sK[j * P + x];
            const bool ok = (k0 + j < a.T) && (!a.causal || k0 + j <= q0 + r);
            sc[jj] = ok ? d : -INFINITY;
            tmax = fmaxf(tmax, sc[jj]);
        }
#pragma unroll
        for (int off = 1; off < 8; off <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
        const float mnew = fmaxf(m, tmax);
        float psum = 0.f;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const float p = (mnew == -INFINITY) ? 0.f : __expf(sc[jj] - mnew);
            sP[r * CT + s + 8 * jj] = p;
            psum += p;
        }
#pragma unroll
        for (int off = 1; off < 8; off <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
        const float alpha = (m == -INFINITY) ? 0.f : __expf(m - mnew);
        l = l * alpha + psum;
        m = mnew;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < MAXD; ++i) o[i] *= alpha;
        for (int j = 0; j < CT; ++j) {
            const float p = sP[r * CT + j];
#pragma unroll
            for (int i = 0; i < MAXD; ++i)
                if (s + 8 * i < HD) o[i] += p * sV[j * P + s + 8 * i];
        }
    }
    if (q0 + r < a.T) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        T* out = (T*)a.o;
#pragma unroll
        for (int i = 0; i < MAXD; ++i)
            if (s + 8 * i < HD)
                out[head_base_o(a, bh) + (long long)(q0 + r) * a.ost + s + 8 * i] = from_f32<T>(o[i] * inv);
        if (s == 0 && a.lse) a.lse[(long long)bh * a.T + q0 + r] = m + logf(l);
    }
}

// delta[bh, t] = sum_d dO * O
template <typename T>
__global__ void attn_delta_kernel(const CmeAttn a) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int rows = a.nb * a.nh * a.T;
    if (row >= rows) return;
    const int bh = row / a.T, t = row % a.T;
    const long long off = head_base_o(a, bh) + (long long)t * a.ost;
    float s = 0.f;
    for (int d = threadIdx.x & 31; d < a.HD; d += 32)
        s += to_f32<T>(((const T*)a.d_o)[off + d]) * to_f32<T>(((const T*)a.o)[off + d]);
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) a.delta[row] = s;
}
// bf16, head size 64, 16-byte aligned rows: 8 lanes per row (one 128-bit load each), 4 rows per warp.
__global__ void attn_delta_hd64_kernel(const CmeAttn a) {
    const int rows = a.nb * a.nh * a.T;
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 3, sub = threadIdx.x & 7;
    float s = 0.f;
    if (row < rows) {
        const int bh = row / a.T, t = row % a.T;
        const long long off = head_base_o(a, bh) + (long long)t * a.ost + sub * 8;
        float x[8], y[8];
        unpack8(*reinterpret_cast<const Bf16x8*>((const __nv_bfloat16*)a.d_o + off), x);
        unpack8(*reinterpret_cast<const Bf16x8*>((const __nv_bfloat16*)a.o + off), y);
#pragma unroll
        for (int i = 0; i < 8; ++i) s += x[i] * y[i];
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    if (row < rows && sub == 0) a.delta[row] = s;
}

// KV = false: block owns RT queries, streams keys:    dQ = scale * sum_j dS_ij K_j
// KV = true : block owns RT keys, streams queries:    dV = sum_i P_ij dO_i ;  dK = scale * sum_i dS_ij Q_i
template <typename T, bool KV>
__global__ void __launch_bounds__(128) attn_bwd_kernel(const CmeAttn a) {
    extern __shared__ float sm[];
    const int HD = a.HD, P = HD + 1;
    float* sA = sm;                    // own rows, first operand   [RT][P]   (Q | K)
    float* sB = sA + RT * P;           // own rows, second operand  [RT][P]   (dO | V)
    float* sC = sB + RT * P;           // streamed, first operand   [CT][P]   (K | Q)
    float* sD = sC + CT * P;           // streamed, second operand  [CT][P]   (V | dO)
    float* sP = sD + CT * P;           // [RT][CT] probabilities
    float* sS = sP + RT * CT;          // [RT][CT] dS
    float* sL = sS + RT * CT;          // [CT] lse of streamed queries (KV) ; unused otherwise
    float* sDl = sL + CT;              // [CT] delta of streamed queries (KV)
    const int bh = blockIdx.y, r0 = blockIdx.x * RT;
    const long long base = head_base(a, bh);
    const int r = threadIdx.x >> 3, s = threadIdx.x & 7;
    const T* q = (const T*)a.q; const T* k = (const T*)a.k; const T* v = (const T*)a.v; const T* d_o = (const T*)a.d_o;
    load_tile<T>(sA, KV ? k : q, base, a.st, r0, RT, a.T, HD, 1.f);
    const long long obase = head_base_o(a, bh);
    if (KV) load_tile<T>(sB, v, base, a.st, r0, RT, a.T, HD, 1.f);
    else load_tile<T>(sB, d_o, obase, a.ost, r0, RT, a.T, HD, 1.f);
    float acc1[MAXD], acc2[MAXD];
#pragma unroll
    for (int i = 0; i < MAXD; ++i) { acc1[i] = 0.f; acc2[i] = 0.f; }
    float my_lse = 0.f, my_delta = 0.f;
    if (!KV && r0 + r < a.T) {
        my_lse = a.lse[(long long)bh * a.T + r0 + r];
        my_delta = a.delta[(long long)bh * a.T + r0 + r];
    }
    // causal: queries see keys <= their index.  dQ blocks stop early; dK/dV blocks start late.
    const int c_begin = (KV && a.causal) ? (r0 / CT) * CT : 0;
    const int c_end = (!KV && a.causal) ? min(a.T, r0 + RT) : a.T;
    for (int c0 = c_begin; c0 < c_end; c0 += CT) {
        __syncthreads();
        load_tile<T>(sC, KV ? q : k, base, a.st, c0, CT, a.T, HD, 1.f);
        if (KV) load_tile<T>(sD, d_o, obase, a.ost, c0, CT, a.T, HD, 1.f);
        else load_tile<T>(sD, v, base, a.st, c0, CT, a.T, HD, 1.f);
        if (KV && threadIdx.x < CT) {
            const int t = c0 + threadIdx.x;
            sL[threadIdx.x] = t < a.T ? a.lse[(long long)bh * a.T + t] : 0.f;
            sDl[threadIdx.x] = t < a.T ? a.delta[(long long)bh * a.T + t] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int j = s + 8 * jj;
            float sc = 0.f, dp = 0.f;
            for (int x = 0; x < HD; ++x) {
                sc += sA[r * P + x] * sC[j * P + x];
                dp += sB[r * P + x] * sD[j * P + x];
            }
            const int qi = KV ? c0 + j : r0 + r, ki = KV ? r0 + r : c0 + j;
            const bool ok = qi < a.T && ki < a.T && (!a.causal || ki <= qi);
            const float lse = KV ? sL[j] : my_lse, dl = KV ? sDl[j] : my_delta;
            const float p = ok ? __expf(sc * a.scale - lse) : 0.f;
            sP[r * CT + j] = p;
            sS[r * CT + j] = p * (dp - dl);
        }
        __syncwarp();
        for (int j = 0; j < CT; ++j) {
            const float p = sP[r * CT + j], ds = sS[r * CT + j];
#pragma unroll
            for (int i = 0; i < MAXD; ++i) {
                if (s + 8 * i < HD) {
                    if (KV) {
                        acc1[i] += p * sD[j * P + s + 8 * i];       // dV += P^T dO
                        acc2[i] += ds * sC[j * P + s + 8 * i];      // dK += dS^T Q
                    } else {
                        acc1[i] += ds * sC[j * P + s + 8 * i];      // dQ += dS K
                    }
                }
            }
        }
    }
    if (r0 + r < a.T) {
        const long long off = base + (long long)(r0 + r) * a.st;
#pragma unroll
        for (int i = 0; i < MAXD; ++i) {
            if (s + 8 * i < HD) {
                if (KV) {
                    ((T*)a.dv)[off + s + 8 * i] = from_f32<T>(acc1[i]);
                    ((T*)a.dk)[off + s + 8 * i] = from_f32<T>(acc2[i] * a.scale);
                } else {
                    ((T*)a.dq)[off + s + 8 * i] = from_f32<T>(acc1[i] * a.scale);
                }
            }
        }
    }
}

template <typename T> int fwd_t(const CmeAttn* a, cudaStream_t st) {
    const size_t smem = ((RT + 2 * CT) * (a->HD + 1) + RT * CT) * sizeof(float);
    auto k = attn_fwd_kernel<T>;
    if (smem > 48 * 1024) CME_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(cme_cdiv(a->T, RT), a->nb * a->nh);
    k<<<grid, 128, smem, st>>>(*a);
    CME_LAUNCH_CHECK();
    return CME_OK;
}
template <typename T> int bwd_t(const CmeAttn* a, cudaStream_t st) {
    const int rows = a->nb * a->nh * a->T;
    attn_delta_kernel<T><<<cme_cdiv(rows, 8), 256, 0, st>>>(*a);
    CME_LAUNCH_CHECK();
    const size_t smem = ((2 * RT + 2 * CT) * (a->HD + 1) + 2 * RT * CT + 2 * CT) * sizeof(float);
    auto k1 = attn_bwd_kernel<T, false>;
    auto k2 = attn_bwd_kernel<T, true>;
    if (smem > 48 * 1024) {
        CME_CUDA(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        CME_CUDA(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    dim3 grid(cme_cdiv(a->T, RT), a->nb * a->nh);
    k1<<<grid, 128, smem, st>>>(*a);
    CME_LAUNCH_CHECK();
    k2<<<grid, 128, smem, st>>>(*a);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

int check(const CmeAttn* a, bool bwd) {
    CME_REQUIRE(a->nb > 0 && a->nh > 0 && a->T > 0 && a->HD > 0, CME_ERR_SHAPE, "attention: empty input");
    CME_REQUIRE(a->HD <= 8 * MAXD, CME_ERR_LIMIT, "attention: head size %d exceeds %d", a->HD, 8 * MAXD);
    CME_REQUIRE(a->lse != nullptr, CME_ERR_SHAPE, "attention: lse buffer is required");
    if (bwd) CME_REQUIRE(a->delta && a->d_o && a->dq && a->dk && a->dv, CME_ERR_SHAPE, "attention backward: missing buffer");
    return CME_OK;
}

}  // namespace

// delta[bh, t] = sum_d dO * O, shared with the tensor-core backward.
int attention_delta_launch(const CmeAttn* a, cudaStream_t st) {
    const int rows = a->nb * a->nh * a->T;
    const bool al = ((reinterpret_cast<uintptr_t>(a->d_o) | reinterpret_cast<uintptr_t>(a->o)) & 15) == 0 &&
                    a->ost % 8 == 0 && a->osh % 8 == 0 && a->osb % 8 == 0;
    if (a->dtype == CME_BF16 && a->HD == 64 && al)
        attn_delta_hd64_kernel<<<cme_cdiv((long long)rows * 8, 256), 256, 0, st>>>(*a);
    else if (a->dtype == CME_BF16) attn_delta_kernel<__nv_bfloat16><<<cme_cdiv(rows, 8), 256, 0, st>>>(*a);
    else attn_delta_kernel<float><<<cme_cdiv(rows, 8), 256, 0, st>>>(*a);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

int attention_simt_fwd(const CmeAttn* a, cudaStream_t st) {
    int rc = check(a, false);
    if (rc) return rc;
    return a->dtype == CME_BF16 ? fwd_t<__nv_bfloat16>(a, st) : fwd_t<float>(a, st);
}
int attention_simt_bwd(const CmeAttn* a, cudaStream_t st) {
    int rc = check(a, true);
    if (rc) return rc;
    return a->dtype == CME_BF16 ? bwd_t<__nv_bfloat16>(a, st) : bwd_t<float>(a, st);
}

// backend: 0 auto (fused tensor-core kernel, else batched-GEMM path, else SIMT), 1 fused tensor-core only,
//          2 SIMT only, 3 batched-GEMM path only
CME_API int cme_attention_fwd(const CmeAttn* a, int backend, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if ((backend == 0 || backend == 1) && attention_tc_supported(a)) return attention_tc_fwd(a, st);
    CME_REQUIRE(backend != 1, CME_ERR_SHAPE, "attention shape not supported by the tensor-core kernel");
    if ((backend == 0 || backend == 3) && attention_gemm_supported(a)) return attention_gemm_fwd(a, st);
    CME_REQUIRE(backend != 3, CME_ERR_SHAPE, "attention shape not supported by the batched-GEMM path");
    return attention_simt_fwd(a, st);
}
CME_API int cme_attention_bwd(const CmeAttn* a, int backend, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if ((backend == 0 || backend == 1) && attention_tc_supported(a)) return attention_tc_bwd(a, st);
    CME_REQUIRE(backend != 1, CME_ERR_SHAPE, "attention shape not supported by the tensor-core kernel");
    if ((backend == 0 || backend == 3) && attention_gemm_supported(a)) return attention_gemm_bwd(a, st);
    CME_REQUIRE(backend != 3, CME_ERR_SHAPE, "attention shape not supported by the batched-GEMM path");
    return attention_simt_bwd(a, st);
}
CME_API long long cme_attention_gemm_ws_bytes(int nb, int T) { return attention_gemm_ws_bytes(nb, T); }
