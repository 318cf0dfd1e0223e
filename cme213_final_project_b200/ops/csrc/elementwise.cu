// Element-wise, bias / activation, column-sum, cast, scale and embedding kernels (bf16 or fp32 I/O).
//
// Counterparts in the reference: FINAL_CLEAN_CODE_/src/kernels/activations.cu:5-357 (ReLU fwd/bwd,
// residual add, bias + residual add, bias add, bias + ReLU, bias backward, fused ReLU-backward +
// bias-backward, scale, float<->half casts) and FINAL_CLEAN_CODE_/src/kernels/embedding.cu:4-79
// (token gather, scatter-add backward, positional add and its backward).  Differences by design:
// token gather and positional add are one kernel; column sums (bias gradients) are reduced in two
// deterministic stages instead of atomicAdd; everything moves 128 bits per thread where alignment allows.
#include "common.h"

namespace {

template <typename T> struct Vw;
template <> struct Vw<float> { static constexpr int N = 4; };
template <> struct Vw<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ void ldv(const T* p, float* f);
template <> __device__ __forceinline__ void ldv<float>(const float* p, float* f) {
    float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void ldv<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
    unpack8(*reinterpret_cast<const Bf16x8*>(p), f);
}
template <typename T> __device__ __forceinline__ void stv(T* p, const float* f);
template <> __device__ __forceinline__ void stv<float>(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <> __device__ __forceinline__ void stv<__nv_bfloat16>(__nv_bfloat16* p, const float* f) {
    *reinterpret_cast<Bf16x8*>(p) = pack8(f);
}

__device__ __forceinline__ float act_f(float v, int act) {
    return act == 1 ? fmaxf(v, 0.f) : act == 2 ? gelu_f(v) : v;
}
__device__ __forceinline__ float dact_f(float pre, int act) {
    return act == 1 ? (pre > 0.f ? 1.f : 0.f) : act == 2 ? dgelu_f(pre) : 1.f;
}

// out[m, n] = act(x[m, n] + bias[n]) + residual[m, n]; any of bias / residual / pre_out may be null.
// One thread per vector of the row-major [rows, cols] matrix; cols is a multiple of the vector width.
template <typename T>
__global__ void bias_act_res_kernel(const T* __restrict__ x, const T* __restrict__ bias, const T* __restrict__ res,
                                    T* __restrict__ pre_out, T* __restrict__ out, long long nvec, int cols, int act) {
    constexpr int W = Vw<T>::N;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
        const long long e = i * W;
        const int c = (int)(e % cols);
        float v[W];
        ldv<T>(x + e, v);
        if (bias) {
            float b[W];
            ldv<T>(bias + c, b);
#pragma unroll
            for (int j = 0; j < W; ++j) v[j] += b[j];
        }
        if (pre_out) stv<T>(pre_out + e, v);
#pragma unroll
        for (int j = 0; j < W; ++j) v[j] = act_f(v[j], act);
        if (res) {
            float r[W];
            ldv<T>(res + e, r);
#pragma unroll
            for (int j = 0; j < W; ++j) v[j] += r[j];
        }
        stv<T>(out + e, v);
    }
}
template <typename T>
__global__ void bias_act_res_scalar_kernel(const T* x, const T* bias, const T* res, T* pre_out, T* out, long long n,
                                           int cols, int act) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        float v = to_f32<T>(x[i]);
        if (bias) v += to_f32<T>(bias[i % cols]);
        if (pre_out) pre_out[i] = from_f32<T>(v);
        v = act_f(v, act);
        if (res) v += to_f32<T>(res[i]);
        out[i] = from_f32<T>(v);
    }
}

// g[m, n] = dout[m, n] * act'(pre[m, n])  (written if g != null)  and partial column sums of g.
// Block = 32 row-lanes x 8 column-lanes; each thread owns one vector of columns.
// grid = (ceil(cols / (8*W)), row_splits); partial is [row_splits][cols].
template <typename T>
__global__ void __launch_bounds__(256)
dact_colsum_kernel(const T* __restrict__ dout, const T* __restrict__ pre, T* __restrict__ g, float* __restrict__ partial,
                   int rows, int cols, int act) {
    constexpr int W = Vw<T>::N;
    __shared__ float sm[32][8 * W + 1];
    pdl_wait();
    const int cl = threadIdx.x & 7, rl = threadIdx.x >> 3;
    const int c0 = (blockIdx.x * 8 + cl) * W;
    float s[W];
#pragma unroll
    for (int j = 0; j < W; ++j) s[j] = 0.f;
    const int rows_per = cme_cdiv_dev(rows, (int)gridDim.y);
    const int r0 = blockIdx.y * rows_per, r1 = min(rows, r0 + rows_per);
    if (c0 < cols) {
        for (int r = r0 + rl; r < r1; r += 32) {
            const long long e = (long long)r * cols + c0;
            float d[W];
            ldv<T>(dout + e, d);
            if (pre) {
                float p[W];
                ldv<T>(pre + e, p);
#pragma unroll
                for (int j = 0; j < W; ++j) d[j] *= dact_f(p[j], act);
            }
            if (g) stv<T>(g + e, d);
#pragma unroll
            for (int j = 0; j < W; ++j) s[j] += d[j];
        }
    }
#pragma unroll
    for (int j = 0; j < W; ++j) sm[rl][cl * W + j] = s[j];
    __syncthreads();
    if (threadIdx.x < 8 * W) {
        float t = 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r) t += sm[r][threadIdx.x];
        const int c = blockIdx.x * 8 * W + threadIdx.x;
        if (c < cols) partial[(long long)blockIdx.y * cols + c] = t;
    }
}
// Scalar twin for column counts that are not a multiple of the vector width.
template <typename T>
__global__ void dact_colsum_scalar_kernel(const T* dout, const T* pre, T* g, float* partial, int rows, int cols,
                                          int act) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const int rows_per = cme_cdiv_dev(rows, (int)gridDim.y);
    const int r0 = blockIdx.y * rows_per, r1 = min(rows, r0 + rows_per);
    float s = 0.f;
    for (int r = r0; r < r1; ++r) {
        const long long e = (long long)r * cols + c;
        float d = to_f32<T>(dout[e]);
        if (pre) d *= dact_f(to_f32<T>(pre[e]), act);
        if (g) g[e] = from_f32<T>(d);
        s += d;
    }
    partial[(long long)blockIdx.y * cols + c] = s;
}
template <typename T>
__global__ void colsum_finalize_kernel(const float* partial, int splits, int cols, T* out, int accumulate) {
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += partial[(long long)k * cols + c];
    out[c] = from_f32<T>(accumulate ? to_f32<T>(out[c]) + s : s);
}

template <typename T> __global__ void scale_kernel(T* x, long long n, float s) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] = from_f32<T>(to_f32<T>(x[i]) * s);
}
template <typename TI, typename TO> __global__ void cast_kernel(const TI* x, TO* y, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        y[i] = from_f32<TO>(to_f32<TI>(x[i]));
}
// out = a + b (element-wise)
template <typename T> __global__ void add_kernel(const T* a, const T* b, T* out, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(to_f32<T>(a[i]) + to_f32<T>(b[i]));
}
// dx = dy where x > 0 else 0
template <typename T> __global__ void relu_bwd_kernel(const T* x, const T* dy, T* dx, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dx[i] = to_f32<T>(x[i]) > 0.f ? dy[i] : from_f32<T>(0.f);
}

// One xorshift round of (seed + i) -> uniform in [-scale, scale], evaluated in fp32.
template <typename T> __global__ void init_uniform_kernel(T* out, long long n, float scale, unsigned seed) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        unsigned s = seed + (unsigned)i;
        s ^= s << 13; s ^= s >> 17; s ^= s << 5;
        const float u = (float)(s & 0x7FFFFFFFu) / (float)0x7FFFFFFF;
        out[i] = from_f32<T>((u * 2.0f - 1.0f) * scale);
    }
}

// ---- embeddings -------------------------------------------------------------------------------
// out[bt, :] = tok[tokens[bt], :] + pos[bt % T, :]
template <typename T>
__global__ void embed_fwd_kernel(const int* __restrict__ tokens, const T* __restrict__ tok, const T* __restrict__ pos,
                                 T* __restrict__ out, int BT, int T_, int D, int V, int vec) {
    constexpr int W = Vw<T>::N;
    if (vec) {
        const int nv = D / W;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)BT * nv;
             i += (long long)gridDim.x * blockDim.x) {
            const int bt = (int)(i / nv), c = (int)(i % nv) * W;
            int id = tokens[bt];
            id = id < 0 ? 0 : (id >= V ? V - 1 : id);
            float a[W], b[W];
            ldv<T>(tok + (long long)id * D + c, a);
            ldv<T>(pos + (long long)(bt % T_) * D + c, b);
#pragma unroll
            for (int j = 0; j < W; ++j) a[j] += b[j];
            stv<T>(out + (long long)bt * D + c, a);
        }
    } else {
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)BT * D;
             i += (long long)gridDim.x * blockDim.x) {
            const int bt = (int)(i / D), c = (int)(i % D);
            int id = tokens[bt];
            id = id < 0 ? 0 : (id >= V ? V - 1 : id);
            out[i] = from_f32<T>(to_f32<T>(tok[(long long)id * D + c]) + to_f32<T>(pos[(long long)(bt % T_) * D + c]));
        }
    }
}
// dpos[t, c] (+)= sum_b dout[b*T + t, c]   (deterministic: one thread per (t, c), loop over b)
template <typename T>
__global__ void pos_bwd_kernel(const T* __restrict__ dout, T* __restrict__ dpos, int B, int T_, int D, int accumulate) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)T_ * D) return;
    float s = accumulate ? to_f32<T>(dpos[i]) : 0.f;
    for (int b = 0; b < B; ++b) s += to_f32<T>(dout[(long long)b * T_ * D + i]);
    dpos[i] = from_f32<T>(s);
}
// Small vocabularies: one block (8 warps) per vocabulary row.  Each warp scans its own contiguous eighth of the
// token list with ballots and sums the matching rows of dout in token order; the eight partial rows are then added
// in warp order.  Deterministic (no atomics) and the scan is 32 tokens per instruction.
//     dtok[v, :] (+)= sum_{bt : tokens[bt] == v} dout[bt, :]
template <typename T>
__global__ void __launch_bounds__(256)
tok_bwd_scan_kernel(const int* __restrict__ tokens, const T* __restrict__ dout, T* __restrict__ dtok, int BT, int D,
                    int accumulate) {
    extern __shared__ float part[];              // [8][D]
    const int v = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per = (BT + 7) / 8, t0 = warp * per, t1 = min(BT, t0 + per);
    for (int c0 = 0; c0 < D; c0 += 32 * 8) {     // 8 columns per lane per pass
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int base = t0; base < t1; base += 32) {
            const int bt = base + lane;
            unsigned hit = __ballot_sync(0xffffffffu, bt < t1 && tokens[bt] == v);
            while (hit) {
                const int src = base + __ffs(hit) - 1;
                hit &= hit - 1;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int c = c0 + lane + 32 * j;
                    if (c < D) acc[j] += to_f32<T>(dout[(long long)src * D + c]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = c0 + lane + 32 * j;
            if (c < D) part[warp * D + c] = acc[j];
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float s2 = accumulate ? to_f32<T>(dtok[(long long)v * D + c]) : 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) s2 += part[w * D + c];
        dtok[(long long)v * D + c] = from_f32<T>(s2);
    }
}
// Large vocabularies: one warp per token, atomic adds into the (already initialised) table gradient.
__device__ __forceinline__ void atomic_add_t(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add_t(__nv_bfloat16* p, float v) { atomicAdd(p, __float2bfloat16_rn(v)); }
template <typename T>
__global__ void tok_bwd_atomic_kernel(const int* __restrict__ tokens, const T* __restrict__ dout, T* __restrict__ dtok,
                                      int BT, int D, int V) {
    const int bt = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (bt >= BT) return;
    const int id = tokens[bt];
    if (id < 0 || id >= V) return;
    if constexpr (sizeof(T) == 2) {
        if (D % 2 == 0) {
            for (int c = (threadIdx.x & 31) * 2; c < D; c += 64) {
                __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(dout + (long long)bt * D + c);
                atomicAdd(reinterpret_cast<__nv_bfloat162*>(dtok + (long long)id * D + c), v);
            }
            return;
        }
    }
    for (int c = threadIdx.x & 31; c < D; c += 32)
        atomic_add_t(dtok + (long long)id * D + c, to_f32<T>(dout[(long long)bt * D + c]));
}

inline int grid_for(long long n, int block = 256, int cap = 148 * 16) {
    long long g = (n + block - 1) / block;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}
template <typename T> bool aligned16(const T* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
int bias_act_res_t(const void* x, const void* bias, const void* res, void* pre, void* out, long long rows, int cols,
                   int act, cudaStream_t st) {
    constexpr int W = Vw<T>::N;
    const long long n = rows * cols;
    const bool vec = cols % W == 0 && aligned16((const T*)x) && aligned16((const T*)out) &&
                     (!bias || aligned16((const T*)bias)) && (!res || aligned16((const T*)res)) &&
                     (!pre || aligned16((const T*)pre));
    if (vec)
        bias_act_res_kernel<T><<<grid_for(n / W), 256, 0, st>>>((const T*)x, (const T*)bias, (const T*)res, (T*)pre,
                                                                 (T*)out, n / W, cols, act);
    else
        bias_act_res_scalar_kernel<T><<<grid_for(n), 256, 0, st>>>((const T*)x, (const T*)bias, (const T*)res,
                                                                    (T*)pre, (T*)out, n, cols, act);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

// dbias[c] (+)= sum over the `slabs` rows of partial[slabs][cols], added in a fixed order: a block covers 32 columns
// with 8 row groups; each thread sums every 8th row (four independent chains), then the 8 groups are added in
// shared memory.  The rows come from a GEMM epilogue that sums its stored output per 32-row slab.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_slabs_finalize_kernel(const float* __restrict__ partial, int slabs, int cols, T* dbias, int accumulate) {
    __shared__ float sm[8][33];
    pdl_wait();
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cx;
    float s = 0.f;
    if (c < cols) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        int r = ry;
        for (; r + 24 < slabs; r += 32) {
            s0 += partial[(long long)r * cols + c];
            s1 += partial[(long long)(r + 8) * cols + c];
            s2 += partial[(long long)(r + 16) * cols + c];
            s3 += partial[(long long)(r + 24) * cols + c];
        }
        for (; r < slabs; r += 8) s0 += partial[(long long)r * cols + c];
        s = (s0 + s1) + (s2 + s3);
    }
    sm[ry][cx] = s;
    __syncthreads();
    if (ry == 0 && c < cols) {
        float t = 0.f;
#pragma unroll
        for (int g = 0; g < 8; ++g) t += sm[g][cx];
        dbias[c] = from_f32<T>(accumulate ? to_f32<T>(dbias[c]) + t : t);
    }
}

template <typename T>
int dact_colsum_t(const void* dout, const void* pre, void* g, void* dbias, float* scratch, int splits, int rows,
                  int cols, int act, int accumulate, cudaStream_t st) {
    constexpr int W = Vw<T>::N;
    const bool vec = cols % W == 0 && aligned16((const T*)dout) && (!pre || aligned16((const T*)pre)) &&
                     (!g || aligned16((const T*)g));
    if (vec) {
        dim3 grid(cme_cdiv(cols, 8 * W), splits);
        CME_CUDA(cme_launch_dependent(dact_colsum_kernel<T>, grid, dim3(256), 0, st, (const T*)dout, (const T*)pre, (T*)g,
                                      scratch, rows, cols, act));
    } else {
        dim3 grid(cme_cdiv(cols, 128), splits);
        dact_colsum_scalar_kernel<T><<<grid, 128, 0, st>>>((const T*)dout, (const T*)pre, (T*)g, scratch, rows, cols,
                                                            act);
    }
    CME_LAUNCH_CHECK();
    if (dbias) {
        CME_CUDA(cme_launch_dependent(colsum_finalize_kernel<T>, dim3(cme_cdiv(cols, 256)), dim3(256), 0, st,
                                      (const float*)scratch, splits, cols, (T*)dbias, accumulate));
        CME_LAUNCH_CHECK();
    }
    return CME_OK;
}

}  // namespace

#define DISPATCH_T(dtype, expr_bf16, expr_f32) ((dtype) == CME_BF16 ? (expr_bf16) : (expr_f32))

// out = act(x + bias) + residual; pre_out receives x + bias.  act: 0 none, 1 relu, 2 gelu.
CME_API int cme_bias_act_residual(int dtype, const void* x, const void* bias, const void* residual, void* pre_out,
                                  void* out, long long rows, int cols, int act, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    CME_REQUIRE(rows > 0 && cols > 0, CME_ERR_SHAPE, "bias_act_residual: empty input");
    return DISPATCH_T(dtype, bias_act_res_t<__nv_bfloat16>(x, bias, residual, pre_out, out, rows, cols, act, st),
                      bias_act_res_t<float>(x, bias, residual, pre_out, out, rows, cols, act, st));
}

// Row splits used by cme_dact_colsum for `rows`; scratch must hold splits * cols floats.
CME_API int cme_colsum_splits(int rows, int cols) {
    int col_blocks = cme_cdiv(cols, 64);
    int s = cme_cdiv(296, col_blocks);
    int max_s = cme_cdiv(rows, 64);
    if (s > max_s) s = max_s;
    return s < 1 ? 1 : s;
}

// g = dout * act'(pre) (pre, g optional) and dbias (+)= column sums of g.
CME_API int cme_dact_colsum(int dtype, const void* dout, const void* pre, void* g, void* dbias, float* scratch,
                            int rows, int cols, int act, int accumulate, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    CME_REQUIRE(rows > 0 && cols > 0, CME_ERR_SHAPE, "dact_colsum: empty input");
    const int splits = cme_colsum_splits(rows, cols);
    return DISPATCH_T(dtype,
                      dact_colsum_t<__nv_bfloat16>(dout, pre, g, dbias, scratch, splits, rows, cols, act, accumulate, st),
                      dact_colsum_t<float>(dout, pre, g, dbias, scratch, splits, rows, cols, act, accumulate, st));
}

// dbias (+)= column sums of partial[slabs][cols] (the per-slab sums a GEMM epilogue left, gemm.h: colsum).
CME_API int cme_colsum_slabs_finalize(int dtype, const float* partial, int slabs, int cols, void* dbias, int accumulate,
                                      void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    CME_REQUIRE(slabs > 0 && cols > 0, CME_ERR_SHAPE, "colsum finalize: empty input");
    if (dtype == CME_BF16)
        CME_CUDA(cme_launch_dependent(colsum_slabs_finalize_kernel<__nv_bfloat16>, dim3(cme_cdiv(cols, 32)), dim3(256), 0,
                                      st, partial, slabs, cols, (__nv_bfloat16*)dbias, accumulate));
    else
        CME_CUDA(cme_launch_dependent(colsum_slabs_finalize_kernel<float>, dim3(cme_cdiv(cols, 32)), dim3(256), 0, st,
                                      partial, slabs, cols, (float*)dbias, accumulate));
    CME_LAUNCH_CHECK();
    return CME_OK;
}

CME_API int cme_scale(int dtype, void* x, long long n, float s, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (n <= 0) return CME_OK;
    if (dtype == CME_BF16) scale_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, st>>>((__nv_bfloat16*)x, n, s);
    else scale_kernel<float><<<grid_for(n), 256, 0, st>>>((float*)x, n, s);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

CME_API int cme_cast(int src_dtype, const void* x, int dst_dtype, void* y, long long n, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (n <= 0) return CME_OK;
    const int g = grid_for(n);
    if (src_dtype == CME_F32 && dst_dtype == CME_BF16)
        cast_kernel<float, __nv_bfloat16><<<g, 256, 0, st>>>((const float*)x, (__nv_bfloat16*)y, n);
    else if (src_dtype == CME_BF16 && dst_dtype == CME_F32)
        cast_kernel<__nv_bfloat16, float><<<g, 256, 0, st>>>((const __nv_bfloat16*)x, (float*)y, n);
    else if (src_dtype == CME_F32)
        cast_kernel<float, float><<<g, 256, 0, st>>>((const float*)x, (float*)y, n);
    else
        cast_kernel<__nv_bfloat16, __nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

CME_API int cme_add(int dtype, const void* a, const void* b, void* out, long long n, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (n <= 0) return CME_OK;
    if (dtype == CME_BF16)
        add_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                                (__nv_bfloat16*)out, n);
    else add_kernel<float><<<grid_for(n), 256, 0, st>>>((const float*)a, (const float*)b, (float*)out, n);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

CME_API int cme_relu_bwd(int dtype, const void* x, const void* dy, void* dx, long long n, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (n <= 0) return CME_OK;
    if (dtype == CME_BF16)
        relu_bwd_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                                     (__nv_bfloat16*)dx, n);
    else relu_bwd_kernel<float><<<grid_for(n), 256, 0, st>>>((const float*)x, (const float*)dy, (float*)dx, n);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

CME_API int cme_init_uniform(int dtype, void* out, long long n, float scale, unsigned seed, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (n <= 0) return CME_OK;
    if (dtype == CME_BF16) init_uniform_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, st>>>((__nv_bfloat16*)out, n, scale, seed);
    else init_uniform_kernel<float><<<grid_for(n), 256, 0, st>>>((float*)out, n, scale, seed);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

CME_API int cme_embedding_fwd(int dtype, const int* tokens, const void* tok, const void* pos, void* out, int BT, int T,
                              int D, int V, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    CME_REQUIRE(BT > 0 && D > 0 && T > 0, CME_ERR_SHAPE, "embedding: empty input");
    if (dtype == CME_BF16) {
        const int vec = D % 8 == 0 && aligned16((const __nv_bfloat16*)tok) && aligned16((const __nv_bfloat16*)pos) &&
                        aligned16((const __nv_bfloat16*)out);
        embed_fwd_kernel<__nv_bfloat16><<<grid_for((long long)BT * D / (vec ? 8 : 1)), 256, 0, st>>>(
            tokens, (const __nv_bfloat16*)tok, (const __nv_bfloat16*)pos, (__nv_bfloat16*)out, BT, T, D, V, vec);
    } else {
        const int vec = D % 4 == 0 && aligned16((const float*)tok) && aligned16((const float*)pos) &&
                        aligned16((const float*)out);
        embed_fwd_kernel<float><<<grid_for((long long)BT * D / (vec ? 4 : 1)), 256, 0, st>>>(
            tokens, (const float*)tok, (const float*)pos, (float*)out, BT, T, D, V, vec);
    }
    CME_LAUNCH_CHECK();
    return CME_OK;
}

// dtok (+)= scatter of dout rows by token id; dpos (+)= sum over the batch.  With accumulate = 0 the
// outputs are overwritten (the scan path writes every row; the atomic path zero-fills first).
CME_API int cme_embedding_bwd(int dtype, const int* tokens, const void* dout, void* dtok, void* dpos, int BT, int T,
                              int D, int V, int accumulate, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    CME_REQUIRE(BT > 0 && D > 0 && T > 0 && BT % T == 0, CME_ERR_SHAPE, "embedding backward: bad shape");
    const size_t esz = dtype == CME_BF16 ? 2 : 4;
    const bool scan = (long long)V * BT <= (1ll << 22) && D <= 1536;
    if (dtok) {
        if (scan) {
            const size_t sm = (size_t)8 * D * sizeof(float);
            CME_REQUIRE(sm <= 48 * 1024, CME_ERR_LIMIT, "embedding backward: hidden size %d too large for the scan path", D);
            if (dtype == CME_BF16)
                tok_bwd_scan_kernel<__nv_bfloat16><<<V, 256, sm, st>>>(tokens, (const __nv_bfloat16*)dout,
                                                                       (__nv_bfloat16*)dtok, BT, D, accumulate);
            else
                tok_bwd_scan_kernel<float><<<V, 256, sm, st>>>(tokens, (const float*)dout, (float*)dtok, BT, D,
                                                               accumulate);
        } else {
            if (!accumulate) CME_CUDA(cudaMemsetAsync(dtok, 0, (size_t)V * D * esz, st));
            if (dtype == CME_BF16)
                tok_bwd_atomic_kernel<__nv_bfloat16><<<cme_cdiv(BT, 8), 256, 0, st>>>(
                    tokens, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dtok, BT, D, V);
            else
                tok_bwd_atomic_kernel<float><<<cme_cdiv(BT, 8), 256, 0, st>>>(tokens, (const float*)dout, (float*)dtok,
                                                                             BT, D, V);
        }
        CME_LAUNCH_CHECK();
    }
    if (dpos) {
        const long long n = (long long)T * D;
        if (dtype == CME_BF16)
            pos_bwd_kernel<__nv_bfloat16><<<cme_cdiv(n, 256), 256, 0, st>>>((const __nv_bfloat16*)dout,
                                                                           (__nv_bfloat16*)dpos, BT / T, T, D, accumulate);
        else
            pos_bwd_kernel<float><<<cme_cdiv(n, 256), 256, 0, st>>>((const float*)dout, (float*)dpos, BT / T, T, D,
                                                                   accumulate);
        CME_LAUNCH_CHECK();
    }
    return CME_OK;
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant of cme_dact_colsum (see noalloc.h for who it is for and the rules of use).
// ---------------------------------------------------------------------------------------------------
#include "noalloc.h"

#include <mutex>

// Scratch for the per-split partial column sums.  In host code this name is only a handle for the runtime
// (it is not a device address); the address kernels may use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_scratch[CME_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device; looked up once per device.
int noalloc_scratch(float** out) {
    int dev = 0;
    CME_CUDA(cudaGetDevice(&dev));
    CME_REQUIRE(dev >= 0 && dev < kMaxDevices, CME_ERR_LIMIT, "noalloc: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {
        float* p = nullptr;
        CME_CUDA(cudaGetSymbolAddress((void**)&p, g_noalloc_scratch));
        CME_REQUIRE(p != nullptr, CME_ERR_CUDA, "noalloc: cudaGetSymbolAddress returned a null address");
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return CME_OK;
}
}  // namespace

CME_API int cme_dact_colsum_noalloc(int dtype, const void* dout, const void* pre, void* g, void* dbias, int rows,
                                    int cols, int act, int accumulate, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    CME_REQUIRE(rows > 0 && cols > 0, CME_ERR_SHAPE, "dact_colsum_noalloc: empty input");
    CME_REQUIRE(dtype == CME_F32 || dtype == CME_BF16, CME_ERR_SHAPE, "dact_colsum_noalloc: unknown dtype %d", dtype);
    const int splits = cme_colsum_splits(rows, cols);
    const long long need = (long long)splits * cols;
    CME_REQUIRE(need <= (long long)CME_NOALLOC_SCRATCH_FLOATS, CME_ERR_LIMIT,
                "dact_colsum_noalloc: %d rows x %d cols needs %lld scratch floats, the built-in scratch holds %d; "
                "use cme_dact_colsum with a caller-provided buffer",
                rows, cols, need, (int)CME_NOALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    int rc = noalloc_scratch(&scratch);
    if (rc) return rc;
    return DISPATCH_T(dtype,
                      dact_colsum_t<__nv_bfloat16>(dout, pre, g, dbias, scratch, splits, rows, cols, act, accumulate, st),
                      dact_colsum_t<float>(dout, pre, g, dbias, scratch, splits, rows, cols, act, accumulate, st));
}
