// LayerNorm forward / backward with fused residual adds, bf16 or fp32 I/O, fp32 statistics.
//
// Covers the reference's five LayerNorm kernels (FINAL_CLEAN_CODE_/src/kernels/layernorm.cu:24-305):
// plain forward, forward saving mean / inverse std, fused residual + LayerNorm forward, backward dx with
// optional fused "gx += dx" residual-gradient add, and the column-wise d(gamma) / d(beta) reduction.
// The reference uses one block per row with a two-pass block reduction and a second kernel with one block
// per column for the weight gradients.  Here one warp owns a row (128-bit loads, shuffles only), and the
// backward kernel produces dx and per-block partial d(gamma)/d(beta) in a single pass over x and dy; a
// small second kernel sums the partials in a fixed order (no atomics, bit-reproducible).
#include "common.h"

namespace {

constexpr int LN_WARPS = 8;            // rows per block iteration
constexpr int LN_MAX_VEC = 4;          // 16-byte vectors per lane kept in registers (D <= 1024 bf16, 512 fp32)

template <typename T> struct VecOf;
template <> struct VecOf<float> { static constexpr int N = 4; };
template <> struct VecOf<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ void load_vec(const T* p, float* f);
template <> __device__ __forceinline__ void load_vec<float>(const float* p, float* f) {
    float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load_vec<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
    unpack8(*reinterpret_cast<const Bf16x8*>(p), f);
}
template <typename T> __device__ __forceinline__ void store_vec(T* p, const float* f);
template <> __device__ __forceinline__ void store_vec<float>(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <> __device__ __forceinline__ void store_vec<__nv_bfloat16>(__nv_bfloat16* p, const float* f) {
    *reinterpret_cast<Bf16x8*>(p) = pack8(f);
}

// y = LN(a [+ b]) * gamma + beta; optionally writes r = a + b, mean and rstd.
// VEC path: D is a multiple of the vector width and D / width <= 32 * LN_MAX_VEC; row kept in registers.
template <typename T, bool VEC>
__global__ void __launch_bounds__(LN_WARPS * 32)
ln_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ r_out, const T* __restrict__ gamma,
              const T* __restrict__ beta, T* __restrict__ y, float* __restrict__ mean_out,
              float* __restrict__ rstd_out, int rows, int D, float eps) {
    constexpr int W = VecOf<T>::N;
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
    if (row >= rows) return;
    const long long off = (long long)row * D;
    if constexpr (VEC) {
        const int nvec = D / W;
        float x[LN_MAX_VEC][W];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < LN_MAX_VEC; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) {
                load_vec<T>(a + off + v * W, x[i]);
                if (b) {
                    float t[W];
                    load_vec<T>(b + off + v * W, t);
#pragma unroll
                    for (int j = 0; j < W; ++j) x[i][j] += t[j];
                    if (r_out) store_vec<T>(r_out + off + v * W, x[i]);
                }
#pragma unroll
                for (int j = 0; j < W; ++j) s += x[i][j];
            }
        }
        const float mean = warp_sum(s) / D;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < LN_MAX_VEC; ++i) {
            if (lane + 32 * i < nvec) {
#pragma unroll
                for (int j = 0; j < W; ++j) { const float d = x[i][j] - mean; q += d * d; }
            }
        }
        const float rstd = rsqrtf(warp_sum(q) / D + eps);
#pragma unroll
        for (int i = 0; i < LN_MAX_VEC; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) {
                float g[W], bt[W], o[W];
                load_vec<T>(gamma + v * W, g);
                load_vec<T>(beta + v * W, bt);
#pragma unroll
                for (int j = 0; j < W; ++j) o[j] = (x[i][j] - mean) * rstd * g[j] + bt[j];
                store_vec<T>(y + off + v * W, o);
            }
        }
        if (lane == 0) {
            if (mean_out) mean_out[row] = mean;
            if (rstd_out) rstd_out[row] = rstd;
        }
    } else {
        float s = 0.f;
        for (int c = lane; c < D; c += 32) {
            float v = to_f32<T>(a[off + c]);
            if (b) {
                v += to_f32<T>(b[off + c]);
                if (r_out) r_out[off + c] = from_f32<T>(v);
            }
            s += v;
        }
        const float mean = warp_sum(s) / D;
        const T* src = (b && r_out) ? r_out : a;
        float q = 0.f;
        for (int c = lane; c < D; c += 32) {
            float v = (b && !r_out) ? to_f32<T>(a[off + c]) + to_f32<T>(b[off + c]) : to_f32<T>(src[off + c]);
            const float d = v - mean;
            q += d * d;
        }
        const float rstd = rsqrtf(warp_sum(q) / D + eps);
        for (int c = lane; c < D; c += 32) {
            float v = (b && !r_out) ? to_f32<T>(a[off + c]) + to_f32<T>(b[off + c]) : to_f32<T>(src[off + c]);
            y[off + c] = from_f32<T>((v - mean) * rstd * to_f32<T>(gamma[c]) + to_f32<T>(beta[c]));
        }
        if (lane == 0) {
            if (mean_out) mean_out[row] = mean;
            if (rstd_out) rstd_out[row] = rstd;
        }
    }
}

template <typename T> __device__ __forceinline__ void unpack_raw(const uint4& r, float* f);
template <> __device__ __forceinline__ void unpack_raw<float>(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
}
template <> __device__ __forceinline__ void unpack_raw<__nv_bfloat16>(const uint4& r, float* f) { unpack8(r, f); }

// Backward for rows that fit NV 16-byte vectors per lane (D = W * 32 * NV at most).  One warp per row, grid-stride.
// Each lane owns fixed columns: the row stays in registers as raw 16-byte words between the two passes (statistics,
// then dx) and the lane's partial d(gamma) / d(beta) accumulate in registers over all rows of the warp; they reach the warp's
// shared-memory slice (slot (i*W + j)*32 + lane: conflict-free) once at the end.  The grid is sized to what is
// resident at once, so every block runs the same number of rounds.
template <typename T, int NV>
__global__ void __launch_bounds__(LN_WARPS * 32, NV <= 2 ? 3 : 2)
ln_bwd_vec_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                  const float* __restrict__ mean, const float* __restrict__ rstd, const T* __restrict__ dres,
                  T* __restrict__ dx, float* __restrict__ partial /*[gridDim.x][2][D]*/, int rows, int D) {
    constexpr int W = VecOf<T>::N;
    constexpr int SLOTS = NV * W * 32;
    extern __shared__ float sm[];     // [LN_WARPS][2][SLOTS]
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nvec = D / W;
    float* wdg = sm + (size_t)warp * 2 * SLOTS;
    float* wdb = wdg + SLOTS;
    float adg[NV][W], adb[NV][W];
    uint4 graw[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int v = lane + 32 * i;
        graw[i] = make_uint4(0, 0, 0, 0);
        if (v < nvec) graw[i] = *reinterpret_cast<const uint4*>(gamma + v * W);
#pragma unroll
        for (int j = 0; j < W; ++j) adg[i][j] = adb[i][j] = 0.f;
    }
    for (int row = blockIdx.x * LN_WARPS + warp; row < rows; row += gridDim.x * LN_WARPS) {
        const long long off = (long long)row * D;
        uint4 xr[NV], dr[NV], rr[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) {
                xr[i] = *reinterpret_cast<const uint4*>(x + off + v * W);
                dr[i] = *reinterpret_cast<const uint4*>(dy + off + v * W);
                if (dres) rr[i] = *reinterpret_cast<const uint4*>(dres + off + v * W);
            }
        }
        const float mu = mean[row], rs = rstd[row];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (lane + 32 * i < nvec) {
                float xv[W], dv[W], g[W];
                unpack_raw<T>(xr[i], xv);
                unpack_raw<T>(dr[i], dv);
                unpack_raw<T>(graw[i], g);
#pragma unroll
                for (int j = 0; j < W; ++j) {
                    const float xh = (xv[j] - mu) * rs, d = dv[j] * g[j];
                    s1 += d;
                    s2 = fmaf(d, xh, s2);
                    adg[i][j] = fmaf(dv[j], xh, adg[i][j]);
                    adb[i][j] += dv[j];
                }
            }
        }
        s1 = warp_sum(s1) / D;
        s2 = warp_sum(s2) / D;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = lane + 32 * i;
            if (v < nvec) {
                float xv[W], dv[W], g[W], o[W];
                unpack_raw<T>(xr[i], xv);
                unpack_raw<T>(dr[i], dv);
                unpack_raw<T>(graw[i], g);
#pragma unroll
                for (int j = 0; j < W; ++j) o[j] = rs * (fmaf(-(xv[j] - mu) * rs, s2, dv[j] * g[j]) - s1);
                if (dres) {
                    float t[W];
                    unpack_raw<T>(rr[i], t);
#pragma unroll
                    for (int j = 0; j < W; ++j) o[j] += t[j];
                }
                store_vec<T>(dx + off + v * W, o);
            }
        }
    }
    // the warp's partial sums go to its shared-memory slice once, after its last row
#pragma unroll
    for (int i = 0; i < NV; ++i) {
#pragma unroll
        for (int j = 0; j < W; ++j) {
            wdg[(i * W + j) * 32 + lane] = adg[i][j];
            wdb[(i * W + j) * 32 + lane] = adb[i][j];
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < 2 * D; c += blockDim.x) {
        const int which = c >= D, col = c - which * D;
        const int v = col / W, j = col % W;
        const int slot = ((v >> 5) * W + j) * 32 + (v & 31);
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < LN_WARPS; ++w) s += sm[(size_t)w * 2 * SLOTS + which * SLOTS + slot];
        partial[(long long)blockIdx.x * 2 * D + c] = s;
    }
}

// Fallback for row lengths the vector kernel does not take (not a multiple of the vector width, or too long):
// same arithmetic with scalar accesses, per-warp partial d(gamma) / d(beta) rows in shared memory.
template <typename T>
__global__ void __launch_bounds__(LN_WARPS * 32)
ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
              const float* __restrict__ mean, const float* __restrict__ rstd, const T* __restrict__ dres,
              T* __restrict__ dx, float* __restrict__ partial /*[gridDim.x][2][D]*/, int rows, int D) {
    extern __shared__ float sm[];     // [LN_WARPS][2][D]
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int c = threadIdx.x; c < LN_WARPS * 2 * D; c += blockDim.x) sm[c] = 0.f;
    __syncthreads();
    for (int row = blockIdx.x * LN_WARPS + warp; row < rows; row += gridDim.x * LN_WARPS) {
        const long long off = (long long)row * D;
        const float mu = mean[row], rs = rstd[row];
        float s1 = 0.f, s2 = 0.f;
        for (int c = lane; c < D; c += 32) {
            const float xh = (to_f32<T>(x[off + c]) - mu) * rs;
            const float dv = to_f32<T>(dy[off + c]);
            const float d = dv * to_f32<T>(gamma[c]);
            s1 += d;
            s2 += d * xh;
            sm[(warp * 2 + 0) * D + c] += dv * xh;
            sm[(warp * 2 + 1) * D + c] += dv;
        }
        s1 = warp_sum(s1) / D;
        s2 = warp_sum(s2) / D;
        for (int c = lane; c < D; c += 32) {
            const float xh = (to_f32<T>(x[off + c]) - mu) * rs;
            const float d = to_f32<T>(dy[off + c]) * to_f32<T>(gamma[c]);
            float o = rs * (d - s1 - xh * s2);
            if (dres) o += to_f32<T>(dres[off + c]);
            dx[off + c] = from_f32<T>(o);
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < 2 * D; c += blockDim.x) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < LN_WARPS; ++w) s += sm[w * 2 * D + c];
        partial[(long long)blockIdx.x * 2 * D + c] = s;
    }
}

// dgamma[c] (+)= sum_b partial[b][0][c];  dbeta[c] (+)= sum_b partial[b][1][c]
// Block (16 columns x 16 block-groups): each thread sums every 16th partial, then a fixed-order shared-memory
// reduction over the 16 groups (deterministic).
template <typename T>
__global__ void __launch_bounds__(256)
ln_bwd_finalize_kernel(const float* __restrict__ partial, int nblocks, int D, T* dgamma, T* dbeta, int accumulate) {
    __shared__ float sm[16][17];
    pdl_wait();
    const int cx = threadIdx.x & 15, ry = threadIdx.x >> 4;
    const int c = blockIdx.x * 16 + cx;
    float s = 0.f;
    if (c < 2 * D) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;      // independent chains: the loads of four blocks overlap
        int b = ry;
        for (; b + 48 < nblocks; b += 64) {
            s0 += partial[(long long)b * 2 * D + c];
            s1 += partial[(long long)(b + 16) * 2 * D + c];
            s2 += partial[(long long)(b + 32) * 2 * D + c];
            s3 += partial[(long long)(b + 48) * 2 * D + c];
        }
        for (; b < nblocks; b += 16) s0 += partial[(long long)b * 2 * D + c];
        s = (s0 + s1) + (s2 + s3);
    }
    sm[ry][cx] = s;
    __syncthreads();
    if (ry == 0 && c < 2 * D) {
        float t = 0.f;
#pragma unroll
        for (int r = 0; r < 16; ++r) t += sm[r][cx];
        T* dst = (c < D) ? dgamma + c : dbeta + (c - D);
        *dst = from_f32<T>(accumulate ? to_f32<T>(*dst) + t : t);
    }
}

template <typename T>
int ln_fwd_t(const void* a, const void* b, void* r, const void* g, const void* be, void* y, float* mean, float* rstd,
             int rows, int D, float eps, cudaStream_t st) {
    constexpr int W = VecOf<T>::N;
    const bool vec = (D % W == 0) && (D / W <= 32 * LN_MAX_VEC);
    const int grid = cme_cdiv(rows, LN_WARPS);
    if (vec)
        CME_CUDA(cme_launch_dependent(ln_fwd_kernel<T, true>, dim3(grid), dim3(LN_WARPS * 32), 0, st, (const T*)a,
                                      (const T*)b, (T*)r, (const T*)g, (const T*)be, (T*)y, mean, rstd, rows, D, eps));
    else
        CME_CUDA(cme_launch_dependent(ln_fwd_kernel<T, false>, dim3(grid), dim3(LN_WARPS * 32), 0, st, (const T*)a,
                                      (const T*)b, (T*)r, (const T*)g, (const T*)be, (T*)y, mean, rstd, rows, D, eps));
    CME_LAUNCH_CHECK();
    return CME_OK;
}

template <typename T, int NV>
int ln_bwd_vec_launch(const T* dy, const T* x, const T* g, const float* mean, const float* rstd, const T* dres, T* dx,
                      float* scratch, int max_blocks, int rows, int D, int* used_blocks, cudaStream_t st) {
    constexpr int W = VecOf<T>::N;
    const size_t smem = (size_t)LN_WARPS * 2 * NV * W * 32 * sizeof(float);
    auto k = ln_bwd_vec_kernel<T, NV>;
    static int resident = 0;          // blocks of this instantiation that fit on the device at once
    if (!resident) {
        int dev = 0, sms = 0, per_sm = 0;
        CME_CUDA(cudaGetDevice(&dev));
        CME_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (smem > 48 * 1024) CME_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        CME_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, LN_WARPS * 32, smem));
        resident = sms * (per_sm > 0 ? per_sm : 1);
    }
    int nb = cme_cdiv(rows, LN_WARPS);
    if (nb > resident) {
        // same number of rounds for every block: ceil(groups / rounds) blocks
        const int rounds = cme_cdiv(nb, resident);
        nb = cme_cdiv(nb, rounds);
    }
    if (nb > max_blocks) nb = max_blocks;
    CME_CUDA(cme_launch_dependent(k, dim3(nb), dim3(LN_WARPS * 32), smem, st, dy, x, g, mean, rstd, dres, dx, scratch, rows,
                                  D));
    *used_blocks = nb;
    return CME_OK;
}

template <typename T>
int ln_bwd_t(const void* dy, const void* x, const void* g, const float* mean, const float* rstd, const void* dres,
             void* dx, void* dgamma, void* dbeta, float* scratch, int nblocks, int rows, int D, int accumulate,
             cudaStream_t st, cudaStream_t fin_st = nullptr, cudaEvent_t fin_ev = nullptr) {
    constexpr int W = VecOf<T>::N;
    const bool vec = (D % W == 0) && (D / W <= 32 * LN_MAX_VEC);
    if (vec) {
        const int nv = cme_cdiv(D / W, 32);
        int rc;
#define CME_LN_NV(N) rc = ln_bwd_vec_launch<T, N>((const T*)dy, (const T*)x, (const T*)g, mean, rstd, (const T*)dres, \
                                                 (T*)dx, scratch, nblocks, rows, D, &nblocks, st)
        if (nv == 1) CME_LN_NV(1); else if (nv == 2) CME_LN_NV(2); else if (nv == 3) CME_LN_NV(3); else CME_LN_NV(4);
#undef CME_LN_NV
        if (rc) return rc;
    } else {
        const size_t smem = (size_t)LN_WARPS * 2 * D * sizeof(float);
        auto k = ln_bwd_kernel<T>;
        if (smem > 48 * 1024) CME_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        CME_CUDA(cme_launch_dependent(k, dim3(nblocks), dim3(LN_WARPS * 32), smem, st, (const T*)dy, (const T*)x,
                                      (const T*)g, mean, rstd, (const T*)dres, (T*)dx, scratch, rows, D));
    }
    CME_LAUNCH_CHECK();
    if (fin_st != nullptr && fin_st != st) {       // the weight gradients are finished on another stream
        CME_CUDA(cudaEventRecord(fin_ev, st));
        CME_CUDA(cudaStreamWaitEvent(fin_st, fin_ev, 0));
        st = fin_st;
    }
    CME_CUDA(cme_launch_dependent(ln_bwd_finalize_kernel<T>, dim3(cme_cdiv(2 * D, 16)), dim3(256), 0, st,
                                  (const float*)scratch, nblocks, D, (T*)dgamma, (T*)dbeta, accumulate));
    CME_LAUNCH_CHECK();
    return CME_OK;
}

}  // namespace

// y = LN(a + b); b, r_out, mean, rstd may be null.
CME_API int cme_layernorm_fwd(int dtype, const void* a, const void* b, void* r_out, const void* gamma,
                              const void* beta, void* y, float* mean, float* rstd, int rows, int D, float eps,
                              void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    CME_REQUIRE(rows > 0 && D > 0, CME_ERR_SHAPE, "layernorm: empty input");
    return dtype == CME_BF16 ? ln_fwd_t<__nv_bfloat16>(a, b, r_out, gamma, beta, y, mean, rstd, rows, D, eps, st)
                             : ln_fwd_t<float>(a, b, r_out, gamma, beta, y, mean, rstd, rows, D, eps, st);
}

// Number of partial blocks the backward uses for `rows`; scratch must hold blocks * 2 * D floats.
CME_API int cme_layernorm_bwd_blocks(int rows) {
    int b = cme_cdiv(rows, LN_WARPS);
    return b < 592 ? b : 592;
}

// dx = LN'(dy) [+ dres]; dgamma/dbeta (+)= column sums.  `scratch`: cme_layernorm_bwd_blocks(rows)*2*D floats.
CME_API int cme_layernorm_bwd(int dtype, const void* dy, const void* x, const void* gamma, const float* mean,
                              const float* rstd, const void* dres, void* dx, void* dgamma, void* dbeta,
                              float* scratch, int rows, int D, int accumulate, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    CME_REQUIRE(rows > 0 && D > 0, CME_ERR_SHAPE, "layernorm: empty input");
    CME_REQUIRE((size_t)LN_WARPS * 2 * D * 4 <= 200 * 1024, CME_ERR_LIMIT, "layernorm backward: D too large (%d)", D);
    const int nb = cme_layernorm_bwd_blocks(rows);
    return dtype == CME_BF16
               ? ln_bwd_t<__nv_bfloat16>(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, scratch, nb, rows, D,
                                         accumulate, st)
               : ln_bwd_t<float>(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, scratch, nb, rows, D, accumulate,
                                 st);
}

// Same, with the small kernel that sums the per-block partial d(gamma) / d(beta) on `fin_stream` (ordered after the main
// kernel through `fin_event`, a cudaEvent_t of the caller): nothing on `stream` needs those sums, so the chain of
// activation-gradient work on `stream` does not wait for them.  `scratch` must stay untouched until that kernel has run.
CME_API int cme_layernorm_bwd_split(int dtype, const void* dy, const void* x, const void* gamma, const float* mean,
                                    const float* rstd, const void* dres, void* dx, void* dgamma, void* dbeta,
                                    float* scratch, int rows, int D, int accumulate, void* stream, void* fin_stream,
                                    void* fin_event) {
    cudaStream_t st = (cudaStream_t)stream;
    CME_REQUIRE(rows > 0 && D > 0, CME_ERR_SHAPE, "layernorm: empty input");
    CME_REQUIRE((size_t)LN_WARPS * 2 * D * 4 <= 200 * 1024, CME_ERR_LIMIT, "layernorm backward: D too large (%d)", D);
    CME_REQUIRE(fin_stream == nullptr || fin_stream == stream || fin_event != nullptr, CME_ERR_SHAPE,
                "layernorm backward: a second stream needs an event");
    const int nb = cme_layernorm_bwd_blocks(rows);
    return dtype == CME_BF16
               ? ln_bwd_t<__nv_bfloat16>(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, scratch, nb, rows, D,
                                         accumulate, st, (cudaStream_t)fin_stream, (cudaEvent_t)fin_event)
               : ln_bwd_t<float>(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, scratch, nb, rows, D, accumulate,
                                 st, (cudaStream_t)fin_stream, (cudaEvent_t)fin_event);
}
