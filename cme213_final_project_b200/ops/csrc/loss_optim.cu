// Fused softmax-cross-entropy (loss + gradient), global gradient norm, and Adam / AdamW on the flat arena.
//
// Reference counterparts: cross_entropy_kernel + reduce_sum_kernel + scale_device_scalar
// (FINAL_CLEAN_CODE_/src/kernels/activations.cu:438-531: one warp per row, loss summed with atomicAdd),
// norm_sq_kernel / clip_scale_kernel (:360-392) and adam_clipped_kernel
// (FINAL_CLEAN_CODE_/src/model/transformer.cu:598-636).  Here: one block per row with an online
// max / sum pass so a 50k-entry vocabulary row is read once for the statistics and once for the gradient,
// the mean loss and the squared norm are reduced in two fixed-order stages (bit-reproducible), and the
// optimizer reads its step counter, learning rate and the squared norm from device memory so that a
// captured CUDA graph of the step stays correct on every replay (the reference bakes the host-computed
// bias corrections into its captured launch).
#include "common.h"
#include <cuda_fp16.h>

namespace {

constexpr int CE_THREADS = 256;

// dlogits[r, :] = (softmax(logits[r, :]) - onehot(target)) * grad_scale; losses[r] = -log(p_target (+ eps)).
// In-place (dlogits == logits) is allowed: each element is read before it is written by the same thread.
template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
cross_entropy_kernel(const T* __restrict__ logits, const int* __restrict__ targets, T* dlogits, float* __restrict__ losses,
                     int V, long long ld, float grad_scale, float prob_eps) {
    __shared__ float scratch[32];
    const long long off = (long long)blockIdx.x * ld;
    const T* row = logits + off;
    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x; i < V; i += CE_THREADS) {
        const float x = to_f32<T>(row[i]);
        if (x > m) { s *= __expf(m - x); m = x; }
        s += __expf(x - m);
    }
    const float row_max = block_max(m, scratch);
    s *= __expf(m - row_max);               // m = -inf with s = 0 gives 0 * 0
    if (m == -INFINITY) s = 0.f;
    const float denom = block_sum(s, scratch);
    const float inv = 1.f / (denom + prob_eps);
    int tgt = targets[blockIdx.x];
    tgt = tgt < 0 ? 0 : (tgt >= V ? V - 1 : tgt);
    if (threadIdx.x == 0) {
        const float p = __expf(to_f32<T>(row[tgt]) - row_max) * inv;
        losses[blockIdx.x] = prob_eps > 0.f ? -logf(p + prob_eps) : -(to_f32<T>(row[tgt]) - row_max - logf(denom));
    }
    __syncthreads();                        // the target logit is read above before anyone overwrites it
    if (dlogits) {
        T* g = dlogits + off;
        for (int i = threadIdx.x; i < V; i += CE_THREADS) {
            float p = __expf(to_f32<T>(row[i]) - row_max) * inv;
            if (i == tgt) p -= 1.f;
            g[i] = from_f32<T>(p * grad_scale);
        }
    }
}


// bf16 rows whose length is a multiple of 8 and whose base is 16-byte aligned: 128-bit loads, the row is kept
// in shared memory between the statistics pass and the gradient pass when it fits (read once from DRAM).
constexpr int CEV_THREADS = 512;
__global__ void __launch_bounds__(CEV_THREADS)
cross_entropy_bf16_vec_kernel(const __nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                              __nv_bfloat16* dlogits, float* __restrict__ losses, int V, long long ld,
                              float grad_scale, float prob_eps, int cache_row) {
    extern __shared__ uint4 srow[];
    __shared__ float scratch[32];
    const long long off = (long long)blockIdx.x * ld;
    const uint4* row = reinterpret_cast<const uint4*>(logits + off);
    const int nv = V / 8;
    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x; i < nv; i += CEV_THREADS) {
        const uint4 u = row[i];
        if (cache_row) srow[i] = u;
        float x[8];
        unpack8(u, x);
        float mx = x[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) mx = fmaxf(mx, x[j]);
        if (mx > m) { s *= __expf(m - mx); m = mx; }
#pragma unroll
        for (int j = 0; j < 8; ++j) s += __expf(x[j] - m);
    }
    const float row_max = block_max(m, scratch);
    s = (m == -INFINITY) ? 0.f : s * __expf(m - row_max);
    const float denom = block_sum(s, scratch);
    const float inv = 1.f / (denom + prob_eps);
    int tgt = targets[blockIdx.x];
    tgt = tgt < 0 ? 0 : (tgt >= V ? V - 1 : tgt);
    if (threadIdx.x == 0) {
        const float xt = __bfloat162float(logits[off + tgt]);
        const float p = __expf(xt - row_max) * inv;
        losses[blockIdx.x] = prob_eps > 0.f ? -logf(p + prob_eps) : -(xt - row_max - logf(denom));
    }
    __syncthreads();
    if (dlogits) {
        uint4* g = reinterpret_cast<uint4*>(dlogits + off);
        for (int i = threadIdx.x; i < nv; i += CEV_THREADS) {
            float x[8];
            unpack8(cache_row ? srow[i] : row[i], x);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float p = __expf(x[j] - row_max) * inv;
                if (i * 8 + j == tgt) p -= 1.f;
                x[j] = p * grad_scale;
            }
            g[i] = pack8(x);
        }
    }
}

// Same contract, for rows of at most CEV_THREADS * CER_MAXV 16-byte vectors (53248 bf16: GPT-2's padded vocabulary
// fits): the row lives in registers from its single read to its single write.  Pass 1 finds the maximum, pass 2
// evaluates exp(x - max) once per element and keeps it as fp16 in the registers that held the logits (values in
// (0, 1], 11 significant bits -- finer than the bf16 the gradient is stored in), pass 3 only scales.  One
// exponential per element instead of two: the kernel is otherwise bound by the special-function unit as much as by
// memory (100 K exponentials per row).
constexpr int CER_MAXV = 13;
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_h2(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
__global__ void __launch_bounds__(CEV_THREADS)
cross_entropy_bf16_reg_kernel(const __nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                              __nv_bfloat16* dlogits, float* __restrict__ losses, int V, long long ld,
                              float grad_scale, float prob_eps) {
    __shared__ float scratch[32];
    const long long off = (long long)blockIdx.x * ld;
    const uint4* row = reinterpret_cast<const uint4*>(logits + off);
    const int nv = V / 8;
    uint4 r[CER_MAXV];
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < CER_MAXV; ++k) {
        const int i = threadIdx.x + k * CEV_THREADS;
        if (i < nv) {
            r[k] = row[i];
            float x[8];
            unpack8(r[k], x);
#pragma unroll
            for (int j = 0; j < 8; ++j) m = fmaxf(m, x[j]);
        }
    }
    const float row_max = block_max(m, scratch);
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < CER_MAXV; ++k) {
        if (threadIdx.x + k * CEV_THREADS < nv) {
            float x[8];
            unpack8(r[k], x);
#pragma unroll
            for (int j = 0; j < 8; ++j) { x[j] = __expf(x[j] - row_max); s += x[j]; }
            r[k] = make_uint4(pack_h2(x[0], x[1]), pack_h2(x[2], x[3]), pack_h2(x[4], x[5]), pack_h2(x[6], x[7]));
        }
    }
    const float denom = block_sum(s, scratch);
    const float inv = 1.f / (denom + prob_eps);
    int tgt = targets[blockIdx.x];
    tgt = tgt < 0 ? 0 : (tgt >= V ? V - 1 : tgt);
    if (threadIdx.x == 0) {
        const float xt = __bfloat162float(logits[off + tgt]);
        const float p = __expf(xt - row_max) * inv;
        losses[blockIdx.x] = prob_eps > 0.f ? -logf(p + prob_eps) : -(xt - row_max - logf(denom));
    }
    __syncthreads();                 // the target's logit has been read before the row is overwritten in place
    if (dlogits) {
        uint4* g = reinterpret_cast<uint4*>(dlogits + off);
        const float sc = inv * grad_scale;
#pragma unroll
        for (int k = 0; k < CER_MAXV; ++k) {
            const int i = threadIdx.x + k * CEV_THREADS;
            if (i < nv) {
                const float2 a = unpack_h2(r[k].x), b = unpack_h2(r[k].y), c = unpack_h2(r[k].z), d = unpack_h2(r[k].w);
                float x[8] = {a.x * sc, a.y * sc, b.x * sc, b.y * sc, c.x * sc, c.y * sc, d.x * sc, d.y * sc};
                const int t = tgt - i * 8;
                if (t >= 0 && t < 8) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (j == t) x[j] -= grad_scale;
                }
                g[i] = pack8(x);
            }
        }
    }
}

// out (+)= weight * sum(x[0..n)); single block, fixed order.
__global__ void __launch_bounds__(1024) reduce_scalar_kernel(const float* __restrict__ x, int n, float weight, float* out,
                                                             int accumulate) {
    __shared__ float scratch[32];
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
    s = block_sum(s, scratch);
    if (threadIdx.x == 0) *out = (accumulate ? *out : 0.f) + s * weight;
}

template <typename T>
__global__ void __launch_bounds__(256) normsq_partial_kernel(const T* __restrict__ g, long long n, float* partial) {
    __shared__ float scratch[32];
    float s = 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = to_f32<T>(g[i]);
        s += v * v;
    }
    s = block_sum(s, scratch);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__global__ void step_inc_kernel(int* step) { *step += 1; }

struct AdamArgs {
    float* master; __nv_bfloat16* compute; const void* grads; float* m; float* v;
    long long n;
    const int* step; const float* lr; const float* normsq;
    float beta1, beta2, eps, weight_decay, grad_scale, clip_norm;
    const long long* nodecay; int n_nodecay;      // sorted [start, end) pairs exempt from weight decay
};

template <typename TG>
__global__ void __launch_bounds__(256) adam_kernel(const AdamArgs a) {
    const int t = *a.step;
    const float lr = *a.lr;
    const float bc1 = 1.f - powf(a.beta1, (float)t), bc2 = 1.f - powf(a.beta2, (float)t);
    float gs = a.grad_scale;
    if (a.normsq && a.clip_norm > 0.f) {
        const float norm = sqrtf(*a.normsq) * a.grad_scale;
        if (norm > a.clip_norm) gs *= a.clip_norm / norm;
    }
    const TG* grads = reinterpret_cast<const TG*>(a.grads);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (long long)gridDim.x * blockDim.x) {
        const float g = to_f32<TG>(grads[i]) * gs;
        const float mi = a.beta1 * a.m[i] + (1.f - a.beta1) * g;
        const float vi = a.beta2 * a.v[i] + (1.f - a.beta2) * g * g;
        a.m[i] = mi;
        a.v[i] = vi;
        float p = a.master[i];
        if (a.weight_decay > 0.f) {
            bool decay = true;
            int lo = 0, hi = a.n_nodecay;          // first segment with end > i
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (a.nodecay[2 * mid + 1] > i) hi = mid; else lo = mid + 1;
            }
            if (lo < a.n_nodecay && a.nodecay[2 * lo] <= i) decay = false;
            if (decay) p *= 1.f - lr * a.weight_decay;
        }
        p -= lr * (mi / bc1) / (sqrtf(vi / bc2) + a.eps);
        a.master[i] = p;
        if (a.compute) a.compute[i] = __float2bfloat16_rn(p);
    }
}


// Four elements per thread-iteration (128-bit accesses on the fp32 state).  Requires n % 4 == 0, 16-byte
// aligned arenas, and no-decay ranges whose ends are multiples of 4 (arena tensors start on 64-element
// boundaries, so a group of four never straddles two tensors).
template <typename TG>
__global__ void __launch_bounds__(256) adam_vec4_kernel(const AdamArgs a) {
    const int t = *a.step;
    const float lr = *a.lr;
    const float bc1 = 1.f - powf(a.beta1, (float)t), bc2 = 1.f - powf(a.beta2, (float)t);
    const float ibc1 = 1.f / bc1, ibc2 = 1.f / bc2;
    float gs = a.grad_scale;
    if (a.normsq && a.clip_norm > 0.f) {
        const float norm = sqrtf(*a.normsq) * a.grad_scale;
        if (norm > a.clip_norm) gs *= a.clip_norm / norm;
    }
    const long long nv = a.n >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
        const long long e = i << 2;
        float g[4];
        if constexpr (sizeof(TG) == 2) {
            const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.grads) + e);
            float2 lo = bf2_to_f2(u.x), hi = bf2_to_f2(u.y);
            g[0] = lo.x; g[1] = lo.y; g[2] = hi.x; g[3] = hi.y;
        } else {
            const float4 u = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.grads) + e);
            g[0] = u.x; g[1] = u.y; g[2] = u.z; g[3] = u.w;
        }
        float4 m4 = *reinterpret_cast<const float4*>(a.m + e);
        float4 v4 = *reinterpret_cast<const float4*>(a.v + e);
        float4 p4 = *reinterpret_cast<const float4*>(a.master + e);
        float decay = 1.f;
        if (a.weight_decay > 0.f) {
            int lo = 0, hi = a.n_nodecay;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (a.nodecay[2 * mid + 1] > e) hi = mid; else lo = mid + 1;
            }
            if (!(lo < a.n_nodecay && a.nodecay[2 * lo] <= e)) decay = 1.f - lr * a.weight_decay;
        }
        float* mp = &m4.x; float* vp = &v4.x; float* pp = &p4.x;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float gj = g[j] * gs;
            mp[j] = a.beta1 * mp[j] + (1.f - a.beta1) * gj;
            vp[j] = a.beta2 * vp[j] + (1.f - a.beta2) * gj * gj;
            pp[j] = pp[j] * decay - lr * (mp[j] * ibc1) / (sqrtf(vp[j] * ibc2) + a.eps);
        }
        *reinterpret_cast<float4*>(a.m + e) = m4;
        *reinterpret_cast<float4*>(a.v + e) = v4;
        *reinterpret_cast<float4*>(a.master + e) = p4;
        if (a.compute)
            *reinterpret_cast<uint2*>(a.compute + e) = make_uint2(f2_to_bf2(p4.x, p4.y), f2_to_bf2(p4.z, p4.w));
    }
}

}  // namespace

// Per-row loss and gradient, then *loss_out (+)= loss_weight * mean(losses).
// prob_eps > 0 selects the reference's form  -log(p + eps), p = e / (sum + eps);  0 the exact log-softmax.
CME_API int cme_cross_entropy(int dtype, const void* logits, const int* targets, void* dlogits, float* losses,
                              float* loss_out, int rows, int V, long long ld, float grad_scale, float prob_eps,
                              float loss_weight, int accumulate_loss, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    CME_REQUIRE(rows > 0 && V > 0, CME_ERR_SHAPE, "cross_entropy: empty input");
    const bool vec = dtype == CME_BF16 && V % 8 == 0 && ld % 8 == 0 && V >= 2048 &&
                     (reinterpret_cast<uintptr_t>(logits) & 15) == 0 &&
                     (!dlogits || (reinterpret_cast<uintptr_t>(dlogits) & 15) == 0);
    if (vec && V / 8 <= CEV_THREADS * CER_MAXV) {
        cross_entropy_bf16_reg_kernel<<<rows, CEV_THREADS, 0, st>>>((const __nv_bfloat16*)logits, targets,
                                                                   (__nv_bfloat16*)dlogits, losses, V, ld, grad_scale,
                                                                   prob_eps);
    } else if (vec) {
        const size_t row_bytes = (size_t)V * 2;
        const int cache = row_bytes <= 110 * 1024;          // two blocks per SM still fit
        static bool attr = false;
        if (!attr) {
            CME_CUDA(cudaFuncSetAttribute(cross_entropy_bf16_vec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          110 * 1024));
            attr = true;
        }
        cross_entropy_bf16_vec_kernel<<<rows, CEV_THREADS, cache ? row_bytes : 0, st>>>(
            (const __nv_bfloat16*)logits, targets, (__nv_bfloat16*)dlogits, losses, V, ld, grad_scale, prob_eps, cache);
    } else if (dtype == CME_BF16)
        cross_entropy_kernel<__nv_bfloat16><<<rows, CE_THREADS, 0, st>>>((const __nv_bfloat16*)logits, targets,
                                                                         (__nv_bfloat16*)dlogits, losses, V, ld,
                                                                         grad_scale, prob_eps);
    else
        cross_entropy_kernel<float><<<rows, CE_THREADS, 0, st>>>((const float*)logits, targets, (float*)dlogits, losses,
                                                                 V, ld, grad_scale, prob_eps);
    CME_LAUNCH_CHECK();
    if (loss_out) {
        reduce_scalar_kernel<<<1, 1024, 0, st>>>(losses, rows, loss_weight / (float)rows, loss_out, accumulate_loss);
        CME_LAUNCH_CHECK();
    }
    return CME_OK;
}

// *out = sum(g^2) over n elements; `partial` holds 1024 floats.
CME_API int cme_grad_normsq(int dtype, const void* g, long long n, float* partial, float* out, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == CME_BF16) normsq_partial_kernel<__nv_bfloat16><<<1024, 256, 0, st>>>((const __nv_bfloat16*)g, n, partial);
    else normsq_partial_kernel<float><<<1024, 256, 0, st>>>((const float*)g, n, partial);
    CME_LAUNCH_CHECK();
    reduce_scalar_kernel<<<1, 1024, 0, st>>>(partial, 1024, 1.f, out, 0);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

// Early loss read-back: bump the sequence number, write the loss and then the sequence number straight into
// pinned, device-mapped host memory.  A host thread that sees the new sequence number also sees the loss.
__global__ void publish_loss_kernel(const float* loss, int* seq, volatile float* host_loss, volatile int* host_seq) {
    const int s = *seq + 1;
    *seq = s;
    *host_loss = *loss;
    __threadfence_system();
    *host_seq = s;
    __threadfence_system();      // push the number out now: inside a CUDA graph nothing else flushes it before the end
}

// Device-side address of a pinned host allocation (once per buffer, outside stream capture).
CME_API int cme_host_device_ptr(void* host, void** dev) {
    CME_CUDA(cudaHostGetDevicePointer(dev, host, 0));
    return CME_OK;
}

CME_API int cme_publish_loss(const float* loss, int* seq, void* host_loss_dev, void* host_seq_dev, void* stream) {
    publish_loss_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(loss, seq, static_cast<volatile float*>(host_loss_dev),
                                                           static_cast<volatile int*>(host_seq_dev));
    CME_LAUNCH_CHECK();
    return CME_OK;
}

CME_API int cme_step_inc(int* step, void* stream) {
    step_inc_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(step);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

// Adam / AdamW over [0, n).  `step` (already incremented), `lr` and `normsq` live in device memory.
// g_eff = grad * grad_scale * min(1, clip_norm / (sqrt(normsq) * grad_scale)); decoupled weight decay
// except inside the `nodecay` ranges; writes the fp32 master and, if given, its bf16 copy.
CME_API int cme_adam(int grad_dtype, float* master, void* compute_bf16, const void* grads, float* m, float* v,
                     long long n, const int* step, const float* lr, const float* normsq, float beta1, float beta2,
                     float eps, float weight_decay, float grad_scale, float clip_norm, const long long* nodecay,
                     int n_nodecay, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (n <= 0) return CME_OK;
    AdamArgs a{master, (__nv_bfloat16*)compute_bf16, grads, m, v, n, step, lr, normsq, beta1, beta2, eps,
               weight_decay, grad_scale, clip_norm, nodecay, n_nodecay};
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    auto al = [](const void* p, int b) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & (b - 1)) == 0; };
    bool vec = n % 4 == 0 && al(master, 16) && al(m, 16) && al(v, 16) && al(compute_bf16, 8) &&
               al(grads, grad_dtype == CME_BF16 ? 8 : 16);
    if (vec) {
        blocks = (n / 4 + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        if (grad_dtype == CME_BF16) adam_vec4_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, st>>>(a);
        else adam_vec4_kernel<float><<<(int)blocks, 256, 0, st>>>(a);
    } else if (grad_dtype == CME_BF16) adam_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, st>>>(a);
    else adam_kernel<float><<<(int)blocks, 256, 0, st>>>(a);
    CME_LAUNCH_CHECK();
    return CME_OK;
}
