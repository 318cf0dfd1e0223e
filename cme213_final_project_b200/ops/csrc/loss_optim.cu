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

}  // namespace

// Per-row loss and gradient, then *loss_out (+)= loss_weight * mean(losses).
// prob_eps > 0 selects the reference's form  -log(p + eps), p = e / (sum + eps);  0 the exact log-softmax.
CME_API int cme_cross_entropy(int dtype, const void* logits, const int* targets, void* dlogits, float* losses,
                              float* loss_out, int rows, int V, long long ld, float grad_scale, float prob_eps,
                              float loss_weight, int accumulate_loss, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    CME_REQUIRE(rows > 0 && V > 0, CME_ERR_SHAPE, "cross_entropy: empty input");
    if (dtype == CME_BF16)
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
    if (grad_dtype == CME_BF16) adam_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, st>>>(a);
    else adam_kernel<float><<<(int)blocks, 256, 0, st>>>(a);
    CME_LAUNCH_CHECK();
    return CME_OK;
}
