// Common runtime for the native library: error reporting, shape helpers, device math, reductions.
//
// Role of the reference's common.h (FINAL_CLEAN_CODE_/include/common.h:20-82): there CUDA_CHECK exits the
// process; here every exported function returns a status code (0 = ok) and records a message that the
// Python side turns into an exception, so a failed launch never takes the interpreter down.
#pragma once
#include <utility>

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#define CME_API extern "C" __attribute__((visibility("default")))

enum CmeStatus : int {
    CME_OK = 0,
    CME_ERR_CUDA = 1,        // a CUDA runtime / driver call failed
    CME_ERR_SHAPE = 2,       // unsupported or inconsistent shape / alignment
    CME_ERR_TIMEOUT = 3,     // a bounded device-side wait ran out (reported through a status word)
    CME_ERR_LIMIT = 4,       // a documented size limit was exceeded
    CME_ERR_UNSUPPORTED = 5,
};

// Data type tags passed through the C ABI.
enum CmeDtype : int { CME_F32 = 0, CME_BF16 = 1 };

void cme_set_error(const char* fmt, ...);
CME_API const char* cme_last_error();

#define CME_CUDA(call)                                                                         \
    do {                                                                                       \
        cudaError_t err__ = (call);                                                            \
        if (err__ != cudaSuccess) {                                                            \
            cme_set_error("%s:%d: %s -> %s", __FILE__, __LINE__, #call, cudaGetErrorString(err__)); \
            return CME_ERR_CUDA;                                                               \
        }                                                                                      \
    } while (0)

// Every kernel launch of the library goes through this check; the counter is what `cme_launch_count` reports.
extern long long g_cme_launches;
#define CME_LAUNCH_CHECK()                  \
    do {                                    \
        ++g_cme_launches;                   \
        CME_CUDA(cudaGetLastError());       \
    } while (0)

#define CME_REQUIRE(cond, code, ...)                                                           \
    do {                                                                                       \
        if (!(cond)) {                                                                         \
            cme_set_error(__VA_ARGS__);                                                        \
            return (code);                                                                     \
        }                                                                                      \
    } while (0)

static inline int cme_cdiv(long long a, long long b) { return (int)((a + b - 1) / b); }

// Per-device facts and status words, created once per device by cme_init_device() -- or by the first launch on
// the device, which must then happen outside stream capture (it allocates).  A process may drive several GPUs:
// everything here is indexed by the current device.
constexpr int CME_MAX_DEVICES = 64;
enum CmeStatusWord : int { CME_STATUS_GEMM = 0, CME_STATUS_ATTENTION = 1, CME_STATUS_WORDS = 4 };
struct CmeDeviceState {
    int num_sms;
    int* status;           // CME_STATUS_WORDS ints in device memory; a kernel whose bounded wait ran out sets its word
    int max_pairs;         // co-resident CTA pairs of the pair GEMM kernel (-1: not queried yet, 0: unusable)
};
int cme_device_state(CmeDeviceState** out);
int cme_check_status_word(int which, int* host_out);

#ifdef __CUDACC__

// Programmatic dependent launch for the many short kernels of a step.  A kernel launched through
// cme_launch_dependent may be scheduled while the previous kernel of the stream is still draining; it must call
// pdl_wait() before it touches anything that kernel wrote (first statement of every such kernel).  The wait
// returns once the previous kernel has completed and its writes are visible, so results are unchanged; what is
// saved is the launch gap between consecutive kernels.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t cme_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                        Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

__host__ __device__ __forceinline__ int cme_cdiv_dev(int a, int b) { return (a + b - 1) / b; }

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum; every thread gets the result.  `scratch` holds at least 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? scratch[lane] : 0.f;
    return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? scratch[lane] : -INFINITY;
    return warp_max(r);
}

// tanh-form GELU and its derivative.
__device__ __forceinline__ float gelu_f(float x) {
    const float k = 0.7978845608028654f;
    float u = k * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
}
__device__ __forceinline__ float dgelu_f(float x) {
    const float k = 0.7978845608028654f;
    float x2 = x * x;
    float u = k * (x + 0.044715f * x * x2);
    float t = tanhf(u);
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x2);
}

// Hardware-tanh variants for bf16 epilogues (one MUFU op instead of a software tanh; ~2^-11 relative error,
// below bf16 resolution).  The fp32 paths keep the accurate forms above.
__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float gelu_fast(float x) {
    const float u = x * fmaf(0.0356774081f, x * x, 0.7978845608f);
    return 0.5f * x * (1.f + tanh_fast(u));
}
__device__ __forceinline__ float dgelu_fast(float x) {
    const float x2 = x * x;
    const float t = tanh_fast(x * fmaf(0.0356774081f, x2, 0.7978845608f));
    const float du = fmaf(0.1070322243f, x2, 0.7978845608f);
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}

// GELU and its derivative from one hardware tanh (the forward epilogue that also leaves the derivative for backward).
__device__ __forceinline__ void gelu_and_grad_fast(float x, float& g, float& d) {
    const float x2 = x * x;
    const float t = tanh_fast(x * fmaf(0.0356774081f, x2, 0.7978845608f));
    const float hx = 0.5f * x;
    g = fmaf(hx, t, hx);
    d = fmaf(hx * fmaf(-t, t, 1.f), fmaf(0.1070322243f, x2, 0.7978845608f), fmaf(0.5f, t, 0.5f));
}

// Packed fp32 pairs (sm_100: add / sub / mul / fma on two fp32 values held in one 64-bit register issue as one
// instruction).  The arithmetic-heavy epilogues are bound by issue slots, so pairs halve their cost.
typedef unsigned long long F32x2;
__device__ __forceinline__ F32x2 f2_pack(float lo, float hi) {
    F32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(F32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ F32x2 f2_splat(float c) { return f2_pack(c, c); }
__device__ __forceinline__ F32x2 f2_fma(F32x2 a, F32x2 b, F32x2 c) {
    F32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ F32x2 f2_mul(F32x2 a, F32x2 b) {
    F32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ F32x2 f2_add(F32x2 a, F32x2 b) {
    F32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// GELU and its derivative for two values at once, from one hardware tanh each.  With a = (1 + t) / 2:
//   gelu = x a,   gelu' = a (1 + 2 x u'(x) (1 - a))   since 1 - t^2 = 4 a (1 - a);   u' = 0.79788 + 0.10703 x^2.
__device__ __forceinline__ void gelu_and_grad_fast2(float& x0, float& x1, float& d0, float& d1) {
    const F32x2 x = f2_pack(x0, x1);
    const F32x2 x2 = f2_mul(x, x);
    const F32x2 u = f2_mul(x, f2_fma(f2_splat(0.0356774081f), x2, f2_splat(0.7978845608f)));
    float u0, u1;
    f2_unpack(u, u0, u1);
    const F32x2 t = f2_pack(tanh_fast(u0), tanh_fast(u1));
    const F32x2 a = f2_fma(f2_splat(0.5f), t, f2_splat(0.5f));
    const F32x2 oma = f2_fma(f2_splat(-0.5f), t, f2_splat(0.5f));
    const F32x2 r = f2_mul(x, f2_fma(f2_splat(0.2140644486f), x2, f2_splat(1.5957691216f)));
    f2_unpack(f2_mul(x, a), x0, x1);
    f2_unpack(f2_mul(a, f2_fma(r, oma, f2_splat(1.f))), d0, d1);
}

// 8 x bf16 <-> 8 x f32 through one 128-bit word (a uint4, so loads and stores stay single 128-bit accesses).
typedef uint4 Bf16x8;
__device__ __forceinline__ float2 bf2_to_f2(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
__device__ __forceinline__ uint32_t f2_to_bf2(float lo, float hi) {
    uint32_t w;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi), "f"(lo));
    return w;
}
__device__ __forceinline__ void unpack8(const Bf16x8& p, float* f) {
    float2 t;
    t = bf2_to_f2(p.x); f[0] = t.x; f[1] = t.y;
    t = bf2_to_f2(p.y); f[2] = t.x; f[3] = t.y;
    t = bf2_to_f2(p.z); f[4] = t.x; f[5] = t.y;
    t = bf2_to_f2(p.w); f[6] = t.x; f[7] = t.y;
}
__device__ __forceinline__ Bf16x8 pack8(const float* f) {
    return make_uint4(f2_to_bf2(f[0], f[1]), f2_to_bf2(f[2], f[3]), f2_to_bf2(f[4], f[5]), f2_to_bf2(f[6], f[7]));
}

#endif  // __CUDACC__
