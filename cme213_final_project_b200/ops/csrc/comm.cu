// Gradient synchronisation over peer memory (NVLink 5 / NVSwitch), from inside the kernel:
//
//   cme_comm_allreduce     in-place sum (x scale) of a symmetric buffer: one-shot (every rank reads every
//                          peer's whole range), two-shot (reduce-scatter my slice, then write it to every peer)
//                          or NVLS (multimem.ld_reduce / multimem.st through the switch);
//   cme_comm_fused_adamw   the per-bucket step of data-parallel training in ONE kernel: barrier, reduce-scatter
//                          of bf16 gradients (128-bit peer loads or multimem.ld_reduce, fp32 accumulation), x 1/world,
//                          AdamW on this rank's fp32 master / moment slice, bf16 parameters written into every
//                          peer's parameter arena (peer stores or multimem.st), barrier.
//
// The reference does this with host-issued library collectives: MPI_Allreduce / MPI_Iallreduce / ncclAllReduce per
// bucket (FINAL_CLEAN_CODE_/src/model/distributed.cpp:183-405), then a scale kernel per bucket (activations.cu:349)
// and, after the last bucket, norm + clip + Adam kernels over the whole arena (transformer.cu:618-636).
//
// Cross-rank ordering uses per-bucket flag words in symmetric memory with monotonically increasing epochs
// (never reset, so a captured CUDA graph can be replayed).  Every wait on a peer is bounded by a wall-clock
// budget read from %globaltimer; on expiry the kernel writes CME_ERR_TIMEOUT to its status word, skips the data
// phase and returns, so a rank that never arrives cannot hang the GPU.
#include "common.h"

#include <cstdlib>

namespace {

constexpr int MAX_RANKS = 16;
// 128-thread CTAs: small enough in registers to share an SM with a resident GEMM or attention CTA, so a
// communication kernel does not have to wait for (or displace) the persistent compute kernels.
constexpr int COMM_THREADS = 128;

struct Peers {
    void* buf[MAX_RANKS];          // the symmetric data buffer as mapped for each rank (index = rank)
    void* buf2[MAX_RANKS];         // second symmetric buffer (parameters) for the fused kernel
    uint32_t* flags[MAX_RANKS];    // symmetric flag array of each rank
    void* mc_buf;                  // multicast address of buf (0 = none)
    void* mc_buf2;                 // multicast address of buf2
    int world, rank;
};

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_peer(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_peer(void* p, uint4 v) {
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
// Sum of 8 bf16 values across all ranks bound to the multicast object, accumulated in fp32 by the switch.
__device__ __forceinline__ uint4 mc_ld_reduce_bf16(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}
__device__ __forceinline__ float4 mc_ld_reduce_f32(const void* mc) {
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
    return v;
}
__device__ __forceinline__ void mc_st(void* mc, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}

// Flag layout per rank: [slot][MAX_RANKS] words; slot = 2 * bucket + phase.  Local bookkeeping (not symmetric):
// ctl[3 * bucket + 0] = epoch of the last completed call, + 1 = CTAs of the current call done with the data phase
// (bit 31: one of them gave up waiting), + 2 = CTAs that have written their partial sum of squares (reduce-only
// calls).  Both counts return to zero when the call completes.
//
// Arrive: tell every peer that this rank reached `phase` of `bucket` in epoch `e`.  One thread per peer.
__device__ __forceinline__ void signal_peers(const Peers& P, int slot, uint32_t e) {
    if (threadIdx.x < P.world) {
        __threadfence_system();
        st_release_sys(P.flags[threadIdx.x] + (size_t)slot * MAX_RANKS + P.rank, e);
    }
}
// Wait until every peer has arrived (epoch >= e); bounded.  Returns false on expiry (whole CTA agrees).
__device__ __forceinline__ bool wait_peers(const Peers& P, int slot, uint32_t e, unsigned long long budget_ns) {
    __shared__ int s_fail;
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    if (threadIdx.x < P.world) {
        const uint32_t* f = P.flags[P.rank] + (size_t)slot * MAX_RANKS + threadIdx.x;
        const unsigned long long t0 = now_ns();
        while ((int)(ld_acquire_sys(f) - e) < 0) {
            if (now_ns() - t0 > budget_ns) { s_fail = 1; break; }
            __nanosleep(64);
        }
    }
    __syncthreads();
    return s_fail == 0;
}

// End of a call.  Every CTA counts itself out of the data phase and returns, except the one that finishes last:
// it announces this rank on `slot1`, waits (bounded) until every peer has done the same -- all ranks have then
// finished reading this rank's inputs and their writes into this rank's outputs have landed -- and advances the
// bucket's epoch.  Only that one CTA waits, so the grid does not have to be resident all at once: CTAs that start
// late never find earlier ones spinning on SM slots they need.  A rank on which some CTA gave up its opening
// wait (its data phase did not run) withholds the announcement, so its peers' closing waits run out too and
// every rank's status word reports the failed step.
__device__ __forceinline__ void finish_call(const Peers& P, uint32_t* ctl, int bucket, int slot1, uint32_t e, bool ok,
                                            int* status, unsigned long long budget_ns,
                                            unsigned long long* tlog = nullptr) {
    __threadfence_system();
    __syncthreads();
    __shared__ int s_last, s_failed;
    if (threadIdx.x == 0) {
        if (!ok) {
            if (status) atomicExch(status, CME_ERR_TIMEOUT);
            atomicOr(&ctl[3 * bucket + 1], 0x80000000u);
        }
        const uint32_t done = atomicAdd(&ctl[3 * bucket + 1], 1u) + 1;
        s_last = ((done & 0x7fffffffu) == gridDim.x);
        s_failed = (int)(done >> 31);
        if (s_last) ctl[3 * bucket + 1] = 0;                        // per-call count: calls may differ in grid size
    }
    __syncthreads();
    if (!s_last) return;
    if (!s_failed) signal_peers(P, slot1, e);
    const bool closed = !s_failed && wait_peers(P, slot1, e, budget_ns);
    if (threadIdx.x == 0) {
        if (!closed && status) atomicExch(status, CME_ERR_TIMEOUT);
        ctl[3 * bucket] = e;                                        // epoch advances once per call
        if (tlog) tlog[2 * bucket + 1] = now_ns();                  // the call is complete on this rank
    }
}

struct ArArgs {
    Peers P;
    long long n;              // elements
    int dtype;                // CME_F32 | CME_BF16
    int algo;                 // 0 one-shot, 1 two-shot, 2 NVLS
    int bucket;
    float scale;
    uint32_t* ctl;
    int* status;
    unsigned long long budget_ns;
};

template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void acc(float* a, uint4 v) {
        a[0] += __uint_as_float(v.x); a[1] += __uint_as_float(v.y); a[2] += __uint_as_float(v.z); a[3] += __uint_as_float(v.w);
    }
    static __device__ __forceinline__ uint4 pack(const float* a, float s) {
        return make_uint4(__float_as_uint(a[0] * s), __float_as_uint(a[1] * s), __float_as_uint(a[2] * s), __float_as_uint(a[3] * s));
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void acc(float* a, uint4 v) {
        float f[8];
        unpack8(v, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] += f[i];
    }
    static __device__ __forceinline__ uint4 pack(const float* a, float s) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = a[i] * s;
        return pack8(f);
    }
};

// Sum of one 16-byte vector over all ranks' buffers, fp32 accumulation in rank order.  The loads of up to eight
// peers are issued before any is consumed, so one thread keeps eight NVLink reads in flight.
template <typename T>
__device__ __forceinline__ void reduce_peers(const Peers& P, long long vec_index, float* acc) {
#pragma unroll
    for (int j = 0; j < Vec16<T>::N; ++j) acc[j] = 0.f;
    for (int r0 = 0; r0 < P.world; r0 += 8) {
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (r0 + k < P.world) v[k] = ld_peer(reinterpret_cast<const uint4*>(P.buf[r0 + k]) + vec_index);
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (r0 + k < P.world) Vec16<T>::acc(acc, v[k]);
    }
}

// All-reduce of P.buf[*][0..n) across ranks into P.buf2[rank][0..n) (out of place: every rank's result lands in
// its own second buffer).  n is a multiple of (16 bytes / element) * world.
template <typename T>
__global__ void __launch_bounds__(COMM_THREADS) allreduce_kernel(const ArArgs a) {
    constexpr int W = Vec16<T>::N;
    const Peers& P = a.P;
    const uint32_t e = a.ctl[3 * a.bucket] + 1;
    const int slot0 = 2 * a.bucket, slot1 = slot0 + 1;
    if (blockIdx.x == 0) signal_peers(P, slot0, e);
    bool ok = wait_peers(P, slot0, e, a.budget_ns);
    if (ok) {
        const long long nvec = a.n / W;
        const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nth = (long long)gridDim.x * blockDim.x;
        if (a.algo == 0) {
            // one-shot: every rank reads the whole range from every peer and keeps the sum; no second phase
            uint4* stage = reinterpret_cast<uint4*>(P.buf2[P.rank]);
            for (long long i = tid; i < nvec; i += nth) {
                float acc[W];
                reduce_peers<T>(P, i, acc);
                stage[i] = Vec16<T>::pack(acc, a.scale);
            }
        } else {
            // two-shot / NVLS: this rank owns slice [rank * per, (rank + 1) * per)
            const long long per = nvec / P.world, v0 = per * P.rank;
            for (long long i = tid; i < per; i += nth) {
                const long long v = v0 + i;
                uint4 out;
                if (a.algo == 2) {
                    if constexpr (W == 8) {
                        uint4 r = mc_ld_reduce_bf16(reinterpret_cast<const uint4*>(P.mc_buf) + v);
                        float f[8];
                        unpack8(r, f);
                        out = Vec16<T>::pack(f, a.scale);
                    } else {
                        float4 r = mc_ld_reduce_f32(reinterpret_cast<const uint4*>(P.mc_buf) + v);
                        float f[4] = {r.x, r.y, r.z, r.w};
                        out = Vec16<T>::pack(f, a.scale);
                    }
                } else {
                    float acc[W];
                    reduce_peers<T>(P, v, acc);
                    out = Vec16<T>::pack(acc, a.scale);
                }
                // the reduced slice goes to the output buffer of every rank
                if (a.algo == 2 && P.mc_buf2) {
                    mc_st(reinterpret_cast<uint4*>(P.mc_buf2) + v, out);
                } else {
                    for (int r = 0; r < P.world; ++r) st_peer(reinterpret_cast<uint4*>(P.buf2[r]) + v, out);
                }
            }
        }
    }
    // closing barrier: every rank has finished reading the inputs and its writes into the peers have landed
    finish_call(P, a.ctl, a.bucket, slot1, e, ok, a.status, a.budget_ns);
}


// Optimizer state and hyper-parameters of the in-kernel AdamW update.
struct OptArgs {
    float* master; float* m; float* v;     // this rank's fp32 state arenas (full length; only the slices it updates are used)
    const int* step; const float* lr;
    float beta1, beta2, eps, weight_decay;
    const long long* nodecay; int n_nodecay;
};

struct FusedArgs {
    Peers P;                  // buf = bf16 gradient arenas, buf2 = bf16 parameter arenas (element 0 = arena start)
    long long start, count;   // bucket range in elements; count is a multiple of 8 * world
    OptArgs o;
    float grad_scale;
    int algo;                 // 0 one-shot: every rank reduces and updates the whole bucket, nothing is sent back;
                              // 1 two-shot: peer loads for this rank's slice, peer stores of the new parameters;
                              // 2 NVLS: multimem.ld_reduce / multimem.st through the switch
    int bucket;
    uint32_t* ctl;
    int* status;
    unsigned long long budget_ns;
    // reduce-only mode (global-norm clipping): no update here
    float* gred;              // fp32 reduced, scaled gradients (full-length arena; this rank's slices are written)
    float* norm_part;         // [gridDim.x] per-CTA partial sums of this call
    float* norm_bucket;       // [bucket] = sum of squares over this rank's slice of the bucket
    unsigned long long* tlog; // optional [2 * buckets] device log: %globaltimer at the start and end of each call
};

// AdamW on eight consecutive elements starting at `el`; `g` already carries every scale factor.
__device__ __forceinline__ uint4 adamw8(const OptArgs& o, long long el, const float* g, float lr, float ibc1,
                                        float ibc2) {
    float decay = 1.f;
    if (o.weight_decay > 0.f) {
        int lo = 0, hi = o.n_nodecay;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (o.nodecay[2 * mid + 1] > el) hi = mid; else lo = mid + 1;
        }
        if (!(lo < o.n_nodecay && o.nodecay[2 * lo] <= el)) decay = 1.f - lr * o.weight_decay;
    }
    // The optimizer state is touched once per step: streaming (evict-first) accesses keep it from displacing the
    // operands of the backward products that run beside this kernel out of L2.
    const float4 m0 = __ldcs(reinterpret_cast<const float4*>(o.m + el)), m1 = __ldcs(reinterpret_cast<const float4*>(o.m + el + 4));
    const float4 v0 = __ldcs(reinterpret_cast<const float4*>(o.v + el)), v1 = __ldcs(reinterpret_cast<const float4*>(o.v + el + 4));
    const float4 p0 = __ldcs(reinterpret_cast<const float4*>(o.master + el)),
                 p1 = __ldcs(reinterpret_cast<const float4*>(o.master + el + 4));
    float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float pp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float gj = g[j];
        mm[j] = o.beta1 * mm[j] + (1.f - o.beta1) * gj;
        vv[j] = o.beta2 * vv[j] + (1.f - o.beta2) * gj * gj;
        pp[j] = pp[j] * decay - lr * (mm[j] * ibc1) / (sqrtf(vv[j] * ibc2) + o.eps);
    }
    __stcs(reinterpret_cast<float4*>(o.m + el), make_float4(mm[0], mm[1], mm[2], mm[3]));
    __stcs(reinterpret_cast<float4*>(o.m + el + 4), make_float4(mm[4], mm[5], mm[6], mm[7]));
    __stcs(reinterpret_cast<float4*>(o.v + el), make_float4(vv[0], vv[1], vv[2], vv[3]));
    __stcs(reinterpret_cast<float4*>(o.v + el + 4), make_float4(vv[4], vv[5], vv[6], vv[7]));
    __stcs(reinterpret_cast<float4*>(o.master + el), make_float4(pp[0], pp[1], pp[2], pp[3]));
    __stcs(reinterpret_cast<float4*>(o.master + el + 4), make_float4(pp[4], pp[5], pp[6], pp[7]));
    return pack8(pp);
}

// New bf16 parameters of eight elements into every rank's parameter arena.
__device__ __forceinline__ void publish8(const Peers& P, long long el, uint4 out, bool nvls) {
    if (nvls && P.mc_buf2) {
        mc_st(reinterpret_cast<__nv_bfloat16*>(P.mc_buf2) + el, out);
    } else {
        for (int r = 0; r < P.world; ++r) st_peer(reinterpret_cast<__nv_bfloat16*>(P.buf2[r]) + el, out);
    }
}

// One bucket of the data-parallel step: barrier -> reduce-scatter (this rank's 1/world slice of the bucket, fp32
// accumulation in rank order) -> x grad_scale -> AdamW on the fp32 master slice -> bf16 parameters into every
// rank's parameter arena -> barrier.  After the kernel every rank holds identical bf16 parameters for the bucket.
//
// UPDATE = false is the first half of the clip-compatible form: the reduced, scaled fp32 gradients of the slice are
// kept (a.gred) together with their sum of squares (a.norm_bucket[bucket], summed over the CTAs in index order, so
// the value does not depend on scheduling); clip_adamw_ag_kernel applies the update once every bucket is reduced
// and the global norm is known.  The reference clips inside its single Adam pass after the last all-reduce
// (FINAL_CLEAN_CODE_/src/model/transformer.cu:618-636).
template <bool UPDATE>
__global__ void __launch_bounds__(COMM_THREADS, 5) fused_rs_adamw_ag_kernel(const FusedArgs a) {
    const Peers& P = a.P;
    const uint32_t e = a.ctl[3 * a.bucket] + 1;
    const int slot0 = 2 * a.bucket, slot1 = slot0 + 1;
    if (a.tlog && blockIdx.x == 0 && threadIdx.x == 0) a.tlog[2 * a.bucket] = now_ns();
    if (blockIdx.x == 0) signal_peers(P, slot0, e);
    bool ok = wait_peers(P, slot0, e, a.budget_ns);
    float sq = 0.f;
    if (ok) {
        const int t = *a.o.step;
        const float lr = *a.o.lr;
        const float ibc1 = 1.f / (1.f - powf(a.o.beta1, (float)t)), ibc2 = 1.f / (1.f - powf(a.o.beta2, (float)t));
        const bool whole = a.algo == 0;                           // one-shot: the whole bucket on every rank
        const bool nvls = a.algo == 2;
        const long long per = whole ? a.count : a.count / P.world;   // elements this rank reduces
        const long long e0 = a.start + (whole ? 0 : per * P.rank);
        const long long nvec = per / 8;
        // Four vectors per thread and trip: the in-switch reductions of all four are requested before the first is
        // consumed, so a thread keeps 64 bytes of NVLink reads in flight instead of 16 (one request per thread was
        // not enough outstanding data to fill the links at their latency).
        constexpr int U = 4;
        const long long stride = (long long)gridDim.x * blockDim.x;
        for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
          uint4 raw[U];
          if (nvls) {
#pragma unroll
              for (int k = 0; k < U; ++k) {
                  const long long ik = i0 + k * stride;
                  if (ik < nvec) raw[k] = mc_ld_reduce_bf16(reinterpret_cast<const __nv_bfloat16*>(P.mc_buf) + e0 + ik * 8);
              }
          }
#pragma unroll
          for (int k = 0; k < U; ++k) {
            const long long i = i0 + k * stride;
            if (i >= nvec) break;
            const long long el = e0 + i * 8;
            float g[8];
            if (nvls) {
                unpack8(raw[k], g);
            } else {
                reduce_peers<__nv_bfloat16>(P, el / 8, g);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) g[j] *= a.grad_scale;
            if constexpr (UPDATE) {
                const uint4 out = adamw8(a.o, el, g, lr, ibc1, ibc2);
                if (whole) *(reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(P.buf2[P.rank]) + el)) = out;
                else publish8(P, el, out, nvls);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) sq += g[j] * g[j];
                *reinterpret_cast<float4*>(a.gred + el) = make_float4(g[0], g[1], g[2], g[3]);
                *reinterpret_cast<float4*>(a.gred + el + 4) = make_float4(g[4], g[5], g[6], g[7]);
            }
          }
        }
    }
    if constexpr (!UPDATE) {
        __shared__ float scratch[32];
        __shared__ int s_norm_last;
        sq = block_sum(sq, scratch);
        if (threadIdx.x == 0) {
            a.norm_part[blockIdx.x] = sq;
            __threadfence();
            // ctl word 2 counts the CTAs whose partial is written; the last one adds them up in index order
            const uint32_t n = atomicAdd(&a.ctl[3 * a.bucket + 2], 1u) + 1;
            s_norm_last = (n == gridDim.x);
            if (s_norm_last) a.ctl[3 * a.bucket + 2] = 0;
        }
        __syncthreads();
        if (s_norm_last && threadIdx.x == 0) {
            __threadfence();
            float tot = 0.f;
            for (unsigned c = 0; c < gridDim.x; ++c) tot += *(volatile float*)(a.norm_part + c);
            a.norm_bucket[a.bucket] = tot;
        }
    }
    finish_call(P, a.ctl, a.bucket, slot1, e, ok, a.status, a.budget_ns, a.tlog);
}

struct ClipArgs {
    Peers P;                  // buf2 = bf16 parameter arenas
    OptArgs o;
    const long long* ranges;  // [n_ranges][2] = (start, count) of every bucket, count a multiple of 8 * world
    int n_ranges;
    const float* gred;        // reduced, scaled fp32 gradients left by the reduce-only kernels
    const float* norm_bucket; // [n_ranges] this rank's sum of squares per bucket
    float clip_norm;
    int use_nvls;
    int bucket;               // flag / control index of this call (one past the gradient buckets)
    int val_slot;             // flag slot whose MAX_RANKS words carry the ranks' partial sums (as float bits)
    uint32_t* ctl;
    int* status;
    unsigned long long budget_ns;
    unsigned long long* tlog;
};

// Second half of the clip-compatible form, one launch per step after every bucket has been reduced: the ranks
// exchange their partial sums of squares through symmetric memory (each writes its value into every peer's slot
// array, then raises the flag; everyone adds the `world` values in rank order, so all ranks compute the same
// norm), then  g *= min(1, clip_norm / ||g||),  AdamW on this rank's slice of every bucket, bf16 parameters into
// every rank's arena, closing barrier.  Same arithmetic as cme_adam with a norm (loss_optim.cu).
__global__ void __launch_bounds__(COMM_THREADS, 5) clip_adamw_ag_kernel(const ClipArgs a) {
    const Peers& P = a.P;
    const uint32_t e = a.ctl[3 * a.bucket] + 1;
    const int slot0 = 2 * a.bucket, slot1 = slot0 + 1;
    if (a.tlog && blockIdx.x == 0 && threadIdx.x == 0) a.tlog[2 * a.bucket] = now_ns();
    if (blockIdx.x == 0 && threadIdx.x < P.world) {
        float local = 0.f;
        for (int b = 0; b < a.n_ranges; ++b) local += a.norm_bucket[b];
        uint32_t* vals = P.flags[threadIdx.x] + (size_t)a.val_slot * MAX_RANKS;
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(vals + P.rank), "r"(__float_as_uint(local)) : "memory");
    }
    if (blockIdx.x == 0) signal_peers(P, slot0, e);               // same thread: value first, then fence + flag
    bool ok = wait_peers(P, slot0, e, a.budget_ns);
    if (ok) {
        const uint32_t* vals = P.flags[P.rank] + (size_t)a.val_slot * MAX_RANKS;
        float total = 0.f;
        for (int r = 0; r < P.world; ++r) {
            uint32_t w;
            asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(w) : "l"(vals + r) : "memory");
            total += __uint_as_float(w);
        }
        const float norm = sqrtf(total);
        const float clipf = (a.clip_norm > 0.f && norm > a.clip_norm) ? a.clip_norm / norm : 1.f;
        const int t = *a.o.step;
        const float lr = *a.o.lr;
        const float ibc1 = 1.f / (1.f - powf(a.o.beta1, (float)t)), ibc2 = 1.f / (1.f - powf(a.o.beta2, (float)t));
        const long long stride = (long long)gridDim.x * blockDim.x;
        for (int b = 0; b < a.n_ranges; ++b) {
            const long long per = a.ranges[2 * b + 1] / P.world;
            const long long e0 = a.ranges[2 * b] + per * P.rank;
            const long long nvec = per / 8;
            for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
                const long long el = e0 + i * 8;
                const float4 g0 = *reinterpret_cast<const float4*>(a.gred + el);
                const float4 g1 = *reinterpret_cast<const float4*>(a.gred + el + 4);
                float g[8] = {g0.x * clipf, g0.y * clipf, g0.z * clipf, g0.w * clipf,
                              g1.x * clipf, g1.y * clipf, g1.z * clipf, g1.w * clipf};
                publish8(P, el, adamw8(a.o, el, g, lr, ibc1, ibc2), a.use_nvls != 0);
            }
        }
    }
    finish_call(P, a.ctl, a.bucket, slot1, e, ok, a.status, a.budget_ns, a.tlog);
}

// A wait that nothing satisfies: used by the failure-detection tests to see the bounded wait give up and report.
__global__ void wait_probe_kernel(const uint32_t* flag, uint32_t expect, unsigned long long budget_ns, int* status,
                                  unsigned long long* waited_ns) {
    const unsigned long long t0 = now_ns();
    bool ok = true;
    while ((int)(ld_acquire_sys(flag) - expect) < 0) {
        if (now_ns() - t0 > budget_ns) { ok = false; break; }
        __nanosleep(64);
    }
    *waited_ns = now_ns() - t0;
    if (!ok) atomicExch(status, CME_ERR_TIMEOUT);
}

void fill_peers(Peers& P, int world, int rank, void* const* buf, void* const* buf2, void* const* flags, void* mc_buf,
                void* mc_buf2) {
    for (int r = 0; r < MAX_RANKS; ++r) {
        P.buf[r] = r < world ? buf[r] : nullptr;
        P.buf2[r] = (r < world && buf2) ? buf2[r] : nullptr;
        P.flags[r] = r < world ? reinterpret_cast<uint32_t*>(flags[r]) : nullptr;
    }
    P.mc_buf = mc_buf; P.mc_buf2 = mc_buf2; P.world = world; P.rank = rank;
}

}  // namespace

// Flag words a rank's symmetric flag array must hold for `buckets` buckets, and local control words.
CME_API int cme_comm_flag_words(int buckets) { return buckets * 2 * MAX_RANKS; }
CME_API int cme_comm_ctl_words(int buckets) { return buckets * 3; }

// All-reduce (sum x scale) of buf[*][offset .. offset+n) into buf2[rank][offset ..), out of place.
// buf / buf2 / flags: arrays of `world` peer pointers (entry r = rank r's buffer as mapped in this process).
// algo: 0 one-shot, 1 two-shot, 2 NVLS (needs mc_buf; mc_buf2 optional).  n must be a multiple of
// (16 / element size) * world and the offset 16-byte aligned.  `ctl`: cme_comm_ctl_words() zeroed uint32 in local
// device memory; `status`: device int that receives CME_ERR_TIMEOUT when a peer did not arrive within budget_ms.
CME_API int cme_comm_allreduce(int dtype, int world, int rank, void* const* buf, void* const* buf2,
                               void* const* flags, void* mc_buf, void* mc_buf2, long long offset, long long n,
                               int algo, float scale, int bucket, int max_buckets, int ctas, void* ctl, int* status,
                               double budget_ms, void* stream) {
    CME_REQUIRE(world >= 1 && world <= MAX_RANKS && rank >= 0 && rank < world, CME_ERR_SHAPE, "comm: bad world/rank");
    const int es = dtype == CME_BF16 ? 2 : 4, w = 16 / es;
    CME_REQUIRE(n > 0 && n % ((long long)w * world) == 0, CME_ERR_SHAPE,
                "comm: element count %lld is not a multiple of %d", n, w * world);
    CME_REQUIRE(algo != 2 || mc_buf != nullptr, CME_ERR_UNSUPPORTED, "comm: NVLS requested without a multicast mapping");
    CME_REQUIRE(bucket >= 0 && bucket < max_buckets, CME_ERR_LIMIT, "comm: bucket %d outside the %d the flags were sized for",
                bucket, max_buckets);
    CME_REQUIRE(ctas >= 1 && ctas <= 740, CME_ERR_SHAPE, "comm: CTA count must be in [1, 740]");
    ArArgs a{};
    void* b1[MAX_RANKS]; void* b2[MAX_RANKS];
    for (int r = 0; r < world; ++r) {
        b1[r] = static_cast<char*>(buf[r]) + offset * es;
        b2[r] = static_cast<char*>(buf2[r]) + offset * es;
    }
    fill_peers(a.P, world, rank, b1, b2, flags, mc_buf ? static_cast<char*>(mc_buf) + offset * es : nullptr,
               mc_buf2 ? static_cast<char*>(mc_buf2) + offset * es : nullptr);
    a.n = n; a.dtype = dtype; a.algo = algo; a.bucket = bucket; a.scale = scale;
    a.ctl = static_cast<uint32_t*>(ctl); a.status = status;
    a.budget_ns = (unsigned long long)(budget_ms * 1e6);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == CME_BF16) allreduce_kernel<__nv_bfloat16><<<ctas, COMM_THREADS, 0, st>>>(a);
    else allreduce_kernel<float><<<ctas, COMM_THREADS, 0, st>>>(a);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

// Fused reduce-scatter + AdamW + all-gather for the bucket [start, start + count) of the arenas.
// grads / params: arrays of `world` peer pointers to the START of each rank's bf16 gradient / parameter arena.
// algo: 0 one-shot (small buckets: every rank reduces and updates the whole bucket, so all ranks must hold the
// optimizer state of the bucket), 1 two-shot over peer loads / stores, 2 NVLS (needs mc_grads).
// gred != null selects the reduce-only form used with global-norm clipping: no update; the reduced, scaled fp32
// gradients of this rank's slice go to gred, their sum of squares to norm_bucket[bucket]; norm_part holds one
// float per CTA.  cme_comm_clip_adamw finishes the step.  `bucket` must be below `max_buckets`, the bucket count
// the flag and control arrays were sized for.
CME_API int cme_comm_fused_adamw(int world, int rank, void* const* grads, void* const* params, void* const* flags,
                                 void* mc_grads, void* mc_params, long long start, long long count, float* master,
                                 float* m, float* v, const int* step, const float* lr, float beta1, float beta2,
                                 float eps, float weight_decay, float grad_scale, const long long* nodecay,
                                 int n_nodecay, int algo, int bucket, int max_buckets, int ctas, void* ctl,
                                 int* status, double budget_ms, float* gred, float* norm_part, float* norm_bucket,
                                 unsigned long long* tlog, void* stream) {
    // Threads per CTA: COMM_THREADS unless CME213_COMM_THREADS asks for thinner CTAs (a multiple of 32 that holds one
    // thread per rank); fewer warps per SM take fewer issue slots from the compute kernels running beside them.
    static const int threads = [] {
        const char* e = getenv("CME213_COMM_THREADS");
        const int t = e ? atoi(e) : COMM_THREADS;
        return (t >= 32 && t <= COMM_THREADS && t % 32 == 0) ? t : COMM_THREADS;
    }();
    CME_REQUIRE(world >= 1 && world <= MAX_RANKS && rank >= 0 && rank < world, CME_ERR_SHAPE, "comm: bad world/rank");
    CME_REQUIRE(count > 0 && count % (8ll * world) == 0 && start % 8 == 0, CME_ERR_SHAPE,
                "comm: bucket [%lld, +%lld) is not aligned to 8 * world elements", start, count);
    CME_REQUIRE(algo >= 0 && algo <= 2, CME_ERR_SHAPE, "comm: unknown algorithm %d", algo);
    CME_REQUIRE(algo != 2 || mc_grads != nullptr, CME_ERR_UNSUPPORTED, "comm: NVLS requested without a multicast mapping");
    CME_REQUIRE(bucket >= 0 && bucket < max_buckets, CME_ERR_LIMIT, "comm: bucket %d outside the %d the flags were sized for",
                bucket, max_buckets);
    CME_REQUIRE(ctas >= 1 && ctas <= 740, CME_ERR_SHAPE, "comm: CTA count must be in [1, 740]");
    CME_REQUIRE(!gred || (algo != 0 && norm_part && norm_bucket), CME_ERR_SHAPE,
                "comm: the reduce-only form needs scratch for the norm and a two-shot or NVLS reduction");
    FusedArgs a{};
    fill_peers(a.P, world, rank, grads, params, flags, mc_grads, mc_params);
    a.start = start; a.count = count;
    a.o = OptArgs{master, m, v, step, lr, beta1, beta2, eps, weight_decay, nodecay, n_nodecay};
    a.grad_scale = grad_scale; a.algo = algo; a.bucket = bucket;
    a.ctl = static_cast<uint32_t*>(ctl); a.status = status;
    a.budget_ns = (unsigned long long)(budget_ms * 1e6);
    a.gred = gred; a.norm_part = norm_part; a.norm_bucket = norm_bucket; a.tlog = tlog;
    const int block = ctas > 296 ? COMM_THREADS : threads;      // the tail call has the GPU to itself: full CTAs
    if (gred) fused_rs_adamw_ag_kernel<false><<<ctas, block, 0, (cudaStream_t)stream>>>(a);
    else fused_rs_adamw_ag_kernel<true><<<ctas, block, 0, (cudaStream_t)stream>>>(a);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

// Global-norm clip + AdamW + all-gather over every bucket, after the reduce-only calls of one step.
// ranges: device array of n_ranges (start, count) pairs; `bucket` / `val_slot`: flag indices reserved for this
// call (bucket < max_buckets, val_slot < 2 * max_buckets, neither used by a gradient bucket).
CME_API int cme_comm_clip_adamw(int world, int rank, void* const* params, void* const* flags, void* mc_params,
                                const long long* ranges, int n_ranges, const float* gred, const float* norm_bucket,
                                float* master, float* m, float* v, const int* step, const float* lr, float beta1,
                                float beta2, float eps, float weight_decay, float clip_norm, const long long* nodecay,
                                int n_nodecay, int use_nvls, int bucket, int val_slot, int max_buckets, int ctas,
                                void* ctl, int* status, double budget_ms, unsigned long long* tlog, void* stream) {
    CME_REQUIRE(world >= 1 && world <= MAX_RANKS && rank >= 0 && rank < world, CME_ERR_SHAPE, "comm: bad world/rank");
    CME_REQUIRE(bucket >= 0 && bucket < max_buckets && val_slot >= 0 && val_slot < 2 * max_buckets, CME_ERR_LIMIT,
                "comm: flag indices %d / %d outside the %d buckets the flags were sized for", bucket, val_slot,
                max_buckets);
    CME_REQUIRE(!use_nvls || mc_params != nullptr, CME_ERR_UNSUPPORTED, "comm: NVLS requested without a multicast mapping");
    CME_REQUIRE(ctas >= 1 && ctas <= 740, CME_ERR_SHAPE, "comm: CTA count must be in [1, 740]");
    ClipArgs a{};
    fill_peers(a.P, world, rank, params, params, flags, nullptr, mc_params);
    a.o = OptArgs{master, m, v, step, lr, beta1, beta2, eps, weight_decay, nodecay, n_nodecay};
    a.ranges = ranges; a.n_ranges = n_ranges; a.gred = gred; a.norm_bucket = norm_bucket; a.clip_norm = clip_norm;
    a.use_nvls = use_nvls; a.bucket = bucket; a.val_slot = val_slot; a.tlog = tlog;
    a.ctl = static_cast<uint32_t*>(ctl); a.status = status;
    a.budget_ns = (unsigned long long)(budget_ms * 1e6);
    clip_adamw_ag_kernel<<<ctas, COMM_THREADS, 0, (cudaStream_t)stream>>>(a);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

// One thread writes %globaltimer to *slot when the stream reaches it: a device-side timestamp that also works inside a
// replayed CUDA graph (where events cannot be read back per replay).
__global__ void record_time_kernel(unsigned long long* slot) { *slot = now_ns(); }

CME_API int cme_record_time(unsigned long long* slot, void* stream) {
    record_time_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(slot);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

// Launches a single-thread kernel that waits (at most budget_ms) for *flag >= expect.  On expiry it stores
// CME_ERR_TIMEOUT in *status and returns normally; *waited_ns receives the time it spent.
CME_API int cme_comm_wait_probe(const void* flag, unsigned expect, double budget_ms, int* status,
                                unsigned long long* waited_ns, void* stream) {
    wait_probe_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(static_cast<const uint32_t*>(flag), expect,
                                                         (unsigned long long)(budget_ms * 1e6), status, waited_ns);
    CME_LAUNCH_CHECK();
    return CME_OK;
}
