// Fused flash-style attention on the 5th-generation tensor cores (head size 64, bf16, causal or not, both
// head layouts): scores, probabilities (forward) and output partials live in TMEM, nothing of size T x T reaches
// global memory, only the per-row log-sum-exp is saved for backward.
//
// Replaces the reference's production attention -- two strided-batched GEMMs around an in-place softmax
// with P, dP and dS materialised as [B*H, T, T] buffers, and four more batched GEMMs plus a dS kernel in
// backward (FINAL_CLEAN_CODE_/src/kernels/attention.cu:138-200, 253-328).
//
// Forward, per CTA = one (batch, head) and 128 queries; 4 softmax warps (thread = query row) + 1 warp whose
// lane 0 issues TMA loads and tcgen05.mma:
//     S_j = Q K_j^T (TMEM) -> copied to registers (the tensor core starts S_{j+1} at once) -> online softmax with a
//     lazily raised reference maximum; a quarter of the exponentials are a packed cubic on the FMA pipe, the rest go
//     to the special-function unit -> P_j (bf16 pairs) written back to tensor memory with tcgen05.st
//     -> O += P_j V_j with the A operand read from tensor memory (P never passes through shared memory; TMEM
//     accumulator, rescaled in place only when the reference maximum is raised)
// Backward, per CTA = one (batch, head) and 128 keys, looping over query blocks (thread = query row, so the
// row's log-sum-exp and delta are two registers):
//     S = Q_i K^T,  dP = dO_i V^T (TMEM)  ->  P, dS (bf16, shared, double buffered)
//     dV += P^T dO_i,  dK += dS^T Q_i (A operand read transposed; TMEM accumulators),  dQ_i = dS K (TMEM).
//     dQ_i gets a part from every key block that sees query block i.  The parts are added to an fp32 scratch with
//     bulk reduce-adds in whatever order the CTAs arrive (fast; the last bits of dQ depend on the order), and
//     either (dq_mode 0, the default) the launch clears the scratch first and a small kernel scales and casts the
//     sums afterwards, or (dq_mode 2) a counter per tile tells the CTA whose part arrived last to do that itself --
//     a spare warp converts the tile and writes zeros back, so no clearing or conversion pass runs; the query
//     blocks are then walked downwards so that the finishing work spreads over the CTAs.  Still slower at large shapes
//     (about 0.05 ms per call at 16 x 12 heads x 1024 tokens: every reduce-add has to complete before its part is
//     counted in, and one warp converts a 32 KB tile).  Deterministic form (dq_mode 1): the
//     highest key block stores its part, each lower one adds its own when the tile's counter says it is its turn,
//     and key block 0, whose turn is last, adds the sum to its part in registers, scales, casts and writes dQ --
//     bit-reproducible, no clearing or conversion pass, but the chain of turns makes CTAs wait for one another
//     (measured 0.32 ms against 0.25 ms per call at 16 x 12 heads x 1024 tokens).
//     The scores of block i+1 are issued before the gradient MMAs of block i, so the arithmetic of block i+1
//     overlaps them.
// Every mbarrier wait is bounded; on expiry the CTA flags the status word, frees TMEM and returns.
#include "attention.h"
#include "sm100_ptx.cuh"

#include <cuda.h>
#include <mutex>

using namespace sm100;

int* cme_attn_status_ptr();

namespace {

constexpr int HD = 64;
constexpr int BQ = 128;            // rows per tile (queries in forward, keys in backward)
constexpr int BKV = 128;           // streamed rows per step
constexpr int TILE_BYTES = 128 * HD * 2;        // 16 KB: 128 rows x 128 bytes
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, const void* src, int c0, int c1, int c2) {
    asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}

// 2^x for two values on the FMA and integer pipes (no special-function unit): x = n + f with n = round(x) taken from
// the mantissa of x + 1.5 * 2^23, 2^f by a cubic on [-0.5, 0.5] (relative error 7.5e-5, far below bf16 resolution),
// and n added into the exponent field.  x is clamped at -126 (masked scores arrive as -inf and come out as 1e-38).
// The softmax loop sends part of its exponentials here so that the special-function unit, which takes 8 cycles per
// warp instruction, is no longer what the loop waits for.
__device__ __forceinline__ void ex2_poly2(float x0, float x1, float& y0, float& y1) {
    const F32x2 x = f2_pack(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
    const F32x2 t = f2_add(x, f2_splat(12582912.f));
    const F32x2 n = f2_add(t, f2_splat(-12582912.f));
    const F32x2 f = f2_fma(n, f2_splat(-1.f), x);
    F32x2 q = f2_fma(f2_splat(0.05517165f), f, f2_splat(0.24261112f));
    q = f2_fma(q, f, f2_splat(0.69326099f));
    q = f2_fma(q, f, f2_splat(0.99992807f));
    float t0, t1, q0, q1;
    f2_unpack(t, t0, t1);
    f2_unpack(q, q0, q1);
    y0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
    y1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
}

// A descriptor whose start address is `bytes` further than that of `base` (the address field counts 16-byte
// units and never carries out of its 14 bits for shared-memory offsets), so the issuing thread spends one add
// per operand instead of re-encoding the descriptor for each of the ~30 MMAs of a block.
__device__ __forceinline__ uint64_t desc_add(uint64_t base, uint32_t bytes) { return base + (uint64_t)(bytes >> 4); }

// Swizzled position of 16-byte chunk `c` of row `r` inside a [rows x 128 B] tile.
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

struct FwdParams {
    int T, nh, causal;
    float scale_log2;              // scale * log2(e)
    float* lse;
    int* status;
};

// ------------------------------------------------------------------------------------------------------
// Forward
// ------------------------------------------------------------------------------------------------------
// shared: Q 16K | K[3] 48K | V[3] 48K | barriers      (P never passes through shared memory)
constexpr int FWD_KV_STAGES = 3;           // a K / V tile is requested two blocks ahead of its use: its ~1200-clock
                                           // latency no longer delays the next S product
constexpr int FWD_SMEM = (1 + 2 * FWD_KV_STAGES) * TILE_BYTES + 128;   // two CTAs per SM: 2 x (this + 1 KB) <= 228 KB
constexpr int FWD_THREADS = 160;
constexpr int FWD_TMEM_COLS = 256;         // S: [0,128)  O accumulator: [128,192)  P (bf16 pairs): [192,256)
static_assert(2 * (FWD_SMEM + 1024) <= 228 * 1024, "two forward CTAs must fit one SM's shared memory");
static_assert(128 + HD + BKV / 2 <= FWD_TMEM_COLS && 2 * FWD_TMEM_COLS <= 512,
              "forward TMEM budget: S + O + P per CTA, two CTAs per SM");
#ifndef CME_ATTN_FWD_POLY_PAIRS
#define CME_ATTN_FWD_POLY_PAIRS 1
#endif
constexpr int FWD_POLY_PAIRS = CME_ATTN_FWD_POLY_PAIRS;   // of every 4 score pairs, how many take 2^x on the FMA pipe
constexpr float RESCALE_THRESHOLD = 8.f;   // log2 units: the running maximum is only raised when it grows by > 2^8

__global__ void __launch_bounds__(FWD_THREADS, 2)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                   const FwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {             // swizzled tiles need a 1024-byte aligned base
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, CME_ERR_SHAPE);
        return;
    }
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + TILE_BYTES;                            // FWD_KV_STAGES stages
    uint8_t* sV = sK + FWD_KV_STAGES * TILE_BYTES;            // FWD_KV_STAGES stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + FWD_KV_STAGES * TILE_BYTES);
    uint64_t* q_full = bars;                  // 1
    uint64_t* kv_full = bars + 1;             // [3]
    uint64_t* kv_empty = bars + 4;            // [3]
    uint64_t* s_full = bars + 7;              // S ready for softmax
    uint64_t* s_free = bars + 8;              // S copied to registers (128 arrivals): the next S may be issued
    uint64_t* p_ready = bars + 9;             // P written to tensor memory, O rescaled (128 arrivals)
    uint64_t* o_full = bars + 10;             // P V accumulated, P consumed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = gridDim.x - 1 - blockIdx.x;               // heavy (late) causal tiles first
    const int q0 = qt * BQ;
    const int bh = blockIdx.y, b = bh / p.nh, h = bh % p.nh;
    const int nkv = p.causal ? min((q0 + BQ + BKV - 1) / BKV, (p.T + BKV - 1) / BKV) : (p.T + BKV - 1) / BKV;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < FWD_KV_STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
        mbar_init(s_full, 1);
        mbar_init(s_free, 128);
        mbar_init(p_ready, 128);
        mbar_init(o_full, 1);
        fence_barrier_init();
    }
    if (warp == 4) { tmem_alloc(tmem_slot, FWD_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 128, tmem_P = tmem_base + 128 + HD;
    pdl_wait();        // barrier set-up and TMEM allocation above may overlap the tail of the previous kernel

    if (warp == 4) {
        if (lane == 0) {
            // ---------------- producer + MMA issuer (one thread) ----------------
            constexpr uint32_t idesc_s = make_idesc(1, false, false, 128, 128);   // Q K^T: both K-major
            constexpr uint32_t idesc_o = make_idesc(1, false, true, 128, HD);     // P V: V is MN-major
            bool ok = true;
            mbar_arrive_expect_tx(q_full, TILE_BYTES);
            tma_load_4d(sQ, &tmQ, q_full, 0, q0, h, b);
            auto load_kv = [&](int j) {
                const int st = j % FWD_KV_STAGES;
                mbar_arrive_expect_tx(&kv_full[st], 2 * TILE_BYTES);
                tma_load_4d(sK + st * TILE_BYTES, &tmK, &kv_full[st], 0, j * BKV, h, b);
                tma_load_4d(sV + st * TILE_BYTES, &tmV, &kv_full[st], 0, j * BKV, h, b);
            };
            const uint64_t dQ_ = make_smem_desc(smem_u32(sQ), 0, 1024);
            const uint64_t dK0 = make_smem_desc(smem_u32(sK), 0, 1024);
            const uint64_t dV0 = make_smem_desc(smem_u32(sV), TILE_BYTES, 1024);
            auto issue_s = [&](int j) {
                const uint64_t kd = desc_add(dK0, (j % FWD_KV_STAGES) * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mma_f16_ss(tmem_S, desc_add(dQ_, k * 32), desc_add(kd, k * 32), idesc_s, k > 0);
                mma_commit(s_full);
            };
            for (int j = 0; j < FWD_KV_STAGES && j < nkv; ++j) load_kv(j);
            ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(&kv_full[0], 0, abort_flag);
            if (ok) { tc_fence_after(); issue_s(0); }
            for (int j = 0; j < nkv && ok; ++j) {
                const int st = j % FWD_KV_STAGES;
                if (j >= 1 && j + 2 < nkv) {
                    // the stage that block j - 1 used is refilled with block j + 2: its P V product was issued one
                    // block ago, so this wait does not hold anything up
                    if (!mbar_wait(&kv_empty[(j - 1) % FWD_KV_STAGES], ((j - 1) / FWD_KV_STAGES) & 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    load_kv(j + 2);
                }
                if (j + 1 < nkv) {
                    // S_j sits in registers now: the tensor core computes S_{j+1} while softmax_j runs
                    if (!mbar_wait(s_free, j & 1, abort_flag) ||
                        !mbar_wait(&kv_full[(j + 1) % FWD_KV_STAGES], ((j + 1) / FWD_KV_STAGES) & 1, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    issue_s(j + 1);
                }
                if (!mbar_wait(p_ready, j & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint64_t vd = desc_add(dV0, st * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k)       // A = P from tensor memory: 16 keys = 8 columns per step
                    mma_f16_ts(tmem_O, tmem_P + k * 8, desc_add(vd, k * 2048), idesc_o, (j > 0 || k > 0));
                mma_commit(o_full);
                mma_commit(&kv_empty[st]);
            }
            if (!ok) for (int i = 0; i < 2000; ++i) __nanosleep(500);
        }
    } else {
        // ---------------- softmax warps: thread = query row ----------------
        const int row = warp * 32 + lane;                 // 0..127 == TMEM lane
        const int q = q0 + row;
        const uint32_t lane_addr = uint32_t(warp * 32) << 16;
        float m_ref = -INFINITY, l = 0.f;                 // reference maximum (log2 units) and running row sum
        bool ok = true;
        for (int j = 0; j < nkv && ok; ++j) {
            if (!mbar_wait(s_full, j & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            uint32_t r[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32(tmem_S + lane_addr + c * 32, r + c * 32);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(s_free);
            const int k0 = j * BKV;
            if ((k0 + BKV > p.T) || (p.causal && k0 + BKV - 1 > q0)) {        // diagonal or ragged block
                // keys [0, lim) of this block are visible to this row: one compare and one select per score
                const int lim = min(p.T, p.causal ? q + 1 : p.T) - k0;
#pragma unroll
                for (int i = 0; i < 128; ++i) r[i] = i < lim ? r[i] : 0xff800000u;     // -inf
            }
            // eight independent chains (a single one would be 128 dependent operations long)
            float mx8[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) mx8[c] = __uint_as_float(r[c]);
#pragma unroll
            for (int i = 8; i < 128; ++i) mx8[i & 7] = fmaxf(mx8[i & 7], __uint_as_float(r[i]));
            float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                             fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
            mx *= p.scale_log2;                            // scale > 0, so the maximum commutes with it
            // Raise the reference maximum only when it would grow by more than the threshold: the accumulated
            // output then needs a rescale, which is rare after the first blocks.
            const bool raise = (j == 0) ? true : (mx > m_ref + RESCALE_THRESHOLD);
            float alpha = 1.f;
            if (raise) {
                alpha = (m_ref == -INFINITY) ? 0.f : ex2_approx(m_ref - mx);
                m_ref = mx;
            }
            if (j > 0) {
                // the previous P V product must be complete before P is overwritten or O is rescaled
                if (!mbar_wait(o_full, (j - 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                if (__any_sync(0xffffffffu, raise)) {
#pragma unroll 1
                    for (int c = 0; c < HD / 16; ++c) {       // 16 columns at a time: the score row stays in registers
                        uint32_t o[16];
                        tmem_ld16(tmem_O + lane_addr + c * 16, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st16(tmem_O + lane_addr + c * 16, o);
                    }
                    tmem_wait_st();
                }
                l *= alpha;
            }
            const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
            // scale-and-shift and the row sum on packed pairs (one instruction per two keys); four independent chains
            const F32x2 sc2 = f2_splat(p.scale_log2), nm2 = f2_splat(-m_use);
            F32x2 sum2[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) sum2[c] = f2_splat(0.f);
            // In passes over 32 keys, so that the 16 scale-and-shifts, then the 32 exponentials, then the sums and
            // stores are each a run of independent instructions (no exponential waits for its own operand or result)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float* x = reinterpret_cast<float*>(r + c * 32);
#pragma unroll
                for (int i = 0; i < 32; i += 2) f2_unpack(f2_fma(f2_pack(x[i], x[i + 1]), sc2, nm2), x[i], x[i + 1]);
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    if ((i & 7) < 2 * FWD_POLY_PAIRS) {
                        ex2_poly2(x[i], x[i + 1], x[i], x[i + 1]);
                    } else {
                        x[i] = ex2_approx(x[i]);
                        x[i + 1] = ex2_approx(x[i + 1]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 32; i += 2) sum2[(i >> 1) & 3] = f2_add(sum2[(i >> 1) & 3], f2_pack(x[i], x[i + 1]));
                // 32 probabilities = 16 columns of bf16 pairs, straight into the A operand of the P V product
                uint32_t pw[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) pw[i] = f2_to_bf2(x[2 * i], x[2 * i + 1]);
                tmem_st16(tmem_P + lane_addr + c * 16, pw);
            }
            tmem_wait_st();
            {
                float s0, s1;
                f2_unpack(f2_add(f2_add(sum2[0], sum2[1]), f2_add(sum2[2], sum2[3])), s0, s1);
                l += s0 + s1;
            }
            tc_fence_before();
            mbar_arrive(p_ready);
        }
        if (ok && nkv > 0) {
            if (mbar_wait(o_full, (nkv - 1) & 1, abort_flag)) {
                tc_fence_after();
                float o[HD];
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t t[32];
                    tmem_ld32(tmem_O + lane_addr + c * 32, t);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c * 32 + i] = __uint_as_float(t[i]);
                }
                const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
                for (int i = 0; i < HD; ++i) o[i] *= inv;
                // stage this warp's 32 rows (every product is complete and no load is in flight: the first K stage is
                // free) and store them with one TMA tile store
                uint8_t* stage = sK + warp * 4096;
#pragma unroll
                for (int g = 0; g < 8; ++g) *reinterpret_cast<uint4*>(stage + swz(lane, g)) = pack8(o + g * 8);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    tma_store_4d(&tmO, stage, 0, q0 + warp * 32, h, b);
                    tma_store_commit();
                    tma_store_wait_read<0>();         // shared memory may go once the copy engine has read the tile
                }
                if (q < p.T) p.lse[(long long)bh * p.T + q] = (m_ref == -INFINITY) ? -INFINITY : (m_ref + log2f(l)) / LOG2E;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, CME_ERR_TIMEOUT);
    if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem_base, FWD_TMEM_COLS); }
}

// ------------------------------------------------------------------------------------------------------
// Backward
// ------------------------------------------------------------------------------------------------------
struct BwdParams {
    int T, nh, causal;
    float scale, scale_log2;
    const float* lse;
    const float* delta;
    float* dq_accum;               // fp32 [nb*nh, T, HD] scratch for the partial sums of dQ
    __nv_bfloat16* dk; __nv_bfloat16* dv;
    long long sb, sh, st;          // strides of dQ / dK / dV
    int* status;
    int* dq_sem;                   // [nb*nh, query blocks] contribution counters (zero between launches); null in mode 0
    __nv_bfloat16* dq;             // final dQ (modes 1 and 2)
    int dq_mode;                   // 0: unordered adds into a scratch the launch cleared, converted by dq_convert_kernel
                                   // 1: ordered adds, key block 0 finishes   2: unordered adds, the last part's CTA finishes
};

// Bounded wait until *sem >= want (acquire).  Lane 0 of the calling warp polls; the warp then synchronises.
__device__ __forceinline__ bool sem_wait_warp(const int* sem, int want, volatile int* abort_flag) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0) {
        uint32_t i = 0;
        for (;; ++i) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(sem) : "memory");
            if (v >= want) break;
            if ((i & 255u) == 255u && *abort_flag) { ok = false; break; }
            if (i >= (1u << 22)) { *abort_flag = 1; ok = false; break; }
            __nanosleep(32);
        }
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    return ok;
}

// shared: K 16K | V 16K | Q[2] 32K | dO[2] 32K | P 32K | dS[2] 64K | dQ staging (fp32) 32K | barriers   (one CTA per SM)
constexpr int BWD_SMEM = 14 * TILE_BYTES + 512;     // tiles | barriers, flags and the finishing warp's ring
constexpr int BWD_MMA_WARP = 16;           // warps 0..15 compute, warp 16 issues TMA loads and MMA,
constexpr int BWD_STORE_WARP = 17;         // warp 17 issues the dQ reduce-stores
constexpr int BWD_FINISH_WARP = 18;        // warp 18 (mode 2) converts the dQ tiles whose last part this CTA added
constexpr int BWD_THREADS = 19 * 32;
constexpr int FIN_RING = CME_ATTN_FINISH_MAX_QBLOCKS;   // a CTA hands over at most one tile per query block
constexpr int BWD_TMEM_COLS = 512;     // S [0,128) dP [128,256) dV [256,320) dK [320,384) dQ [384,448)
static_assert(12 * 8 + 4 + 4 + 4 + FIN_RING * 4 <= 512, "barriers, flags and ring exceed their block");
static_assert(BWD_SMEM <= 227 * 1024, "backward shared-memory carve-up exceeds what one CTA may have");
static_assert(2 * 128 + 3 * HD <= BWD_TMEM_COLS, "backward TMEM budget: S, dP, dV, dK, dQ");

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmdQ, const BwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, CME_ERR_SHAPE);
        return;
    }
    uint8_t* sK = smem;
    uint8_t* sV = sK + TILE_BYTES;
    uint8_t* sQ = sV + TILE_BYTES;             // 2 stages
    uint8_t* sdO = sQ + 2 * TILE_BYTES;        // 2 stages
    uint8_t* sP = sdO + 2 * TILE_BYTES;        // [2 key atoms][128 query rows][128 B]; free again once dV's MMAs ran
    uint8_t* sdS = sP + 2 * TILE_BYTES;        // 2 buffers, same layout
    uint8_t* sdQ = sdS + 4 * TILE_BYTES;       // fp32 dQ staging: [2 column atoms][128 query rows][128 B]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sdQ + 2 * TILE_BYTES);
    uint64_t* kv_full = bars;
    uint64_t* q_full = bars + 1;               // [2]
    uint64_t* q_empty = bars + 3;              // [2]
    uint64_t* s_full = bars + 5;               // S and dP of a query block are in TMEM
    uint64_t* p_ready = bars + 6;              // P, dS written; S, dP, previous dQ consumed (512 arrivals)
    uint64_t* dq_full = bars + 7;              // dV, dK accumulated and dQ of a query block complete
    uint64_t* p_free = bars + 8;               // dV's MMAs of a block have read P
    uint64_t* dqs_full = bars + 9;             // dQ staging written (512 arrivals)
    uint64_t* dqs_free = bars + 10;            // dQ staging read by the reduce-store
    uint64_t* s_free = bars + 11;              // S and dP of a query block are in registers (512 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* fin_count = abort_flag + 1;  // tiles handed to the finishing warp so far; -1 - n once the store warp
                                               // has ended after n tiles
    volatile int* fin_ring = abort_flag + 2;   // [FIN_RING] query-block indices

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Ordered form: higher key blocks are dispatched first, so a CTA only ever waits for the dQ parts of key blocks
    // above its own, which are then resident or finished.  Unordered form: the key blocks with the most query blocks
    // (the lowest) first.
    const int nkb = gridDim.x;
    const bool ordered = p.dq_mode == 1, finish_last = p.dq_mode == 2;
    const int kb = ordered ? nkb - 1 - (int)blockIdx.x : (int)blockIdx.x, k0 = kb * BKV;
    const int bh = blockIdx.y, b = bh / p.nh, h = bh % p.nh;
    const int nq = (p.T + BQ - 1) / BQ;
    // first key block to contribute to query block qi (the highest one that sees it); key block kb's turn comes when
    // first_kb(qi) - kb parts are in, key block 0 finishes the tile
    auto first_kb = [&](int qi) { return p.causal ? min(qi, nkb - 1) : nkb - 1; };
    const int i_begin = p.causal ? kb : 0;     // query blocks that see this key block
    const int n_it = nq - i_begin;
    // Query block of iteration `it`.  Mode 2 walks them downwards: the key blocks of a head start together, so all of
    // them then reach a query tile in the same iteration and whichever comes last finishes it -- the finishing work
    // spreads over the CTAs instead of queueing up on key block 0, which is the last arrival of every tile when all
    // walk upwards.
    auto qblock = [&](int it) { return finish_last ? nq - 1 - it : i_begin + it; };

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        *fin_count = 0;
        mbar_init(kv_full, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
        mbar_init(s_full, 1);
        mbar_init(p_ready, 512);
        mbar_init(dq_full, 1);
        mbar_init(p_free, 1);
        mbar_init(dqs_full, 512);
        mbar_init(dqs_free, 1);
        mbar_init(s_free, 512);
        fence_barrier_init();
    }
    if (warp == BWD_MMA_WARP) { tmem_alloc(tmem_slot, BWD_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 128, tmem_dV = tmem_base + 256,
                   tmem_dK = tmem_base + 320, tmem_dQ = tmem_base + 384;

    if (warp == BWD_MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(1, false, false, 128, 128);    // Q K^T, dO V^T
            constexpr uint32_t idesc_t = make_idesc(1, true, true, 128, HD);       // P^T dO, dS^T Q (A read transposed)
            constexpr uint32_t idesc_q = make_idesc(1, false, true, 128, HD);      // dS K
            bool ok = true;
            mbar_arrive_expect_tx(kv_full, 2 * TILE_BYTES);
            tma_load_4d(sK, &tmK, kv_full, 0, k0, h, b);
            tma_load_4d(sV, &tmV, kv_full, 0, k0, h, b);
            auto load_q = [&](int it) {
                const int st = it & 1;
                mbar_arrive_expect_tx(&q_full[st], 2 * TILE_BYTES);
                tma_load_4d(sQ + st * TILE_BYTES, &tmQ, &q_full[st], 0, qblock(it) * BQ, h, b);
                tma_load_4d(sdO + st * TILE_BYTES, &tmdO, &q_full[st], 0, qblock(it) * BQ, h, b);
            };
            // descriptors are encoded once; per MMA only a byte offset is added
            const uint64_t kK = make_smem_desc(smem_u32(sK), 0, 1024), vK = make_smem_desc(smem_u32(sV), 0, 1024);
            const uint64_t kMN = make_smem_desc(smem_u32(sK), TILE_BYTES, 1024);
            // stage / buffer 1 of each ring lies a fixed distance after stage 0, so its descriptor is base + offset
            const uint64_t qK0 = make_smem_desc(smem_u32(sQ), 0, 1024), oK0 = make_smem_desc(smem_u32(sdO), 0, 1024);
            const uint64_t qMN0 = make_smem_desc(smem_u32(sQ), TILE_BYTES, 1024);
            const uint64_t oMN0 = make_smem_desc(smem_u32(sdO), TILE_BYTES, 1024);
            const uint64_t pMN0 = make_smem_desc(smem_u32(sP), TILE_BYTES, 1024);
            const uint64_t sMN0 = make_smem_desc(smem_u32(sdS), TILE_BYTES, 1024);
            const uint64_t sK0 = make_smem_desc(smem_u32(sdS), 0, 1024);
            auto issue_s = [&](int it) {
                const uint64_t qd = desc_add(qK0, (it & 1) * TILE_BYTES), od = desc_add(oK0, (it & 1) * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mma_f16_ss(tmem_S, desc_add(qd, k * 32), desc_add(kK, k * 32), idesc_s, k > 0);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mma_f16_ss(tmem_dP, desc_add(od, k * 32), desc_add(vK, k * 32), idesc_s, k > 0);
                mma_commit(s_full);
            };
            if (n_it > 0) load_q(0);
            if (n_it > 1) load_q(1);
            ok = mbar_wait(kv_full, 0, abort_flag);
            if (ok && n_it > 0) {
                ok = mbar_wait(&q_full[0], 0, abort_flag);
                if (ok) { tc_fence_after(); issue_s(0); }
            }
            for (int it = 0; it < n_it && ok; ++it) {
                const int st = it & 1;
                if (it + 1 < n_it) {
                    // The next block's S and dP are issued as soon as this block's have been read out of TMEM (the
                    // gradient warps signal that right after their loads), so they are computed while the warps
                    // do this block's arithmetic instead of after it.
                    if (!mbar_wait(s_free, it & 1, abort_flag)) { ok = false; break; }
                    if (!mbar_wait(&q_full[(it + 1) & 1], ((it + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    issue_s(it + 1);
                }
                if (!mbar_wait(p_ready, it & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint64_t pd = pMN0, sd = desc_add(sMN0, st * 2 * TILE_BYTES),
                               sk = desc_add(sK0, st * 2 * TILE_BYTES), qd = desc_add(qMN0, st * TILE_BYTES),
                               od = desc_add(oMN0, st * TILE_BYTES);
                const uint32_t acc = it > 0;
#pragma unroll
                for (int k = 0; k < BQ / 16; ++k)        // dV first: P is single-buffered and is released right after
                    mma_f16_ss(tmem_dV, desc_add(pd, k * 2048), desc_add(od, k * 2048), idesc_t, acc | (k > 0));
                mma_commit(p_free);
#pragma unroll
                for (int k = 0; k < BQ / 16; ++k)        // reduction over the 128 queries of this block
                    mma_f16_ss(tmem_dK, desc_add(sd, k * 2048), desc_add(qd, k * 2048), idesc_t, acc | (k > 0));
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k)       // reduction over the 128 keys of this CTA
                    mma_f16_ss(tmem_dQ, desc_add(sk, (k >> 2) * TILE_BYTES + (k & 3) * 32), desc_add(kMN, k * 2048),
                               idesc_q, k > 0);
                mma_commit(dq_full);
                mma_commit(&q_empty[st]);
                if (it + 2 < n_it) {
                    if (!mbar_wait(&q_empty[st], (it >> 1) & 1, abort_flag)) { ok = false; break; }
                    load_q(it + 2);
                }
            }
            if (!ok) for (int i = 0; i < 2000; ++i) __nanosleep(500);
        }
    } else if (warp == BWD_STORE_WARP) {
        // ---------------- dQ store issuer: moves each staged 128 x 64 fp32 tile into the global scratch.  Ordered form:
        // when it is this key block's turn -- a plain tile store if it is the first part, else a bulk reduce-add --
        // and the tile's counter is raised once the write has completed.  Key block 0 does not come through here.
        if (lane == 0 && !(ordered && kb == 0)) {
            for (int f = 0; f < n_it; ++f) {
                if (!mbar_wait(dqs_full, f & 1, abort_flag)) break;
                const int qi = qblock(f), q0 = qi * BQ;
                int* sem = ordered ? p.dq_sem + (long long)bh * nq + qi : nullptr;
                const int turn = ordered ? first_kb(qi) - kb : 1;
                if (ordered) {
                    bool mine = false;
                    for (uint32_t i = 0; i < (1u << 22); ++i) {
                        int v;
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(sem) : "memory");
                        if (v >= turn) { mine = true; break; }
                        if ((i & 255u) == 255u && *abort_flag) break;
                        __nanosleep(32);
                    }
                    if (!mine) { *abort_flag = 1; break; }
                }
                if (turn == 0) {
                    tma_store_3d(&tmdQ, sdQ, 0, q0, bh);
                    tma_store_3d(&tmdQ, sdQ + TILE_BYTES, 32, q0, bh);
                } else {
                    tma_reduce_add_3d(&tmdQ, sdQ, 0, q0, bh);
                    tma_reduce_add_3d(&tmdQ, sdQ + TILE_BYTES, 32, q0, bh);
                }
                tma_store_commit();
                tma_store_wait_read<0>();
                mbar_arrive(dqs_free);                  // the staging tile may be refilled
                if (ordered) {
                    tma_store_wait<0>();                // the tile is in global memory
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                    __threadfence();
                    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(sem), "r"(turn + 1) : "memory");
                } else if (finish_last) {
                    // count this part in once the adds have been performed; whoever brings the count to the number of
                    // key blocks that see the tile hands it to the finishing warp
                    tma_store_wait<0>();
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                    __threadfence();
                    int before;
                    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;"
                                 : "=r"(before) : "l"(p.dq_sem + (long long)bh * nq + qi) : "memory");
                    if (before + 1 == first_kb(qi) + 1) {
                        const int n = *fin_count;
                        fin_ring[n % FIN_RING] = qi;
                        __threadfence_block();
                        *fin_count = n + 1;
                    }
                }
            }
            tma_store_wait<0>();
            if (finish_last) { __threadfence_block(); *fin_count = -1 - *fin_count; }
        }
    } else if (warp == BWD_FINISH_WARP) {
        // ---------------- finishing warp (mode 2): every part of a handed-over tile is in the scratch; scale and cast the
        // sums to dQ, and leave zeros behind for the next launch.  A tile is 128 x 64 fp32 = 32 KB of contiguous scratch.
        if (finish_last && n_it > 0) {
            int taken = 0;
            bool ok = true;
            for (uint32_t spin = 0; ok;) {
                const int c = *fin_count;
                const int avail = c >= 0 ? c : -1 - c;
                if (taken == avail) {
                    if (c < 0) break;                                   // the store warp has ended and nothing is left
                    if ((++spin & 255u) == 0 && *abort_flag) break;
                    if (spin >= (1u << 24)) { *abort_flag = 1; break; }
                    __nanosleep(200);
                    continue;
                }
                spin = 0;
                __threadfence_block();
                const int qi = fin_ring[taken % FIN_RING];
                ++taken;
                __threadfence();
                asm volatile("fence.proxy.async.global;" ::: "memory");
                const int q0 = qi * BQ;
                const int rows_here = min(BQ, p.T - q0);
                float4* tile = reinterpret_cast<float4*>(p.dq_accum + ((long long)bh * p.T + q0) * HD);
                __nv_bfloat16* dst0 = p.dq + (long long)b * p.sb + (long long)h * p.sh + (long long)q0 * p.st;
                const int n4 = rows_here * (HD / 4);                    // float4 elements of the tile
#pragma unroll 1
                for (int base = 0; base < n4; base += 32 * 8) {
                    float4 v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int i = base + j * 32 + lane;
                        v[j] = i < n4 ? __ldcg(tile + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int i = base + j * 32 + lane;
                        if (i < n4) {
                            const int r = i / (HD / 4), c4 = i % (HD / 4);
                            __nv_bfloat162 lo = __floats2bfloat162_rn(v[j].x * p.scale, v[j].y * p.scale);
                            __nv_bfloat162 hi = __floats2bfloat162_rn(v[j].z * p.scale, v[j].w * p.scale);
                            uint2 out;
                            out.x = *reinterpret_cast<uint32_t*>(&lo);
                            out.y = *reinterpret_cast<uint32_t*>(&hi);
                            *reinterpret_cast<uint2*>(dst0 + (long long)r * p.st + c4 * 4) = out;
                            __stcg(tile + i, make_float4(0.f, 0.f, 0.f, 0.f));
                        }
                    }
                }
                if (lane == 0) p.dq_sem[(long long)bh * nq + qi] = 0;  // nobody else touches it before the next launch
            }
        }
    } else {
        // ---------------- gradient warps: 16 warps; warp w owns TMEM lanes 32*(w&3).. (query rows) and the
        // 32-column group (w>>2) of every S / dP tile, so each scheduler has four warps to hide latency with ----
        const int quarter = warp & 3, cg = warp >> 2;
        const int row = quarter * 32 + lane;            // TMEM lane: query row for S, dP, dQ; key row for dV, dK
        const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
        bool ok = true;
        // dQ of a finished query block: this warp's 16 columns go to the fp32 staging tile (swizzled for TMA); the
        // store warp then adds the tile into the global accumulator with one bulk reduce per 32-column half
        // `signal`: false leaves the proxy fence and the arrival on dqs_full to the caller, who then covers the P / dS
        // stores of the current block and this staging write with one fence
        const bool finisher = ordered && kb == 0;       // this CTA completes dQ of every query block it sees
        auto flush_dq = [&](int f, bool signal) -> bool {
            if (!mbar_wait(dq_full, f & 1, abort_flag)) return false;
            tc_fence_after();
            uint32_t t[16];
            tmem_ld16(tmem_dQ + lane_addr + cg * 16, t);
            tmem_wait_ld();
            if (finisher) {
                // every other key block's part of this query block is in the scratch tile (their counters say so):
                // add it to this thread's 16 columns, scale, cast, store dQ
                const int qi = qblock(f), need = first_kb(qi);
                const int qrow = qi * BQ + row;
                float v[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(t[i]);
                if (need > 0) {
                    if (!sem_wait_warp(p.dq_sem + (long long)bh * nq + qi, need, abort_flag)) return false;
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                    if (qrow < p.T) {
                        const float4* src = reinterpret_cast<const float4*>(p.dq_accum + ((long long)bh * p.T + qrow) * HD + cg * 16);
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const float4 a = __ldcg(src + g);
                            v[4 * g] += a.x; v[4 * g + 1] += a.y; v[4 * g + 2] += a.z; v[4 * g + 3] += a.w;
                        }
                    }
                }
                if (qrow < p.T) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] *= p.scale;
                    __nv_bfloat16* dst = p.dq + (long long)b * p.sb + (long long)h * p.sh + (long long)qrow * p.st + cg * 16;
                    *reinterpret_cast<uint4*>(dst) = pack8(v);
                    *reinterpret_cast<uint4*>(dst + 8) = pack8(v + 8);
                }
                return true;
            }
            if (f > 0 && !mbar_wait(dqs_free, (f - 1) & 1, abort_flag)) return false;
            uint8_t* atom = sdQ + (cg >> 1) * TILE_BYTES;
#pragma unroll
            for (int g = 0; g < 4; ++g)
                *reinterpret_cast<uint4*>(atom + swz(row, (cg & 1) * 4 + g)) =
                    make_uint4(t[4 * g], t[4 * g + 1], t[4 * g + 2], t[4 * g + 3]);
            if (signal) {
                fence_proxy_async();
                mbar_arrive(dqs_full);
            }
            return true;
        };
        // row statistics of a query block are fetched one block ahead: their global-memory latency must not sit
        // between the arrival of S and the first exponential
        auto row_stats = [&](int it2, float& l2, float& d2) {
            const int qc2 = min(qblock(it2) * BQ + row, p.T - 1);
            l2 = p.lse[(long long)bh * p.T + qc2] * LOG2E;
            d2 = p.delta[(long long)bh * p.T + qc2];
        };
        float lse2_n = 0.f, dl_n = 0.f;
        if (n_it > 0) row_stats(0, lse2_n, dl_n);
        for (int it = 0; it < n_it && ok; ++it) {
            const int qi0 = qblock(it) * BQ;
            const int q = qi0 + row;
            const float lse2 = lse2_n, dl = dl_n;
            if (it + 1 < n_it) row_stats(it + 1, lse2_n, dl_n);
            uint8_t* bufP = sP;
            uint8_t* bufS = sdS + (it & 1) * 2 * TILE_BYTES;
            if (!mbar_wait(s_full, it & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const bool need_mask = (qi0 + BQ > p.T) || (k0 + BKV > p.T) || (p.causal && qi0 < k0 + BKV);
            uint32_t rs[32], rd[32];
            tmem_ld32(tmem_S + lane_addr + cg * 32, rs);
            tmem_ld32(tmem_dP + lane_addr + cg * 32, rd);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(s_free);                        // S and dP may be overwritten by the next block's products
            if (it > 0 && !mbar_wait(p_free, (it - 1) & 1, abort_flag)) { ok = false; break; }
            // scale-and-shift, dP - delta and the product on packed pairs (one instruction per two keys)
            const F32x2 sc2 = f2_splat(p.scale_log2), nl2 = f2_splat(-lse2), nd2 = f2_splat(-dl);
            const int lim = (q < p.T ? min(p.T, p.causal ? q + 1 : p.T) : 0) - (k0 + cg * 32);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                float pr[8], ds[8];
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    float a0, a1;
                    f2_unpack(f2_fma(f2_pack(__uint_as_float(rs[g * 8 + i]), __uint_as_float(rs[g * 8 + i + 1])), sc2, nl2),
                              a0, a1);
                    float pv0 = ex2_approx(a0), pv1 = ex2_approx(a1);
                    if (need_mask) {        // this thread's keys [0, lim) of the 32 are visible to its row
                        pv0 = g * 8 + i < lim ? pv0 : 0.f;
                        pv1 = g * 8 + i + 1 < lim ? pv1 : 0.f;
                    }
                    pr[i] = pv0;
                    pr[i + 1] = pv1;
                    f2_unpack(f2_mul(f2_pack(pv0, pv1),
                                     f2_add(f2_pack(__uint_as_float(rd[g * 8 + i]), __uint_as_float(rd[g * 8 + i + 1])), nd2)),
                              ds[i], ds[i + 1]);
                }
                const uint32_t off = (cg >> 1) * TILE_BYTES + swz(row, (cg & 1) * 4 + g);
                *reinterpret_cast<uint4*>(bufP + off) = pack8(pr);
                *reinterpret_cast<uint4*>(bufS + off) = pack8(ds);
            }
            // the previous block's dQ is read here, after this block's arithmetic, so that its MMAs had the whole
            // time of that arithmetic to finish
            if (it > 0 && !flush_dq(it - 1, false)) { ok = false; break; }
            tc_fence_before();
            fence_proxy_async();                        // one fence for P, dS and the dQ staging tile
            if (it > 0 && !finisher) mbar_arrive(dqs_full);
            mbar_arrive(p_ready);
        }
        if (ok && n_it > 0) ok = flush_dq(n_it - 1, true);
        // dK, dV of this key block (all MMAs are complete: the last dq_full wait covered them); this warp stores its
        // 16 columns (32 bytes = one full sector per row) straight from registers
        if (ok) {
            const int key = k0 + row;
            const long long off = (long long)b * p.sb + (long long)h * p.sh + (long long)key * p.st + cg * 16;
            uint32_t t[16];
            float v[16];
            if (n_it > 0) { tmem_ld16(tmem_dV + lane_addr + cg * 16, t); tmem_wait_ld(); }
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = n_it > 0 ? __uint_as_float(t[i]) : 0.f;
            if (key < p.T) {
                *reinterpret_cast<uint4*>(p.dv + off) = pack8(v);
                *reinterpret_cast<uint4*>(p.dv + off + 8) = pack8(v + 8);
            }
            if (n_it > 0) { tmem_ld16(tmem_dK + lane_addr + cg * 16, t); tmem_wait_ld(); }
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = n_it > 0 ? __uint_as_float(t[i]) * p.scale : 0.f;
            if (key < p.T) {
                *reinterpret_cast<uint4*>(p.dk + off) = pack8(v);
                *reinterpret_cast<uint4*>(p.dk + off + 8) = pack8(v + 8);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    // every warp of the finishing CTA is past its waits and no other CTA touches these counters again: back to zero
    // for the next launch
    if (ordered && kb == 0 && (int)threadIdx.x < n_it) p.dq_sem[(long long)bh * nq + i_begin + threadIdx.x] = 0;
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, CME_ERR_TIMEOUT);
    if (warp == BWD_MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, BWD_TMEM_COLS); }
}

// dq[b, h, t, :] = scale * sum over key blocks of the partial dQ slices (bf16, strided destination).
// Causal: only key blocks at or before the query's block contributed (and were written).
__global__ void dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int T, int nh,
                                  long long sb, long long sh, long long st, float scale, long long rows, int nkb,
                                  int causal) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;      // one thread per 8 elements
    if (i >= rows * (HD / 8)) return;
    const long long r = i / (HD / 8);
    const int c = (int)(i % (HD / 8)) * 8;
    const int bh = (int)(r / T), t = (int)(r % T);
    const int last = causal ? min(nkb - 1, t / BKV) : nkb - 1;
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = 0.f;
    for (int kb = 0; kb <= last; ++kb) {
        const float* src = acc + ((long long)kb * rows + r) * HD + c;
        const float4 a = *reinterpret_cast<const float4*>(src);
        const float4 b2 = *reinterpret_cast<const float4*>(src + 4);
        f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
        f[4] += b2.x; f[5] += b2.y; f[6] += b2.z; f[7] += b2.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= scale;
    *reinterpret_cast<uint4*>(dq + (long long)(bh / nh) * sb + (long long)(bh % nh) * sh + (long long)t * st + c) = pack8(f);
}

// ------------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encoder() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// bf16 map over (d, t, h, b) with box (64, rows, 1, 1) and 128-byte swizzle.
int make_map4(CUtensorMap* out, const void* base, int T, int nh, int nb, long long st, long long sh, long long sb,
              int rows) {
    EncodeTiledFn enc = encoder();
    CME_REQUIRE(enc != nullptr, CME_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)T, (cuuint64_t)nh, (cuuint64_t)nb};
    cuuint64_t strides[3] = {(cuuint64_t)st * 2, (cuuint64_t)(nh > 1 ? sh : HD) * 2,
                             (cuuint64_t)(nb > 1 ? sb : (long long)T * st) * 2};
    cuuint32_t box[4] = {(cuuint32_t)HD, (cuuint32_t)rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    CME_REQUIRE(r == CUDA_SUCCESS, CME_ERR_CUDA, "attention: cuTensorMapEncodeTiled failed (%d) T=%d nh=%d nb=%d st=%lld",
                (int)r, T, nh, nb, st);
    return CME_OK;
}

// fp32 map over the dQ accumulator [nbh, T, 64]: box (32 columns = 128 bytes, 128 rows, 1), 128-byte swizzle.
int make_map_dq(CUtensorMap* out, const void* base, int T, int nbh) {
    EncodeTiledFn enc = encoder();
    CME_REQUIRE(enc != nullptr, CME_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)T, (cuuint64_t)nbh};
    cuuint64_t strides[2] = {(cuuint64_t)HD * 4, (cuuint64_t)T * HD * 4};
    cuuint32_t box[3] = {32, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    CME_REQUIRE(r == CUDA_SUCCESS, CME_ERR_CUDA, "attention: dQ tensor map failed (%d)", (int)r);
    return CME_OK;
}

}  // namespace

// Status word of the attention kernels on the current device (null if the device state cannot be set up).
int* cme_attn_status_ptr() {
    CmeDeviceState* ds;
    return cme_device_state(&ds) ? nullptr : ds->status + CME_STATUS_ATTENTION;
}

int attention_tc_supported(const CmeAttn* a) {
    if (a->dtype != CME_BF16 || a->HD != HD) return 0;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (!al16(a->q) || !al16(a->k) || !al16(a->v) || !al16(a->o)) return 0;
    if (a->st % 8 || a->ost % 8 || (a->nh > 1 && (a->sh % 8 || a->osh % 8)) || (a->nb > 1 && (a->sb % 8 || a->osb % 8)))
        return 0;
    return 1;
}

int attention_tc_fwd(const CmeAttn* a, cudaStream_t st) {
    CME_REQUIRE(attention_tc_supported(a), CME_ERR_SHAPE, "attention: shape not supported by the tensor-core kernel");
    CME_REQUIRE(a->lse != nullptr, CME_ERR_SHAPE, "attention: lse buffer is required");
    int* const g_attn_status = cme_attn_status_ptr();
    CME_REQUIRE(g_attn_status != nullptr, CME_ERR_CUDA, "attention: device state unavailable");
    CUtensorMap mq, mk, mv, mo;
    int rc;
    if ((rc = make_map4(&mq, a->q, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 128))) return rc;
    if ((rc = make_map4(&mk, a->k, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 128))) return rc;
    if ((rc = make_map4(&mv, a->v, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 128))) return rc;
    if ((rc = make_map4(&mo, a->o, a->T, a->nh, a->nb, a->ost, a->osh, a->osb, 32))) return rc;
    static bool attr[CME_MAX_DEVICES] = {};               // function attributes are per device
    int dev = 0;
    CME_CUDA(cudaGetDevice(&dev));
    if (!attr[dev % CME_MAX_DEVICES]) {
        CME_CUDA(cudaFuncSetAttribute(attn_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM));
        attr[dev % CME_MAX_DEVICES] = true;
    }
    FwdParams p{a->T, a->nh, a->causal, a->scale * LOG2E, a->lse, g_attn_status};
    dim3 grid(cme_cdiv(a->T, BQ), a->nb * a->nh);
    CME_CUDA(cme_launch_dependent(attn_fwd_tc_kernel, grid, dim3(FWD_THREADS), (size_t)FWD_SMEM, st, mq, mk, mv, mo, p));
    CME_LAUNCH_CHECK();
    return CME_OK;
}

int attention_delta_launch(const CmeAttn* a, cudaStream_t st);

int attention_tc_bwd(const CmeAttn* a, cudaStream_t st) {
    CME_REQUIRE(attention_tc_supported(a), CME_ERR_SHAPE, "attention: shape not supported by the tensor-core kernel");
    CME_REQUIRE(a->lse && a->delta && a->dq_accum && a->d_o && a->dq && a->dk && a->dv, CME_ERR_SHAPE,
                "attention backward: missing buffer");
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    CME_REQUIRE(al16(a->d_o) && al16(a->dq) && al16(a->dk) && al16(a->dv), CME_ERR_SHAPE,
                "attention backward: gradient buffers must be 16-byte aligned");
    int* const g_attn_status = cme_attn_status_ptr();
    CME_REQUIRE(g_attn_status != nullptr, CME_ERR_CUDA, "attention: device state unavailable");
    int rc;
    if ((rc = attention_delta_launch(a, st))) return rc;
    const long long rows = (long long)a->nb * a->nh * a->T;
    CUtensorMap mq, mk, mv, mdo, mdq;
    if ((rc = make_map4(&mq, a->q, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 128))) return rc;
    if ((rc = make_map4(&mk, a->k, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 128))) return rc;
    if ((rc = make_map4(&mv, a->v, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 128))) return rc;
    if ((rc = make_map4(&mdo, a->d_o, a->T, a->nh, a->nb, a->ost, a->osh, a->osb, 128))) return rc;
    if ((rc = make_map_dq(&mdq, a->dq_accum, a->T, a->nb * a->nh))) return rc;
    const int mode = a->dq_mode;
    CME_REQUIRE(mode >= 0 && mode <= 2 && (mode == 0 || a->dq_sem != nullptr), CME_ERR_SHAPE,
                "attention backward: dq_mode 1 and 2 need the counter array");
    CME_REQUIRE(mode != 2 || cme_cdiv(a->T, BQ) <= CME_ATTN_FINISH_MAX_QBLOCKS, CME_ERR_LIMIT,
                "attention backward: dq_mode 2 handles up to %d query blocks", CME_ATTN_FINISH_MAX_QBLOCKS);
    if (mode == 0 && !a->dq_accum_clean) CME_CUDA(cudaMemsetAsync(a->dq_accum, 0, (size_t)rows * HD * sizeof(float), st));
    static bool attr[CME_MAX_DEVICES] = {};               // function attributes are per device
    int dev = 0;
    CME_CUDA(cudaGetDevice(&dev));
    if (!attr[dev % CME_MAX_DEVICES]) {
        CME_CUDA(cudaFuncSetAttribute(attn_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM));
        attr[dev % CME_MAX_DEVICES] = true;
    }
    BwdParams p{a->T, a->nh, a->causal, a->scale, a->scale * LOG2E, a->lse, a->delta, a->dq_accum,
                (__nv_bfloat16*)a->dk, (__nv_bfloat16*)a->dv, a->sb, a->sh, a->st, g_attn_status, a->dq_sem,
                (__nv_bfloat16*)a->dq, mode};
    dim3 grid(cme_cdiv(a->T, BKV), a->nb * a->nh);
    attn_bwd_tc_kernel<<<grid, BWD_THREADS, BWD_SMEM, st>>>(mq, mk, mv, mdo, mdq, p);
    CME_LAUNCH_CHECK();
    if (mode != 0) return CME_OK;                  // dQ was completed inside the kernel
    const long long nthreads = rows * (HD / 8);
    CME_CUDA(cme_launch_dependent(dq_convert_kernel, dim3(cme_cdiv(nthreads, 256)), dim3(256), 0, st,
                                  (const float*)a->dq_accum, (__nv_bfloat16*)a->dq, a->T, a->nh, a->sb, a->sh, a->st,
                                  a->scale, rows, 1, 0));
    CME_LAUNCH_CHECK();
    return CME_OK;
}

// Reads and clears the attention status word (non-zero: a bounded wait ran out).
CME_API int cme_attention_check_status(int* host_out) {
    return cme_check_status_word(CME_STATUS_ATTENTION, host_out);
}
