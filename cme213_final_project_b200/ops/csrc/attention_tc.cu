// Fused flash-style attention on the 5th-generation tensor cores (head size 64, bf16, causal or not, both
// head layouts): scores and output partials live in TMEM, probabilities go to the second MMA through shared
// memory, nothing of size T x T reaches global memory, only the per-row log-sum-exp is saved for backward.
//
// Replaces the reference's production attention -- two strided-batched GEMMs around an in-place softmax
// with P, dP and dS materialised as [B*H, T, T] buffers, and four more batched GEMMs plus a dS kernel in
// backward (FINAL_CLEAN_CODE_/src/kernels/attention.cu:138-200, 253-328).
//
// Forward, per CTA = one (batch, head) and 128 queries; 4 softmax warps (thread = query row) + 1 warp whose
// lane 0 issues TMA loads and tcgen05.mma:
//     S = Q K_j^T (TMEM)  ->  online softmax in registers  ->  P_j (bf16, shared, swizzled K-major)
//     O_j = P_j V_j (TMEM, fresh each block)  ->  o = o * alpha + O_j in registers
// Backward, per CTA = one (batch, head) and 128 keys, looping over query blocks:
//     S^T = K Q_i^T,  dP^T = V dO_i^T (TMEM)  ->  P^T, dS^T (bf16, shared)
//     dV += P^T dO_i,  dK += dS^T Q_i (TMEM accumulators)  dQ_i = dS K (TMEM, added to fp32 global with
//     vector reductions; a small kernel scales and casts dQ at the end)
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
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

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
// shared: Q 16K | K[2] 32K | V[2] 32K | P 32K | barriers
constexpr int FWD_SMEM = 7 * TILE_BYTES + 128;      // two CTAs per SM must fit: 2 x (this + 1 KB reserved) <= 228 KB
constexpr int FWD_THREADS = 160;
constexpr int FWD_TMEM_COLS = 256;         // S: [0,128)  O partial: [128,192)

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
    uint8_t* sK = sQ + TILE_BYTES;            // 2 stages
    uint8_t* sV = sK + 2 * TILE_BYTES;        // 2 stages
    uint8_t* sP = sV + 2 * TILE_BYTES;        // 2 atoms of 64 keys (also the output staging area)
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * TILE_BYTES);
    uint64_t* q_full = bars;                  // 1
    uint64_t* kv_full = bars + 1;             // [2]
    uint64_t* kv_empty = bars + 3;            // [2]
    uint64_t* s_full = bars + 5;              // S ready for softmax
    uint64_t* p_ready = bars + 6;             // P written (128 arrivals), S consumed
    uint64_t* o_full = bars + 7;              // O partial ready, P consumed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = gridDim.x - 1 - blockIdx.x;               // heavy (late) causal tiles first
    const int q0 = qt * BQ;
    const int bh = blockIdx.y, b = bh / p.nh, h = bh % p.nh;
    const int nkv = p.causal ? min((q0 + BQ + BKV - 1) / BKV, (p.T + BKV - 1) / BKV) : (p.T + BKV - 1) / BKV;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
        mbar_init(s_full, 1);
        mbar_init(p_ready, 128);
        mbar_init(o_full, 1);
        fence_barrier_init();
    }
    if (warp == 4) { tmem_alloc(tmem_slot, FWD_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 128;

    if (warp == 4) {
        if (lane == 0) {
            // ---------------- producer + MMA issuer (one thread) ----------------
            constexpr uint32_t idesc_s = make_idesc(1, false, false, 128, 128);   // Q K^T: both K-major
            constexpr uint32_t idesc_o = make_idesc(1, false, true, 128, HD);     // P V: V is MN-major
            bool ok = true;
            mbar_arrive_expect_tx(q_full, TILE_BYTES);
            tma_load_4d(sQ, &tmQ, q_full, 0, q0, h, b);
            auto load_kv = [&](int j) {
                const int st = j & 1;
                mbar_arrive_expect_tx(&kv_full[st], 2 * TILE_BYTES);
                tma_load_4d(sK + st * TILE_BYTES, &tmK, &kv_full[st], 0, j * BKV, h, b);
                tma_load_4d(sV + st * TILE_BYTES, &tmV, &kv_full[st], 0, j * BKV, h, b);
            };
            auto issue_s = [&](int j) {
                const uint32_t a = smem_u32(sQ), bb = smem_u32(sK + (j & 1) * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mma_f16_ss(tmem_S, make_smem_desc(a + k * 32, 0, 1024), make_smem_desc(bb + k * 32, 0, 1024),
                               idesc_s, k > 0);
                mma_commit(s_full);
            };
            load_kv(0);
            if (nkv > 1) load_kv(1);
            ok = mbar_wait(q_full, 0, abort_flag) && mbar_wait(&kv_full[0], 0, abort_flag);
            if (ok) { tc_fence_after(); issue_s(0); }
            for (int j = 0; j < nkv && ok; ++j) {
                const int st = j & 1;
                // P_j written and S_j consumed
                if (!mbar_wait(p_ready, j & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t pa = smem_u32(sP), vb = smem_u32(sV + st * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k)
                    mma_f16_ss(tmem_O, make_smem_desc(pa + (k >> 2) * TILE_BYTES + (k & 3) * 32, 0, 1024),
                               make_smem_desc(vb + k * 2048, TILE_BYTES, 1024), idesc_o, k > 0);
                mma_commit(o_full);
                mma_commit(&kv_empty[st]);
                if (j + 1 < nkv) {
                    if (!mbar_wait(&kv_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    issue_s(j + 1);
                }
                if (j + 2 < nkv) {
                    if (!mbar_wait(&kv_empty[st], (j >> 1) & 1, abort_flag)) { ok = false; break; }
                    load_kv(j + 2);
                }
            }
            if (!ok) for (int i = 0; i < 2000; ++i) __nanosleep(500);
        }
    } else {
        // ---------------- softmax warps: thread = query row ----------------
        const int row = warp * 32 + lane;                 // 0..127 == TMEM lane
        const int q = q0 + row;
        const uint32_t lane_addr = uint32_t(warp * 32) << 16;
        float m = -INFINITY, l = 0.f, o[HD];
#pragma unroll
        for (int i = 0; i < HD; ++i) o[i] = 0.f;
        bool ok = true;
        for (int j = 0; j < nkv && ok; ++j) {
            if (!mbar_wait(s_full, j & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int k0 = j * BKV;
            const bool need_mask = (k0 + BKV > p.T) || (p.causal && k0 + BKV - 1 > q0);
            // pass 1: row maximum
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_S + lane_addr + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float s = __uint_as_float(r[i]) * p.scale_log2;
                    if (need_mask) {
                        const int key = k0 + c * 32 + i;
                        if (key >= p.T || (p.causal && key > q)) s = -INFINITY;
                    }
                    mx = fmaxf(mx, s);
                }
            }
            const float m_new = fmaxf(m, mx);
            const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            // the previous block's P V product must be finished before P is overwritten; fold it in
            if (j > 0) {
                if (!mbar_wait(o_full, (j - 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_O + lane_addr + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(r[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < HD; ++i) o[i] *= alpha;
            // pass 2: probabilities -> shared (bf16), row sum
            float sum = 0.f;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_S + lane_addr + c * 32, r);
                tmem_wait_ld();
                float pr[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float s = __uint_as_float(r[i]) * p.scale_log2;
                    if (need_mask) {
                        const int key = k0 + c * 32 + i;
                        if (key >= p.T || (p.causal && key > q)) s = -INFINITY;
                    }
                    pr[i] = exp2f(s - m_use);
                    sum += pr[i];
                }
                uint8_t* atom = sP + (c >> 1) * TILE_BYTES;
#pragma unroll
                for (int g = 0; g < 4; ++g)
                    *reinterpret_cast<uint4*>(atom + swz(row, (c & 1) * 4 + g)) = pack8(pr + g * 8);
            }
            l = l * alpha + sum;
            m = m_new;
            tc_fence_before();
            fence_proxy_async();
            mbar_arrive(p_ready);
        }
        // last block's product
        if (ok && nkv > 0) {
            if (mbar_wait(o_full, (nkv - 1) & 1, abort_flag)) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_O + lane_addr + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(r[i]);
                }
                const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
                for (int i = 0; i < HD; ++i) o[i] *= inv;
                // stage this warp's 32 rows (P is free now) and store them with one TMA tile store
                uint8_t* stage = sP + warp * 4096;
#pragma unroll
                for (int g = 0; g < 8; ++g) *reinterpret_cast<uint4*>(stage + swz(lane, g)) = pack8(o + g * 8);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    tma_store_4d(&tmO, stage, 0, q0 + warp * 32, h, b);
                    tma_store_commit();
                    tma_store_wait<0>();
                }
                if (q < p.T) p.lse[(long long)bh * p.T + q] = (m == -INFINITY) ? -INFINITY : (m + log2f(l)) / LOG2E;
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
    float* dq_accum;               // fp32 [nb*nh, T, HD], zeroed by the launcher
    int* status;
};

// shared: K 16K | V 16K | Q[2] 32K | dO[2] 32K | P^T 32K | dS^T 32K | barriers
constexpr int BWD_SMEM = 10 * TILE_BYTES + 128;
constexpr int BWD_THREADS = 160;
constexpr int BWD_TMEM_COLS = 512;     // S^T [0,128) dP^T [128,256) dV [256,320) dK [320,384) dQ [384,448)

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                   const BwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, CME_ERR_SHAPE);
        return;
    }
    uint8_t* sK = smem;
    uint8_t* sV = sK + TILE_BYTES;
    uint8_t* sQ = sV + TILE_BYTES;             // 2 stages
    uint8_t* sdO = sQ + 2 * TILE_BYTES;        // 2 stages
    uint8_t* sPt = sdO + 2 * TILE_BYTES;       // [2 query atoms][128 key rows][128 B]
    uint8_t* sdSt = sPt + 2 * TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sdSt + 2 * TILE_BYTES);
    uint64_t* kv_full = bars;
    uint64_t* q_full = bars + 1;               // [2]
    uint64_t* q_empty = bars + 3;              // [2]
    uint64_t* s_full = bars + 5;
    uint64_t* p_ready = bars + 6;              // 128 arrivals
    uint64_t* dq_full = bars + 7;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb = blockIdx.x, k0 = kb * BKV;
    const int bh = blockIdx.y, b = bh / p.nh, h = bh % p.nh;
    const int nq = (p.T + BQ - 1) / BQ;
    const int i_begin = p.causal ? kb : 0;     // query blocks that see this key block
    const int n_it = nq - i_begin;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(kv_full, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
        mbar_init(s_full, 1);
        mbar_init(p_ready, 128);
        mbar_init(dq_full, 1);
        fence_barrier_init();
    }
    if (warp == 4) { tmem_alloc(tmem_slot, BWD_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_St = tmem_base, tmem_dPt = tmem_base + 128, tmem_dV = tmem_base + 256,
                   tmem_dK = tmem_base + 320, tmem_dQ = tmem_base + 384;

    if (warp == 4) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(1, false, false, 128, 128);    // K Q^T, V dO^T
            constexpr uint32_t idesc_kv = make_idesc(1, false, true, 128, HD);     // P^T dO, dS^T Q
            constexpr uint32_t idesc_dq = make_idesc(1, true, true, 128, HD);      // dS K (A read transposed)
            bool ok = true;
            mbar_arrive_expect_tx(kv_full, 2 * TILE_BYTES);
            tma_load_4d(sK, &tmK, kv_full, 0, k0, h, b);
            tma_load_4d(sV, &tmV, kv_full, 0, k0, h, b);
            auto load_q = [&](int it) {
                const int st = it & 1;
                mbar_arrive_expect_tx(&q_full[st], 2 * TILE_BYTES);
                tma_load_4d(sQ + st * TILE_BYTES, &tmQ, &q_full[st], 0, (i_begin + it) * BQ, h, b);
                tma_load_4d(sdO + st * TILE_BYTES, &tmdO, &q_full[st], 0, (i_begin + it) * BQ, h, b);
            };
            auto issue_s = [&](int it) {
                const int st = it & 1;
                const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
                const uint32_t qb = smem_u32(sQ + st * TILE_BYTES), ob = smem_u32(sdO + st * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mma_f16_ss(tmem_St, make_smem_desc(ka + k * 32, 0, 1024), make_smem_desc(qb + k * 32, 0, 1024),
                               idesc_s, k > 0);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    mma_f16_ss(tmem_dPt, make_smem_desc(va + k * 32, 0, 1024), make_smem_desc(ob + k * 32, 0, 1024),
                               idesc_s, k > 0);
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
                if (!mbar_wait(p_ready, it & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t pt = smem_u32(sPt), dst = smem_u32(sdSt), ka = smem_u32(sK);
                const uint32_t qb = smem_u32(sQ + st * TILE_BYTES), ob = smem_u32(sdO + st * TILE_BYTES);
#pragma unroll
                for (int k = 0; k < BQ / 16; ++k) {     // reduction over the 128 queries of this block
                    const uint32_t a_off = (k >> 2) * TILE_BYTES + (k & 3) * 32;
                    mma_f16_ss(tmem_dV, make_smem_desc(pt + a_off, 0, 1024),
                               make_smem_desc(ob + k * 2048, TILE_BYTES, 1024), idesc_kv, (it > 0 || k > 0));
                    mma_f16_ss(tmem_dK, make_smem_desc(dst + a_off, 0, 1024),
                               make_smem_desc(qb + k * 2048, TILE_BYTES, 1024), idesc_kv, (it > 0 || k > 0));
                }
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k)      // reduction over the 128 keys of this CTA
                    mma_f16_ss(tmem_dQ, make_smem_desc(dst + k * 2048, TILE_BYTES, 1024),
                               make_smem_desc(ka + k * 2048, TILE_BYTES, 1024), idesc_dq, k > 0);
                mma_commit(dq_full);
                mma_commit(&q_empty[st]);
                if (it + 1 < n_it) {
                    if (!mbar_wait(&q_full[(it + 1) & 1], ((it + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    issue_s(it + 1);
                }
                if (it + 2 < n_it) {
                    if (!mbar_wait(&q_empty[st], (it >> 1) & 1, abort_flag)) { ok = false; break; }
                    load_q(it + 2);
                }
            }
            if (!ok) for (int i = 0; i < 2000; ++i) __nanosleep(500);
        }
    } else {
        const int row = warp * 32 + lane;               // key row for S^T / dP^T, query row for dQ
        const int key = k0 + row;
        const uint32_t lane_addr = uint32_t(warp * 32) << 16;
        bool ok = true;
        for (int it = 0; it < n_it && ok; ++it) {
            const int qi0 = (i_begin + it) * BQ;
            // per-query statistics are read straight from global memory: every lane of a warp asks for the
            // same address, so each read is one broadcast transaction (no block-wide barrier to get stuck in)
            const float* lse_row = p.lse + (long long)bh * p.T;
            const float* dl_row = p.delta + (long long)bh * p.T;
            if (!mbar_wait(s_full, it & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const bool need_mask = (qi0 + BQ > p.T) || (k0 + BKV > p.T) || (p.causal && qi0 < k0 + BKV);
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t rs[32], rd[32];
                tmem_ld32(tmem_St + lane_addr + c * 32, rs);
                tmem_ld32(tmem_dPt + lane_addr + c * 32, rd);
                tmem_wait_ld();
                float pr[32], ds[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int qq = c * 32 + i;
                    const int qc = min(qi0 + qq, p.T - 1);
                    float pv = exp2f(__uint_as_float(rs[i]) * p.scale_log2 - __ldg(lse_row + qc) * LOG2E);
                    if (need_mask) {
                        const int q = qi0 + qq;
                        if (q >= p.T || key >= p.T || (p.causal && key > q)) pv = 0.f;
                    }
                    pr[i] = pv;
                    ds[i] = pv * (__uint_as_float(rd[i]) - __ldg(dl_row + qc));
                }
                const uint32_t atom = (c >> 1) * TILE_BYTES;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint32_t off = atom + swz(row, (c & 1) * 4 + g);
                    *reinterpret_cast<uint4*>(sPt + off) = pack8(pr + g * 8);
                    *reinterpret_cast<uint4*>(sdSt + off) = pack8(ds + g * 8);
                }
            }
            tc_fence_before();
            fence_proxy_async();
            mbar_arrive(p_ready);
            // dQ partial of this query block: add into the fp32 accumulator
            if (!mbar_wait(dq_full, it & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            {
                const int q = qi0 + row;
                float* dst = p.dq_accum + ((long long)bh * p.T + q) * HD;
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_dQ + lane_addr + c * 32, r);
                    tmem_wait_ld();
                    if (q < p.T) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            red_add_v4(dst + c * 32 + i, __uint_as_float(r[i]), __uint_as_float(r[i + 1]),
                                       __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                    }
                }
            }
            tc_fence_before();
        }
        // dK, dV of this key block (all MMAs are complete: the last dq_full wait covered them)
        if (ok) {
            float v[HD];
            uint8_t* stage = sPt + warp * 8192;           // P^T / dS^T are free now
            if (n_it > 0) {
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_dV + lane_addr + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[c * 32 + i] = __uint_as_float(r[i]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < HD; ++i) v[i] = 0.f;
            }
#pragma unroll
            for (int g = 0; g < 8; ++g) *reinterpret_cast<uint4*>(stage + swz(lane, g)) = pack8(v + g * 8);
            if (n_it > 0) {
#pragma unroll
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_dK + lane_addr + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[c * 32 + i] = __uint_as_float(r[i]) * p.scale;
                }
            }
#pragma unroll
            for (int g = 0; g < 8; ++g) *reinterpret_cast<uint4*>(stage + 4096 + swz(lane, g)) = pack8(v + g * 8);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_4d(&tmdV, stage, 0, k0 + warp * 32, h, b);
                tma_store_4d(&tmdK, stage + 4096, 0, k0 + warp * 32, h, b);
                tma_store_commit();
                tma_store_wait<0>();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, CME_ERR_TIMEOUT);
    if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem_base, BWD_TMEM_COLS); }
}

// dq[b, h, t, :] = dq_accum[bh, t, :] * scale  (bf16, strided destination)
__global__ void dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int T, int nh,
                                  long long sb, long long sh, long long st, float scale, long long rows) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;      // one thread per 8 elements
    if (i >= rows * (HD / 8)) return;
    const long long r = i / (HD / 8);
    const int c = (int)(i % (HD / 8)) * 8;
    const int bh = (int)(r / T), t = (int)(r % T);
    float f[8];
    const float4 a = *reinterpret_cast<const float4*>(acc + r * HD + c);
    const float4 b2 = *reinterpret_cast<const float4*>(acc + r * HD + c + 4);
    f[0] = a.x * scale; f[1] = a.y * scale; f[2] = a.z * scale; f[3] = a.w * scale;
    f[4] = b2.x * scale; f[5] = b2.y * scale; f[6] = b2.z * scale; f[7] = b2.w * scale;
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

int* g_attn_status = nullptr;

}  // namespace

int* cme_attn_status_ptr() { return g_attn_status; }

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
    if (!g_attn_status) {
        CME_CUDA(cudaMalloc(&g_attn_status, sizeof(int)));
        CME_CUDA(cudaMemset(g_attn_status, 0, sizeof(int)));
    }
    CUtensorMap mq, mk, mv, mo;
    int rc;
    if ((rc = make_map4(&mq, a->q, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 128))) return rc;
    if ((rc = make_map4(&mk, a->k, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 128))) return rc;
    if ((rc = make_map4(&mv, a->v, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 128))) return rc;
    if ((rc = make_map4(&mo, a->o, a->T, a->nh, a->nb, a->ost, a->osh, a->osb, 32))) return rc;
    static bool attr = false;
    if (!attr) {
        CME_CUDA(cudaFuncSetAttribute(attn_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM));
        attr = true;
    }
    FwdParams p{a->T, a->nh, a->causal, a->scale * LOG2E, a->lse, g_attn_status};
    dim3 grid(cme_cdiv(a->T, BQ), a->nb * a->nh);
    attn_fwd_tc_kernel<<<grid, FWD_THREADS, FWD_SMEM, st>>>(mq, mk, mv, mo, p);
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
    if (!g_attn_status) {
        CME_CUDA(cudaMalloc(&g_attn_status, sizeof(int)));
        CME_CUDA(cudaMemset(g_attn_status, 0, sizeof(int)));
    }
    int rc;
    if ((rc = attention_delta_launch(a, st))) return rc;
    const long long rows = (long long)a->nb * a->nh * a->T;
    CME_CUDA(cudaMemsetAsync(a->dq_accum, 0, (size_t)rows * HD * sizeof(float), st));
    CUtensorMap mq, mk, mv, mdo, mdk, mdv;
    if ((rc = make_map4(&mq, a->q, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 128))) return rc;
    if ((rc = make_map4(&mk, a->k, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 128))) return rc;
    if ((rc = make_map4(&mv, a->v, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 128))) return rc;
    if ((rc = make_map4(&mdo, a->d_o, a->T, a->nh, a->nb, a->ost, a->osh, a->osb, 128))) return rc;
    if ((rc = make_map4(&mdk, a->dk, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 32))) return rc;
    if ((rc = make_map4(&mdv, a->dv, a->T, a->nh, a->nb, a->st, a->sh, a->sb, 32))) return rc;
    static bool attr = false;
    if (!attr) {
        CME_CUDA(cudaFuncSetAttribute(attn_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM));
        attr = true;
    }
    BwdParams p{a->T, a->nh, a->causal, a->scale, a->scale * LOG2E, a->lse, a->delta, a->dq_accum, g_attn_status};
    dim3 grid(cme_cdiv(a->T, BKV), a->nb * a->nh);
    attn_bwd_tc_kernel<<<grid, BWD_THREADS, BWD_SMEM, st>>>(mq, mk, mv, mdo, mdk, mdv, p);
    CME_LAUNCH_CHECK();
    const long long nthreads = rows * (HD / 8);
    dq_convert_kernel<<<cme_cdiv(nthreads, 256), 256, 0, st>>>(a->dq_accum, (__nv_bfloat16*)a->dq, a->T, a->nh, a->sb,
                                                              a->sh, a->st, a->scale, rows);
    CME_LAUNCH_CHECK();
    return CME_OK;
}

// Reads and clears the attention status word (non-zero: a bounded wait ran out).
CME_API int cme_attention_check_status(int* host_out) {
    *host_out = 0;
    if (!g_attn_status) return CME_OK;
    CME_CUDA(cudaMemcpy(host_out, g_attn_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*host_out) CME_CUDA(cudaMemset(g_attn_status, 0, sizeof(int)));
    return CME_OK;
}
