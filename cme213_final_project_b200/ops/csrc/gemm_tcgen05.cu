// bf16 GEMM on the 5th-generation tensor cores: TMA-fed, mbarrier-pipelined, accumulators in TMEM,
// persistent over output tiles with a double-buffered accumulator so the epilogue of tile i overlaps the
// main loop of tile i+1.
//
// Replaces every GEMM variant of the reference (FINAL_CLEAN_CODE_/src/kernels/gemm.cu:483-1998: NN / TN /
// NT, accumulate twins, atomic split-K, strided-batched) and the cuBLAS / cuBLASLt wrappers (:111-481).
// The reference's split-K adds partial sums with atomicAdd into a zeroed C (:1028-1144); here split-K
// writes fp32 partials to a workspace and a second kernel sums them in a fixed order, so weight
// gradients are bit-reproducible.
//
// Structure per CTA (192 threads, 1 CTA per SM):
//   warp 0      one lane issues TMA tile loads into a ring of shared-memory stages
//   warp 1      allocates TMEM; one lane issues tcgen05.mma (128 x BN x 16 per instruction)
//   warps 2..5  epilogue: tcgen05.ld of their 32-lane quarter of the accumulator, fused epilogue, stores
// Operands may be K-major or MN-major in global memory; MN-major tiles are fetched as 64-wide column
// groups so that shared memory holds the canonical 128-byte-swizzled layout either way.
// Every mbarrier wait is bounded: on expiry the CTA sets the abort flag, leaves its loops, reports
// through the status word, frees its TMEM and returns.
#include "gemm.h"
#include "sm100_ptx.cuh"

#include <cuda.h>
#include <dlfcn.h>
#include <mutex>

using namespace sm100;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BM * BK * 2;
constexpr int NUM_THREADS = 192;

template <int BN> struct Cfg {
    static constexpr int B_TILE_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128) ? 6 : 8;
    static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
    static constexpr int STAGING_BYTES = 4 * 2 * 4096;     // per epilogue warp: two 32-row x 128-byte buffers
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

struct EpiParams {
    int M, N, K, batch;
    int tiles_m, tiles_n, splits, kb_per_split, num_kb;
    int a_batched, b_batched;
    void* C; long long ldc, strideC; int c_f32;
    const __nv_bfloat16* bias;
    const void* residual; long long ldres;
    void* aux_out; const void* aux_in; long long ldaux;
    int act, dact, accumulate;
    int tma_store;                 // outputs go through shared memory and TMA tile stores
    int* status;
};

__device__ __forceinline__ void epilogue_chunk(const EpiParams& p, float* acc, long long row_off_c,
                                               long long row_off_res, long long row_off_aux, int n, int ncols,
                                               bool vec_ok) {
    // acc: 32 fp32 values of one output row, columns [n, n+32); ncols = how many are inside N.
    if (p.bias) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < ncols) acc[j] += __bfloat162float(p.bias[n + j]);
    }
    const bool full = vec_ok && ncols == 32;
    if (p.c_f32) {
        float* C = reinterpret_cast<float*>(p.C) + row_off_c + n;
        if (p.accumulate) {
            if (full) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    float4 o = *reinterpret_cast<const float4*>(C + j);
                    acc[j] += o.x; acc[j + 1] += o.y; acc[j + 2] += o.z; acc[j + 3] += o.w;
                }
            } else {
                _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) acc[j] += C[j];
            }
        }
        if (full) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(C + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        } else {
            _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) C[j] = acc[j];
        }
        return;
    }
    __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C) + row_off_c + n;
    if (p.aux_out) {
        __nv_bfloat16* X = reinterpret_cast<__nv_bfloat16*>(p.aux_out) + row_off_aux + n;
        if (full) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) *reinterpret_cast<Bf16x8*>(X + j) = pack8(acc + j);
        } else {
            _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) X[j] = __float2bfloat16_rn(acc[j]);
        }
    }
    if (p.act == CME_ACT_RELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = fmaxf(acc[j], 0.f);
    } else if (p.act == CME_ACT_GELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = gelu_fast(acc[j]);
    }
    if (p.dact) {
        const __nv_bfloat16* X = reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + row_off_aux + n;
        float x[32];
        if (full) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) unpack8(*reinterpret_cast<const Bf16x8*>(X + j), x + j);
        } else {
            _Pragma("unroll") for (int j = 0; j < 32; ++j) x[j] = (j < ncols) ? __bfloat162float(X[j]) : 0.f;
        }
        if (p.dact == CME_ACT_RELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = x[j] > 0.f ? acc[j] : 0.f;
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] *= dgelu_fast(x[j]);
        }
    }
    if (p.residual) {
        const __nv_bfloat16* R = reinterpret_cast<const __nv_bfloat16*>(p.residual) + row_off_res + n;
        if (full) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                float r[8];
                unpack8(*reinterpret_cast<const Bf16x8*>(R + j), r);
#pragma unroll
                for (int q = 0; q < 8; ++q) acc[j + q] += r[q];
            }
        } else {
            _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) acc[j] += __bfloat162float(R[j]);
        }
    }
    if (p.accumulate) {
        if (full) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                float r[8];
                unpack8(*reinterpret_cast<const Bf16x8*>(C + j), r);
#pragma unroll
                for (int q = 0; q < 8; ++q) acc[j + q] += r[q];
            }
        } else {
            _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) acc[j] += __bfloat162float(C[j]);
        }
    }
    if (full) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) *reinterpret_cast<Bf16x8*>(C + j) = pack8(acc + j);
    } else {
        _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) C[j] = __float2bfloat16_rn(acc[j]);
    }
}


// Guarded 8-wide bf16 row read: vector when the group is inside the matrix, scalar at the ragged edge.
__device__ __forceinline__ void load8_guard(const __nv_bfloat16* rowp, int n, int N, bool row_ok, float* f) {
    if (row_ok && n + 8 <= N) {
        unpack8(*reinterpret_cast<const Bf16x8*>(rowp + n), f);
    } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) f[q] = (row_ok && n + q < N) ? __bfloat162float(rowp[n + q]) : 0.f;
    }
}

// Fused epilogue arithmetic on 32 columns of one row (bf16 outputs).  `pre` receives the pre-activation.
// `in_raw` (when `in_ok`) holds the 32 bf16 of this row's primary input operand for these columns -- the activation
// input of the derivative (dact) or else the residual -- loaded one step ahead by the caller, so the global-memory
// latency of those row reads overlaps the previous step's arithmetic.
__device__ __forceinline__ void epilogue_math(const EpiParams& p, float* acc, float* pre, bool row_ok, long long offc,
                                              long long offr, long long offa, int n, const uint4* in_raw, bool in_ok) {
    if (p.bias) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float b[8];
            load8_guard(p.bias, n + g * 8, p.N, true, b);
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[g * 8 + q] += b[q];
        }
    }
    if (p.aux_out) {
#pragma unroll
        for (int j = 0; j < 32; ++j) pre[j] = acc[j];
    }
    if (p.act == CME_ACT_RELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = fmaxf(acc[j], 0.f);
    } else if (p.act == CME_ACT_GELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = gelu_fast(acc[j]);
    }
    if (p.dact) {
        const __nv_bfloat16* X = reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + offa;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float x[8];
            if (in_ok) unpack8(in_raw[g], x); else load8_guard(X, n + g * 8, p.N, row_ok, x);
#pragma unroll
            for (int q = 0; q < 8; ++q)
                acc[g * 8 + q] = (p.dact == CME_ACT_RELU) ? (x[q] > 0.f ? acc[g * 8 + q] : 0.f)
                                                          : acc[g * 8 + q] * dgelu_fast(x[q]);
        }
    }
    if (p.residual) {
        const __nv_bfloat16* R = reinterpret_cast<const __nv_bfloat16*>(p.residual) + offr;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float x[8];
            if (in_ok && !p.dact) unpack8(in_raw[g], x); else load8_guard(R, n + g * 8, p.N, row_ok, x);
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[g * 8 + q] += x[q];
        }
    }
    if (p.accumulate) {
        const __nv_bfloat16* Cp = reinterpret_cast<const __nv_bfloat16*>(p.C) + offc;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float x[8];
            load8_guard(Cp, n + g * 8, p.N, row_ok, x);
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[g * 8 + q] += x[q];
        }
    }
}

template <int BN, bool A_MN, bool B_MN, bool SIMPLE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmX, const EpiParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* staging = smem + C::STAGES * C::STAGE_BYTES;       // 1024-byte aligned
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + C::STAGING_BYTES);
    uint64_t* full_bar = bars;                       // [STAGES]  TMA -> MMA
    uint64_t* empty_bar = bars + C::STAGES;          // [STAGES]  MMA -> TMA
    uint64_t* tfull_bar = bars + 2 * C::STAGES;      // [2]       MMA -> epilogue
    uint64_t* tempty_bar = bars + 2 * C::STAGES + 2; // [2]       epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull_bar[b], 1);
            mbar_init(&tempty_bar[b], 128);
        }
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch: everything above (barrier init, TMEM allocation, descriptor prefetch) may run
    // while the previous kernel of the stream is still finishing; its results are only touched after this point.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int tiles_mn = p.tiles_m * p.tiles_n;
    const int total_tiles = tiles_mn * p.batch * p.splits;

    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int mn = tile % tiles_mn, rest = tile / tiles_mn;
                const int bidx = rest % p.batch, split = rest / p.batch;
                const int m0 = (mn % p.tiles_m) * BM, n0 = (mn / p.tiles_m) * BN;
                const int kb0 = split * p.kb_per_split;
                const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
                const int za = p.a_batched ? bidx : 0, zb = p.b_batched ? bidx : 0;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* sA = smem + stage * C::STAGE_BYTES;
                    uint8_t* sB = sA + A_TILE_BYTES;
                    mbar_arrive_expect_tx(&full_bar[stage], C::STAGE_BYTES);
                    if (!A_MN) {
                        tma_load_3d(sA, &tmA, &full_bar[stage], kb * BK, m0, za);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j)
                            tma_load_3d(sA + j * (64 * BK * 2), &tmA, &full_bar[stage], m0 + j * 64, kb * BK, za);
                    }
                    if (!B_MN) {
                        tma_load_3d(sB, &tmB, &full_bar[stage], kb * BK, n0, zb);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_3d(sB + j * (64 * BK * 2), &tmB, &full_bar[stage], n0 + j * 64, kb * BK, zb);
                    }
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // Give copies that are still in flight time to land before shared memory is released.
                for (int i = 0; i < 2000; ++i) __nanosleep(500);
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ---------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(1 /*bf16*/, A_MN, B_MN, BM, BN);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
                const int rest = tile / tiles_mn;
                const int split = rest / p.batch;
                const int kb0 = split * p.kb_per_split;
                const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
                const int buf = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!mbar_wait(&tempty_bar[buf], acc_phase ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sA = smem_u32(smem + stage * C::STAGE_BYTES);
                    const uint32_t sB = sA + A_TILE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // K-major: step 16 elements (32 bytes) inside the 128-byte row.
                        // MN-major: step 16 k-rows of 128 bytes; 64-wide groups are BK*128 bytes apart.
                        const uint64_t da = A_MN ? make_smem_desc(sA + k * UMMA_K * 128, BK * 128, 1024)
                                                 : make_smem_desc(sA + k * UMMA_K * 2, 0, 1024);
                        const uint64_t db = B_MN ? make_smem_desc(sB + k * UMMA_K * 128, BK * 128, 1024)
                                                 : make_smem_desc(sB + k * UMMA_K * 2, 0, 1024);
                        mma_f16_ss(tmem_d, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    mma_commit(&empty_bar[stage]);      // stage is free once these MMAs have read it
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) mma_commit(&tfull_bar[buf]);    // accumulator complete
            }
        }
    } else {
        // ------------------------------- epilogue -----------------------------------
        const int quarter = warp & 3;                   // TMEM lanes [32*quarter, 32*quarter+32)
        const bool vec_ok = (p.N % 8 == 0) && (p.ldc % 8 == 0) &&
                            (!p.residual || p.ldres % 8 == 0) && ((!p.aux_in && !p.aux_out) || p.ldaux % 8 == 0);
        int it = 0;
        uint32_t store_cnt = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
            const int mn = tile % tiles_mn, rest = tile / tiles_mn;
            const int bidx = rest % p.batch, split = rest / p.batch;
            const int m0 = (mn % p.tiles_m) * BM, n0 = (mn / p.tiles_m) * BN;
            const int buf = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            if (!mbar_wait(&tfull_bar[buf], acc_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const long long zoff = (long long)(split * p.batch + bidx);
            const long long offc = zoff * p.strideC + (long long)row * p.ldc;
            const long long offr = (long long)bidx * p.strideC + (long long)row * p.ldres;
            const long long offa = (long long)bidx * p.strideC + (long long)row * p.ldaux;
            // primary input operand of the epilogue (read per thread along its own row), prefetched in halves
            const __nv_bfloat16* in_row =
                p.c_f32 ? nullptr
                        : (p.dact ? reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + offa
                                  : (p.residual ? reinterpret_cast<const __nv_bfloat16*>(p.residual) + offr : nullptr));
            uint4 in_cur[4];
            bool cur_ok = false;
            auto load_in = [&](int nn, uint4* dst) {
                if (in_row && row < p.M && nn + 32 <= p.N) {
                    const uint4* src = reinterpret_cast<const uint4*>(in_row + nn);
#pragma unroll
                    for (int g = 0; g < 4; ++g) dst[g] = __ldg(src + g);
                }
            };
            const uint32_t tmem_row = tmem_base + (uint32_t(quarter * 32) << 16) + buf * BN;
            if constexpr (SIMPLE) {
                // Plain bf16 output (no fused arithmetic): the TMEM loads of chunk c+1 are in flight while chunk c is
                // converted and staged, and the accumulator is handed back to the MMA warp as soon as the last load
                // has landed in registers, before the stores are issued.
                uint32_t ra[64], rb[64];
                int nchunks = (p.N - n0 + 63) / 64;
                nchunks = nchunks < BN / 64 ? nchunks : BN / 64;
                tmem_ld32(tmem_row, ra);
                tmem_ld32(tmem_row + 32, ra + 32);
#pragma unroll
                for (int c2 = 0; c2 < BN / 64; ++c2) {
                    if (c2 < nchunks) {
                        uint32_t* cur = (c2 & 1) ? rb : ra;
                        uint32_t* nxt = (c2 & 1) ? ra : rb;
                        tmem_wait_ld();
                        if (c2 + 1 < nchunks) {
                            tmem_ld32(tmem_row + (c2 + 1) * 64, nxt);
                            tmem_ld32(tmem_row + (c2 + 1) * 64 + 32, nxt + 32);
                        } else {
                            tc_fence_before();
                            mbar_arrive(&tempty_bar[buf]);          // accumulator fully read
                        }
                        uint8_t* sb = staging + quarter * 8192 + (store_cnt & 1) * 4096;
                        if (lane == 0) tma_store_wait_read<1>();
                        __syncwarp();
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const uint4 v = make_uint4(
                                f2_to_bf2(__uint_as_float(cur[8 * q]), __uint_as_float(cur[8 * q + 1])),
                                f2_to_bf2(__uint_as_float(cur[8 * q + 2]), __uint_as_float(cur[8 * q + 3])),
                                f2_to_bf2(__uint_as_float(cur[8 * q + 4]), __uint_as_float(cur[8 * q + 5])),
                                f2_to_bf2(__uint_as_float(cur[8 * q + 6]), __uint_as_float(cur[8 * q + 7])));
                            *reinterpret_cast<uint4*>(sb + lane * 128 + ((q ^ (lane & 7)) * 16)) = v;
                        }
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_3d(&tmC, sb, n0 + c2 * 64, m0 + quarter * 32, (int)zoff);
                            tma_store_commit();
                        }
                        ++store_cnt;
                    }
                }
                continue;
            }
            if (!p.tma_store) {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_row + c * 32, r);
                    tmem_wait_ld();
                    const int n = n0 + c * 32;
                    if (row < p.M && n < p.N) {
                        float acc[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(r[j]);
                        epilogue_chunk(p, acc, offc, offr, offa, n, min(32, p.N - n), vec_ok);
                    }
                }
            } else if (p.c_f32) {
                // fp32 output (split-K partials, fp32 C): 32 columns = one 128-byte staging row per TMA store
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int n = n0 + c * 32;
                    if (n >= p.N) break;
                    uint32_t r[32];
                    tmem_ld32(tmem_row + c * 32, r);
                    tmem_wait_ld();
                    if (p.accumulate) {
                        const float* Cp = reinterpret_cast<const float*>(p.C) + offc;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (row < p.M && n + j < p.N) r[j] = __float_as_uint(__uint_as_float(r[j]) + Cp[n + j]);
                    }
                    uint8_t* sb = staging + quarter * 8192 + (store_cnt & 1) * 4096;
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<uint4*>(sb + lane * 128 + ((q ^ (lane & 7)) * 16)) =
                            make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_3d(&tmC, sb, n, m0 + quarter * 32, (int)zoff);
                        tma_store_commit();
                    }
                    ++store_cnt;
                }
            } else {
                // bf16 output: 64 columns = one 128-byte staging row per TMA store
                const bool row_ok = row < p.M;
#pragma unroll 1
                for (int c2 = 0; c2 < BN / 64; ++c2) {
                    const int n = n0 + c2 * 64;
                    if (n >= p.N) break;
                    if (c2 == 0) { load_in(n, in_cur); cur_ok = in_row && row_ok && n + 32 <= p.N; }
                    uint8_t* sbC = staging + quarter * 8192 + (store_cnt & 1) * 4096;
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
                    __nv_bfloat16* Xrow = p.aux_out ? reinterpret_cast<__nv_bfloat16*>(p.aux_out) + offa : nullptr;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t r[32];
                        tmem_ld32(tmem_row + c2 * 64 + h * 32, r);
                        tmem_wait_ld();
                        float acc[32], pre[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(r[j]);
                        // start the next half's input reads before this half's arithmetic
                        uint4 in_nxt[4];
                        const int nn = n + h * 32 + 32;
                        const bool nxt_ok = in_row && row_ok && nn + 32 <= p.N && nn < n0 + BN;
                        if (nxt_ok) load_in(nn, in_nxt);
                        epilogue_math(p, acc, pre, row_ok, offc, offr, offa, n + h * 32, in_cur, cur_ok);
#pragma unroll
                        for (int g = 0; g < 4; ++g) in_cur[g] = in_nxt[g];
                        cur_ok = nxt_ok;
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const int q = h * 4 + g;
                            *reinterpret_cast<uint4*>(sbC + lane * 128 + ((q ^ (lane & 7)) * 16)) = pack8(acc + g * 8);
                            // the pre-activation goes straight to global memory: 16 bytes per store, 64 contiguous
                            // bytes per thread and chunk (two full sectors), no second staging buffer to wait on
                            if (Xrow) {
                                const int col = n + h * 32 + g * 8;
                                if (row_ok && col + 8 <= p.N) {
                                    *reinterpret_cast<uint4*>(Xrow + col) = pack8(pre + g * 8);
                                } else if (row_ok) {
#pragma unroll
                                    for (int e2 = 0; e2 < 8; ++e2)
                                        if (col + e2 < p.N) Xrow[col + e2] = __float2bfloat16_rn(pre[g * 8 + e2]);
                                }
                            }
                        }
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_3d(&tmC, sbC, n, m0 + quarter * 32, (int)zoff);
                        tma_store_commit();
                    }
                    ++store_cnt;
                }
            }
            tc_fence_before();
            mbar_arrive(&tempty_bar[buf]);
        }
        if (p.tma_store && lane == 0) tma_store_wait<0>();   // stores complete before shared memory goes away
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, CME_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// Sums split-K partials in a fixed order and applies the accumulate flag:  C (+)= sum_s P[s].
__global__ void splitk_reduce_kernel(const float* __restrict__ P, int splits, long long per_split, void* Cout,
                                     int c_f32, int accumulate, int M, int N, long long ldc, long long strideC,
                                     int batch) {
    const long long total = (long long)batch * M * N;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < splits; ++k) s += P[k * per_split + i];
        const long long b = i / ((long long)M * N), rem = i % ((long long)M * N);
        const long long off = b * strideC + (rem / N) * ldc + (rem % N);
        if (c_f32) {
            float* C = reinterpret_cast<float*>(Cout);
            C[off] = accumulate ? C[off] + s : s;
        } else {
            __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(Cout);
            C[off] = __float2bfloat16_rn(accumulate ? __bfloat162float(C[off]) + s : s);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encoder() {
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

// 3-D tensor map: dims (inner, rows, batch), 128-byte swizzle, box (128 bytes of inner, box_rows, 1).
int make_tmap(CUtensorMap* out, const void* base, long long inner, long long rows, long long ld, long long batch,
              long long batch_stride, int box_rows, bool f32 = false) {
    EncodeTiledFn enc = get_encoder();
    CME_REQUIRE(enc != nullptr, CME_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const int es = f32 ? 4 : 2;
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)(batch > 0 ? batch : 1)};
    cuuint64_t strides[2] = {(cuuint64_t)ld * es, (cuuint64_t)(batch_stride > 0 ? batch_stride : ld * rows) * es};
    cuuint32_t box[3] = {(cuuint32_t)(128 / es), (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    CME_REQUIRE(r == CUDA_SUCCESS, CME_ERR_CUDA,
                "cuTensorMapEncodeTiled failed (%d): inner=%lld rows=%lld ld=%lld batch=%lld bstride=%lld box_rows=%d",
                (int)r, inner, rows, ld, batch, batch_stride, box_rows);
    return CME_OK;
}

int g_num_sms = 0;
int* g_status = nullptr;     // device status word shared by all launches on this device

template <int BN, bool A_MN, bool B_MN, bool SIMPLE>
int launch_cfg(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tx,
               const EpiParams& ep, int grid, cudaStream_t st) {
    auto kern = gemm_tc_kernel<BN, A_MN, B_MN, SIMPLE>;
    static bool attr_set = false;
    if (!attr_set) {
        CME_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::SMEM_BYTES));
        attr_set = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = Cfg<BN>::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CME_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, tx, ep));
    CME_LAUNCH_CHECK();
    return CME_OK;
}

template <int BN, bool SIMPLE>
int launch_bn(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
              const CUtensorMap& tx, const EpiParams& ep, int grid, cudaStream_t st) {
    if (!a_mn && !b_mn) return launch_cfg<BN, false, false, SIMPLE>(ta, tb, tc, tx, ep, grid, st);
    if (!a_mn && b_mn) return launch_cfg<BN, false, true, SIMPLE>(ta, tb, tc, tx, ep, grid, st);
    if (a_mn && !b_mn) return launch_cfg<BN, true, false, SIMPLE>(ta, tb, tc, tx, ep, grid, st);
    return launch_cfg<BN, true, true, SIMPLE>(ta, tb, tc, tx, ep, grid, st);
}

}  // namespace

CME_API int cme_gemm_status_word(int** out) {
    if (!g_status) {
        CME_CUDA(cudaMalloc(&g_status, sizeof(int)));
        CME_CUDA(cudaMemset(g_status, 0, sizeof(int)));
    }
    *out = g_status;
    return CME_OK;
}

int gemm_tcgen05_supported(const CmeGemm* g) {
    if (g->ab_dtype != CME_BF16) return 0;
    if (g->M <= 0 || g->N <= 0 || g->K <= 0 || g->batch <= 0) return 0;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (!al16(g->A) || !al16(g->B) || !al16(g->C)) return 0;
    if (g->lda % 8 || g->ldb % 8 || g->strideA % 8 || g->strideB % 8) return 0;
    // inner extents must make a legal map (>= one 16-byte unit) -- tiny shapes go to the SIMT kernel
    const long long innerA = g->a_trans ? g->M : g->K, innerB = g->b_trans ? g->K : g->N;
    if (innerA % 8 || innerB % 8) return 0;
    if (g->c_dtype == CME_F32 && (g->act || g->dact || g->residual || g->aux_out)) return 0;
    return 1;
}

int gemm_tcgen05_launch(const CmeGemm* g, cudaStream_t stream) {
    CME_REQUIRE(gemm_tcgen05_supported(g), CME_ERR_SHAPE, "gemm shape/alignment not supported by the tcgen05 kernel");
    if (!g_num_sms) {
        int dev = 0;
        CME_CUDA(cudaGetDevice(&dev));
        CME_CUDA(cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev));
    }
    if (!g_status) {
        int* dummy;
        int rc = cme_gemm_status_word(&dummy);
        if (rc) return rc;
    }
    const int tiles_m = cme_cdiv(g->M, BM);
    const int num_kb = cme_cdiv(g->K, BK);
    // Tile width and K splits: minimise  waves x k-blocks per unit x cost(bn)  (+ fixed per-tile and
    // per-split overheads).  cost(bn) per 16-deep MMA is max(tensor time bn/2, shared-memory read time
    // (128 + bn)/4) in clocks: 128 / 64 / 48 for bn = 256 / 128 / 64.
    const bool plain_epi = !g->bias && !g->residual && !g->aux_out && !g->act && !g->dact;
    int bn = g->force_bn, splits = g->force_splits;
    if (!bn || !splits) {
        double best = 1e30;
        int best_bn = 128, best_s = 1;
        const int bns[3] = {256, 128, 64};
        const double cost[3] = {128.0, 80.0, 64.0};     // narrower tiles re-read A more often than they compute
        for (int i = 0; i < 3; ++i) {
            if (g->force_bn && bns[i] != g->force_bn) continue;
            if (bns[i] > 64 && g->N <= bns[i] / 2) continue;            // tile mostly padding
            const long long t = (long long)tiles_m * cme_cdiv(g->N, bns[i]) * g->batch;
            for (int s = 1; s <= 16; ++s) {
                if (g->force_splits && s != g->force_splits) continue;
                if (s > 1 && (!plain_epi || !g->workspace || num_kb / s < 4 ||
                              (long long)s * g->batch * g->M * g->N * 4 > g->workspace_bytes)) break;
                const long long units = t * s;
                const double waves = (double)((units + g_num_sms - 1) / g_num_sms);
                const double kb = (double)cme_cdiv(num_kb, s);
                // 4 MMAs per k-block; epilogue / pipeline fill ~ 6 k-blocks of the widest tile per unit;
                // a split adds one fp32 write + read of the output per split
                double est = waves * ((kb + 2.0) * 4.0 * cost[i] + 6.0 * 4.0 * bns[i] / 2.0);
                if (s > 1) est += 6000.0 + (double)s * g->M * g->N * g->batch / g_num_sms / 16.0;   // + one more launch
                if (est < best) { best = est; best_bn = bns[i]; best_s = s; }
            }
        }
        if (!bn) bn = best_bn;
        if (!splits) splits = best_s;
    }
    CME_REQUIRE(bn == 64 || bn == 128 || bn == 256, CME_ERR_SHAPE, "tile width must be 64, 128 or 256");
    const int tiles_n = cme_cdiv(g->N, bn);
    const long long tiles = (long long)tiles_m * tiles_n * g->batch;
    if (splits > 1) {
        CME_REQUIRE(plain_epi, CME_ERR_SHAPE, "split-K supports only the plain / accumulate epilogue");
        CME_REQUIRE(g->workspace && (long long)splits * g->batch * g->M * g->N * 4 <= g->workspace_bytes,
                    CME_ERR_LIMIT, "split-K workspace too small");
    }
    int kb_per = cme_cdiv(num_kb, splits);
    splits = cme_cdiv(num_kb, kb_per);

    CUtensorMap ta, tb;
    int rc;
    // A: K-major -> map (K, M), box (64, 128); MN-major -> map (M, K), box (64, 64)
    if (!g->a_trans) rc = make_tmap(&ta, g->A, g->K, g->M, g->lda, g->strideA ? g->batch : 1, g->strideA, BM);
    else             rc = make_tmap(&ta, g->A, g->M, g->K, g->lda, g->strideA ? g->batch : 1, g->strideA, BK);
    if (rc) return rc;
    // B: stored [N, K] (b_trans) is K-major -> map (K, N), box (64, bn); stored [K, N] -> map (N, K), box (64, 64)
    if (g->b_trans) rc = make_tmap(&tb, g->B, g->K, g->N, g->ldb, g->strideB ? g->batch : 1, g->strideB, bn);
    else            rc = make_tmap(&tb, g->B, g->N, g->K, g->ldb, g->strideB ? g->batch : 1, g->strideB, BK);
    if (rc) return rc;

    EpiParams ep{};
    ep.M = g->M; ep.N = g->N; ep.K = g->K; ep.batch = g->batch;
    ep.tiles_m = tiles_m; ep.tiles_n = tiles_n; ep.splits = splits; ep.kb_per_split = kb_per; ep.num_kb = num_kb;
    ep.a_batched = g->strideA != 0 && g->batch > 1; ep.b_batched = g->strideB != 0 && g->batch > 1;
    ep.status = g_status;
    if (splits > 1) {
        ep.C = g->workspace; ep.ldc = g->N; ep.strideC = (long long)g->M * g->N; ep.c_f32 = 1;
    } else {
        ep.C = g->C; ep.ldc = g->ldc; ep.strideC = g->strideC; ep.c_f32 = g->c_dtype == CME_F32;
        ep.bias = reinterpret_cast<const __nv_bfloat16*>(g->bias);
        ep.residual = g->residual; ep.ldres = g->ldres;
        ep.aux_out = g->aux_out; ep.aux_in = g->aux_in; ep.ldaux = g->ldaux;
        ep.act = g->act; ep.dact = g->dact; ep.accumulate = g->accumulate;
    }
    // Outputs through shared-memory staging + TMA tile stores when rows are 16-byte addressable.
    CUtensorMap tc = ta, tx = ta;
    {
        const int es = ep.c_f32 ? 4 : 2;
        auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
        const long long nb = (long long)splits * g->batch;
        bool ok = al16(ep.C) && (ep.ldc * es) % 16 == 0 && (nb == 1 || (ep.strideC * es) % 16 == 0);
        if (ep.aux_out) ok = ok && al16(ep.aux_out) && (ep.ldaux * 2) % 16 == 0;
        if (ok) {
            rc = make_tmap(&tc, ep.C, g->N, g->M, ep.ldc, nb, nb > 1 ? ep.strideC : 0, 32, ep.c_f32 != 0);
            if (rc) return rc;
            if (ep.aux_out) {
                rc = make_tmap(&tx, ep.aux_out, g->N, g->M, ep.ldaux, g->batch, g->batch > 1 ? ep.strideC : 0, 32);
                if (rc) return rc;
            }
            ep.tma_store = 1;
        }
    }
    const long long total = tiles * splits;
    const int grid = (int)(total < g_num_sms ? total : g_num_sms);
    const bool a_mn = g->a_trans != 0, b_mn = g->b_trans == 0;
    const bool simple = ep.tma_store && !ep.c_f32 && !ep.bias && !ep.residual && !ep.aux_out && !ep.aux_in &&
                        !ep.act && !ep.dact && !ep.accumulate;
    if (simple) {
        if (bn == 256) rc = launch_bn<256, true>(a_mn, b_mn, ta, tb, tc, tx, ep, grid, stream);
        else if (bn == 128) rc = launch_bn<128, true>(a_mn, b_mn, ta, tb, tc, tx, ep, grid, stream);
        else rc = launch_bn<64, true>(a_mn, b_mn, ta, tb, tc, tx, ep, grid, stream);
    } else {
        if (bn == 256) rc = launch_bn<256, false>(a_mn, b_mn, ta, tb, tc, tx, ep, grid, stream);
        else if (bn == 128) rc = launch_bn<128, false>(a_mn, b_mn, ta, tb, tc, tx, ep, grid, stream);
        else rc = launch_bn<64, false>(a_mn, b_mn, ta, tb, tc, tx, ep, grid, stream);
    }
    if (rc) return rc;
    if (splits > 1) {
        const long long per = (long long)g->batch * g->M * g->N;
        const int blocks = (int)((per + 255) / 256 < 4096 ? (per + 255) / 256 : 4096);
        splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(g->workspace), splits, per,
                                                         g->C, g->c_dtype == CME_F32, g->accumulate, g->M, g->N,
                                                         g->ldc, g->strideC, g->batch);
        CME_LAUNCH_CHECK();
    }
    return CME_OK;
}

// Reads and clears the device status word (0 = every bounded wait completed).
CME_API int cme_gemm_check_status(int* host_out) {
    *host_out = 0;
    if (!g_status) return CME_OK;
    CME_CUDA(cudaMemcpy(host_out, g_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*host_out) CME_CUDA(cudaMemset(g_status, 0, sizeof(int)));
    return CME_OK;
}
