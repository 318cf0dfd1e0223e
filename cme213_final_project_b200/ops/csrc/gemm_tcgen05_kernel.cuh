// bf16 (and, for fp32 storage, tf32) GEMM on the 5th-generation tensor cores: TMA-fed, mbarrier-pipelined, accumulators in TMEM,
// persistent over output tiles with a double-buffered accumulator so the epilogue of tile i overlaps the
// main loop of tile i+1.
//
// Replaces every GEMM variant of the reference (FINAL_CLEAN_CODE_/src/kernels/gemm.cu:483-1998: NN / TN /
// NT, accumulate twins, atomic split-K, strided-batched) and the cuBLAS / cuBLASLt wrappers (:111-481).
// The reference's split-K adds partial sums with atomicAdd into a zeroed C (:1028-1144); here split-K
// writes fp32 partials to a workspace and a second kernel sums them in a fixed order, so weight
// gradients are bit-reproducible.
//
// Structure per CTA (192 threads -- 320 with eight epilogue warps for the arithmetic-heavy epilogues; 1 CTA per SM):
//   warp 0      one lane issues TMA tile loads into a ring of shared-memory stages
//   warp 1      allocates TMEM; one lane issues tcgen05.mma (128 x BN x 16 per instruction)
//   warps 2..5  epilogue: tcgen05.ld of their 32-lane quarter of the accumulator, fused epilogue, stores
//   (warps 6..9  a second epilogue set on the same four quarters, taking every other 64-column chunk)
// Operands may be K-major or MN-major in global memory; MN-major tiles are fetched as 64-wide column
// groups so that shared memory holds the canonical 128-byte-swizzled layout either way.
// Every mbarrier wait is bounded: on expiry the CTA sets the abort flag, leaves its loops, reports
// through the status word, frees its TMEM and returns.
//
// This header holds the kernel template and its launcher; the instantiations are spread over several translation
// units (gemm_tc_inst_*.cu) so that they compile in parallel, and gemm_tcgen05.cu plans and dispatches.
#pragma once
#include "gemm.h"
#include "sm100_ptx.cuh"

#include <cuda.h>

namespace gemm_tc {

using namespace sm100;


constexpr int BM = 128;
constexpr int BK_BYTES = 128;          // a k-block is one 128-byte swizzle row of K: 64 bf16 or 32 fp32 (tf32) elements
constexpr int MMA_K_BYTES = 32;        // one MMA consumes 32 bytes of K per row: 16 bf16 or 8 tf32 elements
constexpr int A_TILE_BYTES = BM * BK_BYTES;
// Operand element type of a kernel variant: SPEC bit 14 set = fp32 storage multiplied as tf32 (kind::tf32), output
// fp32.  The tile geometry is the same in bytes; only element counts and the instruction kind differ.
constexpr bool spec_tf32(int spec) { return spec >= 0 && ((spec >> 14) & 1) != 0; }
constexpr int NUM_THREADS = 192;          // TMA warp + MMA warp + 4 epilogue warps
constexpr int NUM_THREADS_WIDE = 320;     // ... + 8 epilogue warps (two per scheduler) for the arithmetic-heavy epilogues

// PAIR: two CTAs of a cluster share one 256 x BN tile.  Each stages 128 rows of A and BN/2 columns of B, the
// leader issues cta_group::2 MMAs, and each holds its own 128 accumulator rows.  Per SM that is 2/3 of the
// shared-memory fill traffic of a 128 x 256 tile for the same tensor work.
// Epilogue shared memory: per epilogue warp a ring of NB buffers of 32 rows x 128 bytes.  A buffer receives the
// warp's slice of the epilogue's input operand by TMA (residual, activation input of a derivative, or the old C),
// is overwritten in place with the result and is then the source of the TMA store.  While the main loops keep
// hundreds of KB per SM in flight, a new request to L2 takes microseconds, so the fused epilogues fetch NB - 1
// chunks ahead (across tile boundaries), and the bias of the next tile is read while the current one is processed.
// The plain epilogue only stores (NB = 2).
constexpr int SMEM_LIMIT = 232448;     // 227 KB per CTA
// Ring buffers per epilogue warp of the compile-time variants with a TMA-fed input / a second output.  Deeper rings
// (3 / 4) were measured slower at the GPT-2 small shapes: they cost the main loop one of its four stages
// (bias + GELU + derivative 86 -> 98 us, bias + residual 68 -> 74 us).
#ifndef CME_GEMM_NB_IN
#define CME_GEMM_NB_IN 2
#endif
#ifndef CME_GEMM_NB_AUX
#define CME_GEMM_NB_AUX 2
#endif
template <int BN, bool PAIR, bool SIMPLE, int SPEC = -1> struct Cfg {
    static constexpr int BN_LOCAL = PAIR ? BN / 2 : BN;       // B columns staged by this CTA
    static constexpr bool TF32 = spec_tf32(SPEC);
    static constexpr int ES = TF32 ? 4 : 2;                   // operand element size
    static constexpr int BK = BK_BYTES / ES;                  // K elements per k-block
    static constexpr int GW = 128 / ES;                       // elements per 128-byte row of an MN-major operand tile
    static constexpr int B_TILE_BYTES = BN_LOCAL * BK_BYTES;
    static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
    // Compile-time variants with a TMA-fed input or a second (pre-activation) output run eight epilogue warps, two
    // per warp scheduler, each set taking every other 64-column chunk: their dependent chains (TMEM load, shared
    // memory, MUFU) then overlap instead of leaving the scheduler idle.  Two buffers per warp there; three for the
    // run-time epilogue; two where the epilogue only stores.
    static constexpr bool WIDE = !SIMPLE && SPEC >= 0 && (((SPEC >> 8) & 3) != 0 || ((SPEC >> 10) & 1) != 0);
    static constexpr int EPI_WARPS = WIDE ? 8 : 4;
    static constexpr int THREADS = WIDE ? NUM_THREADS_WIDE : NUM_THREADS;
    static constexpr bool IN_FED = !SIMPLE && SPEC >= 0 && ((SPEC >> 8) & 3) != 0;     // an operand arrives through the ring
    static constexpr bool AUX_RING = !SIMPLE && SPEC >= 0 && ((SPEC >> 10) & 1) != 0;  // a second output leaves through it
    static constexpr int NB = SIMPLE ? 2 : SPEC < 0 ? 3 : AUX_RING ? CME_GEMM_NB_AUX : IN_FED ? CME_GEMM_NB_IN : 2;
    static constexpr int AUX_ALLOW = (NB - 2) / 2;    // bulk groups that may still be reading when a chunk takes 2 buffers
    static constexpr int WARP_RING_BYTES = NB * 4096;
    static constexpr int STAGING_BYTES = EPI_WARPS * WARP_RING_BYTES;
    static constexpr int BIAS_BYTES = SIMPLE ? 0 : 3 * 256 * 2;          // three tiles' worth, shared by the warps
    static constexpr int BAR_BYTES = 512;
    static constexpr int FIXED_BYTES = STAGING_BYTES + BIAS_BYTES + 1024 /*align slack*/ + BAR_BYTES;
    static constexpr int FIT = (SMEM_LIMIT - FIXED_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = FIT > 8 ? 8 : FIT;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + FIXED_BYTES;
    static_assert(STAGES >= 3, "too few main-loop stages");
    static_assert(SMEM_BYTES <= SMEM_LIMIT, "shared-memory carve-up exceeds what one CTA may have");
    static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "two accumulators must fit TMEM (power of two)");
    static_assert(STAGE_BYTES % 1024 == 0 && A_TILE_BYTES % 1024 == 0, "swizzled tiles need 1024-byte aligned bases");
    static_assert(BAR_BYTES >= (2 * 8 + 4 + EPI_WARPS * NB) * 8 + 8, "barrier block too small");
};

struct EpiParams {
    int M, N, K, batch;
    int tiles_m, tiles_n, splits, kb_per_split, num_kb;
    int stream_aux;                // the auxiliary tensors (activation derivative written by forward, read once by backward)
                                   // go through L2 with the evict-first policy
    int n_fast;                    // tile order: 0 = consecutive tiles walk down M (share a B stripe), 1 = across N (share A rows)
    int a_batched, b_batched;
    void* C; long long ldc, strideC; int c_f32;
    const __nv_bfloat16* bias;
    const void* residual; long long ldres;
    void* aux_out; const void* aux_in; long long ldaux;
    int act, dact, accumulate;
    int aux_deriv;                 // aux tensors hold the activation's derivative instead of the pre-activation
    float* colsum;                 // [ceil(M / 32)][N] partial column sums of the stored C, or null
    int tma_store;                 // outputs go through shared memory and TMA tile stores
    int in_kind;                   // operand delivered by TMA through tmI: 0 none, 1 aux_in, 2 residual, 3 old C
    int aux_ring;                  // aux_out leaves through the ring + tmX (else direct 16-byte stores)
    int* status;
};

// Tile index -> (row block, column block).  Co-running CTAs work on consecutive tiles, so the order decides which operand
// they share in L2: walking down M they share a stripe of B and every row block of A is fetched once per column block;
// walking across N they share rows of A.  The launcher picks the order with the smaller DRAM traffic.
__device__ __forceinline__ void tile_mn(const EpiParams& p, int mn, int& tm, int& tn) {
    if (p.n_fast) { tn = mn % p.tiles_n; tm = mn / p.tiles_n; }
    else          { tm = mn % p.tiles_m; tn = mn / p.tiles_m; }
}

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
        float xo[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) xo[j] = (p.aux_deriv && p.act == CME_ACT_GELU) ? dgelu_fast(acc[j]) : acc[j];
        if (full) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) *reinterpret_cast<Bf16x8*>(X + j) = pack8(xo + j);
        } else {
            _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) X[j] = __float2bfloat16_rn(xo[j]);
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
            for (int j = 0; j < 32; ++j) acc[j] *= p.aux_deriv ? x[j] : dgelu_fast(x[j]);
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

// Which parts of the fused epilogue a kernel contains.  SPEC < 0: decided at run time from the parameters (one
// kernel holds every combination -- large code whose instruction fetches miss in the caches while L2 is saturated
// by the main loops).  SPEC >= 0: a bit set fixed at compile time, so the hot loop holds only what it executes:
//   bit 0 bias | bits 1-2 act | bits 3-4 dact | bit 5 residual | bit 6 accumulate | bit 7 aux_out |
//   bits 8-9 in_kind | bit 10 aux_ring | bit 11 fp32 output (split-K partials; nothing else set) |
//   bit 12 aux tensors hold the activation's derivative | bit 13 column sums of C |
//   bit 14 fp32 operands multiplied as tf32 (with bit 11: fp32 output)
constexpr int spec_pack(bool bias, int act, int dact, bool res, bool accum, bool aux, int in_kind, bool aux_ring,
                        bool aux_deriv = false, bool colsum = false) {
    return int(bias) | (act << 1) | (dact << 3) | (int(res) << 5) | (int(accum) << 6) | (int(aux) << 7) |
           (in_kind << 8) | (int(aux_ring) << 10) | (int(aux_deriv) << 12) | (int(colsum) << 13);
}
template <int SPEC> struct Spec {
    static constexpr bool RT = SPEC < 0;
    __device__ __forceinline__ static bool bias(const EpiParams& p) { return RT ? p.bias != nullptr : (SPEC & 1) != 0; }
    __device__ __forceinline__ static int act(const EpiParams& p) { return RT ? p.act : (SPEC >> 1) & 3; }
    __device__ __forceinline__ static int dact(const EpiParams& p) { return RT ? p.dact : (SPEC >> 3) & 3; }
    __device__ __forceinline__ static bool residual(const EpiParams& p) {
        return RT ? p.residual != nullptr : ((SPEC >> 5) & 1) != 0;
    }
    __device__ __forceinline__ static bool accumulate(const EpiParams& p) {
        return RT ? p.accumulate != 0 : ((SPEC >> 6) & 1) != 0;
    }
    __device__ __forceinline__ static bool aux_out(const EpiParams& p) {
        return RT ? p.aux_out != nullptr : ((SPEC >> 7) & 1) != 0;
    }
    __device__ __forceinline__ static int in_kind(const EpiParams& p) { return RT ? p.in_kind : (SPEC >> 8) & 3; }
    __device__ __forceinline__ static bool aux_ring(const EpiParams& p) {
        return RT ? p.aux_ring != 0 : ((SPEC >> 10) & 1) != 0;
    }
    __device__ __forceinline__ static bool c_f32(const EpiParams& p) {
        return RT ? p.c_f32 != 0 : ((SPEC >> 11) & 1) != 0;
    }
    __device__ __forceinline__ static bool aux_deriv(const EpiParams& p) {
        return RT ? p.aux_deriv != 0 : ((SPEC >> 12) & 1) != 0;
    }
    // column sums exist only in compile-time variants
    __device__ __forceinline__ static bool colsum(const EpiParams&) { return !RT && ((SPEC >> 13) & 1) != 0; }
};

// Fused epilogue arithmetic on 32 columns of one row (bf16 outputs).  `pre` receives the pre-activation.
// `bias8` points at the 32 bias values of these columns in shared memory.  `in_raw` holds the 32 bf16 of this row
// of the operand named by `in_kind` (1 activation input of the derivative, 2 residual, 3 old C), fetched by TMA
// well ahead of use; any further operand is read from global memory here.
template <int SPEC>
__device__ __forceinline__ void epilogue_math(const EpiParams& p, float* acc, float* pre, bool row_ok, long long offc,
                                              long long offr, long long offa, int n, const __nv_bfloat16* bias8,
                                              const uint4* in_raw, int in_kind) {
    using S = Spec<SPEC>;
    const int act = S::act(p), dact = S::dact(p);
    if (S::bias(p)) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float b[8];
            unpack8(*reinterpret_cast<const uint4*>(bias8 + g * 8), b);
#pragma unroll
            for (int q = 0; q < 8; q += 2)
                f2_unpack(f2_add(f2_pack(acc[g * 8 + q], acc[g * 8 + q + 1]), f2_pack(b[q], b[q + 1])), acc[g * 8 + q],
                          acc[g * 8 + q + 1]);
        }
    }
    const bool deriv = S::aux_deriv(p);
    if (S::aux_out(p) && deriv && act == CME_ACT_GELU) {
        // activation and its derivative from one tanh; the derivative is what backward multiplies by
#pragma unroll
        for (int j = 0; j < 32; j += 2) gelu_and_grad_fast2(acc[j], acc[j + 1], pre[j], pre[j + 1]);
    } else {
        if (S::aux_out(p)) {
#pragma unroll
            for (int j = 0; j < 32; ++j) pre[j] = acc[j];
        }
        if (act == CME_ACT_RELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = fmaxf(acc[j], 0.f);
        } else if (act == CME_ACT_GELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = gelu_fast(acc[j]);
        }
    }
    if (dact) {
        const __nv_bfloat16* X = reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + offa;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float x[8];
            if (in_kind == 1) unpack8(in_raw[g], x); else load8_guard(X, n + g * 8, p.N, row_ok, x);
            if (dact != CME_ACT_RELU && deriv) {
#pragma unroll
                for (int q = 0; q < 8; q += 2)
                    f2_unpack(f2_mul(f2_pack(acc[g * 8 + q], acc[g * 8 + q + 1]), f2_pack(x[q], x[q + 1])), acc[g * 8 + q],
                              acc[g * 8 + q + 1]);
            } else {
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    acc[g * 8 + q] = (dact == CME_ACT_RELU) ? (x[q] > 0.f ? acc[g * 8 + q] : 0.f)
                                                            : acc[g * 8 + q] * dgelu_fast(x[q]);
            }
        }
    }
    if (S::residual(p)) {
        const __nv_bfloat16* R = reinterpret_cast<const __nv_bfloat16*>(p.residual) + offr;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float x[8];
            if (in_kind == 2) unpack8(in_raw[g], x); else load8_guard(R, n + g * 8, p.N, row_ok, x);
#pragma unroll
            for (int q = 0; q < 8; q += 2)
                f2_unpack(f2_add(f2_pack(acc[g * 8 + q], acc[g * 8 + q + 1]), f2_pack(x[q], x[q + 1])), acc[g * 8 + q],
                          acc[g * 8 + q + 1]);
        }
    }
    if (S::accumulate(p)) {
        const __nv_bfloat16* Cp = reinterpret_cast<const __nv_bfloat16*>(p.C) + offc;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float x[8];
            if (in_kind == 3) unpack8(in_raw[g], x); else load8_guard(Cp, n + g * 8, p.N, row_ok, x);
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[g * 8 + q] += x[q];
        }
    }
}

template <int BN, bool A_MN, bool B_MN, bool SIMPLE, bool PAIR, int SPEC>
__global__ void __launch_bounds__((Cfg<BN, PAIR, SIMPLE, SPEC>::THREADS), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmX,
               const __grid_constant__ CUtensorMap tmI, const EpiParams p) {
    using C = Cfg<BN, PAIR, SIMPLE, SPEC>;
    using S = Spec<SPEC>;
    constexpr int BK = C::BK, GW = C::GW;
    constexpr int GROUP_BYTES = BK * 128;           // one GW-wide column group of an MN-major tile: BK rows of 128 bytes
    static_assert(!PAIR || BN == 256, "CTA pairs use 256-wide tiles");
    static_assert(!SIMPLE || SPEC < 0, "the plain epilogue has no compile-time variants");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* staging = smem + C::STAGES * C::STAGE_BYTES;       // 1024-byte aligned
    __nv_bfloat16* bias_smem = reinterpret_cast<__nv_bfloat16*>(staging + C::STAGING_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + C::STAGING_BYTES + C::BIAS_BYTES);
    uint64_t* full_bar = bars;                       // [STAGES]  TMA -> MMA
    uint64_t* empty_bar = bars + C::STAGES;          // [STAGES]  MMA -> TMA
    uint64_t* tfull_bar = bars + 2 * C::STAGES;      // [2]       MMA -> epilogue
    uint64_t* tempty_bar = bars + 2 * C::STAGES + 2; // [2]       epilogue -> MMA
    uint64_t* in_bar = bars + 2 * C::STAGES + 4;     // [4 warps][NB]  TMA input loads -> epilogue warp
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(in_bar + C::EPI_WARPS * C::NB);
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
            mbar_init(&tempty_bar[b], (PAIR ? 2 : 1) * C::EPI_WARPS);   // one arrival per epilogue warp (of both CTAs)
        }
        for (int b = 0; b < C::EPI_WARPS * C::NB; ++b) mbar_init(&in_bar[b], 1);
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    if (warp == 1) {
        if constexpr (PAIR) { tmem_alloc_pair(tmem_slot, C::TMEM_COLS); tmem_relinquish_pair(); }
        else                { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
    }
    tc_fence_before();
    // In a pair, the peer's barriers and TMEM must exist before anything is signalled across.
    if constexpr (PAIR) cluster_sync_all(); else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
    const int tile0 = PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x);
    const int tile_step = PAIR ? int(gridDim.x >> 1) : int(gridDim.x);
    constexpr int BMT = PAIR ? 2 * BM : BM;                  // rows of one scheduled tile
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
            for (int tile = tile0; tile < total_tiles && ok; tile += tile_step) {
                const int mn = tile % tiles_mn, rest = tile / tiles_mn;
                const int bidx = rest % p.batch, split = rest / p.batch;
                int tm, tn;
                tile_mn(p, mn, tm, tn);
                const int m0 = tm * BMT + int(cta_rank) * BM;
                const int n0 = tn * BN + int(cta_rank) * C::BN_LOCAL;
                const int kb0 = split * p.kb_per_split;
                const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
                const int za = p.a_batched ? bidx : 0, zb = p.b_batched ? bidx : 0;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* sA = smem + stage * C::STAGE_BYTES;
                    uint8_t* sB = sA + A_TILE_BYTES;
                    if constexpr (PAIR) {
                        // both CTAs' bytes are credited to the leader's barrier, which its MMA thread waits on
                        if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * C::STAGE_BYTES);
                        const uint32_t fb = mapa_u32(&full_bar[stage], 0);
                        if (!A_MN) {
                            tma_load_3d_pair(sA, &tmA, fb, kb * BK, m0, za);
                        } else {
#pragma unroll
                            for (int j = 0; j < BM / GW; ++j)
                                tma_load_3d_pair(sA + j * GROUP_BYTES, &tmA, fb, m0 + j * GW, kb * BK, za);
                        }
                        if (!B_MN) {
                            tma_load_3d_pair(sB, &tmB, fb, kb * BK, n0, zb);
                        } else {
#pragma unroll
                            for (int j = 0; j < C::BN_LOCAL / GW; ++j)
                                tma_load_3d_pair(sB + j * GROUP_BYTES, &tmB, fb, n0 + j * GW, kb * BK, zb);
                        }
                    } else {
                        mbar_arrive_expect_tx(&full_bar[stage], C::STAGE_BYTES);
                        if (!A_MN) {
                            tma_load_3d(sA, &tmA, &full_bar[stage], kb * BK, m0, za);
                        } else {
#pragma unroll
                            for (int j = 0; j < BM / GW; ++j)
                                tma_load_3d(sA + j * GROUP_BYTES, &tmA, &full_bar[stage], m0 + j * GW, kb * BK, za);
                        }
                        if (!B_MN) {
                            tma_load_3d(sB, &tmB, &full_bar[stage], kb * BK, n0, zb);
                        } else {
#pragma unroll
                            for (int j = 0; j < BN / GW; ++j)
                                tma_load_3d(sB + j * GROUP_BYTES, &tmB, &full_bar[stage], n0 + j * GW, kb * BK, zb);
                        }
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
        if (lane == 0 && cta_rank == 0) {
            constexpr uint32_t idesc = make_idesc(C::TF32 ? 2 /*tf32*/ : 1 /*bf16*/, A_MN, B_MN, BMT, BN);
            constexpr int KROWS = MMA_K_BYTES / C::ES;      // k-rows one MMA consumes of an MN-major tile: 16 or 8
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = tile0; tile < total_tiles && ok; tile += tile_step, ++it) {
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
                    for (int k = 0; k < BK_BYTES / MMA_K_BYTES; ++k) {
                        // K-major: step 32 bytes (16 bf16 / 8 tf32 elements) inside the 128-byte row.
                        // MN-major: step KROWS k-rows of 128 bytes; column groups are GROUP_BYTES apart.
                        const uint64_t da = A_MN ? make_smem_desc(sA + k * KROWS * 128, GROUP_BYTES, 1024)
                                                 : make_smem_desc(sA + k * MMA_K_BYTES, 0, 1024);
                        const uint64_t db = B_MN ? make_smem_desc(sB + k * KROWS * 128, GROUP_BYTES, 1024)
                                                 : make_smem_desc(sB + k * MMA_K_BYTES, 0, 1024);
                        const uint32_t accf = (kb > kb0 || k > 0) ? 1u : 0u;
                        if constexpr (C::TF32) {
                            if constexpr (PAIR) mma_tf32_ss_pair(tmem_d, da, db, idesc, accf);
                            else                mma_tf32_ss(tmem_d, da, db, idesc, accf);
                        } else {
                            if constexpr (PAIR) mma_f16_ss_pair(tmem_d, da, db, idesc, accf);
                            else                mma_f16_ss(tmem_d, da, db, idesc, accf);
                        }
                    }
                    // stage is free (in both CTAs of a pair) once these MMAs have read it
                    if constexpr (PAIR) mma_commit_pair(&empty_bar[stage], 3); else mma_commit(&empty_bar[stage]);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) {                               // accumulator complete
                    if constexpr (PAIR) mma_commit_pair(&tfull_bar[buf], 3); else mma_commit(&tfull_bar[buf]);
                }
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
        // the accumulator goes back to the (leader's) MMA thread: one arrival per warp
        auto acc_release = [&](int b) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR) mbar_arrive_cluster(mapa_u32(&tempty_bar[b], 0));
                else                mbar_arrive(&tempty_bar[b]);
            }
        };
        // Ring of this warp's epilogue buffers and the cursor of the input prefetch (fused bf16 epilogues only).  The
        // cursor runs over (tile, 64-column chunk) in the order the warp will consume them, NB - 1 chunks ahead, and
        // crosses tile boundaries, so the first chunks of a tile are already in flight while its main loop runs.
        constexpr int ESETS = C::EPI_WARPS / 4;         // warp sets; set s takes the chunks c with c % ESETS == s
        const int eset = (warp - 2) >> 2;
        const int wslot = eset * 4 + quarter;
        uint8_t* ring = staging + wslot * C::WARP_RING_BYTES;
        uint64_t* my_in_bar = in_bar + wslot * C::NB;
        // Bias values of three consecutive tiles, [3][256].  Every epilogue warp writes the same values (and reads
        // only after its own writes); three slots because a warp may finish tile i + 1, and park the bias of tile
        // i + 2, while another is still reading that of tile i.
        __nv_bfloat16* bias_w = bias_smem;
        const bool ring_epi = !SIMPLE && (SPEC >= 0 ? !S::c_f32(p) : (p.tma_store && !p.c_f32));
        const int in_kind = ring_epi ? S::in_kind(p) : 0;
        uint32_t slot = 0;                              // ring buffers handed out so far
        int f_tile = tile0, f_c = eset;
        uint32_t f_cnt = 0;
        auto fetch_next = [&]() {
            int fmn = 0, fn0 = 0, fm_blk = 0;
            while (f_tile < total_tiles) {              // next tile that has a chunk for this warp set
                fmn = f_tile % tiles_mn;
                int ftm, ftn;
                tile_mn(p, fmn, ftm, ftn);
                fn0 = ftn * BN;
                fm_blk = ftm;
                int nchf = (p.N - fn0 + 63) / 64;
                nchf = nchf < BN / 64 ? nchf : BN / 64;
                if (f_c < nchf) break;
                f_c = eset;
                f_tile += tile_step;
            }
            if (f_tile >= total_tiles) return;
            const int fb = (f_tile / tiles_mn) % p.batch;
            const int fm0 = fm_blk * BMT + int(cta_rank) * BM + quarter * 32;
            if (lane == 0) {
                const uint32_t b = f_cnt % C::NB;
                mbar_arrive_expect_tx(&my_in_bar[b], 4096);
                if (p.stream_aux && in_kind == 1)
                    tma_load_3d_hint(ring + b * 4096, &tmI, &my_in_bar[b], fn0 + f_c * 64, fm0, fb, l2_policy_evict_first());
                else
                    tma_load_3d(ring + b * 4096, &tmI, &my_in_bar[b], fn0 + f_c * 64, fm0, fb);
            }
            ++f_cnt;
            f_c += ESETS;
        };
        constexpr bool FETCH_AT_TOP = C::NB == 2;
        if (in_kind) {
            for (int i = 0; i < C::NB - 1; ++i) fetch_next();
        }
        const bool stage_bias = !SIMPLE && ring_epi && S::bias(p);
        auto bias_fetch = [&](int t) {                  // this lane's 8 bias values of tile t (zeros past N)
            float b8[8];
            int btm, btn;
            tile_mn(p, t % tiles_mn, btm, btn);
            const int tn0 = btn * BN;
            load8_guard(p.bias, tn0 + lane * 8, p.N, true, b8);
            return pack8(b8);
        };
        if (stage_bias && tile0 < total_tiles) {
            *reinterpret_cast<uint4*>(bias_w + lane * 8) = bias_fetch(tile0);
            __syncwarp();
        }
        for (int tile = tile0; tile < total_tiles && ok; tile += tile_step, ++it) {
            const int mn = tile % tiles_mn, rest = tile / tiles_mn;
            const int bidx = rest % p.batch, split = rest / p.batch;
            int etm, etn;
            tile_mn(p, mn, etm, etn);
            const int m0 = etm * BMT + int(cta_rank) * BM, n0 = etn * BN;
            const int buf = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const __nv_bfloat16* bias_s = bias_w + (it % 3) * 256;
            // the next tile's bias values are requested now and parked in shared memory after this tile's chunks
            uint4 bias_next = make_uint4(0, 0, 0, 0);
            const bool have_next = stage_bias && tile + tile_step < total_tiles;
            if (have_next) bias_next = bias_fetch(tile + tile_step);
            if (!mbar_wait(&tfull_bar[buf], acc_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const long long zoff = (long long)(split * p.batch + bidx);
            const long long offc = zoff * p.strideC + (long long)row * p.ldc;
            const long long offr = (long long)bidx * p.strideC + (long long)row * p.ldres;
            const long long offa = (long long)bidx * p.strideC + (long long)row * p.ldaux;
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
                            acc_release(buf);                       // accumulator fully read
                        }
                        uint8_t* sb = ring + (store_cnt & 1) * 4096;
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
            if (SPEC < 0 && !p.tma_store) {
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
            } else if (S::c_f32(p)) {
                // fp32 output (split-K partials, fp32 C): 32 columns = one 128-byte staging row per TMA store
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int n = n0 + c * 32;
                    if (n >= p.N) break;
                    uint32_t r[32];
                    tmem_ld32(tmem_row + c * 32, r);
                    tmem_wait_ld();
                    if (SPEC < 0 && p.accumulate) {
                        const float* Cp = reinterpret_cast<const float*>(p.C) + offc;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (row < p.M && n + j < p.N) r[j] = __float_as_uint(__uint_as_float(r[j]) + Cp[n + j]);
                    }
                    uint8_t* sb = ring + (store_cnt & 1) * 4096;
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
                // bf16 output, fused epilogue: per 64-column chunk one ring buffer (two when the pre-activation also
                // leaves through the ring).  With a TMA-fed input the buffer already holds this warp's 32 x 64 slice
                // of it; every thread replaces its own 16-byte groups in place with the result.
                const bool row_ok = row < p.M;
                const bool aux_ring = S::aux_ring(p);
                __nv_bfloat16* Xrow = (S::aux_out(p) && !aux_ring) ? reinterpret_cast<__nv_bfloat16*>(p.aux_out) + offa
                                                                   : nullptr;
#pragma unroll 1
                for (int c2 = eset; c2 < BN / 64; c2 += ESETS) {
                    const int n = n0 + c2 * 64;
                    if (n >= p.N) break;
                    uint8_t* sbC = ring + (slot % C::NB) * 4096;
                    uint8_t* sbX = ring + ((slot + 1) % C::NB) * 4096;
                    if (in_kind && FETCH_AT_TOP) {
                        // Two buffers: the other one holds the previous chunk, whose copy-out was issued a moment ago.  As
                        // soon as the copy engine has read it (a short wait) the next chunk's input is requested into it,
                        // and arrives while this chunk is processed -- instead of being requested after this chunk and
                        // awaited at once with its full latency.
                        if (lane == 0) tma_store_wait_read<0>();
                        __syncwarp();
                        fetch_next();
                    }
                    if (in_kind) {
                        if (!mbar_wait(&my_in_bar[slot % C::NB], (slot / C::NB) & 1, abort_flag)) { ok = false; break; }
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t r[32];
                        tmem_ld32(tmem_row + c2 * 64 + h * 32, r);
                        uint4 in_raw[4];
                        if (in_kind) {
#pragma unroll
                            for (int g = 0; g < 4; ++g)
                                in_raw[g] = *reinterpret_cast<const uint4*>(sbC + lane * 128 +
                                                                            (((h * 4 + g) ^ (lane & 7)) * 16));
                        }
                        tmem_wait_ld();
                        float acc[32], pre[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(r[j]);
                        epilogue_math<SPEC>(p, acc, pre, row_ok, offc, offr, offa, n + h * 32,
                                            bias_s + c2 * 64 + h * 32, in_raw, in_kind);
                        if (h == 0 && !in_kind) {
                            // buffers written by plain stores: their previous TMA stores must have been read out.
                            // One bulk group per chunk; the aux variant takes two buffers per chunk.
                            if (lane == 0) {
                                if (aux_ring) tma_store_wait_read<C::AUX_ALLOW>();
                                else tma_store_wait_read<C::NB - 1>();
                            }
                            __syncwarp();
                        }
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const int q = h * 4 + g;
                            *reinterpret_cast<uint4*>(sbC + lane * 128 + ((q ^ (lane & 7)) * 16)) = pack8(acc + g * 8);
                            if (aux_ring) {
                                *reinterpret_cast<uint4*>(sbX + lane * 128 + ((q ^ (lane & 7)) * 16)) =
                                    pack8(pre + g * 8);
                            } else if (Xrow) {
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
                        if (aux_ring) {
                            if (p.stream_aux) tma_store_3d_hint(&tmX, sbX, n, m0 + quarter * 32, bidx, l2_policy_evict_first());
                            else tma_store_3d(&tmX, sbX, n, m0 + quarter * 32, bidx);
                        }
                        tma_store_commit();
                    }
                    if (S::colsum(p)) {
                        // Column sums of the 32 x 64 slab just staged (the bf16 values that are stored): lane l owns
                        // columns 2l, 2l + 1 and walks down the rows; for a fixed row the lanes read the 32 words of
                        // one 128-byte line, so there are no bank conflicts.  The buffer is not refilled before the
                        // next chunk ends, and the TMA store only reads it.
                        const int row0 = m0 + quarter * 32;
                        const int nvalid = min(32, p.M - row0);
                        float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
                        for (int r = 0; r < 32; ++r) {
                            if (r < nvalid) {
                                const uint32_t w = *reinterpret_cast<const uint32_t*>(
                                    sbC + r * 128 + (((lane >> 2) ^ (r & 7)) * 16) + (lane & 3) * 4);
                                const float2 f = bf2_to_f2(w);
                                s0 += f.x; s1 += f.y;
                            }
                        }
                        const int col = n + 2 * lane;
                        float* dst = p.colsum + (long long)(row0 >> 5) * p.N + col;
                        if (nvalid > 0) {
                            if (col + 1 < p.N && (p.N & 1) == 0) *reinterpret_cast<float2*>(dst) = make_float2(s0, s1);
                            else { if (col < p.N) dst[0] = s0; if (col + 1 < p.N) dst[1] = s1; }
                        }
                    }
                    slot += aux_ring ? 2 : 1;
                    if (in_kind && !FETCH_AT_TOP) {
                        // three buffers: refill the one stored one chunk ago with the chunk two ahead
                        if (lane == 0) tma_store_wait_read<1>();
                        __syncwarp();
                        fetch_next();
                    }
                }
                if (!ok) break;
            }
            if (have_next) {
                *reinterpret_cast<uint4*>(bias_w + ((it + 1) % 3) * 256 + lane * 8) = bias_next;
                __syncwarp();
            }
            acc_release(buf);
        }
        if (!ok && in_kind) {
            // input copies may still be in flight: give them time to land before shared memory is released
            for (int i = 0; i < 2000; ++i) __nanosleep(500);
        }
        if (p.tma_store && lane == 0) tma_store_wait<0>();   // stores complete before shared memory goes away
    }

    __syncwarp();
    tc_fence_before();
    // A pair leaves together: neither CTA may exit while the other can still signal its barriers or read its tiles.
    if constexpr (PAIR) cluster_sync_all(); else __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, CME_ERR_TIMEOUT);
    if (warp == 1) {
        tc_fence_after();
        if constexpr (PAIR) tmem_dealloc_pair(tmem_base, C::TMEM_COLS); else tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

template <int BN, bool A_MN, bool B_MN, bool SIMPLE, bool PAIR, int SPEC>
int launch_cfg(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tx,
               const CUtensorMap& ti, const EpiParams& ep, int grid, cudaStream_t st) {
    auto kern = gemm_tc_kernel<BN, A_MN, B_MN, SIMPLE, PAIR, SPEC>;
    static bool attr_set[CME_MAX_DEVICES] = {};          // function attributes are per device
    int dev = 0;
    CME_CUDA(cudaGetDevice(&dev));
    if (!attr_set[dev % CME_MAX_DEVICES]) {
        CME_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN, PAIR, SIMPLE, SPEC>::SMEM_BYTES));
        attr_set[dev % CME_MAX_DEVICES] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(Cfg<BN, PAIR, SIMPLE, SPEC>::THREADS);
    cfg.dynamicSmemBytes = Cfg<BN, PAIR, SIMPLE, SPEC>::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (PAIR) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    CME_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, tx, ti, ep));
    CME_LAUNCH_CHECK();
    return CME_OK;
}

template <int BN, bool SIMPLE, bool PAIR, int SPEC = -1>
int launch_bn(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
              const CUtensorMap& tx, const CUtensorMap& ti, const EpiParams& ep, int grid, cudaStream_t st) {
    if (!a_mn && !b_mn) return launch_cfg<BN, false, false, SIMPLE, PAIR, SPEC>(ta, tb, tc, tx, ti, ep, grid, st);
    if (!a_mn && b_mn) return launch_cfg<BN, false, true, SIMPLE, PAIR, SPEC>(ta, tb, tc, tx, ti, ep, grid, st);
    if (a_mn && !b_mn) return launch_cfg<BN, true, false, SIMPLE, PAIR, SPEC>(ta, tb, tc, tx, ti, ep, grid, st);
    return launch_cfg<BN, true, true, SIMPLE, PAIR, SPEC>(ta, tb, tc, tx, ti, ep, grid, st);
}

// Epilogue combinations with a compile-time kernel : the ones a transformer layer uses.
constexpr int SPEC_BIAS = spec_pack(true, 0, 0, false, false, false, 0, false);
constexpr int SPEC_BIAS_RES = spec_pack(true, 0, 0, true, false, false, 2, false);
constexpr int SPEC_BIAS_GELU_AUX = spec_pack(true, CME_ACT_GELU, 0, false, false, true, 0, true);
constexpr int SPEC_DGELU = spec_pack(false, 0, CME_ACT_GELU, false, false, false, 1, false);
constexpr int SPEC_BIAS_RELU = spec_pack(true, CME_ACT_RELU, 0, false, false, false, 0, false);
constexpr int SPEC_DRELU = spec_pack(false, 0, CME_ACT_RELU, false, false, false, 1, false);
constexpr int SPEC_RES = spec_pack(false, 0, 0, true, false, false, 2, false);
constexpr int SPEC_F32 = 1 << 11;
constexpr int SPEC_TF32 = (1 << 11) | (1 << 14);      // fp32 operands multiplied as tf32, fp32 output
// the pair the transformer's MLP uses: forward leaves GELU'(pre-activation), backward multiplies by it and sums columns
constexpr int SPEC_BIAS_GELU_AUXD = spec_pack(true, CME_ACT_GELU, 0, false, false, true, 0, true, true);
constexpr int SPEC_DMUL_COLSUM = spec_pack(false, 0, CME_ACT_GELU, false, false, false, 1, false, true, true);
constexpr int SPEC_DMUL = spec_pack(false, 0, CME_ACT_GELU, false, false, false, 1, false, true, false);
constexpr int SPEC_DRELU_COLSUM = spec_pack(false, 0, CME_ACT_RELU, false, false, false, 1, false, false, true);
constexpr int SPEC_ACC = spec_pack(false, 0, 0, false, true, false, 3, false);

}  // namespace gemm_tc
