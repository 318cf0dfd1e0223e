// Host side of the tcgen05 GEMM: tile / split-K planning, tensor maps, dispatch to the kernel instantiation that
// matches the layout and the fused epilogue, split-K reduction kernels and the status word.  The kernel itself is in
// gemm_tcgen05_kernel.cuh; its instantiations live in gemm_tc_inst_*.cu.
#include "gemm_tcgen05_kernel.cuh"

#include <dlfcn.h>
#include <mutex>

using namespace gemm_tc;

// Instantiated elsewhere (one line per launcher; each covers the four operand layouts).
#define CME_GEMM_TC_EXTERN(BN, SIMPLE, PAIR, SPEC)                                                                  \
    extern template int gemm_tc::launch_bn<BN, SIMPLE, PAIR, SPEC>(bool, bool, const CUtensorMap&, const CUtensorMap&, \
                                                                   const CUtensorMap&, const CUtensorMap&,             \
                                                                   const CUtensorMap&, const EpiParams&, int, cudaStream_t);
#include "gemm_tc_inst_list.h"
#undef CME_GEMM_TC_EXTERN

namespace {

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

// Same, four consecutive columns per thread (N, ldc and strideC multiples of 4): 16-byte reads of every partial.
__global__ void splitk_reduce_vec4_kernel(const float4* __restrict__ P, int splits, long long per_split4, void* Cout,
                                          int c_f32, int accumulate, int M, int N4, long long ldc, long long strideC,
                                          int batch) {
    pdl_wait();
    const long long total = (long long)batch * M * N4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        float4 s = P[i];
        for (int k = 1; k < splits; ++k) {
            const float4 v = P[k * per_split4 + i];
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        const long long mn4 = (long long)M * N4;
        const long long b = i / mn4, rem = i - b * mn4;
        const long long r = rem / N4, c = (rem - r * N4) * 4;
        const long long off = b * strideC + r * ldc + c;
        if (c_f32) {
            float4* C = reinterpret_cast<float4*>(reinterpret_cast<float*>(Cout) + off);
            if (accumulate) { const float4 o = *C; s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w; }
            *C = s;
        } else {
            uint2* C = reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(Cout) + off);
            if (accumulate) {
                const uint2 o = *C;
                const float2 a = bf2_to_f2(o.x), d = bf2_to_f2(o.y);
                s.x += a.x; s.y += a.y; s.z += d.x; s.w += d.y;
            }
            *C = make_uint2(f2_to_bf2(s.x, s.y), f2_to_bf2(s.z, s.w));
        }
    }
}

// out[b][c][r] = in[b][r][c] for fp32 matrices (32 x 32 tiles through shared memory).  The tf32 products take
// K-major operands only -- with an MN-major fp32 operand the tensor core returned zeros here -- so operands stored
// the other way are copied into the workspace transposed first.
__global__ void __launch_bounds__(256) transpose_f32_kernel(const float* __restrict__ in, float* __restrict__ out, int rows,
                                                            int cols, long long ld_in, long long stride_in,
                                                            long long stride_out) {
    __shared__ float tile[32][33];
    pdl_wait();
    const float* src = in + (long long)blockIdx.z * stride_in;
    float* dst = out + (long long)blockIdx.z * stride_out;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int j = ty; j < 32; j += 8)
        if (r0 + j < rows && c0 + tx < cols) tile[j][tx] = src[(long long)(r0 + j) * ld_in + c0 + tx];
    __syncthreads();
#pragma unroll
    for (int j = ty; j < 32; j += 8)
        if (c0 + j < cols && r0 + tx < rows) dst[(long long)(c0 + j) * rows + r0 + tx] = tile[tx][j];
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
              long long batch_stride, int box_rows, bool f32 = false, bool round_tf32 = false) {
    EncodeTiledFn enc = get_encoder();
    CME_REQUIRE(enc != nullptr, CME_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const int es = f32 ? 4 : 2;
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)(batch > 0 ? batch : 1)};
    cuuint64_t strides[2] = {(cuuint64_t)ld * es, (cuuint64_t)(batch_stride > 0 ? batch_stride : ld * rows) * es};
    cuuint32_t box[3] = {(cuuint32_t)(128 / es), (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    // operands of a tf32 product are rounded to tf32 (to nearest) by the copy engine on their way into shared
    // memory; the tensor core would otherwise just drop the low mantissa bits, a one-sided error
    const CUtensorMapDataType dt = !f32 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                        : round_tf32 ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    CUresult r = enc(out, dt, 3,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    CME_REQUIRE(r == CUDA_SUCCESS, CME_ERR_CUDA,
                "cuTensorMapEncodeTiled failed (%d): inner=%lld rows=%lld ld=%lld batch=%lld bstride=%lld box_rows=%d",
                (int)r, inner, rows, ld, batch, batch_stride, box_rows);
    return CME_OK;
}

// How many CTA pairs of the pair kernel can be resident at once (the persistent grid must not exceed it: a pair
// that is not resident would only start when another has finished all of its tiles).
int query_max_pairs(int num_sms) {
    auto kern = gemm_tc_kernel<256, false, false, true, true, -1>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<256, true, true>::SMEM_BYTES) !=
        cudaSuccess) { cudaGetLastError(); return 0; }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * num_sms);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = Cfg<256, true, true>::SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

}  // namespace

CME_API int cme_gemm_status_word(int** out) {
    CmeDeviceState* ds;
    int rc = cme_device_state(&ds);
    if (rc) return rc;
    *out = ds->status + CME_STATUS_GEMM;
    return CME_OK;
}

// Tile shape and K splits for a product: minimise  waves x k-blocks per unit x cost(tile)  (+ fixed per-tile and
// per-split overheads), with measured clocks per 16-deep MMA step for each tile shape.  Pure host arithmetic.
//   force_bn: 0 = choose; 64 / 128 / 256 = tile width on one CTA; 512 = the 256 x 256 tile on a CTA pair
//   force_splits: 0 = choose.  Split-K needs the plain epilogue, a workspace for the fp32 partials and at least
//   four 64-deep k-blocks per split.
static void plan_tiles(int M, int N, int K, int batch, bool plain_epi, long long workspace_bytes, int num_sms,
                       int max_pairs, int force_bn, int force_splits, int* bn_out, bool* pair_out, int* splits_out,
                       int bk = 64) {
    const int num_kb = cme_cdiv(K, bk);
    int bn = force_bn, splits = force_splits;
    bool pair = false;
    if (bn == 512) { bn = 256; pair = true; }
    if (!bn || !splits) {
        double best = 1e30;
        int best_bn = 128, best_s = 1;
        bool best_pair = false;
        const int bns[4] = {256, 256, 128, 64};
        // clocks per 16-deep MMA step and SM: the 128-row tiles are limited by how fast shared memory can be
        // refilled from L2 ((128 + bn) x 32 bytes per step), the pair tile (128 + 128 per SM) by the tensor pipe
        const double cost[4] = {136.0, 168.0, 100.0, 72.0};
        for (int i = 0; i < 4; ++i) {
            const bool pr = i == 0;
            if (pr && (max_pairs <= 0 || M <= BM)) continue;
            if (force_bn && (force_bn == 512 ? !pr : (pr || bns[i] != force_bn))) continue;
            if (bns[i] > 64 && N <= bns[i] / 2) continue;            // tile mostly padding
            const long long t = (long long)cme_cdiv(M, pr ? 2 * BM : BM) * cme_cdiv(N, bns[i]) * batch;
            const int slots = pr ? max_pairs : num_sms;
            for (int s = 1; s <= 16; ++s) {
                if (force_splits && s != force_splits) continue;
                if (s > 1 && (!plain_epi || num_kb / s < 4 || (long long)s * batch * M * N * 4 > workspace_bytes)) break;
                const long long units = t * s;
                const double waves = (double)((units + slots - 1) / slots);
                const double kb = (double)cme_cdiv(num_kb, s);
                // 4 MMAs per k-block; epilogue / pipeline fill ~ 6 k-blocks of the widest tile per unit;
                // a split adds one fp32 write + read of the output per split
                double est = waves * ((kb + 2.0) * 4.0 * cost[i] + 6.0 * 4.0 * bns[i] / 2.0);
                if (s > 1) est += 6000.0 + (double)s * M * N * batch / num_sms / 16.0;   // + one more launch
                if (est < best) { best = est; best_bn = bns[i]; best_s = s; best_pair = pr; }
            }
        }
        if (!bn) { bn = best_bn; pair = best_pair; }
        if (!splits) splits = best_s;
    }
    *bn_out = bn; *pair_out = pair; *splits_out = splits;
}

// The plan the launcher would choose, without a device: `num_sms` SMs, `max_pairs` co-resident CTA pairs (0 = no
// cluster launches).  out = {tile width, pair (0/1), splits}.
CME_API int cme_gemm_plan(int M, int N, int K, int batch, int plain_epilogue, long long workspace_bytes, int num_sms,
                          int max_pairs, int force_bn, int force_splits, int* out) {
    CME_REQUIRE(M > 0 && N > 0 && K > 0 && batch > 0 && num_sms > 0, CME_ERR_SHAPE, "gemm plan: empty problem");
    int bn = 0, splits = 0;
    bool pair = false;
    plan_tiles(M, N, K, batch, plain_epilogue != 0, workspace_bytes, num_sms, max_pairs, force_bn, force_splits, &bn,
               &pair, &splits);
    out[0] = bn; out[1] = pair ? 1 : 0; out[2] = splits;
    return CME_OK;
}

int gemm_tcgen05_supported(const CmeGemm* g) {
    const bool tf32 = g->ab_dtype == CME_F32;
    // fp32 operands run as tf32, and only where the caller allows the reduced input precision: plain products
    // (fp32 output, optionally accumulated), rows of C addressable in 16-byte units
    if (tf32 && (!g->allow_tf32 || g->c_dtype != CME_F32 || g->bias || g->residual || g->aux_out || g->aux_in ||
                 g->act || g->dact || g->N % 4 || g->ldc % 4 || (g->batch > 1 && g->strideC % 4)))
        return 0;
    if (tf32 && (g->a_trans || !g->b_trans)) {
        // an operand stored MN-major is transposed into the workspace first: its new row pitch is K
        const long long na = g->a_trans ? (long long)(g->strideA ? g->batch : 1) * g->M * g->K : 0;
        const long long nb = !g->b_trans ? (long long)(g->strideB ? g->batch : 1) * g->N * g->K : 0;
        if (g->K % 4 || !g->workspace || (na + nb) * 4 + 512 > g->workspace_bytes / 2) return 0;
    }
    if (!tf32 && g->ab_dtype != CME_BF16) return 0;
    if (g->M <= 0 || g->N <= 0 || g->K <= 0 || g->batch <= 0) return 0;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (!al16(g->A) || !al16(g->B) || !al16(g->C)) return 0;
    const int unit = tf32 ? 4 : 8;                           // elements per 16 bytes
    if (g->lda % unit || g->ldb % unit || g->strideA % unit || g->strideB % unit) return 0;
    // Extents need not be multiples of the 16-byte unit: row pitches are (checked above), and a box that reaches
    // past an extent reads zeros.  Degenerate extents go to the SIMT kernel.
    const long long innerA = g->a_trans ? g->M : g->K, innerB = g->b_trans ? g->K : g->N;
    if (innerA < unit || innerB < unit) return 0;
    if (g->c_dtype == CME_F32 && (g->act || g->dact || g->residual || g->aux_out)) return 0;
    return 1;
}

int gemm_tcgen05_launch(const CmeGemm* g, cudaStream_t stream) {
    CME_REQUIRE(gemm_tcgen05_supported(g), CME_ERR_SHAPE, "gemm shape/alignment not supported by the tcgen05 kernel");
    CmeDeviceState* ds;
    {
        int rc0 = cme_device_state(&ds);
        if (rc0) return rc0;
    }
    if (ds->max_pairs < 0) {
        const char* e = getenv("CME213_GEMM_PAIR");
        ds->max_pairs = (e && e[0] == '0') ? 0 : query_max_pairs(ds->num_sms);
    }
    const int g_num_sms = ds->num_sms, g_max_pairs = ds->max_pairs;
    int* const g_status = ds->status + CME_STATUS_GEMM;
    const bool tf32 = g->ab_dtype == CME_F32;
    if (tf32 && (g->a_trans || !g->b_trans)) {
        // K-major copies of the operands that are stored MN-major (see transpose_f32_kernel), carved from the front
        // of the workspace; the product then runs on the copies with what is left of the workspace
        CmeGemm gg = *g;
        char* w = static_cast<char*>(g->workspace);
        auto carve = [&](long long floats) {
            float* p = reinterpret_cast<float*>(w);
            w += (floats * 4 + 255) / 256 * 256;
            return p;
        };
        if (g->a_trans) {                                     // stored [K, M] -> [M, K]
            const int nb = g->strideA ? g->batch : 1;
            float* t = carve((long long)nb * g->M * g->K);
            CME_CUDA(cme_launch_dependent(transpose_f32_kernel, dim3(cme_cdiv(g->M, 32), cme_cdiv(g->K, 32), nb), dim3(256),
                                          0, stream, static_cast<const float*>(g->A), t, g->K, g->M, g->lda, g->strideA,
                                          (long long)g->M * g->K));
            CME_LAUNCH_CHECK();
            gg.A = t; gg.lda = g->K; gg.a_trans = 0; gg.strideA = g->strideA ? (long long)g->M * g->K : 0;
        }
        if (!g->b_trans) {                                    // stored [K, N] -> [N, K]
            const int nb = g->strideB ? g->batch : 1;
            float* t = carve((long long)nb * g->N * g->K);
            CME_CUDA(cme_launch_dependent(transpose_f32_kernel, dim3(cme_cdiv(g->N, 32), cme_cdiv(g->K, 32), nb), dim3(256),
                                          0, stream, static_cast<const float*>(g->B), t, g->K, g->N, g->ldb, g->strideB,
                                          (long long)g->N * g->K));
            CME_LAUNCH_CHECK();
            gg.B = t; gg.ldb = g->K; gg.b_trans = 1; gg.strideB = g->strideB ? (long long)g->N * g->K : 0;
        }
        gg.workspace = w;
        gg.workspace_bytes = g->workspace_bytes - (w - static_cast<char*>(g->workspace));
        return gemm_tcgen05_launch(&gg, stream);
    }
    const int BK = tf32 ? 32 : 64;                            // K elements per 128-byte k-block
    int tiles_m = cme_cdiv(g->M, BM);
    const int num_kb = cme_cdiv(g->K, BK);
    const bool plain_epi = !g->bias && !g->residual && !g->aux_out && !g->act && !g->dact;
    int bn = 0, splits = 0;
    bool pair = false;
    plan_tiles(g->M, g->N, g->K, g->batch, plain_epi, g->workspace ? g->workspace_bytes : 0, g_num_sms, g_max_pairs,
               g->force_bn, g->force_splits, &bn, &pair, &splits, BK);
    // A tf32 product that accumulates into C goes through the fp32 workspace like a split-K product (one "split"
    // is then added to C by the reduction kernel): the tf32 kernel variants only store.
    const bool via_ws = splits > 1 || (tf32 && g->accumulate);
    if (tf32 && g->accumulate)
        CME_REQUIRE(g->workspace && (long long)splits * g->batch * g->M * g->N * 4 <= g->workspace_bytes, CME_ERR_LIMIT,
                    "tf32 accumulate needs an fp32 workspace of M x N");
    CME_REQUIRE(bn == 64 || bn == 128 || bn == 256, CME_ERR_SHAPE, "tile width must be 64, 128, 256 or 512 (pair)");
    CME_REQUIRE(!pair || g_max_pairs > 0, CME_ERR_SHAPE, "CTA-pair tiles are not available on this device");
    if (pair) tiles_m = cme_cdiv(g->M, 2 * BM);
    static const bool trace = getenv("CME213_GEMM_TRACE") != nullptr;
    if (trace)
        fprintf(stderr, "[gemm] M=%d N=%d K=%d batch=%d at=%d bt=%d -> bn=%d pair=%d splits=%d\n", g->M, g->N, g->K,
                g->batch, g->a_trans, g->b_trans, bn, (int)pair, splits);
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
    if (!g->a_trans) rc = make_tmap(&ta, g->A, g->K, g->M, g->lda, g->strideA ? g->batch : 1, g->strideA, BM, tf32, tf32);
    else             rc = make_tmap(&ta, g->A, g->M, g->K, g->lda, g->strideA ? g->batch : 1, g->strideA, BK, tf32, tf32);
    if (rc) return rc;
    // B: stored [N, K] (b_trans) is K-major -> map (K, N), box (64, bn); stored [K, N] -> map (N, K), box (64, 64)
    if (g->b_trans) rc = make_tmap(&tb, g->B, g->K, g->N, g->ldb, g->strideB ? g->batch : 1, g->strideB,
                                   pair ? bn / 2 : bn, tf32, tf32);
    else            rc = make_tmap(&tb, g->B, g->N, g->K, g->ldb, g->strideB ? g->batch : 1, g->strideB, BK, tf32, tf32);
    if (rc) return rc;

    EpiParams ep{};
    ep.M = g->M; ep.N = g->N; ep.K = g->K; ep.batch = g->batch;
    ep.tiles_m = tiles_m; ep.tiles_n = tiles_n; ep.splits = splits; ep.kb_per_split = kb_per; ep.num_kb = num_kb;
    ep.a_batched = g->strideA != 0 && g->batch > 1; ep.b_batched = g->strideB != 0 && g->batch > 1;
    {
        // Tile order by estimated DRAM traffic.  The CTAs that run together walk K at about the same pace, so the
        // operand they share is fetched once per wave of tiles from DRAM and served to the others from L2; the
        // operand they do not share is needed again a wave later and comes from DRAM again unless it stays in L2
        // (taken as half of its 126 MB).  So the order that shares the operand too large for L2 wins.
        const int es = tf32 ? 4 : 2;
        const double a_bytes = (double)g->M * g->K * es, b_bytes = (double)g->N * g->K * es, l2 = 63.0e6;
        const double slots = pair ? (double)g_max_pairs : (double)g_num_sms;
        const double waves = (double)tiles_m * tiles_n / slots > 1.0 ? (double)tiles_m * tiles_n / slots : 1.0;
        const double ra = waves < tiles_n ? waves : tiles_n, rb = waves < tiles_m ? waves : tiles_m;
        const double m_fast = a_bytes * (a_bytes > l2 ? ra : 1.0) + b_bytes;         // B stripe shared, A rows distinct
        const double n_fast = b_bytes * (b_bytes > l2 ? rb : 1.0) + a_bytes;         // A rows shared
        static const char* force = getenv("CME213_GEMM_NFAST");
        ep.n_fast = force ? (force[0] == '1') : (n_fast < m_fast && tiles_n > 1);
        // the stored derivative is written once by forward and read once by backward, a layer's worth of other work
        // apart: keep it from displacing what the neighbouring kernels re-read (CME213_GEMM_STREAM_AUX=0: off)
        static const bool stream_aux = !(getenv("CME213_GEMM_STREAM_AUX") && getenv("CME213_GEMM_STREAM_AUX")[0] == '0');
        ep.stream_aux = (stream_aux && g->aux_deriv && (g->act == CME_ACT_GELU || g->dact == CME_ACT_GELU)) ? 1 : 0;
    }
    ep.status = g_status;
    if (via_ws) {
        ep.C = g->workspace; ep.ldc = g->N; ep.strideC = (long long)g->M * g->N; ep.c_f32 = 1;
    } else {
        ep.C = g->C; ep.ldc = g->ldc; ep.strideC = g->strideC; ep.c_f32 = g->c_dtype == CME_F32;
        ep.bias = reinterpret_cast<const __nv_bfloat16*>(g->bias);
        ep.residual = g->residual; ep.ldres = g->ldres;
        ep.aux_out = g->aux_out; ep.aux_in = g->aux_in; ep.ldaux = g->ldaux;
        ep.act = g->act; ep.dact = g->dact; ep.accumulate = g->accumulate;
        ep.aux_deriv = (g->aux_deriv && (g->act == CME_ACT_GELU || g->dact == CME_ACT_GELU)) ? 1 : 0;
    }
    if (g->colsum_slabs) *g->colsum_slabs = 0;
    // Outputs through shared-memory staging + TMA tile stores when rows are 16-byte addressable.
    CUtensorMap tc = ta, tx = ta, ti = ta;
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
            // The operand the fused epilogue reads per output element comes in by TMA, chunk by chunk, ahead of use.
            if (!ep.c_f32) {
                const void* ib = nullptr;
                long long ild = 0;
                int kind = 0;
                if (ep.dact) { ib = ep.aux_in; ild = ep.ldaux; kind = 1; }
                else if (ep.residual) { ib = ep.residual; ild = ep.ldres; kind = 2; }
                else if (ep.accumulate) { ib = ep.C; ild = ep.ldc; kind = 3; }
                if (kind && al16(ib) && (ild * 2) % 16 == 0 && (g->batch == 1 || (ep.strideC * 2) % 16 == 0)) {
                    rc = make_tmap(&ti, ib, g->N, g->M, ild, g->batch, g->batch > 1 ? ep.strideC : 0, 32);
                    if (rc) return rc;
                    ep.in_kind = kind;
                }
                ep.aux_ring = ep.aux_out && !ep.in_kind;
            }
        }
    }
    const long long total = tiles * splits;
    const int grid = pair ? 2 * (int)(total < g_max_pairs ? total : g_max_pairs)
                          : (int)(total < g_num_sms ? total : g_num_sms);
    const bool a_mn = g->a_trans != 0, b_mn = g->b_trans == 0;
    const bool simple = ep.tma_store && !ep.c_f32 && !ep.bias && !ep.residual && !ep.aux_out && !ep.aux_in &&
                        !ep.act && !ep.dact && !ep.accumulate;
    int spec = -1, spec_colsum = -1;
    if (!simple) {
        if (ep.tma_store && !ep.c_f32) {
            spec = spec_pack(ep.bias != nullptr, ep.act, ep.dact, ep.residual != nullptr, ep.accumulate != 0,
                             ep.aux_out != nullptr, ep.in_kind, ep.aux_ring != 0, ep.aux_deriv != 0, false);
            // column sums ride in the variants whose input arrives through the ring (one output buffer per chunk)
            if (g->colsum && g->colsum_slabs && splits == 1 && g->batch == 1 && ep.in_kind == 1 && ep.dact)
                spec_colsum = spec | (1 << 13);
        } else if (ep.tma_store && ep.c_f32 && !ep.accumulate) {
            spec = tf32 ? SPEC_TF32 : SPEC_F32;
        }
    }
    CME_REQUIRE(!tf32 || spec == SPEC_TF32, CME_ERR_SHAPE, "tf32 product: output rows are not 16-byte addressable");
    // the instantiation with this tile, pairing and compile-time epilogue (first with the column sums, if asked
    // for); else the run-time epilogue of that tile
    rc = -1;
    for (int attempt = 0; attempt < 3 && rc == -1; ++attempt) {
        const int want = attempt == 0 ? spec_colsum : attempt == 1 ? spec : -1;
        if (attempt == 0 && want < 0) continue;
        ep.colsum = attempt == 0 ? g->colsum : nullptr;
#define CME_GEMM_TC_EXTERN(BN, SIMPLE, PAIR, SPEC)                                              \
    if (rc == -1 && bn == BN && simple == SIMPLE && pair == PAIR && want == SPEC)               \
        rc = launch_bn<BN, SIMPLE, PAIR, SPEC>(a_mn, b_mn, ta, tb, tc, tx, ti, ep, grid, stream);
#include "gemm_tc_inst_list.h"
#undef CME_GEMM_TC_EXTERN
        if (rc == CME_OK && attempt == 0) *g->colsum_slabs = cme_cdiv(g->M, 32);
    }
    CME_REQUIRE(rc != -1, CME_ERR_SHAPE, "gemm: no kernel instantiation for tile %d pair %d", bn, (int)pair);
    if (rc) return rc;
    if (via_ws) {
        const long long per = (long long)g->batch * g->M * g->N;
        const bool f32 = g->c_dtype == CME_F32;
        const bool vec = g->N % 4 == 0 && g->ldc % 4 == 0 && (g->batch == 1 || g->strideC % 4 == 0) &&
                         (reinterpret_cast<uintptr_t>(g->C) & (f32 ? 15 : 7)) == 0 &&
                         (reinterpret_cast<uintptr_t>(g->workspace) & 15) == 0;
        if (vec) {
            const long long per4 = per / 4;
            const int blocks = (int)((per4 + 255) / 256 < 8 * g_num_sms ? (per4 + 255) / 256 : 8 * g_num_sms);
            CME_CUDA(cme_launch_dependent(splitk_reduce_vec4_kernel, dim3(blocks), dim3(256), 0, stream,
                                          reinterpret_cast<const float4*>(g->workspace), splits, per4, g->C, (int)f32,
                                          g->accumulate, g->M, g->N / 4, g->ldc, g->strideC, g->batch));
        } else {
            const int blocks = (int)((per + 255) / 256 < 4096 ? (per + 255) / 256 : 4096);
            splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float*>(g->workspace), splits, per,
                                                             g->C, f32, g->accumulate, g->M, g->N, g->ldc, g->strideC,
                                                             g->batch);
        }
        CME_LAUNCH_CHECK();
    }
    return CME_OK;
}

// Reads and clears the device status word (0 = every bounded wait completed).
CME_API int cme_gemm_check_status(int* host_out) { return cme_check_status_word(CME_STATUS_GEMM, host_out); }
