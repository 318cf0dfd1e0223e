// Native model executor: forward and backward of the transformer over the flat arenas, every op one of
// this library's kernels, every launch on the caller's stream (so a whole step can be captured in a
// CUDA graph by the caller).
//
// Role of the reference's TransformerModel::forward_no_sync / backward_bucketed
// (FINAL_CLEAN_CODE_/src/model/transformer.cu:337-408, 417-590).  Differences by design:
//   * N blocks, ReLU or GELU, causal or not, flat or split heads, tied or untied head, optional final LN;
//   * bias / activation / residual adds ride in GEMM epilogues instead of separate kernels
//     (the reference launches bias_relu, residual_add_with_bias, residual+LayerNorm kernels);
//   * the ReLU / GELU derivative rides in the dgrad GEMM epilogue; bias gradients are column sums;
//   * weight gradients overwrite (or accumulate, for micro-batches after the first), so there is no
//     gradient memset per step (the reference zeroes all gradients because split-K uses atomics);
//   * `bucket_ready(index)` is called on the host right after the launches that complete a natural gradient
//     bucket have been enqueued, in arena order -- the hook the reference calls sync_bucket (:428-457);
//   * weight-gradient products (and the bias column sums) can run on a second stream beside the chain of
//     input-gradient kernels that the next layer waits for: a persistent GEMM leaves SMs idle during its last,
//     partial wave of tiles, and CTAs of the other stream's kernel start on them.  Dependencies in both
//     directions are CUDA events, so the whole backward pass is still one capturable graph.
#include "attention.h"
#include "gemm.h"

#include <cstdlib>
#include <new>
#include <vector>

extern "C" {
int cme_layernorm_fwd(int, const void*, const void*, void*, const void*, const void*, void*, float*, float*, int, int,
                      float, void*);
int cme_layernorm_bwd_blocks(int);
int cme_layernorm_bwd(int, const void*, const void*, const void*, const float*, const float*, const void*, void*, void*,
                      void*, float*, int, int, int, void*);
int cme_layernorm_bwd_split(int, const void*, const void*, const void*, const float*, const float*, const void*, void*,
                            void*, void*, float*, int, int, int, void*, void*, void*);
int cme_colsum_splits(int, int);
int cme_dact_colsum(int, const void*, const void*, void*, void*, float*, int, int, int, int, void*);
int cme_colsum_slabs_finalize(int, const float*, int, int, void*, int, void*);
int cme_bias_act_residual(int, const void*, const void*, const void*, void*, void*, long long, int, int, void*);
int cme_embedding_fwd(int, const int*, const void*, const void*, void*, int, int, int, int, void*);
int cme_embedding_bwd(int, const int*, const void*, void*, void*, int, int, int, int, int, void*);
int cme_cross_entropy(int, const void*, const int*, void*, float*, float*, int, int, long long, float, float, float,
                      int, void*);
int cme_attention_fwd(const CmeAttn*, int, void*);
int cme_attention_bwd(const CmeAttn*, int, void*);
int cme_gemm(const CmeGemm*, int, void*);
int cme_cast(int, const void*, int, void*, long long, void*);
}

struct CmeEngineDesc {
    int V, T, D, H, FF, L, B;
    int act;             // CME_ACT_RELU | CME_ACT_GELU
    int causal, head_flat, tied, final_ln, fused_qkv;
    int allow_tf32;      // fp32 storage: plain products may run on the tensor cores with tf32 inputs
    int fuse_epilogues;  // 0: bias / activation / residual adds and the activation derivative run as separate kernels
                         // after plain products (the ablation the reference measures with CME213_LT_FUSION)
    int ffn_lowp;        // fp32 storage only.  1: the feed-forward activation is rounded to bf16 where it is stored (the
                         // reference's CME213_FP16_STORAGE_ONLY experiment); 2: the four feed-forward products of a
                         // layer take bf16 copies of their operands and give fp32 results (its CME213_FFN_FP16)
    float ln_eps, prob_eps;
    int dtype;           // CME_BF16 | CME_F32
    int gemm_backend;    // 0 auto, 1 tcgen05, 2 simt
    int attn_backend;    // 0 auto, 1 tensor-core, 2 simt
};

// Element offsets into the parameter / gradient arenas; -1 = tensor absent.
struct CmeLayerSlots { long long W2, b2, W1, b1, ln2g, ln2b, Wo, Wq, Wk, Wv, Wqkv, ln1g, ln1b; };
struct CmeGlobalSlots { long long Wout, lnfg, lnfb, tok, pos; };

typedef void (*CmeBucketFn)(void* user, int natural_bucket);

namespace {

struct LayerAct {
    char *ln1, *qkv, *attn, *xmid, *ln2, *ffpre, *ffact;
    float *mean1, *rstd1, *mean2, *rstd2, *lse;
};

struct Engine {
    CmeEngineDesc d;
    size_t es;
    int BT, BH;
    std::vector<CmeLayerSlots> ls;
    CmeGlobalSlots gs;
    char* params = nullptr;
    char* grads = nullptr;
    char* ws = nullptr;
    size_t ws_bytes = 0;
    // activations
    std::vector<char*> x;          // L+1 residual-stream buffers
    std::vector<LayerAct> la;
    char *xf, *logits;
    char* wout_pad = nullptr;      // untied output projection [D, V] re-pitched to [D, VL] when V is not a multiple of
                                   // 8 (bf16): refreshed at the start of every forward, read by forward and dX
    long long VL;                  // row pitch of the logits buffer: the vocabulary rounded up to 8 elements, so every
                                   // row starts 16-byte aligned and the LM-head products run on the TMA-fed GEMM
    float *meanf, *rstdf, *losses;
    // backward temporaries
    char *dxa, *dxb, *dff, *dln, *dqkv, *dattn;
    float *delta, *dq_accum, *ln_scratch, *col_scratch;
    float* dq_accum2 = nullptr;     // second dQ scratch: the layers alternate, so that a layer's scratch can be cleared on the
                                    // second stream while the layer above still uses the other one
    std::vector<cudaEvent_t> ev_ln;  // one per LayerNorm site: its main kernel has run (the sums follow on the second stream)
    size_t ln_scratch_stride = 0;    // floats per LayerNorm site in ln_scratch (2 L + 1 sites)
    cudaEvent_t ev_dq[4] = {};      // [0..1] scratch b was converted (main stream)   [2..3] scratch b is clear (second stream)
    int* dq_sem = nullptr;          // per (batch, head, query block) counters ordering the dQ parts; zero between launches
    void* attn_ws; long long attn_ws_bytes;
    void* gemm_ws; long long gemm_ws_bytes;
    void* gemm_ws_side; long long gemm_ws_side_bytes;     // split-K partials of the products on the second stream
    float* col_scratch_side;
    float* slab_scratch;                                   // [ceil(BT / 32)][FF] column sums left by a GEMM epilogue
    char *lp_x = nullptr, *lp_h = nullptr, *lp_w = nullptr;  // bf16 copies for ffn_lowp: [BT, D], [BT, FF], [D, FF]
    // second stream for the weight-gradient work (null: everything on the caller's stream)
    cudaStream_t side = nullptr;
    std::vector<cudaEvent_t> ev;                           // [L + 1][8]: four "inputs ready" + four "done" per layer

    char* P(long long off) const { return params + off * (long long)es; }
    char* G(long long off) const { return grads + off * (long long)es; }
};

size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }

// One pass computes the carve-up; with base == nullptr it only measures.
size_t carve(Engine& e, char* base) {
    const CmeEngineDesc& d = e.d;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        char* p = base ? base + off : nullptr;
        off += align_up(bytes);
        return p;
    };
    const size_t BT = e.BT, D = d.D, FF = d.FF, es = e.es;
    e.x.resize(d.L + 1);
    for (int l = 0; l <= d.L; ++l) e.x[l] = take(BT * D * es);
    e.la.resize(d.L);
    for (int l = 0; l < d.L; ++l) {
        LayerAct& a = e.la[l];
        a.ln1 = take(BT * D * es);
        a.qkv = take(3 * BT * D * es);
        a.attn = take(BT * D * es);
        a.xmid = take(BT * D * es);
        a.ln2 = take(BT * D * es);
        a.ffpre = d.act == CME_ACT_GELU ? take(BT * FF * es) : nullptr;
        a.ffact = take(BT * FF * es);
        a.mean1 = (float*)take(BT * 4); a.rstd1 = (float*)take(BT * 4);
        a.mean2 = (float*)take(BT * 4); a.rstd2 = (float*)take(BT * 4);
        a.lse = (float*)take((size_t)e.BH * d.T * 4);
    }
    e.xf = d.final_ln ? take(BT * D * es) : nullptr;
    e.meanf = (float*)take(BT * 4); e.rstdf = (float*)take(BT * 4);
    e.VL = ((long long)d.V + 7) / 8 * 8;
    e.logits = take(BT * (size_t)e.VL * es);
    e.losses = (float*)take(BT * 4);
    e.wout_pad = (!d.tied && d.dtype == CME_BF16 && e.VL != d.V) ? take(D * (size_t)e.VL * es) : nullptr;
    e.dxa = take(BT * D * es); e.dxb = take(BT * D * es);
    e.dff = take(BT * FF * es);
    e.dln = take(BT * D * es);
    e.dqkv = take(3 * BT * D * es);
    e.dattn = take(BT * D * es);
    e.delta = (float*)take((size_t)e.BH * d.T * 4);
    e.dq_accum = (float*)take(BT * D * 4);
    e.dq_accum2 = (float*)take(BT * D * 4);
    e.dq_sem = (int*)take((size_t)e.BH * ((d.T + 127) / 128) * 4);
    e.attn_ws_bytes = (d.head_flat && d.T <= 512) ? attention_gemm_ws_bytes(e.BH, d.T) : 0;
    e.attn_ws = e.attn_ws_bytes ? take((size_t)e.attn_ws_bytes) : nullptr;
    const size_t widest = FF > D ? FF : D;
    // one region per LayerNorm site: the sums of a site's partials run on the second stream, after the next site's
    // main kernel may already have started
    e.ln_scratch_stride = (size_t)cme_layernorm_bwd_blocks((int)BT) * 2 * D;
    e.ln_scratch = (float*)take(e.ln_scratch_stride * 4 * (2 * (size_t)d.L + 1));
    e.col_scratch = (float*)take((size_t)(cme_colsum_splits((int)BT, (int)D) + cme_colsum_splits((int)BT, (int)FF)) *
                                 widest * 4);
    // split-K partials (fp32): room for four splits of the widest activation-gradient product, e.g. the LM-head
    // input gradient whose 192 pair tiles fill 74 CTA pairs unevenly unless K is split three ways
    const long long want_ws = 4ll * (long long)BT * (long long)widest * 4ll;
    e.gemm_ws_bytes = want_ws > (64ll << 20) ? want_ws : (64ll << 20);
    e.gemm_ws = take((size_t)e.gemm_ws_bytes);
    // the second stream's own scratch: eight splits of the largest per-layer weight gradient, column-sum partials
    const long long side_ws = 8ll * (long long)D * (long long)widest * 4ll;
    e.gemm_ws_side_bytes = side_ws > (64ll << 20) ? side_ws : (64ll << 20);
    e.gemm_ws_side = take((size_t)e.gemm_ws_side_bytes);
    e.slab_scratch = (float*)take((size_t)((BT + 31) / 32) * widest * 4);
    e.col_scratch_side = (float*)take((size_t)(cme_colsum_splits((int)BT, (int)D) + cme_colsum_splits((int)BT, (int)FF)) *
                                      widest * 4);
    if (d.ffn_lowp) {
        e.lp_x = take(BT * D * 2);
        e.lp_h = take(BT * FF * 2);
        e.lp_w = take(D * FF * 2);
    }
    return off;
}

int gemm(const Engine& e, cudaStream_t st, int M, int N, int K, const void* A, long long lda, int a_trans,
         const void* B, long long ldb, int b_trans, void* C, long long ldc, int accumulate = 0,
         const void* bias = nullptr, int act = 0, void* aux_out = nullptr, int dact = 0, const void* aux_in = nullptr,
         long long ldaux = 0, const void* residual = nullptr, long long ldres = 0, int batch = 1, long long sA = 0,
         long long sB = 0, long long sC = 0, int aux_deriv = 0, float* colsum = nullptr, int* colsum_slabs = nullptr) {
    CmeGemm g{};
    g.M = M; g.N = N; g.K = K; g.batch = batch;
    g.A = A; g.lda = lda; g.strideA = sA; g.a_trans = a_trans;
    g.B = B; g.ldb = ldb; g.strideB = sB; g.b_trans = b_trans;
    g.C = C; g.ldc = ldc; g.strideC = sC; g.c_dtype = e.d.dtype; g.ab_dtype = e.d.dtype;
    g.bias = bias; g.residual = residual; g.ldres = ldres;
    g.aux_out = aux_out; g.aux_in = aux_in; g.ldaux = ldaux;
    g.act = act; g.dact = dact; g.accumulate = accumulate;
    g.aux_deriv = aux_deriv; g.colsum = colsum; g.colsum_slabs = colsum_slabs;
    g.allow_tf32 = e.d.allow_tf32;
    const bool on_side = e.side != nullptr && st == e.side;
    g.workspace = on_side ? e.gemm_ws_side : e.gemm_ws;
    g.workspace_bytes = on_side ? e.gemm_ws_side_bytes : e.gemm_ws_bytes;
    return cme_gemm(&g, e.d.gemm_backend, st);
}

// A plain product of bf16 operands with an fp32 result (the reduced-precision feed-forward experiment).
int gemm_lp(const Engine& e, cudaStream_t st, int M, int N, int K, const void* A, long long lda, int a_trans,
            const void* B, long long ldb, int b_trans, void* C, long long ldc, int accumulate = 0) {
    CmeGemm g{};
    g.M = M; g.N = N; g.K = K; g.batch = 1;
    g.A = A; g.lda = lda; g.a_trans = a_trans;
    g.B = B; g.ldb = ldb; g.b_trans = b_trans;
    g.C = C; g.ldc = ldc; g.c_dtype = CME_F32; g.ab_dtype = CME_BF16;
    g.accumulate = accumulate;
    g.workspace = e.gemm_ws; g.workspace_bytes = e.gemm_ws_bytes;
    return cme_gemm(&g, 0, st);
}

int to_bf16(const void* x, void* y, long long n, cudaStream_t st) { return cme_cast(CME_F32, x, CME_BF16, y, n, st); }

// CME213_DETERMINISTIC=1: the attention backward adds the key blocks' parts of dQ in a fixed order (bit-reproducible
// gradients, about 0.07 ms per layer slower at GPT-2 small shapes); default: unordered reduce-adds.
bool attn_ordered_dq() {
    static const bool on = getenv("CME213_DETERMINISTIC") && getenv("CME213_DETERMINISTIC")[0] == '1';
    return on;
}

// CME213_ATTN_DQ_MODE=2: dQ finished inside the attention backward by the CTA whose part of a tile arrives last
// (no clearing and no conversion pass: two launches fewer per layer).  Off by default: the store warp then waits for
// every reduce-add to complete before it counts the part in, and one warp converts each finished tile, which costs
// more than the two passes it saves at GPT-2 small shapes (17.2 against 16.6 ms per training step).
bool attn_dq_finish() {
    static const bool on = getenv("CME213_ATTN_DQ_MODE") && getenv("CME213_ATTN_DQ_MODE")[0] == '2';
    return on;
}

void fill_attn(const Engine& e, int l, CmeAttn& a) {
    const CmeEngineDesc& d = e.d;
    const int HD = d.D / d.H;
    const long long BT = e.BT, D = d.D;
    a = CmeAttn{};
    a.T = d.T; a.HD = HD; a.causal = d.causal; a.scale = 1.0f / sqrtf((float)HD); a.dtype = d.dtype;
    char* qkv = e.la[l].qkv;
    if (d.fused_qkv) {            // [BT, 3D] rows: Q | K | V
        a.nb = d.B; a.nh = d.H; a.sb = (long long)d.T * 3 * D; a.sh = HD; a.st = 3 * D;
        a.q = qkv; a.k = qkv + D * e.es; a.v = qkv + 2 * D * e.es;
        a.dq = e.dqkv; a.dk = e.dqkv + D * e.es; a.dv = e.dqkv + 2 * D * e.es;
    } else {                      // three [BT, D] planes
        if (d.head_flat) { a.nb = d.B * d.H; a.nh = 1; a.sb = (long long)d.T * HD; a.sh = 0; a.st = HD; }
        else { a.nb = d.B; a.nh = d.H; a.sb = (long long)d.T * D; a.sh = HD; a.st = D; }
        a.q = qkv; a.k = qkv + BT * D * e.es; a.v = qkv + 2 * BT * D * e.es;
        a.dq = e.dqkv; a.dk = e.dqkv + BT * D * e.es; a.dv = e.dqkv + 2 * BT * D * e.es;
    }
    if (d.head_flat) { a.osb = (long long)d.T * HD; a.osh = 0; a.ost = HD; }
    else { a.osb = (long long)d.T * D; a.osh = HD; a.ost = D; }
    a.lse = e.la[l].lse; a.delta = e.delta; a.dq_accum = e.dq_accum;
    // dQ: parts added in arrival order to a scratch that the launch clears and a second kernel converts (mode 0);
    // on request the deterministic form (mode 1) or the form finished inside the kernel (mode 2)
    a.dq_sem = e.dq_sem;
    a.dq_mode = attn_ordered_dq() ? 1 : attn_dq_finish() && (d.T + 127) / 128 <= CME_ATTN_FINISH_MAX_QBLOCKS ? 2 : 0;
    a.ws = e.attn_ws; a.ws_bytes = e.attn_ws_bytes;
}

#define TRY(expr) do { int rc__ = (expr); if (rc__) return rc__; } while (0)

// CME213_FFN_COLSUM=0: the gradient of b1 as a column-sum kernel on the second stream instead of inside the epilogue
// of the product that makes d ff_pre (for A/B measurements).
bool ffn_colsum() {
    static const bool on = !(getenv("CME213_FFN_COLSUM") && getenv("CME213_FFN_COLSUM")[0] == '0');
    return on;
}

// CME213_FFN_DERIV=0 goes back to keeping the pre-activation and re-evaluating the derivative in backward, with the
// bias gradient as a separate column-sum kernel (for A/B measurements of the fused form).
bool ffn_deriv() {
    static const bool on = !(getenv("CME213_FFN_DERIV") && getenv("CME213_FFN_DERIV")[0] == '0');
    return on;
}

}  // namespace

CME_API int cme_engine_create(const CmeEngineDesc* desc, const CmeLayerSlots* layers, const CmeGlobalSlots* globals,
                              void** out) {
    CME_REQUIRE(desc->L >= 1 && desc->D % desc->H == 0, CME_ERR_SHAPE, "engine: bad model shape");
    CME_REQUIRE(!(desc->fused_qkv && desc->head_flat), CME_ERR_SHAPE, "engine: fused QKV needs split heads");
    CME_REQUIRE(!desc->head_flat || desc->T % desc->H == 0, CME_ERR_SHAPE, "engine: flat heads need T %% H == 0");
    CME_REQUIRE(desc->ffn_lowp >= 0 && desc->ffn_lowp <= 2 && (!desc->ffn_lowp || desc->dtype == CME_F32), CME_ERR_SHAPE,
                "engine: the reduced-precision feed-forward modes need fp32 storage");
    Engine* e = new (std::nothrow) Engine();
    CME_REQUIRE(e != nullptr, CME_ERR_CUDA, "engine: out of host memory");
    e->d = *desc;
    e->es = desc->dtype == CME_BF16 ? 2 : 4;
    e->BT = desc->B * desc->T;
    e->BH = desc->B * desc->H;
    e->ls.assign(layers, layers + desc->L);
    e->gs = *globals;
    e->ws_bytes = carve(*e, nullptr);
    *out = e;
    return CME_OK;
}

CME_API long long cme_engine_workspace_bytes(void* h) { return (long long)static_cast<Engine*>(h)->ws_bytes; }

CME_API int cme_engine_bind(void* h, void* params, void* grads, void* workspace, long long workspace_bytes) {
    Engine* e = static_cast<Engine*>(h);
    CME_REQUIRE((size_t)workspace_bytes >= e->ws_bytes, CME_ERR_LIMIT, "engine: workspace too small");
    CME_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, CME_ERR_SHAPE, "engine: workspace must be 256-byte aligned");
    e->params = (char*)params; e->grads = (char*)grads; e->ws = (char*)workspace;
    carve(*e, e->ws);
    // the attention backward's counters and its dQ scratch start at zero; every launch leaves them at zero again
    CME_CUDA(cudaMemset(e->dq_sem, 0, (size_t)e->BH * ((e->d.T + 127) / 128) * 4));
    CME_CUDA(cudaMemset(e->dq_accum, 0, (size_t)e->BT * e->d.D * 4));
    CME_CUDA(cudaMemset(e->dq_accum2, 0, (size_t)e->BT * e->d.D * 4));
    return CME_OK;
}

CME_API void cme_engine_destroy(void* h) {
    Engine* e = static_cast<Engine*>(h);
    for (cudaEvent_t v : e->ev) cudaEventDestroy(v);
    for (cudaEvent_t v : e->ev_dq) if (v) cudaEventDestroy(v);
    for (cudaEvent_t v : e->ev_ln) cudaEventDestroy(v);
    if (e->side) cudaStreamDestroy(e->side);
    delete e;
}

// Turns the second stream for weight-gradient work on (creating it and its events on the current device) or off.
// Call outside stream capture.
CME_API int cme_engine_set_overlap(void* h, int on) {
    Engine* e = static_cast<Engine*>(h);
    if (on && !e->side) {
        CME_CUDA(cudaStreamCreateWithFlags(&e->side, cudaStreamNonBlocking));
        e->ev.resize((size_t)(e->d.L + 1) * 8);
        for (cudaEvent_t& v : e->ev) CME_CUDA(cudaEventCreateWithFlags(&v, cudaEventDisableTiming));
        for (cudaEvent_t& v : e->ev_dq) CME_CUDA(cudaEventCreateWithFlags(&v, cudaEventDisableTiming));
        e->ev_ln.resize(2 * (size_t)e->d.L + 1);
        for (cudaEvent_t& v : e->ev_ln) CME_CUDA(cudaEventCreateWithFlags(&v, cudaEventDisableTiming));
    } else if (!on && e->side) {
        CME_CUDA(cudaStreamSynchronize(e->side));
        for (cudaEvent_t v : e->ev) cudaEventDestroy(v);
        for (cudaEvent_t& v : e->ev_dq) { cudaEventDestroy(v); v = nullptr; }
        for (cudaEvent_t v : e->ev_ln) cudaEventDestroy(v);
        e->ev_ln.clear();
        e->ev.clear();
        CME_CUDA(cudaStreamDestroy(e->side));
        e->side = nullptr;
    }
    return CME_OK;
}

// Makes `target` wait for everything enqueued so far on `stream` and on the engine's second stream: what a
// gradient-synchronisation stream needs before it may read a bucket that backward has just completed.
CME_API int cme_engine_fence(void* h, void* stream, void* target) {
    Engine* e = static_cast<Engine*>(h);
    cudaEvent_t v;
    CME_CUDA(cudaEventCreateWithFlags(&v, cudaEventDisableTiming));
    CME_CUDA(cudaEventRecord(v, (cudaStream_t)stream));
    CME_CUDA(cudaStreamWaitEvent((cudaStream_t)target, v, 0));
    if (e->side) {
        CME_CUDA(cudaEventRecord(v, e->side));
        CME_CUDA(cudaStreamWaitEvent((cudaStream_t)target, v, 0));
    }
    CME_CUDA(cudaEventDestroy(v));           // released once the recorded work has completed
    return CME_OK;
}

CME_API void* cme_engine_logits(void* h) { return static_cast<Engine*>(h)->logits; }
CME_API long long cme_engine_logits_ld(void* h) { return static_cast<Engine*>(h)->VL; }
CME_API void* cme_engine_activation(void* h, int layer, int which) {
    Engine* e = static_cast<Engine*>(h);
    if (which == 0) return e->x[layer];
    const LayerAct& a = e->la[layer];
    switch (which) {
        case 1: return a.ln1; case 2: return a.qkv; case 3: return a.attn; case 4: return a.xmid;
        case 5: return a.ln2; case 6: return a.ffact; default: return nullptr;
    }
}

// Forward: logits, per-token losses, and *loss_out (+)= loss_weight * mean loss.  With targets == null
// only the logits are produced.  The cross-entropy kernel leaves d(logits) * grad_scale in the logits
// buffer, ready for backward.
CME_API int cme_engine_forward(void* h, const int* tokens, const int* targets, float* loss_out, float loss_weight,
                               int accumulate_loss, float grad_scale, void* stream) {
    Engine& e = *static_cast<Engine*>(h);
    const CmeEngineDesc& d = e.d;
    cudaStream_t st = (cudaStream_t)stream;
    CME_REQUIRE(e.ws != nullptr, CME_ERR_SHAPE, "engine: not bound");
    const int BT = e.BT, D = d.D, FF = d.FF, V = d.V, dt = d.dtype;
    const bool fused = d.fuse_epilogues != 0;
    TRY(cme_embedding_fwd(dt, tokens, e.P(e.gs.tok), e.P(e.gs.pos), e.x[0], BT, d.T, D, V, st));
    for (int l = 0; l < d.L; ++l) {
        const CmeLayerSlots& s = e.ls[l];
        LayerAct& a = e.la[l];
        TRY(cme_layernorm_fwd(dt, e.x[l], nullptr, nullptr, e.P(s.ln1g), e.P(s.ln1b), a.ln1, a.mean1, a.rstd1, BT, D,
                              d.ln_eps, st));
        if (d.fused_qkv)
            TRY(gemm(e, st, BT, 3 * D, D, a.ln1, D, 0, e.P(s.Wqkv), 3 * D, 0, a.qkv, 3 * D));
        else      // three weight matrices back to back, one shared A: a batch of 3
            TRY(gemm(e, st, BT, D, D, a.ln1, D, 0, e.P(s.Wq), D, 0, a.qkv, D, 0, nullptr, 0, nullptr, 0, nullptr, 0,
                     nullptr, 0, 3, 0, (long long)D * D, (long long)BT * D));
        CmeAttn at;
        fill_attn(e, l, at);
        at.o = a.attn;
        TRY(cme_attention_fwd(&at, d.attn_backend, st));
        // x_mid = x + attn @ Wo
        if (fused) {
            TRY(gemm(e, st, BT, D, D, a.attn, D, 0, e.P(s.Wo), D, 0, a.xmid, D, 0, nullptr, 0, nullptr, 0, nullptr, 0,
                     e.x[l], D));
        } else {
            TRY(gemm(e, st, BT, D, D, a.attn, D, 0, e.P(s.Wo), D, 0, a.xmid, D));
            TRY(cme_bias_act_residual(dt, a.xmid, nullptr, e.x[l], nullptr, a.xmid, BT, D, 0, st));
        }
        TRY(cme_layernorm_fwd(dt, a.xmid, nullptr, nullptr, e.P(s.ln2g), e.P(s.ln2b), a.ln2, a.mean2, a.rstd2, BT, D,
                              d.ln_eps, st));
        // ff_act = act(ln2 @ W1 + b1)   (GELU also keeps GELU'(pre-activation), from the same tanh, for backward)
        if (d.ffn_lowp == 2) {
            // bf16 copies of the operands, fp32 products, fp32 element-wise work
            // (FINAL_CLEAN_CODE_/src/model/transformer.cu:297-306)
            TRY(to_bf16(a.ln2, e.lp_x, (long long)BT * D, st));
            TRY(to_bf16(e.P(s.W1), e.lp_w, (long long)D * FF, st));
            TRY(gemm_lp(e, st, BT, FF, D, e.lp_x, D, 0, e.lp_w, FF, 0, a.ffact, FF));
            TRY(cme_bias_act_residual(dt, a.ffact, e.P(s.b1), nullptr, a.ffpre, a.ffact, BT, FF, d.act, st));
            TRY(to_bf16(a.ffact, e.lp_h, (long long)BT * FF, st));
            TRY(to_bf16(e.P(s.W2), e.lp_w, (long long)D * FF, st));
            TRY(gemm_lp(e, st, BT, D, FF, e.lp_h, FF, 0, e.lp_w, D, 0, e.x[l + 1], D));
            TRY(cme_bias_act_residual(dt, e.x[l + 1], e.P(s.b2), a.xmid, nullptr, e.x[l + 1], BT, D, 0, st));
        } else if (fused && d.ffn_lowp == 0) {
            TRY(gemm(e, st, BT, FF, D, a.ln2, D, 0, e.P(s.W1), FF, 0, a.ffact, FF, 0, e.P(s.b1), d.act, a.ffpre, 0,
                     nullptr, FF, nullptr, 0, 1, 0, 0, 0, /*aux_deriv=*/ffn_deriv() ? 1 : 0));
            // x_next = x_mid + ff_act @ W2 + b2
            TRY(gemm(e, st, BT, D, FF, a.ffact, FF, 0, e.P(s.W2), D, 0, e.x[l + 1], D, 0, e.P(s.b2), 0, nullptr, 0,
                     nullptr, 0, a.xmid, D));
        } else {
            // plain products, then the reference's element-wise kernels: bias + activation (keeping the
            // pre-activation), and bias + residual add (FINAL_CLEAN_CODE_/src/model/transformer.cu:387-399)
            TRY(gemm(e, st, BT, FF, D, a.ln2, D, 0, e.P(s.W1), FF, 0, a.ffact, FF));
            TRY(cme_bias_act_residual(dt, a.ffact, e.P(s.b1), nullptr, a.ffpre, a.ffact, BT, FF, d.act, st));
            if (d.ffn_lowp == 1) {
                // the stored activation keeps bf16 precision: what the second product and backward read is the
                // rounded value (FINAL_CLEAN_CODE_/src/model/transformer.cu:317-320)
                TRY(to_bf16(a.ffact, e.lp_h, (long long)BT * FF, st));
                TRY(cme_cast(CME_BF16, e.lp_h, CME_F32, a.ffact, (long long)BT * FF, st));
            }
            TRY(gemm(e, st, BT, D, FF, a.ffact, FF, 0, e.P(s.W2), D, 0, e.x[l + 1], D));
            TRY(cme_bias_act_residual(dt, e.x[l + 1], e.P(s.b2), a.xmid, nullptr, e.x[l + 1], BT, D, 0, st));
        }
    }
    const void* xlast = e.x[d.L];
    if (d.final_ln) {
        TRY(cme_layernorm_fwd(dt, e.x[d.L], nullptr, nullptr, e.P(e.gs.lnfg), e.P(e.gs.lnfb), e.xf, e.meanf, e.rstdf,
                              BT, D, d.ln_eps, st));
        xlast = e.xf;
    }
    if (d.tied) {
        TRY(gemm(e, st, BT, V, D, xlast, D, 0, e.P(e.gs.tok), D, 1, e.logits, e.VL));
    } else if (e.wout_pad) {
        CME_CUDA(cudaMemcpy2DAsync(e.wout_pad, (size_t)e.VL * e.es, e.P(e.gs.Wout), (size_t)V * e.es, (size_t)V * e.es, D,
                                   cudaMemcpyDeviceToDevice, st));
        TRY(gemm(e, st, BT, V, D, xlast, D, 0, e.wout_pad, e.VL, 0, e.logits, e.VL));
    } else {
        TRY(gemm(e, st, BT, V, D, xlast, D, 0, e.P(e.gs.Wout), V, 0, e.logits, e.VL));
    }
    if (targets)
        TRY(cme_cross_entropy(dt, e.logits, targets, e.logits, e.losses, loss_out, BT, V, e.VL, grad_scale, d.prob_eps,
                              loss_weight, accumulate_loss, st));
    return CME_OK;
}

// Backward from d(logits) left in the logits buffer by forward.  accumulate != 0 adds into the gradient
// arena (micro-batches after the first); otherwise every gradient is overwritten.
//
// With the second stream on, the chain  dX products -> LayerNorm / attention backward  stays on `stream` and every
// weight-gradient product and bias column sum goes to the second stream.  Event k of a layer's first four marks
// "the k-th input of the side work exists" (recorded on `stream`), of its last four "the k-th piece of side work is
// done" (recorded on the second stream); the main chain waits for a "done" event only where it is about to
// overwrite a buffer that piece reads, which is up to one layer later.
CME_API int cme_engine_backward(void* h, const int* tokens, int accumulate, CmeBucketFn bucket_ready, void* user,
                                void* stream) {
    Engine& e = *static_cast<Engine*>(h);
    const CmeEngineDesc& d = e.d;
    cudaStream_t st = (cudaStream_t)stream;
    const bool ov = e.side != nullptr;
    cudaStream_t ws = ov ? e.side : st;                     // stream of the weight-gradient work
    const int BT = e.BT, D = d.D, FF = d.FF, V = d.V, dt = d.dtype;
    int bucket = 0;
    auto emit = [&]() { if (bucket_ready) bucket_ready(user, bucket); ++bucket; };
    // slot L = output head, slot l = layer l; k in [0, 4) inputs ready, [4, 8) side work done
    auto evt = [&](int slot, int k) { return e.ev[(size_t)slot * 8 + k]; };
    auto ready = [&](int slot, int k) -> int {              // side work may start: its inputs are enqueued on `st`
        if (!ov) return CME_OK;
        CME_CUDA(cudaEventRecord(evt(slot, k), st));
        CME_CUDA(cudaStreamWaitEvent(ws, evt(slot, k), 0));
        return CME_OK;
    };
    auto done = [&](int slot, int k) -> int {               // marks the end of a piece of side work
        if (!ov) return CME_OK;
        CME_CUDA(cudaEventRecord(evt(slot, 4 + k), ws));
        return CME_OK;
    };
    auto need = [&](int slot, int k) -> int {               // `st` is about to overwrite what that piece reads
        if (!ov) return CME_OK;
        CME_CUDA(cudaStreamWaitEvent(st, evt(slot, 4 + k), 0));
        return CME_OK;
    };
    float* col_s = ov ? e.col_scratch_side : e.col_scratch;
    // LayerNorm backward at `site` (2 l + 1: LN2 of block l, 2 l: LN1, 2 L: final): dx on `st`; the sums of the
    // per-block partial d(gamma) / d(beta) follow on the second stream when there is one
    auto ln_bwd = [&](int site, const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                      const void* dres, void* dxo, void* dgamma, void* dbeta) -> int {
        float* scr = e.ln_scratch + (size_t)site * e.ln_scratch_stride;
        if (!ov) return cme_layernorm_bwd(dt, dy, x, gamma, mean, rstd, dres, dxo, dgamma, dbeta, scr, BT, D, accumulate, st);
        return cme_layernorm_bwd_split(dt, dy, x, gamma, mean, rstd, dres, dxo, dgamma, dbeta, scr, BT, D, accumulate, st, ws,
                                       e.ev_ln[(size_t)site]);
    };
    const void* xlast = d.final_ln ? e.xf : e.x[d.L];
    char* dx = e.dxa;       // gradient w.r.t. the residual stream entering the part being processed
    char* dx_other = e.dxb;
    // ---- output head (the logits buffer holds d(logits); forward already ran on `st`)
    TRY(ready(d.L, 0));
    if (d.tied) {
        TRY(gemm(e, st, BT, D, V, e.logits, e.VL, 0, e.P(e.gs.tok), D, 0, dx, D));                 // dX = dL @ tok
        TRY(gemm(e, ws, V, D, BT, e.logits, e.VL, 1, xlast, D, 0, e.G(e.gs.tok), D, accumulate));  // dtok = dL^T @ X
        TRY(done(d.L, 0));
    } else {
        if (e.wout_pad) TRY(gemm(e, st, BT, D, V, e.logits, e.VL, 0, e.wout_pad, e.VL, 1, dx, D));   // dX = dL @ Wout^T
        else TRY(gemm(e, st, BT, D, V, e.logits, e.VL, 0, e.P(e.gs.Wout), V, 1, dx, D));
        TRY(gemm(e, ws, D, V, BT, xlast, D, 1, e.logits, e.VL, 0, e.G(e.gs.Wout), V, accumulate)); // dWout = X^T @ dL
        TRY(done(d.L, 0));
        emit();
    }
    if (d.final_ln) {
        TRY(ln_bwd(2 * d.L, dx, e.x[d.L], e.P(e.gs.lnfg), e.meanf, e.rstdf, nullptr, dx_other, e.G(e.gs.lnfg),
                   e.G(e.gs.lnfb)));
        std::swap(dx, dx_other);
        emit();
    }
    for (int l = d.L - 1; l >= 0; --l) {
        const CmeLayerSlots& s = e.ls[l];
        LayerAct& a = e.la[l];
        const bool below_top = l < d.L - 1;     // the layer above left side work that reads the shared temporaries
        // ---- FFN2:  x_next = x_mid + ff_act @ W2 + b2
        // a.ffpre holds GELU'(pre-activation); relu'(pre) == (act > 0).  The product's epilogue also sums d ff_pre
        // over rows (the gradient of b1) when the kernel that runs can; the sums are finished on the side stream.
        const void* aux = d.act == CME_ACT_GELU ? a.ffpre : a.ffact;
        const bool fused = d.fuse_epilogues != 0 && d.ffn_lowp == 0;
        const bool deriv = fused && ffn_deriv();
        int slabs = 0;
        TRY(ready(l, 0));                                                   // dx exists
        if (below_top) TRY(need(l + 1, 1));                                 // dff is still read by the layer above's dW1
        bool db1_done = false;
        if (d.ffn_lowp == 2) {
            // the four feed-forward gradient products on bf16 copies, all on the caller's stream (the copies are
            // shared temporaries); FINAL_CLEAN_CODE_/src/model/transformer.cu:468-489
            TRY(to_bf16(dx, e.lp_x, (long long)BT * D, st));
            TRY(to_bf16(e.P(s.W2), e.lp_w, (long long)D * FF, st));
            TRY(gemm_lp(e, st, BT, FF, D, e.lp_x, D, 0, e.lp_w, D, 1, e.dff, FF));
            TRY(cme_dact_colsum(dt, e.dff, aux, e.dff, e.G(s.b1), e.col_scratch, BT, FF, d.act, accumulate, st));
            TRY(to_bf16(a.ffact, e.lp_h, (long long)BT * FF, st));
            TRY(gemm_lp(e, st, FF, D, BT, e.lp_h, FF, 1, e.lp_x, D, 0, e.G(s.W2), D, accumulate));
            TRY(cme_dact_colsum(dt, dx, nullptr, nullptr, e.G(s.b2), e.col_scratch, BT, D, 0, accumulate, st));
            TRY(ready(l, 0));
            TRY(done(l, 0));
            emit();
            TRY(to_bf16(e.dff, e.lp_h, (long long)BT * FF, st));
            TRY(to_bf16(e.P(s.W1), e.lp_w, (long long)D * FF, st));
            TRY(gemm_lp(e, st, BT, D, FF, e.lp_h, FF, 0, e.lp_w, FF, 1, e.dln, D));
            TRY(to_bf16(a.ln2, e.lp_x, (long long)BT * D, st));
            TRY(gemm_lp(e, st, D, FF, BT, e.lp_x, D, 1, e.lp_h, FF, 0, e.G(s.W1), FF, accumulate));
            TRY(ready(l, 1));
            TRY(done(l, 1));
            emit();
        } else {
            if (fused) {
                TRY(gemm(e, st, BT, FF, D, dx, D, 0, e.P(s.W2), D, 1, e.dff, FF, 0, nullptr, 0, nullptr, d.act, aux, FF, nullptr,
                         0, 1, 0, 0, 0, /*aux_deriv=*/deriv ? 1 : 0, deriv && ffn_colsum() ? e.slab_scratch : nullptr,
                         &slabs));
            } else {
                // plain product, then the derivative and the bias gradient in one element-wise pass (the reference's
                // fused_relu_backward_bias_backward_kernel, FINAL_CLEAN_CODE_/src/kernels/activations.cu:247-283)
                TRY(gemm(e, st, BT, FF, D, dx, D, 0, e.P(s.W2), D, 1, e.dff, FF));
                TRY(cme_dact_colsum(dt, e.dff, aux, e.dff, e.G(s.b1), e.col_scratch, BT, FF, d.act, accumulate, st));
                db1_done = true;
            }
            TRY(gemm(e, ws, FF, D, BT, a.ffact, FF, 1, dx, D, 0, e.G(s.W2), D, accumulate));
            TRY(cme_dact_colsum(dt, dx, nullptr, nullptr, e.G(s.b2), col_s, BT, D, 0, accumulate, ws));
            TRY(done(l, 0));
            emit();
            // ---- FFN1:  ff_pre = ln2 @ W1 + b1   (e.dff now holds d ff_pre)
            TRY(ready(l, 1));                                                   // dff exists
            TRY(gemm(e, st, BT, D, FF, e.dff, FF, 0, e.P(s.W1), FF, 1, e.dln, D));
            TRY(gemm(e, ws, D, FF, BT, a.ln2, D, 1, e.dff, FF, 0, e.G(s.W1), FF, accumulate));
            if (slabs) TRY(cme_colsum_slabs_finalize(dt, e.slab_scratch, slabs, FF, e.G(s.b1), accumulate, ws));
            else if (!db1_done) TRY(cme_dact_colsum(dt, e.dff, nullptr, nullptr, e.G(s.b1), col_s, BT, FF, 0, accumulate, ws));
            TRY(done(l, 1));
            emit();
        }
        // ---- LN2 (+ residual gradient): d x_mid = LN'(d ln2) + dx
        if (below_top) TRY(need(l + 1, 2));                                 // dx_other is read by the layer above's dWo
        TRY(ln_bwd(2 * l + 1, e.dln, a.xmid, e.P(s.ln2g), a.mean2, a.rstd2, dx, dx_other, e.G(s.ln2g), e.G(s.ln2b)));
        std::swap(dx, dx_other);                                            // dx = d x_mid
        emit();
        // ---- attention output projection:  x_mid = x + attn @ Wo
        TRY(ready(l, 2));                                                   // d x_mid exists
        TRY(gemm(e, st, BT, D, D, dx, D, 0, e.P(s.Wo), D, 1, e.dattn, D));
        TRY(gemm(e, ws, D, D, BT, a.attn, D, 1, dx, D, 0, e.G(s.Wo), D, accumulate));
        TRY(done(l, 2));
        emit();
        // ---- attention
        CmeAttn at;
        fill_attn(e, l, at);
        at.o = a.attn; at.d_o = e.dattn;
        if (below_top) TRY(need(l + 1, 3));                                 // dqkv is read by the layer above's dWqkv
        // dQ scratch of the tensor-core kernel (arrival-order form): the layers alternate between two buffers, and a
        // buffer is cleared on the second stream as soon as its sums have been converted -- two layers before it is
        // needed again -- instead of by a clear in front of every launch on this stream.  Both start clear (bind), and
        // a step ends with both cleared again, since the caller joins the second stream before the next step.
        const bool side_clear = ov && at.dq_mode == 0 && (d.attn_backend == 0 || d.attn_backend == 1) &&
                                attention_tc_supported(&at);
        const int b01 = l & 1;
        if (side_clear) {
            at.dq_accum = b01 ? e.dq_accum2 : e.dq_accum;
            at.dq_accum_clean = 1;
            if (l + 2 <= d.L - 1) CME_CUDA(cudaStreamWaitEvent(st, e.ev_dq[2 + b01], 0));   // cleared after layer l + 2
        }
        TRY(cme_attention_bwd(&at, d.attn_backend, st));
        if (side_clear) {
            CME_CUDA(cudaEventRecord(e.ev_dq[b01], st));
            CME_CUDA(cudaStreamWaitEvent(ws, e.ev_dq[b01], 0));
            CME_CUDA(cudaMemsetAsync(at.dq_accum, 0, (size_t)BT * D * 4, ws));
            CME_CUDA(cudaEventRecord(e.ev_dq[2 + b01], ws));
        }
        // ---- QKV projection
        TRY(ready(l, 3));                                                   // dqkv exists
        if (d.fused_qkv) {
            TRY(gemm(e, st, BT, D, 3 * D, e.dqkv, 3 * D, 0, e.P(s.Wqkv), 3 * D, 1, e.dln, D));
            TRY(gemm(e, ws, D, 3 * D, BT, a.ln1, D, 1, e.dqkv, 3 * D, 0, e.G(s.Wqkv), 3 * D, accumulate));
        } else {
            const long long pl = (long long)BT * D * e.es, wm = (long long)D * D * e.es;
            for (int i = 0; i < 3; ++i)
                TRY(gemm(e, st, BT, D, D, e.dqkv + i * pl, D, 0, e.P(s.Wq) + i * wm, D, 1, e.dln, D, i > 0));
            TRY(gemm(e, ws, D, D, BT, a.ln1, D, 1, e.dqkv, D, 0, e.G(s.Wq), D, accumulate, nullptr, 0, nullptr, 0,
                     nullptr, 0, nullptr, 0, 3, 0, (long long)BT * D, (long long)D * D));
        }
        TRY(done(l, 3));
        emit();
        // ---- LN1 (+ residual gradient): d x = LN'(d ln1) + d x_mid
        TRY(need(l, 0));                                                    // dx_other is still read by this layer's dW2
        TRY(ln_bwd(2 * l, e.dln, e.x[l], e.P(s.ln1g), a.mean1, a.rstd1, dx, dx_other, e.G(s.ln1g), e.G(s.ln1b)));
        std::swap(dx, dx_other);
        emit();
    }
    // ---- embeddings (tied: the table gradient already holds the output-head part, so the scatter adds).  Everything
    // on the second stream joins here: the head's table gradient before the scatter adds to it, and the rest so that
    // the caller's stream alone orders the end of backward.
    if (ov) {
        cudaEvent_t fin = evt(d.L, 5);
        CME_CUDA(cudaEventRecord(fin, ws));
        CME_CUDA(cudaStreamWaitEvent(st, fin, 0));
    }
    // the two tables are independent: the position table's sums run on the second stream beside the token scatter,
    // and join before the last bucket is handed over
    if (ov) {
        cudaEvent_t dx0 = evt(d.L, 6), posd = evt(d.L, 7);
        CME_CUDA(cudaEventRecord(dx0, st));
        CME_CUDA(cudaStreamWaitEvent(ws, dx0, 0));
        TRY(cme_embedding_bwd(dt, tokens, dx, nullptr, e.G(e.gs.pos), BT, d.T, D, V, accumulate, ws));
        CME_CUDA(cudaEventRecord(posd, ws));
        TRY(cme_embedding_bwd(dt, tokens, dx, e.G(e.gs.tok), nullptr, BT, d.T, D, V, (d.tied || accumulate) ? 1 : 0, st));
        CME_CUDA(cudaStreamWaitEvent(st, posd, 0));
    } else {
        TRY(cme_embedding_bwd(dt, tokens, dx, e.G(e.gs.tok), nullptr, BT, d.T, D, V, (d.tied || accumulate) ? 1 : 0, st));
        TRY(cme_embedding_bwd(dt, tokens, dx, nullptr, e.G(e.gs.pos), BT, d.T, D, V, accumulate, st));
    }
    emit();
    return CME_OK;
}
