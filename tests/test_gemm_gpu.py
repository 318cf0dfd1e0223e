"""tcgen05 / SIMT GEMM against a plain PyTorch fp32 reference of the same product.

Strategy of the reference's GEMM unit test (FINAL_CLEAN_CODE_/tests/test_gemm.cu:28-105: CPU triple loop
vs the dispatched kernel at 64^3 ... 512^3, backend-dependent tolerance), widened to every storage
combination, batches, split-K, odd sizes and every epilogue."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from cme213_final_project_b200 import ops
    return ops


def _ref(a, b, a_trans, b_trans):
    A = a.float().transpose(-1, -2) if a_trans else a.float()
    B = b.float().transpose(-1, -2) if b_trans else b.float()
    return A @ B


def _mk(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * 0.5).to(torch.bfloat16)


def _check(out, ref, tol=2e-2):
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= tol * scale, f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("a_trans,b_trans", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (384, 192, 320), (2048, 128, 128), (200, 136, 72)])
def test_tcgen05_layouts(M, N, K, a_trans, b_trans):
    ops = _ops()
    a = _mk((K, M) if a_trans else (M, K), 1)
    b = _mk((N, K) if b_trans else (K, N), 2)
    out = ops.gemm(a, b, a_trans=a_trans, b_trans=b_trans, backend="tcgen05")
    torch.cuda.synchronize()
    assert ops.gemm_check_status() == 0
    _check(out, _ref(a, b, a_trans, b_trans))


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_tcgen05_tile_widths_and_persistence(bn):
    ops = _ops()
    a, b = _mk((1024, 512), 3), _mk((512, 2304), 4)       # more tiles than one wave at bn = 64
    out = ops.gemm(a, b, backend="tcgen05", force_bn=bn)
    torch.cuda.synchronize()
    assert ops.gemm_check_status() == 0
    _check(out, _ref(a, b, False, False))


def test_tcgen05_many_tiles_per_cta():
    ops = _ops()
    a, b = _mk((4096, 256), 5), _mk((256, 4096), 6)        # 32 x 32 tiles of 128 x 128 -> ~7 per CTA
    out = ops.gemm(a, b, backend="tcgen05", force_bn=128)
    torch.cuda.synchronize()
    assert ops.gemm_check_status() == 0
    _check(out, _ref(a, b, False, False))


def test_tcgen05_batched_shared_a():
    ops = _ops()
    a, b = _mk((512, 128), 7), _mk((3, 128, 128), 8)       # the QKV projection: one A, three weight matrices
    out = ops.gemm(a, b, backend="tcgen05")
    torch.cuda.synchronize()
    _check(out, a.float() @ b.float())


def test_tcgen05_batched_both():
    ops = _ops()
    a, b = _mk((4, 256, 64), 9), _mk((4, 192, 64), 10)
    out = ops.gemm(a, b, b_trans=True, backend="tcgen05")
    torch.cuda.synchronize()
    _check(out, a.float() @ b.float().transpose(1, 2))


def test_tcgen05_split_k_wgrad():
    ops = _ops()
    x, dy = _mk((8192, 256), 11), _mk((8192, 128), 12)     # dW[256,128] = x^T dy, K = 8192 tokens
    ref = x.float().t() @ dy.float()
    for splits in (0, 1, 4, 7):
        out = ops.gemm(x, dy, a_trans=True, backend="tcgen05", force_splits=splits)
        torch.cuda.synchronize()
        assert ops.gemm_check_status() == 0
        _check(out, ref)
    base = _mk((256, 128), 13)
    out = base.clone()
    ops.gemm(x, dy, a_trans=True, out=out, accumulate=True, backend="tcgen05", force_splits=4)
    _check(out, ref + base.float())
    again = base.clone()
    ops.gemm(x, dy, a_trans=True, out=again, accumulate=True, backend="tcgen05", force_splits=4)
    assert torch.equal(out, again), "split-K must be bit-reproducible"


@pytest.mark.parametrize("backend", ["tcgen05", "simt"])
def test_epilogues(backend):
    ops = _ops()
    M, N, K = 384, 256, 128
    a, b = _mk((M, K), 14), _mk((K, N), 15)
    bias, res = _mk((N,), 16), _mk((M, N), 17)
    ref = a.float() @ b.float()
    pre = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    out = ops.gemm(a, b, bias=bias, act="gelu", aux_out=pre, residual=res, backend=backend)
    refpre = ref + bias.float()
    _check(pre, refpre)
    _check(out, torch.nn.functional.gelu(refpre, approximate="tanh") + res.float())
    out = ops.gemm(a, b, bias=bias, act="relu", backend=backend)
    _check(out, torch.relu(refpre))
    # activation backward fused into a dgrad product
    x = _mk((M, N), 18)
    out = ops.gemm(a, b, dact="gelu", aux_in=x, backend=backend)
    xf = x.float().requires_grad_(True)
    torch.nn.functional.gelu(xf, approximate="tanh").sum().backward()
    _check(out, ref * xf.grad)
    out = ops.gemm(a, b, dact="relu", aux_in=x, backend=backend)
    _check(out, ref * (x.float() > 0))
    acc = res.clone()
    ops.gemm(a, b, out=acc, accumulate=True, backend=backend)
    _check(acc, ref + res.float())
    o32 = ops.gemm(a, b, out_dtype=torch.float32, backend=backend)
    _check(o32, ref, tol=1e-3)


@pytest.mark.parametrize("M,N,K", [(64, 64, 64), (128, 65, 128), (100, 65, 37), (512, 512, 512)])
def test_simt_fp32_matches_reference(M, N, K):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(20)
    a = torch.randn(M, K, generator=g, device="cuda")
    b = torch.randn(K, N, generator=g, device="cuda")
    out = ops.gemm(a, b, backend="simt")
    ref = (a.double() @ b.double()).float()
    assert (out - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())
    out = ops.gemm(a.t().contiguous(), b.t().contiguous(), a_trans=True, b_trans=True, backend="simt")
    assert (out - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())


def test_auto_dispatch_falls_back_for_vocab_65():
    ops = _ops()
    a, b = _mk((256, 128), 21), _mk((128, 65), 22)          # the reference's output head shape
    out = ops.gemm(a, b)
    _check(out, a.float() @ b.float())


@pytest.mark.parametrize("a_trans,b_trans", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 256), (384, 320, 192), (1000, 520, 328), (2304, 256, 4096)])
def test_cta_pair_tiles(M, N, K, a_trans, b_trans):
    """force_bn=512: the 256 x 256 tile on a CTA pair (cta_group::2), including edges where the second CTA of a
    pair has only padding rows or columns, and many tiles per pair."""
    ops = _ops()
    a = _mk((K, M) if a_trans else (M, K), 31)
    b = _mk((N, K) if b_trans else (K, N), 32)
    out = ops.gemm(a, b, a_trans=a_trans, b_trans=b_trans, backend="tcgen05", force_bn=512)
    assert ops.gemm_check_status() == 0
    _check(out, _ref(a, b, a_trans, b_trans))


@pytest.mark.parametrize("bn", [64, 128, 512])
def test_compile_time_epilogue_variants(bn):
    """Each fused epilogue that has its own kernel instantiation (per tile width), against the same arithmetic in
    fp32; two output tiles per CTA in every direction so the prefetch ring crosses tile boundaries."""
    ops = _ops()
    M, N, K = 1024, 1536 if bn == 512 else 512, 192
    a, b = _mk((M, K), 41), _mk((K, N), 42)
    bias, res, x = _mk((N,), 43), _mk((M, N), 44), _mk((M, N), 45)
    ref = a.float() @ b.float()
    refb = ref + bias.float()
    gelu = lambda t: torch.nn.functional.gelu(t, approximate="tanh")
    kw = dict(backend="tcgen05", force_bn=bn)
    _check(ops.gemm(a, b, bias=bias, **kw), refb)
    _check(ops.gemm(a, b, bias=bias, act="relu", **kw), torch.relu(refb))
    _check(ops.gemm(a, b, residual=res, **kw), ref + res.float())
    _check(ops.gemm(a, b, bias=bias, residual=res, **kw), refb + res.float())
    pre = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    _check(ops.gemm(a, b, bias=bias, act="gelu", aux_out=pre, **kw), gelu(refb))
    _check(pre, refb)
    xf = x.float().requires_grad_(True)
    gelu(xf).sum().backward()
    _check(ops.gemm(a, b, dact="gelu", aux_in=x, **kw), ref * xf.grad)
    _check(ops.gemm(a, b, dact="relu", aux_in=x, **kw), ref * (x.float() > 0))
    acc = res.clone()
    ops.gemm(a, b, out=acc, accumulate=True, **kw)
    _check(acc, ref + res.float())
    _check(ops.gemm(a, b, out_dtype=torch.float32, force_splits=2, **kw).float(), ref, tol=1e-3)
    assert ops.gemm_check_status() == 0


def test_output_narrower_than_a_vector_unit_on_the_tensor_core_path():
    """[M, 65] logits from a tied [65, D] embedding: K-major operands with legal pitches, an output whose rows are
    not 16-byte addressable (direct-store epilogue, no TMA store)."""
    ops = _ops()
    M, V, D = 512, 65, 128
    x, w = _mk((M, D), 53), _mk((V, D), 52)
    logits = ops.gemm(x, w, b_trans=True, backend="tcgen05")
    assert ops.gemm_check_status() == 0
    _check(logits, x.float() @ w.float().t())


@pytest.mark.parametrize("bn", [64, 128, 512])
@pytest.mark.parametrize("M,N", [(1024, 512), (1000, 520)])
def test_derivative_kept_by_forward_and_bias_gradient_in_the_epilogue(bn, M, N):
    """The MLP pair: the forward product stores GELU'(pre-activation) beside the activation (one tanh for both), the
    backward product multiplies by the stored derivative and also sums its output over rows -- the bias gradient
    (the reference's cuBLASLt DRELU_BGRAD epilogue, FINAL_CLEAN_CODE_/src/kernels/gemm.cu:243, and its fused
    ReLU-backward + bias-backward kernel, src/kernels/activations.cu:247-283).  M = 1000 leaves a ragged last slab."""
    ops = _ops()
    K = 192
    if bn == 512:
        N = N * 3
    a, b, bias = _mk((M, K), 61), _mk((K, N), 62), _mk((N,), 63)
    kw = dict(backend="tcgen05", force_bn=bn)
    pre = (a.float() @ b.float() + bias.float()).requires_grad_(True)
    act = torch.nn.functional.gelu(pre, approximate="tanh")
    act.sum().backward()
    d = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    out = ops.gemm(a, b, bias=bias, act="gelu", aux_out=d, aux_deriv=True, **kw)
    _check(out, act.detach())
    _check(d, pre.grad)
    # backward: dC = (g @ w) * d, with its column sums
    g, w = _mk((M, 128), 64), _mk((128, N), 65)
    ref = (g.float() @ w.float()) * d.float()
    for dact, aux, want in (("gelu", d, ref), ("relu", d, (g.float() @ w.float()) * (d.float() > 0))):
        dbias = torch.zeros(N, dtype=torch.bfloat16, device="cuda")
        got = ops.gemm(g, w, dact=dact, aux_in=aux, aux_deriv=True, dbias=dbias, **kw)
        torch.cuda.synchronize()
        assert ops.gemm_check_status() == 0
        _check(got, want)
        assert ops.gemm.last_colsum_slabs == (M + 31) // 32, "the epilogue variant with column sums did not run"
        colref = got.float().sum(0)                      # sums of the stored (bf16) values, like the separate kernel
        err = (dbias.float() - colref).abs().max().item()
        assert err <= 1e-2 * colref.abs().max().item() + 1e-3, err
        again = torch.zeros_like(dbias)
        ops.gemm(g, w, dact=dact, aux_in=aux, aux_deriv=True, dbias=again, **kw)
        assert torch.equal(dbias, again), "column sums must be bit-reproducible"
    # the SIMT kernel honours the same flags (column sums then come from the separate pass)
    dbias = torch.zeros(N, dtype=torch.bfloat16, device="cuda")
    got = ops.gemm(g, w, dact="gelu", aux_in=d, aux_deriv=True, dbias=dbias, backend="simt")
    _check(got, ref)
    assert ops.gemm.last_colsum_slabs == 0
    _check(dbias, got.float().sum(0), tol=1e-2)


@pytest.mark.parametrize("a_trans,b_trans", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K,bn", [(128, 128, 64, 0), (256, 512, 256, 0), (384, 192, 320, 64), (1000, 520, 328, 128),
                                      (1024, 256, 4096, 0), (512, 768, 256, 512), (1024, 1024, 96, 256)])
def test_tf32_products_on_fp32_storage(M, N, K, bn, a_trans, b_trans):
    """fp32 operands multiplied as tf32 on the tcgen05 kernel (every tile shape, both storage orders of both operands
    -- the tensor core takes tf32 operands K-major only, the launcher transposes the others into the workspace --
    split-K through the workspace, ragged edges) against an fp64 product.  tf32 keeps 10 mantissa bits of each
    input: the tolerance is the reference's for its tensor-core backend on fp32 data (5e-3 of the output scale,
    FINAL_CLEAN_CODE_/tests/test_gemm.cu:28-105)."""
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(70)
    a = torch.randn((K, M) if a_trans else (M, K), generator=g, device="cuda") * 0.5
    b = torch.randn((N, K) if b_trans else (K, N), generator=g, device="cuda") * 0.5
    ref = _ref(a.double(), b.double(), a_trans, b_trans)
    out = ops.gemm(a, b, a_trans=a_trans, b_trans=b_trans, backend="tcgen05", force_bn=bn)
    torch.cuda.synchronize()
    assert ops.gemm_check_status() == 0 and out.dtype == torch.float32
    err = (out.double() - ref.double()).abs().max().item()
    assert err <= 2e-3 * ref.abs().max().item(), err
    # accumulate goes through the workspace
    base = torch.randn(M, N, generator=g, device="cuda")
    acc = base.clone()
    ops.gemm(a, b, a_trans=a_trans, b_trans=b_trans, out=acc, accumulate=True, backend="tcgen05", force_bn=bn)
    assert (acc.double() - (ref.double() + base.double())).abs().max().item() <= 2e-3 * ref.abs().max().item()
    # without the permission the tensor-core kernel refuses fp32 data and the dispatcher uses the exact kernel
    exact = ops.gemm(a, b, a_trans=a_trans, b_trans=b_trans, allow_tf32=False)
    assert (exact.double() - ref.double()).abs().max().item() <= 1e-4 * ref.abs().max().item()
