"""Element-wise, LayerNorm, embedding, loss and optimizer kernels against PyTorch fp32 references.

Covers what the reference checks in FINAL_CLEAN_CODE_/tests/test_layernorm.cu, test_fusion_benchmark.cu
(fused vs unfused equivalence) and NEW_code/tests/test_embedding.cu, test_softmax_ce.cu, plus backward
kernels, which the reference only exercises through its integration test."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def _ops():
    from cme213_final_project_b200 import ops
    return ops


def _tol(dtype):
    return 1e-4 if dtype == torch.float32 else 3e-2


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(dtype)


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    ref = b.float().abs().max().item() + 1e-6
    assert err <= tol * max(ref, 1.0), f"err {err} ref {ref}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,D", [(2048, 128), (512, 768), (100, 1024), (33, 100), (64, 2048)])
def test_layernorm_forward_backward(dtype, rows, D):
    ops = _ops()
    x, res = _rand((rows, D), dtype, 1), _rand((rows, D), dtype, 2)
    g, b = _rand((D,), dtype, 3) + 1, _rand((D,), dtype, 4)
    y, mean, rstd, summed = ops.layernorm_fwd(x, g, b, 1e-5, residual=res, save_sum=True)
    xs = x.float() + res.float()
    _close(summed, xs, _tol(dtype))
    xs = summed.float().requires_grad_(True)
    gf, bf = g.float().requires_grad_(True), b.float().requires_grad_(True)
    ref = F.layer_norm(xs, (D,), gf, bf, 1e-5)
    _close(y, ref, _tol(dtype))
    y2, _, _, _ = ops.layernorm_fwd(summed, g, b, 1e-5)
    _close(y2, ref, _tol(dtype))
    dy, dres = _rand((rows, D), dtype, 5), _rand((rows, D), dtype, 6)
    ref.backward(dy.float())
    dx, dg, db = ops.layernorm_bwd(dy, summed, g, mean, rstd, dres=dres)
    _close(dx, xs.grad + dres.float(), _tol(dtype))
    _close(dg, gf.grad, _tol(dtype) * 4)
    _close(db, bf.grad, _tol(dtype) * 4)
    dx2, dg2, db2 = ops.layernorm_bwd(dy, summed, g, mean, rstd, dres=dres)
    assert torch.equal(dg, dg2) and torch.equal(db, db2) and torch.equal(dx, dx2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["relu", "gelu", None])
@pytest.mark.parametrize("rows,cols", [(2048, 512), (31, 100)])
def test_bias_act_residual_and_backward(dtype, act, rows, cols):
    ops = _ops()
    x, bias, res = _rand((rows, cols), dtype, 7), _rand((cols,), dtype, 8), _rand((rows, cols), dtype, 9)
    out, pre = ops.bias_act_residual(x, bias, act, res, save_pre=True)
    p = x.float() + bias.float()
    a = torch.relu(p) if act == "relu" else F.gelu(p, approximate="tanh") if act == "gelu" else p
    _close(pre, p, _tol(dtype))
    _close(out, a + res.float(), _tol(dtype))
    dout = _rand((rows, cols), dtype, 10)
    g, dbias = ops.dact_colsum(dout, pre, act)
    pf = pre.float().requires_grad_(True)
    a = torch.relu(pf) if act == "relu" else F.gelu(pf, approximate="tanh") if act == "gelu" else pf * 1.0
    a.backward(dout.float())
    _close(g, pf.grad, _tol(dtype))
    _close(dbias, g.float().sum(0), _tol(dtype) * 8)
    _, db_only = ops.dact_colsum(dout)
    _close(db_only, dout.float().sum(0), _tol(dtype) * 8)


@pytest.mark.parametrize("dtype", DTYPES)
def test_fused_equals_unfused(dtype):
    """bias+activation+residual in one kernel equals the three-kernel pipeline bit for bit in fp32."""
    ops = _ops()
    x, bias, res = _rand((2048, 512), dtype, 11), _rand((512,), dtype, 12), _rand((2048, 512), dtype, 13)
    fused, _ = ops.bias_act_residual(x, bias, "relu", res)
    step1, _ = ops.bias_act_residual(x, bias, None, None)
    step2, _ = ops.bias_act_residual(step1, None, "relu", None)
    unfused = ops.add(step2, res)
    tol = 0 if dtype == torch.float32 else 6.25e-2   # one bf16 ulp at |x| < 8
    assert (fused.float() - unfused.float()).abs().max().item() <= tol


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,D,B,T", [(65, 128, 32, 64), (7, 8, 2, 4), (50304, 64, 2, 128)])
def test_embedding(dtype, V, D, B, T):
    ops = _ops()
    tok, pos = _rand((V, D), dtype, 14), _rand((T, D), dtype, 15)
    ids = torch.randint(0, V, (B * T,), device="cuda", dtype=torch.int32, generator=torch.Generator(device="cuda").manual_seed(1))
    out = ops.embedding_fwd(ids, tok, pos)
    ref = tok.float()[ids.long()] + pos.float().repeat(B, 1)
    _close(out, ref, _tol(dtype))
    dout = _rand((B * T, D), dtype, 16)
    dtok, dpos = ops.embedding_bwd(ids, dout, V, T)
    rt = torch.zeros(V, D, device="cuda").index_add_(0, ids.long(), dout.float())
    _close(dtok, rt, _tol(dtype) * 2)
    _close(dpos, dout.float().view(B, T, D).sum(0), _tol(dtype) * 4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,V", [(256, 512), (128, 4096), (64, 65), (16, 50304)])
def test_cross_entropy(dtype, rows, V):
    ops = _ops()
    logits = _rand((rows, V), dtype, 17, 2.0)
    tg = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    loss, dl, losses = ops.cross_entropy(logits, tg)
    lf = logits.float().requires_grad_(True)
    ref = F.cross_entropy(lf, tg.long())
    ref.backward()
    assert abs(loss.item() - ref.item()) <= 1e-4 * max(1.0, abs(ref.item()))
    _close(dl, lf.grad, 1e-5 if dtype == torch.float32 else 2e-2)
    loss2, _, _ = ops.cross_entropy(logits, tg, prob_eps=1e-9)       # the reference's -log(p + 1e-9) form
    e = torch.exp(logits.double() - logits.double().max(-1, keepdim=True).values)
    pt = e.gather(1, tg.long()[:, None]).squeeze(1) / (e.sum(-1) + 1e-9)
    ref2 = -(torch.log(pt + 1e-9)).mean().item()
    assert abs(loss2.item() - ref2) <= 1e-4 * max(1.0, abs(ref2))
    l3, dl3, _ = ops.cross_entropy(logits.clone(), tg, inplace=True)
    assert torch.equal(dl3, dl)


def test_adam_matches_closed_form_and_torch():
    ops = _ops()
    n = 10007
    p0 = _rand((n,), torch.float32, 18)
    g = _rand((n,), torch.float32, 19, 0.1)
    step = torch.ones(1, dtype=torch.int32, device="cuda")
    lr = torch.full((1,), 1e-3, device="cuda")
    # first Adam step in closed form (FINAL_CLEAN_CODE_/tests/test_model_reference.cu:320-342)
    p, m, v = p0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    nsq = ops.grad_normsq(g)
    assert abs(nsq.item() - g.double().pow(2).sum().item()) <= 1e-4 * nsq.item()
    ops.adam_step(p, g, m, v, step, lr, normsq=nsq, clip_norm=1.0)
    clip = min(1.0, 1.0 / nsq.sqrt().item())
    ge = g * clip
    ref = p0 - 1e-3 * ge / (ge.abs() + 1e-8)
    assert (p - ref).abs().max().item() <= 5e-6
    # AdamW, several steps, bf16 grads, bf16 compute copy, no-decay ranges, vs torch.optim.AdamW
    pt = torch.nn.Parameter(p0.clone())
    nd = torch.nn.Parameter(p0[:100].clone())
    opt = torch.optim.AdamW([{"params": [pt], "weight_decay": 0.1}, {"params": [nd], "weight_decay": 0.0}],
                            lr=1e-3, betas=(0.9, 0.95), eps=1e-8)
    p, m, v = p0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    comp = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    nodecay = torch.tensor([[0, 100]], dtype=torch.int64, device="cuda")
    for t in range(1, 6):
        gb = _rand((n,), torch.bfloat16, 100 + t, 0.1)
        pt.grad, nd.grad = gb.float().clone(), gb.float()[:100].clone()
        opt.step()
        step.fill_(t)
        ops.adam_step(p, gb, m, v, step, lr, compute=comp, beta1=0.9, beta2=0.95, weight_decay=0.1, nodecay=nodecay)
    assert (p[100:] - pt.data[100:]).abs().max().item() <= 1e-5
    assert (p[:100] - nd.data).abs().max().item() <= 1e-5
    assert torch.equal(comp, p.to(torch.bfloat16))


def test_init_uniform_matches_host_formula():
    ops = _ops()
    from cme213_final_project_b200.arena import xorshift_uniform
    out = torch.empty(5000, device="cuda")
    ops.init_uniform_(out, 0.02, 42 + 10)
    assert torch.equal(out.cpu(), xorshift_uniform(5000, 52))


def test_scale_cast_relu_bwd():
    ops = _ops()
    x = _rand((1000,), torch.float32, 30)
    y = ops.cast(x, torch.bfloat16)
    assert torch.equal(y, x.to(torch.bfloat16))
    ops.scale_(x, 0.25)
    dy = _rand((1000,), torch.float32, 31)
    assert torch.equal(ops.relu_bwd(x, dy), dy * (x > 0))
