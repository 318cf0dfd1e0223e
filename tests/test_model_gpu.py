"""Native engine against the PyTorch oracle model.

Protocol of the reference's integration test (FINAL_CLEAN_CODE_/tests/test_model_reference.cu:212-350):
a tiny model with deterministic parameters, loss and logits against a float64 CPU model (tolerance 2e-5),
gradients against the oracle (the reference uses finite differences of its CPU model; autograd of the
float64 oracle is the same quantity without the truncation error), one optimizer step against the closed
form.  Then the bf16 production path at the reference's H128 shape and a GPT-mode model."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(cfg, optim, strict, seed=42):
    from cme213_final_project_b200.config import RunConfig
    from cme213_final_project_b200.models.engine import NativeEngine
    from cme213_final_project_b200.models.reference import ReferenceModel
    eng = NativeEngine(cfg, optim, RunConfig(compute_dtype="fp32" if strict else "bf16"), device="cuda", seed=seed)
    ref = ReferenceModel(cfg, optim, device="cpu", dtype=torch.float64, seed=seed, layout=eng.layout)
    return eng, ref


def _sincos_params(layout):
    flat = torch.zeros(layout.total, dtype=torch.float64)
    for s in layout.specs:
        i = torch.arange(s.numel, dtype=torch.float64)
        if s.kind == "ln_gamma":
            v = 1.0 + 0.1 * torch.sin(0.37 * i)
        else:
            v = 0.3 * torch.sin(0.13 * i + s.offset * 0.01) + 0.2 * torch.cos(0.07 * i)
        flat[s.offset:s.offset + s.numel] = v
    return flat


def _tokens(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    n = cfg.tokens_per_step
    x = torch.randint(0, cfg.vocab_size, (n,), generator=g, dtype=torch.int32)
    y = torch.randint(0, cfg.vocab_size, (n,), generator=g, dtype=torch.int32)
    return x, y


def _rel(a, b):
    return ((a.double() - b.double()).norm() / (b.double().norm() + 1e-30)).item()


@pytest.mark.parametrize("mode", ["parity", "gpt"])
def test_strict_fp32_tiny_model_matches_fp64_oracle(mode):
    from cme213_final_project_b200.config import ModelConfig, OptimConfig
    if mode == "parity":
        cfg = ModelConfig(vocab_size=7, seq_len=4, hidden=8, heads=2, ff=16, batch_size=2)
        optim = OptimConfig(lr=1e-3)
    else:
        cfg = ModelConfig(mode="gpt", vocab_size=11, seq_len=8, hidden=16, heads=2, ff=32, layers=2, batch_size=3,
                          activation="gelu", causal=True, head_layout="split", tied_embeddings=True,
                          final_layernorm=True, init="normal")
        optim = OptimConfig(lr=1e-3, beta2=0.95, weight_decay=0.1, clip_norm=0.0)
    eng, ref = _mk(cfg, optim, strict=True)
    p0 = _sincos_params(eng.layout)
    eng.set_params(p0.float())
    with torch.no_grad():
        ref.params.copy_(p0.float().double())
    x, y = _tokens(cfg)
    loss_ref = ref.forward(x, y)
    logits_ref = ref.logits.detach()
    eng.forward(x.cuda(), None)
    assert (eng.logits().cpu().double() - logits_ref).abs().max().item() < 2e-5
    eng.train_step([x.cuda()], [y.cuda()])
    assert abs(eng.read_loss() - loss_ref.item()) < 2e-5
    ref.zero_grad()
    ref.backward()
    g = eng.grads.cpu().double()
    for s in eng.layout.specs:
        sl = slice(s.offset, s.offset + s.numel)
        err = (g[sl] - ref.grads[sl]).abs().max().item()
        assert err < 2e-5 + 1e-4 * ref.grads[sl].abs().max().item(), (s.name, err)
    # one optimizer step
    eng.update()
    ref.update()
    assert (eng.master.cpu().double() - ref.params.detach()).abs().max().item() < 5e-5
    if optim.clip_norm > 0 and optim.weight_decay == 0:      # closed form of the first clipped Adam step
        norm = ref.grads.norm().item()
        ge = ref.grads * min(1.0, optim.clip_norm / norm)
        closed = p0.float().double() - optim.lr * ge / (ge.abs() + optim.eps)
        assert (eng.master.cpu().double() - closed).abs().max().item() < 5e-5


def _cos(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return (a @ b / (a.norm() * b.norm() + 1e-300)).item()


@pytest.mark.parametrize("preset_name", ["parity-h128", "tiny-gpt"])
def test_bf16_engine_tracks_oracle(preset_name):
    """bf16 production path vs the float64 oracle on the same bf16-rounded weights.  With random targets on
    an untrained model the gradient is a small residual of cancelling terms, so bf16 activations cost a few
    percent per tensor; direction and loss must still agree."""
    from cme213_final_project_b200.config import preset
    cfg, optim = preset(preset_name)
    eng, ref = _mk(cfg, optim, strict=False)
    with torch.no_grad():
        ref.params.copy_(eng.params.float().cpu().double())        # same bf16-rounded weights on both sides
    x, y = _tokens(cfg)
    loss_ref = ref.forward(x, y)
    eng.train_step([x.cuda()], [y.cuda()])
    assert abs(eng.read_loss() - loss_ref.item()) < 2e-2
    ref.zero_grad()
    ref.backward()
    g = eng.grads.float().cpu()
    assert _cos(g, ref.grads) > 0.98
    for s in eng.layout.specs:
        sl = slice(s.offset, s.offset + s.numel)
        if ref.grads[sl].abs().max() < 1e-7:
            continue
        assert _cos(g[sl], ref.grads[sl]) > 0.9, (s.name, _cos(g[sl], ref.grads[sl]))
    from cme213_final_project_b200 import ops
    assert ops.gemm_check_status() == 0


@pytest.mark.parametrize("preset_name", ["parity-h128", "parity-h256", "tiny-gpt"])
def test_tcgen05_engine_equals_simt_engine_in_bf16(preset_name):
    """Same bf16 rounding points, different GEMM kernels: only fp32 summation order may differ.  A pre-activation
    that lands on the other side of zero flips its ReLU derivative, which moves single elements of the small bias
    gradients by more than rounding; those tensors must still point the same way."""
    from cme213_final_project_b200.config import RunConfig, preset
    from cme213_final_project_b200.models.engine import NativeEngine
    cfg, optim = preset(preset_name)
    a = NativeEngine(cfg, optim, RunConfig(gemm_backend="tcgen05"), device="cuda")
    b = NativeEngine(cfg, optim, RunConfig(gemm_backend="simt"), device="cuda")
    x, y = _tokens(cfg)
    a.train_step([x.cuda()], [y.cuda()])
    b.train_step([x.cuda()], [y.cuda()])
    assert abs(a.read_loss() - b.read_loss()) < 1e-3
    ga, gb = a.grads.float(), b.grads.float()
    for s in a.layout.specs:
        sl = slice(s.offset, s.offset + s.numel)
        if gb[sl].abs().max() < 1e-9:
            continue
        assert _rel(ga[sl], gb[sl]) < 3e-2 or _cos(ga[sl].double(), gb[sl].double()) > 0.995, \
            (s.name, _rel(ga[sl], gb[sl]), _cos(ga[sl].double(), gb[sl].double()))


def test_gradient_accumulation_equals_big_batch_mean():
    from cme213_final_project_b200.config import ModelConfig, OptimConfig
    cfg = ModelConfig(vocab_size=7, seq_len=4, hidden=8, heads=2, ff=16, batch_size=2)
    eng, _ = _mk(cfg, OptimConfig(), strict=True)
    x1, y1 = _tokens(cfg, 1)
    x2, y2 = _tokens(cfg, 2)
    eng.train_step([x1.cuda()], [y1.cuda()])
    g1, l1 = eng.grads.clone(), eng.read_loss()
    eng.train_step([x2.cuda()], [y2.cuda()])
    g2, l2 = eng.grads.clone(), eng.read_loss()
    eng.train_step([x1.cuda(), x2.cuda()], [y1.cuda(), y2.cuda()])
    assert (eng.grads - 0.5 * (g1 + g2)).abs().max().item() < 1e-6
    assert abs(eng.read_loss() - 0.5 * (l1 + l2)) < 1e-6


def test_training_reduces_loss_and_bucket_callbacks_fire_in_arena_order():
    from cme213_final_project_b200.config import preset
    from cme213_final_project_b200.data import synthetic_batches
    cfg, optim = preset("tiny-gpt")
    eng, _ = _mk(cfg, optim, strict=False)
    x, y = synthetic_batches(cfg.vocab_size, cfg.seq_len, cfg.batch_size, 2, seed=0)
    x, y = x.cuda(), y.cuda()
    seen = []
    buckets = eng.layout.coalesced_buckets(0)
    eng.train_step([x[0]], [y[0]], lambda b: seen.append(b.index), buckets)
    assert seen == list(range(len(buckets)))
    coarse = eng.layout.coalesced_buckets(200000)
    seen.clear()
    eng.train_step([x[0]], [y[0]], lambda b: seen.append((b.start, b.end)), coarse)
    assert seen == [(b.start, b.end) for b in coarse]
    first = eng.read_loss()
    for _ in range(30):
        eng.train_step([x[0]], [y[0]])
        eng.update()
    assert eng.read_loss() < first - 0.5


@pytest.mark.parametrize("graph", [False, True])
def test_early_loss_readback_and_host_batches(graph):
    """``Trainer.step`` takes pinned host batches; ``wait_loss`` returns the step's loss from pinned memory as soon
    as the forward pass has produced it and agrees with the synchronising read, in eager steps and graph replays."""
    from cme213_final_project_b200.config import RunConfig, preset
    from cme213_final_project_b200.data import synthetic_batches
    from cme213_final_project_b200.parallel.dist import DistributedContext
    from cme213_final_project_b200.trainer import Trainer
    cfg, optim = preset("tiny-gpt")
    eng, _ = _mk(cfg, optim, strict=False)
    ctx = DistributedContext()
    ctx.device = torch.device("cuda", 0)
    tr = Trainer(eng, ctx, RunConfig(cuda_graph=graph), optim)
    if graph:
        assert tr.enable_cuda_graph(warmup_steps=2)
    x, y = synthetic_batches(cfg.vocab_size, cfg.seq_len, cfg.batch_size, 6, seed=0)
    x, y = x.pin_memory(), y.pin_memory()
    seen = []
    for i in range(6):
        tr.step([x[i]], [y[i]])
        early = eng.wait_loss()
        torch.cuda.synchronize()
        assert early == eng.read_loss()
        seen.append(early)
    assert len(set(seen)) > 1 and all(math.isfinite(v) for v in seen)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout,causal", [("flat", False), ("split", True), ("split", False)])
@pytest.mark.parametrize("B,H,T,HD", [(2, 4, 64, 32), (1, 2, 100, 64), (2, 1, 37, 128)])
def test_attention_simt_forward_backward(dtype, layout, causal, B, H, T, HD):
    from cme213_final_project_b200 import ops
    from cme213_final_project_b200.config import ModelConfig
    from cme213_final_project_b200.models.reference import attention
    if layout == "flat" and T % H:
        pytest.skip("flat layout needs T % H == 0")
    D = H * HD
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v, do = (torch.randn(B * T, D, generator=g, device="cuda").to(dtype) for _ in range(4))
    cfg = ModelConfig(mode="gpt" if layout == "split" else "parity", seq_len=T, hidden=D, heads=H, causal=causal,
                      head_layout=layout)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = attention(qf, kf, vf, cfg, B)
    ref.backward(do.float())
    out, lse = ops.attention_fwd(q, k, v, B, H, T, layout, causal, backend="simt")
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert (out.float() - ref).abs().max().item() < tol
    dq, dk, dv = ops.attention_bwd(q, k, v, out, lse, do, B, H, T, layout, causal, backend="simt")
    for got, want in ((dq, qf.grad), (dk, kf.grad), (dv, vf.grad)):
        assert (got.float() - want).abs().max().item() < tol * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("preset_name", ["parity-h128", "tiny-gpt"])
def test_tf32_engine_tracks_oracle(preset_name):
    """fp32 storage with tf32 tensor-core products (the reference's default precision: fp32 data, tensor-core math)
    against the float64 oracle on the same weights: loss, every gradient tensor (relative error and direction; tf32
    keeps 10 mantissa bits of each input and the gradients are residuals of cancelling terms), and the loss after
    ten optimizer steps against the strict-fp32 engine."""
    from cme213_final_project_b200 import ops
    from cme213_final_project_b200.config import RunConfig, preset
    from cme213_final_project_b200.models.engine import NativeEngine
    from cme213_final_project_b200.models.reference import ReferenceModel
    cfg, optim = preset(preset_name)
    eng = NativeEngine(cfg, optim, RunConfig(compute_dtype="tf32"), device="cuda", seed=42)
    strict = NativeEngine(cfg, optim, RunConfig(compute_dtype="fp32"), device="cuda", seed=42)
    ref = ReferenceModel(cfg, optim, device="cpu", dtype=torch.float64, seed=42, layout=eng.layout)
    with torch.no_grad():
        ref.params.copy_(eng.master.cpu().double())
    x, y = _tokens(cfg)
    loss_ref = ref.forward(x, y)
    eng.train_step([x.cuda()], [y.cuda()])
    assert abs(eng.read_loss() - loss_ref.item()) < 2e-3
    ref.zero_grad()
    ref.backward()
    g = eng.grads.cpu().double()
    # Direction of the whole gradient and of every tensor.  The bounds are those of an ill-conditioned problem, not of
    # tf32 arithmetic (3e-4 relative per product, tests/test_gemm_gpu.py): on an untrained model with random targets the
    # gradients are residuals of cancelling terms, and a pre-activation that rounds across zero flips its ReLU
    # derivative -- the strict-fp32 engine itself is only within 1e-2 of the float64 oracle on the deeper tensors of
    # the wider reference shapes.
    assert _cos(g, ref.grads) > 0.97
    gmax = ref.grads.abs().max().item()
    for s in eng.layout.specs:
        sl = slice(s.offset, s.offset + s.numel)
        if ref.grads[sl].abs().max() < 1e-7:
            continue
        small = (g[sl] - ref.grads[sl]).abs().max().item() < 1e-3 * gmax
        assert _cos(g[sl], ref.grads[sl]) > 0.9 or small, (s.name, _cos(g[sl], ref.grads[sl]))
    # training follows the strict-fp32 engine: same loss after ten optimizer steps on the same batch (parameter-wise
    # comparison is meaningless under Adam, which moves every parameter by about lr per step whatever the size of its
    # gradient, so near-zero gradients that change sign under tf32 rounding differ by whole steps)
    for _ in range(10):
        for m in (eng, strict):
            m.train_step([x.cuda()], [y.cuda()])
            m.update()
    torch.cuda.synchronize()
    assert abs(eng.read_loss() - strict.read_loss()) < 2e-2 and eng.read_loss() < loss_ref.item()
    assert ops.gemm_check_status() == 0


@pytest.mark.parametrize("base", ["fp32", "tf32"])
@pytest.mark.parametrize("mode", ["store", "bf16"])
@pytest.mark.parametrize("preset_name", ["parity-h128", "tiny-gpt"])
def test_reduced_precision_feed_forward_modes(preset_name, mode, base):
    """fp32 storage with the feed-forward part at reduced precision (the reference's CME213_FP16_STORAGE_ONLY and
    CME213_FFN_FP16 experiments, FINAL_CLEAN_CODE_/src/model/transformer.cu:297-324,468-489, with bf16 as the 16-bit
    type): ``store`` rounds the stored activation to bf16, ``bf16`` runs the four feed-forward products of a block
    on bf16 copies of their operands.  Both stay close to the float64 oracle, differ from the full-precision engine
    (the switch does something) by no more than rounding, and train."""
    from cme213_final_project_b200 import ops
    from cme213_final_project_b200.config import RunConfig, preset
    from cme213_final_project_b200.models.engine import NativeEngine
    from cme213_final_project_b200.models.reference import ReferenceModel
    cfg, optim = preset(preset_name)
    eng = NativeEngine(cfg, optim, RunConfig(compute_dtype=base, ffn_precision=mode), device="cuda", seed=42)
    full = NativeEngine(cfg, optim, RunConfig(compute_dtype=base), device="cuda", seed=42)
    ref = ReferenceModel(cfg, optim, device="cpu", dtype=torch.float64, seed=42, layout=eng.layout)
    with torch.no_grad():
        ref.params.copy_(eng.master.cpu().double())
    x, y = _tokens(cfg)
    loss_ref = ref.forward(x, y)
    for m in (eng, full):
        m.train_step([x.cuda()], [y.cuda()])
    torch.cuda.synchronize()
    assert ops.gemm_check_status() == 0
    assert abs(eng.read_loss() - loss_ref.item()) < 5e-3
    ref.zero_grad()
    ref.backward()
    g, gf = eng.grads.cpu().double(), full.grads.cpu().double()
    assert torch.isfinite(g).all()
    assert _cos(g, ref.grads) > 0.97
    assert not torch.equal(g, gf)                        # the mode changes the arithmetic ...
    assert _cos(g, gf) > 0.97                            # ... by rounding, not by more
    # ten optimizer steps on one batch: the loss falls and follows the full-precision engine
    for _ in range(10):
        for m in (eng, full):
            m.train_step([x.cuda()], [y.cuda()])
            m.update()
    torch.cuda.synchronize()
    assert eng.read_loss() < loss_ref.item() and abs(eng.read_loss() - full.read_loss()) < 3e-2


def test_engine_at_gpt2_small_width_tracks_the_oracle():
    """The production kernels at the width of the headline model -- CTA-pair GEMM tiles with their fused epilogues,
    the tensor-core attention at 12 heads x 1024 tokens x head size 64, the register-resident cross-entropy at a
    50304-token vocabulary, the tied head -- assembled by the engine (2 blocks, 2 sequences) against the float64
    oracle on the same bf16-rounded weights: loss, and every gradient tensor by relative error and direction."""
    from cme213_final_project_b200 import ops
    from cme213_final_project_b200.config import ModelConfig, OptimConfig, RunConfig
    from cme213_final_project_b200.models.engine import NativeEngine
    from cme213_final_project_b200.models.reference import ReferenceModel
    cfg = ModelConfig(mode="gpt", vocab_size=50304, seq_len=1024, hidden=768, heads=12, ff=3072, layers=2, batch_size=2,
                      activation="gelu", causal=True, head_layout="split", tied_embeddings=True, final_layernorm=True,
                      init="normal")
    optim = OptimConfig(lr=3e-4, beta2=0.95, weight_decay=0.1, clip_norm=0.0)
    eng = NativeEngine(cfg, optim, RunConfig(), device="cuda", seed=5)
    ref = ReferenceModel(cfg, optim, device="cuda", dtype=torch.float64, seed=5, layout=eng.layout)
    with torch.no_grad():
        ref.params.copy_(eng.params.double())
    x, y = _tokens(cfg, seed=9)
    loss_ref = ref.forward(x.cuda(), y.cuda())
    eng.train_step([x.cuda()], [y.cuda()])
    torch.cuda.synchronize()
    assert ops.gemm_check_status() == 0 and ops.attention_check_status() == 0
    assert abs(eng.read_loss() - loss_ref.item()) < 2e-2
    ref.zero_grad()
    ref.backward()
    g = eng.grads.double()
    assert _cos(g, ref.grads) > 0.99
    worst = ("", 0.0)
    for s in eng.layout.specs:
        sl = slice(s.offset, s.offset + s.numel)
        if ref.grads[sl].abs().max() < 1e-9:
            continue
        r = _rel(g[sl], ref.grads[sl])
        if r > worst[1]:
            worst = (s.name, r)
        assert _cos(g[sl], ref.grads[sl]) > 0.97, (s.name, _cos(g[sl], ref.grads[sl]))
        assert r < 0.25, (s.name, r)
    print(f"worst per-tensor relative gradient error: {worst[0]} {worst[1]:.4f}")
