"""Out-of-bounds writes: every kernel's outputs are placed inside a larger buffer filled with a sentinel, the kernel
runs on shapes that do not fill its tiles (ragged rows, columns, sequence lengths), and the sentinel around the
output must be intact afterwards.

The reference has no memory checking of any kind (no sanitizer run in its Makefile or scripts); on this hardware the
tile kernels write through TMA tile stores, bulk reduces and 128-bit vector stores whose bounds come from tensor maps
and hand-written guards, which is exactly where an off-by-one-tile error would land outside the tensor."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
GUARD = 4096
SENTINEL = -12345.0


class Guarded:
    """A tensor of `shape` carved from the middle of a sentinel-filled buffer."""

    def __init__(self, shape, dtype, fill=None):
        n = 1
        for s in shape:
            n *= s
        self.big = torch.full((GUARD + n + GUARD,), SENTINEL, dtype=dtype, device="cuda")
        self.t = self.big[GUARD:GUARD + n].view(*shape)
        if fill is not None:
            self.t.copy_(fill)
        self.n = n

    def intact(self):
        return bool((self.big[:GUARD] == SENTINEL).all().item() and (self.big[GUARD + self.n:] == SENTINEL).all().item())


def _rand(shape, dtype=torch.bfloat16, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * 0.5).to(dtype)


@pytest.mark.parametrize("M,N,K,bn", [(1000, 520, 328, 0), (130, 72, 40, 64), (300, 264, 200, 128), (520, 776, 136, 512),
                                      (129, 8, 64, 0)])
def test_gemm_outputs_stay_inside_their_tensors(M, N, K, bn):
    from cme213_final_project_b200 import ops
    a, b, bias = _rand((M, K), seed=1), _rand((K, N), seed=2), _rand((N,), seed=3)
    res, x = _rand((M, N), seed=4), _rand((M, N), seed=5)
    kw = dict(backend="tcgen05", force_bn=bn)
    cases = [dict(), dict(bias=bias), dict(bias=bias, act="relu"), dict(residual=res), dict(bias=bias, residual=res),
             dict(dact="gelu", aux_in=x), dict(dact="relu", aux_in=x), dict(dact="gelu", aux_in=x, aux_deriv=True)]
    for c in cases:
        out = Guarded((M, N), torch.bfloat16)
        ops.gemm(a, b, out=out.t, **c, **kw)
        torch.cuda.synchronize()
        assert out.intact(), c.keys()
    for deriv in (False, True):
        out, aux = Guarded((M, N), torch.bfloat16), Guarded((M, N), torch.bfloat16)
        ops.gemm(a, b, out=out.t, bias=bias, act="gelu", aux_out=aux.t, aux_deriv=deriv, **kw)
        torch.cuda.synchronize()
        assert out.intact() and aux.intact()
    out, db = Guarded((M, N), torch.bfloat16), Guarded((N,), torch.bfloat16)
    ops.gemm(a, b, out=out.t, dact="gelu", aux_in=x, aux_deriv=True, dbias=db.t, **kw)
    torch.cuda.synchronize()
    assert out.intact() and db.intact()
    acc = Guarded((M, N), torch.bfloat16, fill=res)
    ops.gemm(a, b, out=acc.t, accumulate=True, **kw)
    o32 = Guarded((M, N), torch.float32)
    ops.gemm(a, b, out=o32.t, **kw)
    torch.cuda.synchronize()
    assert acc.intact() and o32.intact()
    if N % 4 == 0 and K % 4 == 0:                         # fp32 storage, tf32 products (and their transposed copies)
        o = Guarded((M, N), torch.float32)
        ops.gemm(a.float(), b.float(), out=o.t, **kw)
        torch.cuda.synchronize()
        assert o.intact()
    assert ops.gemm_check_status() == 0


def test_split_k_weight_gradient_stays_inside():
    from cme213_final_project_b200 import ops
    x, dy = _rand((4000, 200), seed=6), _rand((4000, 136), seed=7)
    for splits in (0, 3, 5):
        out = Guarded((200, 136), torch.bfloat16)
        ops.gemm(x, dy, a_trans=True, out=out.t, backend="tcgen05", force_splits=splits)
        torch.cuda.synchronize()
        assert out.intact()


def test_row_kernels_stay_inside():
    from cme213_final_project_b200 import ops
    rows, D = 301, 776
    x, dy, g, b = _rand((rows, D), seed=8), _rand((rows, D), seed=9), _rand((D,), seed=10), _rand((D,), seed=11)
    y, mean, rstd = ops.layernorm_fwd(x, g, b)[:3]
    dg, dbt = Guarded((D,), torch.bfloat16), Guarded((D,), torch.bfloat16)
    ops.layernorm_bwd(dy, x, g, mean, rstd, dgamma=dg.t, dbeta=dbt.t)
    db = Guarded((D,), torch.bfloat16)
    ops.dact_colsum(dy, x, "gelu", dbias=db.t)
    # cross-entropy in place on a row pitch that is not a power of two
    V = 4104
    logits = Guarded((rows, V), torch.bfloat16, fill=_rand((rows, V), seed=12))
    tgt = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    ops.cross_entropy(logits.t, tgt, inplace=True)
    torch.cuda.synchronize()
    assert dg.intact() and dbt.intact() and db.intact() and logits.intact()


def test_embedding_and_optimizer_stay_inside():
    from cme213_final_project_b200 import ops
    V, T, D, B = 67, 24, 136, 5
    tokens = torch.randint(0, V, (B * T,), device="cuda", dtype=torch.int32)
    dout = _rand((B * T, D), seed=13)
    dtok, dpos = Guarded((V, D), torch.bfloat16, fill=torch.zeros(V, D)), Guarded((T, D), torch.bfloat16, fill=torch.zeros(T, D))
    ops.embedding_bwd(tokens, dout, V, T, dtok=dtok.t, dpos=dpos.t)
    n = 1000 * 4
    master, m, v = (Guarded((n,), torch.float32, fill=torch.zeros(n)) for _ in range(3))
    comp = Guarded((n,), torch.bfloat16, fill=torch.zeros(n))
    grads = _rand((n,), seed=14)
    step = torch.ones(1, dtype=torch.int32, device="cuda")
    lr = torch.full((1,), 1e-3, device="cuda")
    ops.adam_step(master.t, grads, m.t, v.t, step, lr, compute=comp.t)
    torch.cuda.synchronize()
    assert dtok.intact() and dpos.intact() and master.intact() and m.intact() and v.intact() and comp.intact()


@pytest.mark.parametrize("T,causal", [(200, True), (129, False), (384, True)])
def test_attention_outputs_stay_inside(T, causal):
    """Ragged sequence lengths through the tensor-core kernels: O, the log-sum-exp, dQ (through its fp32 scratch), dK
    and dV; all three ways the backward completes dQ."""
    from cme213_final_project_b200 import ops
    B, H = 2, 3
    D = H * 64
    q, k, v, do = (_rand((B * T, D), seed=20 + i) for i in range(4))
    a = ops._attn_desc(q, B, H, T, "split", causal)
    out, lse = Guarded((B * T, D), torch.bfloat16), Guarded((B * H * T,), torch.float32)
    a.q, a.k, a.v, a.o, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.t.data_ptr(), lse.t.data_ptr()
    ops._check(ops.lib().cme_attention_fwd(ctypes.byref(a), 1, ops._stream()))
    torch.cuda.synchronize()
    assert out.intact() and lse.intact()
    for mode in (0, 1, 2):        # cleared scratch + conversion kernel | ordered adds | last part finishes
        dq, dk, dv = (Guarded((B * T, D), torch.bfloat16) for _ in range(3))
        delta = Guarded((B * H * T,), torch.float32)
        acc = Guarded((B * T * D,), torch.float32, fill=torch.zeros(B * T * D))
        sem = Guarded((B * H * ((T + 127) // 128),), torch.int32, fill=torch.zeros(B * H * ((T + 127) // 128), dtype=torch.int32))
        a.d_o, a.dq, a.dk, a.dv = do.data_ptr(), dq.t.data_ptr(), dk.t.data_ptr(), dv.t.data_ptr()
        a.delta, a.dq_accum = delta.t.data_ptr(), acc.t.data_ptr()
        a.dq_sem, a.dq_mode = sem.t.data_ptr(), mode
        ops._check(ops.lib().cme_attention_bwd(ctypes.byref(a), 1, ops._stream()))
        torch.cuda.synchronize()
        assert ops.attention_check_status() == 0
        assert dq.intact() and dk.intact() and dv.intact() and delta.intact() and acc.intact() and sem.intact(), mode
        if mode:
            assert int(sem.t.abs().sum().item()) == 0, "the counters must be left at zero"
        if mode == 2:
            assert acc.t.abs().max().item() == 0.0, "the scratch must be left clear"
