"""The allocation-free bias-gradient entry point, called through its exported C symbol.

Some users of the native library cannot get device memory when they need a bias gradient: they run where
another allocator already owns the GPU's free memory, or under a host contract that forbids cudaMalloc /
cudaFree (both synchronise the device), or from plain C without any caching allocator.  For them the
library carries a fixed 1 MiB scratch array of its own.  This file checks that the entry point that uses it
gives the same numbers as the regular one (which takes a caller-allocated scratch buffer), on two calls in a
row that share the array, and that it refuses problems that do not fit.  The file name sorts last so a run
that stops at the first failure has already run everything else."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, ops, dout, pre, act, want_g, dbias=None, accumulate=False):
    rows, cols = dout.shape
    g = torch.empty_like(dout) if want_g else None
    if dbias is None:
        dbias = torch.empty(cols, dtype=dout.dtype, device=dout.device)
    ptr = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())
    rc = lib.cme_dact_colsum_noalloc(ops._dt(dout), ptr(dout), ptr(pre), ptr(g), ptr(dbias), rows, cols,
                                     ops.ACT[act], int(accumulate),
                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, g, dbias


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_matches_regular_entry_point_twice(dtype):
    from cme213_final_project_b200 import ops
    lib = ops.lib()
    gen = torch.Generator(device="cuda").manual_seed(5)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    # two calls back to back on the shared scratch: different shapes, so stale partial sums would show
    for rows, cols, act in ((4096, 512, "gelu"), (300, 136, "relu")):
        dout = torch.randn(rows, cols, generator=gen, device="cuda").to(dtype)
        pre = torch.randn(rows, cols, generator=gen, device="cuda").to(dtype)
        g_ref, db_ref = ops.dact_colsum(dout, pre, act)
        rc, g, db = _call(lib, ops, dout, pre, act, True)
        assert rc == 0, lib.cme_last_error().decode()
        torch.cuda.synchronize()
        assert (g.float() - g_ref.float()).abs().max().item() <= tol
        scale = max(1.0, db_ref.float().abs().max().item())
        assert (db.float() - db_ref.float()).abs().max().item() <= tol * scale
        # and against the same arithmetic in plain PyTorch fp32 (not only against the sibling entry point)
        x = pre.float().requires_grad_(True)
        (torch.nn.functional.gelu(x, approximate="tanh") if act == "gelu" else torch.relu(x)).sum().backward()
        g_torch = dout.float() * x.grad
        assert (g.float() - g_torch).abs().max().item() <= tol * max(1.0, g_torch.abs().max().item())
        db_torch = g.float().sum(0)                 # column sums of the values the kernel stored
        assert (db.float() - db_torch).abs().max().item() <= tol * max(1.0, db_torch.abs().max().item())
    # plain column sum with accumulation into an existing gradient
    dout = torch.randn(1000, 72, generator=gen, device="cuda").to(dtype)
    base = torch.randn(72, generator=gen, device="cuda").to(dtype)
    _, want = ops.dact_colsum(dout, dbias=base.clone(), accumulate=True)
    rc, _, got = _call(lib, ops, dout, None, None, False, dbias=base.clone(), accumulate=True)
    assert rc == 0
    assert (got.float() - want.float()).abs().max().item() <= tol * max(1.0, want.float().abs().max().item())
    ref = base.float() + dout.float().sum(0)
    assert (got.float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())


def test_noalloc_refuses_sizes_beyond_its_scratch():
    from cme213_final_project_b200 import ops
    lib = ops.lib()
    cols = 400000                                   # splits * cols > 2**18 floats
    dout = torch.zeros(64, cols, device="cuda")
    rc, _, _ = _call(lib, ops, dout, None, None, False)
    assert rc == 4                                  # CME_ERR_LIMIT
    msg = lib.cme_last_error().decode()
    assert "scratch" in msg and str(cols) in msg
