"""Peer-memory collectives and the fused synchronisation path on 2+ GPUs (child processes, one rank per GPU),
plus the single-GPU degenerate case of the fused kernel."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_fused_kernel_world_of_one_equals_unfused_update():
    from cme213_final_project_b200.config import RunConfig, preset
    from cme213_final_project_b200.models.engine import NativeEngine
    from cme213_final_project_b200.parallel.dist import DistributedContext
    from cme213_final_project_b200.parallel.fused_sync import attach_fused_sync
    cfg, optim = preset("tiny-gpt")
    ctx = DistributedContext()
    ctx.device = torch.device("cuda", 0)
    a = NativeEngine(cfg, optim, RunConfig(), device="cuda", seed=3)
    b = NativeEngine(cfg, optim, RunConfig(bucket_kb=128), device="cuda", seed=3)
    fs = attach_fused_sync(b, ctx, RunConfig(bucket_kb=128, sync_mode="overlap"))
    g = torch.Generator().manual_seed(1)
    n = cfg.tokens_per_step
    for _ in range(3):
        x = torch.randint(0, cfg.vocab_size, (n,), generator=g, dtype=torch.int32).cuda()
        y = torch.randint(0, cfg.vocab_size, (n,), generator=g, dtype=torch.int32).cuda()
        a.train_step([x], [y]); a.update()
        b.train_step([x], [y]); b.update()
    torch.cuda.synchronize()
    assert fs.comm.check_status() == 0 and fs.launched == 3 * len(fs.buckets)
    assert (a.master - b.master).abs().max().item() < 1e-6
    # the two kernels contract their multiply-adds differently: fp32 state agrees to ~1 ulp, so the bf16 copies may
    # differ by one bf16 ulp on a few elements
    assert torch.allclose(a.params.float(), b.params.float(), rtol=8e-3, atol=1e-6)


def test_two_phase_clip_kernels_world_of_one_equal_norm_plus_adam():
    """The clip-compatible fused form (reduce-only kernels that keep fp32 gradients and their sum of squares, then
    one clip + Adam kernel) against the separate norm and Adam kernels, on the reference's model and optimizer
    (Adam, global-norm clip), with a threshold low enough that the clip is active."""
    import dataclasses
    from cme213_final_project_b200.config import RunConfig, preset
    from cme213_final_project_b200.models.engine import NativeEngine
    from cme213_final_project_b200.parallel.dist import DistributedContext
    from cme213_final_project_b200.parallel.fused_sync import attach_fused_sync
    cfg, optim = preset("parity-h128")
    optim = dataclasses.replace(optim, clip_norm=0.05)
    ctx = DistributedContext()
    ctx.device = torch.device("cuda", 0)
    a = NativeEngine(cfg, optim, RunConfig(), device="cuda", seed=3)
    b = NativeEngine(cfg, optim, RunConfig(bucket_kb=64), device="cuda", seed=3)
    fs = attach_fused_sync(b, ctx, RunConfig(bucket_kb=64, sync_mode="overlap"))
    assert fs.clip and len(fs.buckets) > 1
    g = torch.Generator().manual_seed(1)
    n = cfg.tokens_per_step
    p0 = a.master.clone()
    for _ in range(3):
        x = torch.randint(0, cfg.vocab_size, (n,), generator=g, dtype=torch.int32).cuda()
        y = torch.randint(0, cfg.vocab_size, (n,), generator=g, dtype=torch.int32).cuda()
        a.train_step([x], [y]); a.update()
        b.train_step([x], [y]); b.update()
    torch.cuda.synchronize()
    assert fs.check_status() == 0 and fs.launched == 3 * (len(fs.buckets) + 1)
    upd = (a.master - p0).abs().max().item()
    # the norm is accumulated in a different order (per bucket and CTA instead of over the whole arena)
    assert (a.master - b.master).abs().max().item() < 1e-3 * upd + 1e-7
    assert torch.allclose(a.params.float(), b.params.float(), rtol=8e-3, atol=1e-6)
    tl = fs.timeline()
    assert len(tl["buckets"]) == len(fs.buckets) + 1 and all(e >= s for s, e in tl["buckets"])


def test_blocking_mode_on_the_fused_path_is_one_call_after_backward():
    from cme213_final_project_b200.config import RunConfig, preset
    from cme213_final_project_b200.models.engine import NativeEngine
    from cme213_final_project_b200.parallel.dist import DistributedContext
    from cme213_final_project_b200.parallel.fused_sync import attach_fused_sync
    cfg, optim = preset("tiny-gpt")
    ctx = DistributedContext()
    ctx.device = torch.device("cuda", 0)
    a = NativeEngine(cfg, optim, RunConfig(), device="cuda", seed=3)
    b = NativeEngine(cfg, optim, RunConfig(), device="cuda", seed=3)
    fs = attach_fused_sync(b, ctx, RunConfig(sync_mode="blocking", bucket_kb=64))
    assert len(fs.buckets) == 1 and fs.buckets[0].numel == b.layout.total and not fs.overlap
    g = torch.Generator().manual_seed(2)
    n = cfg.tokens_per_step
    for _ in range(2):
        x = torch.randint(0, cfg.vocab_size, (n,), generator=g, dtype=torch.int32).cuda()
        y = torch.randint(0, cfg.vocab_size, (n,), generator=g, dtype=torch.int32).cuda()
        a.train_step([x], [y]); a.update()
        b.train_step([x], [y]); b.update()
    torch.cuda.synchronize()
    assert fs.check_status() == 0 and fs.launched == 2
    assert (a.master - b.master).abs().max().item() < 1e-6


def test_bounded_wait_reports_instead_of_hanging():
    """A device-side wait on a flag that nothing sets gives up after its budget and reports through the status word."""
    import ctypes
    from cme213_final_project_b200 import ops
    lib = ops.lib()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    ops._check(lib.cme_comm_wait_probe(ops._p(flag), 1, ctypes.c_double(200.0), ops._p(status), ops._p(waited),
                                       ops._stream()))
    torch.cuda.synchronize()
    assert status.item() == 3                       # CME_ERR_TIMEOUT
    assert 0.15e9 < waited.item() < 1.5e9           # about the 200 ms budget, and the context is still usable
    flag.fill_(1)
    status.zero_()
    ops._check(lib.cme_comm_wait_probe(ops._p(flag), 1, ctypes.c_double(200.0), ops._p(status), ops._p(waited),
                                       ops._stream()))
    torch.cuda.synchronize()
    assert status.item() == 0 and waited.item() < 0.1e9


def test_allreduce_calls_on_one_bucket_may_change_their_grid_size():
    """Consecutive calls on the same bucket with different CTA counts (a size sweep) must each complete their
    barriers: the per-call CTA counters start from zero every time."""
    from cme213_final_project_b200.parallel.fused_sync import PeerComm
    from cme213_final_project_b200.parallel.symm import LocalPeers
    dev = torch.device("cuda", 0)
    comm = PeerComm(dev, max_buckets=2, budget_ms=200.0, single=True)
    src = LocalPeers(torch.randn(1 << 16, device=dev).to(torch.bfloat16))
    dst = LocalPeers(torch.zeros(1 << 16, device=dev, dtype=torch.bfloat16))
    for ctas, n in ((1, 512), (1, 512), (4, 8192), (3, 8192), (16, 1 << 16), (1, 512)):
        for algo in ("one_shot", "two_shot"):
            dst.tensor.zero_()
            comm.allreduce(src, dst, n, algo=algo, bucket=0, ctas=ctas)
            torch.cuda.synchronize()
            assert comm.check_status() == 0
            assert torch.equal(dst.tensor[:n], src.tensor[:n])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_peer_memory_collectives_and_fused_sync():
    n = min(torch.cuda.device_count(), 8)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29641", os.path.join(ROOT, "tests", "mp_fused_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "MP_RESULT" in r.stdout
    print("\n".join(l for l in r.stdout.splitlines() if l.startswith("MP_RESULT")))     # shown with pytest -s


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_training_driver_runs_the_fused_path_in_one_graph(tmp_path):
    """The command-line driver on several GPUs: `--comm-backend fused --cuda-graph` attaches the fused kernels,
    captures the multi-GPU step, keeps the ranks' parameters identical and writes a checkpoint (gathered from the
    sharded optimizer state).  Clipping stays on (the reference's optimizer), so the two-phase form runs."""
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    ck = str(tmp_path / "fused.ckpt")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29643", "-m", "cme213_final_project_b200.train",
           "--preset", "parity-h128", "--synthetic", "--epochs", "1", "--max-steps", "12", "--sync-mode", "overlap",
           "--bucket-kb", "64", "--comm-backend", "fused", "--cuda-graph", "--log-every", "4",
           "--save-checkpoint", ck]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "DP gradient backend: fused" in r.stdout and "CUDA Graph: enabled" in r.stdout, r.stdout[-2000:]
    assert "checksum_span=0.000e+00" in r.stdout, r.stdout[-2000:]
    assert os.path.exists(ck)
