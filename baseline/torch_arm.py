"""PyTorch comparator of bench.py (``--impl torch``): the same GPT configuration, synthetic data and timing
protocol as the framework's own arm, built from stock PyTorch parts only -- ``nn.Linear`` / ``torch.matmul``
(cuBLAS), ``F.scaled_dot_product_attention``, ``F.layer_norm``, tanh GELU, ``F.cross_entropy``, bf16 autocast over
fp32 parameters, ``torch.optim.AdamW(fused=True)`` and, for N > 1, ``DistributedDataParallel`` over NCCL with
25 MB buckets.  None of this framework's kernels, engine or synchronisation code is on this path.

It is an independent same-box anchor for configurations the reference cannot express (the reference ships such a
comparison for its own shape, ``FINAL_CLEAN_CODE_/scripts/run_pytorch_baseline.sh:30``); it is NOT the reference
arm and does not answer to ``--impl reference``.
"""
from __future__ import annotations

import json
import os
import sys


def run_torch(a) -> int:
    import torch
    import torch.distributed as dist
    import torch.nn as nn
    import torch.nn.functional as F

    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, here)
    from cme213_final_project_b200.config import preset
    from cme213_final_project_b200.data import synthetic_batches
    from cme213_final_project_b200.utils.clocks import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus:
        print(f"bench.py: --gpus {a.gpus} but WORLD_SIZE={world}", file=sys.stderr)
        return 2
    cfg, optim = preset(a.config)
    if cfg.mode != "gpt":
        print(json.dumps({"impl": "torch", "unavailable": "the PyTorch comparator covers the GPT presets", "n_gpus": world}))
        return 0
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    accum = a.grad_accum or (4 if a.config == "gpt2-medium" else 1)
    D, H, L, FF, V, T, B = cfg.hidden, cfg.heads, cfg.layers, cfg.ff, cfg.vocab_size, cfg.seq_len, cfg.batch_size

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.ln1, self.ln2 = nn.LayerNorm(D), nn.LayerNorm(D)
            self.qkv, self.proj = nn.Linear(D, 3 * D, bias=False), nn.Linear(D, D, bias=False)
            self.fc1, self.fc2 = nn.Linear(D, FF), nn.Linear(FF, D)

        def forward(self, x):
            b, t, _ = x.shape
            q, k, v = self.qkv(self.ln1(x)).view(b, t, 3, H, D // H).permute(2, 0, 3, 1, 4)
            y = F.scaled_dot_product_attention(q, k, v, is_causal=cfg.causal)
            x = x + self.proj(y.transpose(1, 2).reshape(b, t, D))
            return x + self.fc2(F.gelu(self.fc1(self.ln2(x)), approximate="tanh"))

    class GPT(nn.Module):
        def __init__(self):
            super().__init__()
            self.tok, self.pos = nn.Embedding(V, D), nn.Embedding(T, D)
            self.blocks = nn.ModuleList(Block() for _ in range(L))
            self.lnf = nn.LayerNorm(D)

        def forward(self, idx, tgt):
            x = self.tok(idx) + self.pos.weight[: idx.shape[1]]
            for blk in self.blocks:
                x = blk(x)
            logits = F.linear(self.lnf(x), self.tok.weight)              # tied output head
            return F.cross_entropy(logits.view(-1, V).float(), tgt.reshape(-1).long())

    torch.manual_seed(42)
    model = GPT().to(dev)
    for p in model.parameters():
        if p.dim() > 1:
            nn.init.normal_(p, 0.0, 0.02)
    decay = [p for p in model.parameters() if p.dim() > 1]
    nodecay = [p for p in model.parameters() if p.dim() <= 1]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": optim.weight_decay},
                             {"params": nodecay, "weight_decay": 0.0}], lr=optim.lr, betas=(optim.beta1, optim.beta2),
                            eps=optim.eps, fused=True)
    net = nn.parallel.DistributedDataParallel(model, device_ids=[local], bucket_cap_mb=a.bucket_mb,
                                              gradient_as_bucket_view=True) if world > 1 else model

    total = a.warmup + a.steps
    hx, hy = synthetic_batches(V, T, B, total * accum, seed=rank)
    hx, hy = hx.pin_memory(), hy.pin_memory()
    dx, dy = hx.to(dev).view(-1, B, T), hy.to(dev).view(-1, B, T)          # int32 token ids
    sx = torch.empty(accum, B, T, dtype=torch.int32, device=dev)
    sy = torch.empty_like(sx)
    loss_box = [None]

    def step(xs, ys):
        opt.zero_grad(set_to_none=True)
        for i in range(accum):
            ctx = net.no_sync() if (world > 1 and i < accum - 1) else _null()
            with ctx, torch.autocast("cuda", dtype=torch.bfloat16):
                loss = net(xs[i], ys[i]) / accum
            loss.backward()
        opt.step()
        loss_box[0] = loss.detach()

    class _null:
        def __enter__(self): return None
        def __exit__(self, *e): return False

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    def timed(run_step):
        for s in range(a.warmup):
            run_step(s)
        barrier()
        sampler = ClockSampler(local).start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(a.warmup, total):
            run_step(s)
        e1.record()
        barrier()
        clocks = sampler.stop()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() / a.steps, clocks

    ms_step, clocks = timed(lambda s: step(dx[s * accum:(s + 1) * accum], dy[s * accum:(s + 1) * accum]))
    last = [0.0]

    def step_e2e(s):
        for i in range(accum):                                   # int32 token ids from pinned host memory, every step
            sx[i].copy_(hx[s * accum + i].view(B, T), non_blocking=True)
            sy[i].copy_(hy[s * accum + i].view(B, T), non_blocking=True)
        step(sx, sy)
        last[0] = float(loss_box[0].item()) * accum              # 4 bytes back per step

    ms_e2e, clocks_e2e = timed(step_e2e)
    tokens = B * T * accum * world
    bad = [r for r in clocks["reasons"] if r in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")]
    if rank == 0:
        print(json.dumps({
            "metric": "train tokens/sec (device-timed, max over ranks)", "impl": "torch",
            "value": tokens / (ms_step / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 autocast over fp32 parameters", "data": "synthetic uniform token ids (seed = rank), random-init weights",
            "config": {"model": a.config, "global_batch": B * accum * world, "seq_len": T, "micro_batch_per_gpu": B,
                       "grad_accum": accum, "parallelism": f"dp{world}",
                       "sync": f"DDP/NCCL bucket_cap_mb={a.bucket_mb}" if world > 1 else "none",
                       "stack": f"torch {torch.__version__}: SDPA, cuBLAS matmul, fused AdamW, eager",
                       "l2": "per-step working set is far larger than the 126 MB L2"},
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"]},
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": 2 * accum * B * T * 4, "d2h_bytes_per_step": 4},
            "loss": last[0], "rejected": bool(bad)}), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0
