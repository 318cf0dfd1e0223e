"""Two gloo ranks on CPU: data-parallel plumbing against a single-process reference.  Run by test_dp_cpu.py."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    mode = sys.argv[1]
    from cme213_final_project_b200.config import RunConfig, preset
    from cme213_final_project_b200.data import synthetic_batches
    from cme213_final_project_b200.models.reference import ReferenceModel
    from cme213_final_project_b200.parallel.dist import DistributedContext
    from cme213_final_project_b200.trainer import Trainer
    torch.set_num_threads(2)
    cfg, optim = preset("tiny-gpt")
    run = RunConfig(sync_mode="blocking" if mode == "blocking" else "overlap", bucket_kb=64 if mode != "blocking" else 0,
                    device="cpu")
    ctx = DistributedContext().init(backend="gloo", device="cpu", comm_thread=(mode == "thread"),
                                    defer_grad_avg=(mode == "defer"), timeout_s=60)
    W, R = ctx.world_size, ctx.rank
    model = ReferenceModel(cfg, optim, device="cpu", dtype=torch.float32, seed=42)
    single = ReferenceModel(cfg, optim, device="cpu", dtype=torch.float32, seed=42)
    tr = Trainer(model, ctx, run, optim)
    steps = 10
    x, y = synthetic_batches(cfg.vocab_size, cfg.seq_len, cfg.batch_size, steps * W, seed=0)
    worst_g = worst_l = 0.0
    if mode == "drop":
        ctx.drop_next_bucket = (R == 1)           # injected fault: rank 1 loses one bucket hand-off
    for s in range(steps):
        tr.step([x[s * W + R]], [y[s * W + R]])
        # single-process reference: mean gradient over both ranks' batches
        single.zero_grad()
        losses = []
        for r in range(W):
            single.forward(x[s * W + r], y[s * W + r])
            losses.append(single.read_loss())
            single.backward(scale=1.0 / W)
        if mode != "drop":
            g = model.grads if not ctx.defer_gradient_average else model.grads / W
            worst_g = max(worst_g, (g - single.grads).abs().max().item())
            worst_l = max(worst_l, abs(model.read_loss() - losses[R]))
        single.update()
    span = ctx.max_double(float(model.params.double().sum())) - ctx.min_double(float(model.params.double().sum()))
    diff = (model.params.detach() - single.params.detach()).abs().max().item()
    if R == 0:
        print("DP_RESULT " + json.dumps({"mode": mode, "grad_err": worst_g, "loss_err": worst_l, "span": span,
                                         "param_err": diff, "overlap": tr.use_overlap, "buckets": len(tr.buckets),
                                         "start_ms": tr.async_start_ms_sum, "sync_ms": tr.comm_ms_sum}), flush=True)
    ctx.finalize()


if __name__ == "__main__":
    main()
