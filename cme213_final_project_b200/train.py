"""Command-line training driver: ``python -m cme213_final_project_b200.train [data] [flags]``.

Flow and output follow the reference driver (``FINAL_CLEAN_CODE_/src/main.cu:134-495``): environment
banner, configuration validation (``--validate-config`` exits 0 after ``Configuration validation: PASS``,
an invalid combination exits 2), tokenizer + dataset, model build, every batch preloaded to the device,
rank-strided batches, per-epoch wall-clock throughput (max over ranks) and cross-rank parameter
checksum span, optional per-step ``TRAJECTORY`` lines, optional whole-step CUDA graph.
"""
from __future__ import annotations

import sys
import time
from typing import List, Optional, Sequence

import torch

from . import checkpoint as ckpt
from .arena import ArenaLayout
from .config import (RunConfig, environment_report, parse_args, validate_environment, validate_run)
from .data import CharTokenizer, Dataset, ShardPlan, read_file, synthetic_batches
from .parallel.dist import DistributedContext
from .trainer import Trainer
from .utils import logfmt


def fused_sync_obstacle(model_cfg, optim_cfg, run: RunConfig, dist_ctx: DistributedContext) -> Optional[str]:
    """Why this run cannot use the fused device synchronisation path, or ``None`` if it can.  A single rank uses it
    too: its world-of-one form is the optimizer applied bucket by bucket on a second stream while backward is still
    running, instead of one pass over the whole arena afterwards."""
    if dist_ctx.device.type != "cuda":
        return "the fused device path needs GPUs"
    if dist_ctx.world_size <= 1 and run.sync_mode != "overlap":
        return "a single rank keeps the one-pass optimizer unless --sync-mode overlap asks for the bucketed one"
    if run.comm_backend not in ("auto", "fused"):
        return f"comm backend '{run.comm_backend}' was requested"
    if run.engine not in ("auto", "native"):
        return "the fused path is part of the native engine"
    if run.compute_dtype != "bf16":
        return "the fused kernels reduce bf16 gradients (--compute-dtype bf16)"
    if run.comm_thread:
        return "--comm-thread drives host-issued collectives"
    return None


def build_model(model_cfg, optim_cfg, run: RunConfig, dist_ctx: DistributedContext, seed: int):
    """Native sm_100a engine on a GPU, PyTorch oracle model otherwise (or on request).  With several GPU ranks the
    engine gets the fused synchronisation path (peer-memory reduce-scatter + optimizer + all-gather kernels, the
    multi-GPU step capturable as one CUDA graph) unless an option rules it out; the reason is then recorded in
    ``dist_ctx.backend_note`` and host-issued NCCL all-reduces are used."""
    use_native = run.engine == "native" or (run.engine == "auto" and dist_ctx.device.type == "cuda")
    if use_native:
        from .models.engine import NativeEngine
        why = fused_sync_obstacle(model_cfg, optim_cfg, run, dist_ctx)
        if why is None:
            from .parallel.fused_sync import attach_fused_sync, shard_align
            model = NativeEngine(model_cfg, optim_cfg, run, dist_ctx, seed=seed, align=shard_align(dist_ctx.world_size))
            attach_fused_sync(model, dist_ctx, run)
            if dist_ctx.world_size > 1:
                dist_ctx.backend = "fused"
            dist_ctx.backend_note = model.fused.describe()
            return model
        if dist_ctx.world_size > 1:
            dist_ctx.fall_back(why)
        return NativeEngine(model_cfg, optim_cfg, run, dist_ctx, seed=seed)
    if dist_ctx.world_size > 1:
        dist_ctx.fall_back("the fused path is part of the native engine")
    from .models.reference import ReferenceModel
    return ReferenceModel(model_cfg, optim_cfg, device=dist_ctx.device, dtype=torch.float32, seed=seed)


def main(argv: Optional[Sequence[str]] = None) -> int:
    model_cfg, optim_cfg, run = parse_args(argv)
    d = DistributedContext()
    try:
        d.init(backend=run.comm_backend, device=run.device, comm_thread=run.comm_thread,
               defer_grad_avg=run.defer_grad_avg)
    except Exception as e:                                            # rendezvous failure
        print(f"Error: distributed initialisation failed: {e}", file=sys.stderr)
        return 1
    root = d.is_root()
    say = (lambda *a: print(*a, flush=True)) if root else (lambda *a: None)
    for line in environment_report(gemm_requested=run.gemm_backend):
        say(line)
    errs, warns = validate_environment(d.world_size)
    errs += validate_run(model_cfg, run, d.world_size)
    for w in warns:
        if root:
            print(w, file=sys.stderr)
    if errs:
        for e in errs:
            if root:
                print(f"Invalid CME213 configuration: {e}", file=sys.stderr)
        d.finalize()
        return 2
    if run.validate_config:
        say("Configuration validation: PASS")
        d.finalize()
        return 0

    # ---- data ----------------------------------------------------------------------------------
    if run.synthetic:
        n_batches = max(run.max_steps if run.max_steps > 0 else 64, 1) * d.world_size * run.grad_accum
        all_x, all_y = synthetic_batches(model_cfg.vocab_size, model_cfg.seq_len, model_cfg.batch_size,
                                         n_batches, seed=0)
        say(f"Dataset: synthetic uniform tokens, vocab_size={model_cfg.vocab_size}, seq_len={model_cfg.seq_len}, "
            f"batch_size={model_cfg.batch_size}")
    else:
        try:
            text = read_file(run.data_path)
        except OSError:
            print(f"Error: cannot open {run.data_path}", file=sys.stderr)
            d.finalize()
            return 1
        tok = CharTokenizer().build(text)
        say(f"Vocabulary size: {tok.vocab_size}")
        model_cfg.vocab_size = tok.vocab_size
        ds = Dataset(tok.encode(text), model_cfg.seq_len, model_cfg.batch_size)
        say(f"Dataset: {len(ds.tokens)} tokens, vocab_size={tok.vocab_size}, seq_len={model_cfg.seq_len}, "
            f"batch_size={model_cfg.batch_size}")
        all_x, all_y = ds.all_batches()

    model = build_model(model_cfg, optim_cfg, run, d, run.seed)
    for line in d.banner() if d.world_size > 1 else []:
        say(line)
    start_step = 0
    if run.load_checkpoint:
        _, p, m, v, start_step, _ = ckpt.load_checkpoint(run.load_checkpoint, model.layout)
        model.load_state(p, m, v, start_step) if hasattr(model, "load_state") else _load_into(model, p, m, v, start_step)
        say(f"Checkpoint: loaded {run.load_checkpoint} at optimizer step {start_step}")
    trainer = Trainer(model, d, run, optim_cfg)

    say(logfmt.model_line(model_cfg))
    say(logfmt.params_line(model.layout.num_params()))
    say(logfmt.training_line(run.epochs, optim_cfg.lr, run.max_steps, d.world_size, run.sync_mode,
                             trainer.use_overlap, run.bucket_kb, run.auto_overlap_max_mb))
    if run.trace_trajectory:
        say("Trajectory trace: enabled, reporting loss and parameter statistics after each step")
    if d.world_size > 1:
        say("Gradient averaging: %s" % ("deferred_to_adam" if d.defer_gradient_average else "post_allreduce"))

    per_step = d.world_size * run.grad_accum
    plan = ShardPlan(all_x.shape[0], per_step)
    if plan.local_batches <= 0:
        if root:
            print(f"Error: dataset has {all_x.shape[0]} batches but world_size={d.world_size}", file=sys.stderr)
        d.finalize()
        return 1
    steps_per_epoch = plan.local_batches
    if 0 < run.max_steps < steps_per_epoch:
        steps_per_epoch = run.max_steps
    say(logfmt.batches_line(all_x.shape[0], plan.local_batches, steps_per_epoch, plan.dropped))

    all_x = all_x.to(d.device)
    all_y = all_y.to(d.device)
    if run.cuda_graph and d.device.type == "cuda":
        if trainer.enable_cuda_graph(warmup_steps=3):
            say("CUDA Graph: enabled, capture after 3 warmup steps")
        elif root:
            print("Warning: --cuda-graph needs the native engine and, with several ranks, the fused sync path"
                  + (f" ({d.backend_note})" if d.backend_note else "") + "; running eagerly", file=sys.stderr)

    BT = model_cfg.tokens_per_step
    step_loss = 0.0
    for epoch in range(run.epochs):
        logged_sum, logged_n = 0.0, 0
        trainer.reset_timers()
        d.barrier()
        t0 = time.perf_counter()
        for step in range(steps_per_epoch):
            base = step * per_step + d.rank * run.grad_accum
            xs = [all_x[base + i] for i in range(run.grad_accum)]
            ys = [all_y[base + i] for i in range(run.grad_accum)]
            trainer.step(xs, ys)
            if run.trace_trajectory:
                if d.device.type == "cuda":
                    torch.cuda.synchronize()
                # fp32 master values: under the fused path every rank owns a slice of them, so they are gathered
                # (a collective all ranks enter; tracing mode only)
                if getattr(model, "fused", None) is not None and d.world_size > 1:
                    traced = model.state()[0]
                else:
                    traced = model.master_params() if hasattr(model, "master_params") else model.params
                st = ckpt.param_stats(traced)
                spans = tuple(d.max_double(x) - d.min_double(x) for x in (st.sum, st.sumsq, st.max_abs))
                if root:
                    step_loss = model.read_loss()
                    print(ckpt.trajectory_line(epoch + 1, step + 1, step_loss, st, spans), flush=True)
            if (step + 1) % run.log_every == 0 or step + 1 == steps_per_epoch:
                trainer.check_device_status()                   # raises if a bounded device-side wait ran out
                if trainer.watchdog is not None:
                    trainer.watchdog.beat()                     # the status read synchronised: the device answers
            if root and ((step + 1) % run.log_every == 0 or step + 1 == steps_per_epoch):
                step_loss = model.read_loss()
                logged_sum += step_loss
                logged_n += 1
                print(logfmt.step_line(epoch + 1, step + 1, steps_per_epoch, step_loss), flush=True)
        if d.device.type == "cuda":
            torch.cuda.synchronize()
        d.barrier()
        max_ms = d.max_double((time.perf_counter() - t0) * 1e3)
        sync_ms = d.max_double(trainer.comm_ms_sum / max(steps_per_epoch, 1))
        start_ms = d.max_double(trainer.async_start_ms_sum / max(steps_per_epoch, 1))
        p = model.master_params() if hasattr(model, "master_params") else model.params
        checksum = float(p.detach().double().sum())
        span = d.max_double(checksum) - d.min_double(checksum)
        tokens = float(steps_per_epoch) * BT * run.grad_accum * d.world_size
        say(logfmt.epoch_line(epoch + 1, logged_sum / logged_n if logged_n else step_loss, steps_per_epoch,
                              max_ms, tokens / (max_ms / 1e3), d.world_size, trainer.use_overlap,
                              start_ms, sync_ms, span))
        if getattr(model, "fused", None) is not None:
            # device timestamps of the last step's bucket kernels (ms relative to the end of backward) and the exposed
            # synchronisation time, max over ranks; parsed by benchmarks/run_experiments.py
            import json
            tl = model.fused.timeline()
            tl["exposed_ms"] = d.max_double(tl["exposed_ms"])
            say("SYNC_TIMELINE " + json.dumps(tl))

    if run.save_checkpoint:
        # every rank takes part: under the fused path the optimizer state is sharded and `state` gathers it
        p, m, v, t = model.state() if hasattr(model, "state") else (model.params, model.adam_m, model.adam_v,
                                                                     model.step_count)
        if root:
            st = ckpt.save_checkpoint(run.save_checkpoint, model.layout, p, m, v, t)
            say(f"Checkpoint: wrote {run.save_checkpoint} step={t} param_hash={st.hex_hash()}")
    if trainer.watchdog is not None:
        trainer.watchdog.stop()
    d.finalize()
    return 0


def _load_into(model, p, m, v, step) -> None:
    with torch.no_grad():
        model.params.data.copy_(p.to(model.params.device, model.params.dtype))
        model.adam_m.copy_(m.to(model.adam_m.device, model.adam_m.dtype))
        model.adam_v.copy_(v.to(model.adam_v.device, model.adam_v.dtype))
    model.step_count = step


if __name__ == "__main__":
    sys.exit(main())
