"""One training step under every synchronisation policy, for any model that exposes the flat-arena
interface (``zero_grad / forward / backward / update / read_loss`` plus ``params``, ``grads``, ``layout``).

Mirrors the step structure of the reference driver (``FINAL_CLEAN_CODE_/src/main.cu:357-394``):

    zero_grad -> forward -> backward (plain, or bucketed with asynchronous sync) -> [blocking sync] -> update

and adds gradient accumulation (several micro-batches per optimizer step; only the last one synchronises).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .arena import Bucket
from .config import OptimConfig, RunConfig, effective_overlap, min_bucket_elems
from .parallel.dist import DistributedContext
from .utils.nvtx import nvtx_range


class StepWatchdog:
    """Host-side watchdog: if no step completes for ``timeout_s`` seconds the process is ended with a message.

    The reference bounds every run from outside (``timeout --kill-after`` per case, ``scripts/common_env.sh:31-40``)
    and has no detection of its own; here a stalled step -- a rank that never arrives at a collective, a device that
    stopped answering -- ends the process from inside instead of leaving the job hanging until someone notices.
    ``beat()`` is called after every step the trainer hands to the device and after every synchronising read.
    ``on_expire`` (tests) replaces the default action, which prints to stderr and exits with status 3."""

    def __init__(self, timeout_s: float, on_expire=None, poll_s: float = 0.25) -> None:
        import threading
        import time
        self.timeout_s, self.on_expire, self.poll_s = timeout_s, on_expire, poll_s
        self._last = time.monotonic()
        self._stop = threading.Event()
        self.expired = False
        self._thread = threading.Thread(target=self._run, name="step-watchdog", daemon=True)
        self._thread.start()

    def beat(self) -> None:
        import time
        self._last = time.monotonic()

    def stop(self) -> None:
        self._stop.set()

    def _run(self) -> None:
        import os
        import sys
        import time
        while not self._stop.wait(self.poll_s):
            if time.monotonic() - self._last > self.timeout_s:
                self.expired = True
                if self.on_expire is not None:
                    self.on_expire()
                    return
                print(f"Error: no training step completed for {self.timeout_s:.0f} s; ending the process",
                      file=sys.stderr, flush=True)
                os._exit(3)


class Trainer:
    def __init__(self, model, dist_ctx: DistributedContext, run: RunConfig, optim: OptimConfig) -> None:
        self.model = model
        self.dist = dist_ctx
        self.run = run
        self.optim = optim
        elem_bytes = model.grads.element_size()
        self.grad_mb = model.layout.total * elem_bytes / (1024.0 * 1024.0)
        self.use_overlap = effective_overlap(run, self.grad_mb, dist_ctx.world_size)
        self.buckets: List[Bucket] = model.layout.coalesced_buckets(min_bucket_elems(run.bucket_kb, elem_bytes))
        self.comm_ms_sum = 0.0
        self.async_start_ms_sum = 0.0
        self.steps = 0
        self.graphed = None
        self.watchdog = StepWatchdog(run.step_timeout_s) if getattr(run, "step_timeout_s", 0) > 0 else None

    def enable_cuda_graph(self, warmup_steps: int = 3) -> bool:
        """Replay the whole step as one CUDA graph after ``warmup_steps`` eager steps (the reference's
        ``CME213_USE_CUDA_GRAPH=1``, ``main.cu:299-355``).  Host-issued collectives with host waits cannot be
        captured, so with more than one rank this needs the fused device synchronisation path."""
        m = self.model
        if not hasattr(m, "train_step") or m.device.type != "cuda":
            return False
        if self.dist.world_size > 1 and not getattr(m, "handles_sync", False):
            return False
        from .graph import GraphedStep
        self.graphed = GraphedStep(self._step, m.cfg.tokens_per_step, max(self.run.grad_accum, 1), m.device,
                                   warmup=warmup_steps)
        return True

    # ---------------------------------------------------------------------------------------------
    def _bucket_ready(self, b: Bucket) -> None:
        m = self.model
        if hasattr(m, "fence") and m.grads.is_cuda:
            # the bucket's last producer may sit on the engine's second stream: order the current stream behind it,
            # since the communication path takes its dependency from the current stream
            m.fence(torch.cuda.current_stream(m.device))
        self.dist.start_async_gradient_sync(m.grads[b.start:b.end])

    def step(self, tokens: Sequence[torch.Tensor], targets: Sequence[torch.Tensor]) -> None:
        """One optimizer step over ``len(tokens)`` micro-batches (``grad_accum`` of them)."""
        if isinstance(tokens, torch.Tensor):
            tokens, targets = [tokens], [targets]
        if hasattr(self.model, "seq_expected"):
            self.model.seq_expected += 1
        mdev = getattr(self.model, "device", None)
        if (self.graphed is None and len(tokens) and not tokens[0].is_cuda and mdev is not None
                and torch.device(mdev).type == "cuda"):
            tokens, targets = self._stage(tokens, targets)       # host (pinned) batches: one async copy each
        if self.graphed is not None:
            self.graphed(tokens, targets)
            self.steps += 1
        else:
            self._step(tokens, targets)
        if self.watchdog is not None:
            self.watchdog.beat()

    def _stage(self, tokens, targets):
        dev = self.model.device
        if getattr(self, "_stage_x", None) is None or self._stage_x.shape != (len(tokens), tokens[0].numel()):
            self._stage_x = torch.empty(len(tokens), tokens[0].numel(), dtype=torch.int32, device=dev)
            self._stage_y = torch.empty_like(self._stage_x)
        for i, (x, y) in enumerate(zip(tokens, targets)):
            self._stage_x[i].copy_(x.reshape(-1), non_blocking=True)
            self._stage_y[i].copy_(y.reshape(-1), non_blocking=True)
        return [self._stage_x[i] for i in range(len(tokens))], [self._stage_y[i] for i in range(len(tokens))]

    def _step(self, tokens: Sequence[torch.Tensor], targets: Sequence[torch.Tensor]) -> None:
        m, d = self.model, self.dist
        if hasattr(m, "train_step"):                 # native engine: one call enqueues every micro-batch
            d.begin_step()
            with nvtx_range("backward_bucketed" if self.use_overlap else "forward_backward", self.run.profile):
                if getattr(m, "handles_sync", False):
                    m.train_step(tokens, targets)
                elif self.use_overlap:
                    m.train_step(tokens, targets, self._bucket_ready, self.buckets)
                    d.finish_async_gradient_syncs()
                else:
                    m.train_step(tokens, targets)
                    if d.world_size > 1 and not getattr(m, "handles_sync", False):
                        with nvtx_range("gradient_sync", self.run.profile):
                            d.sync_gradients(m.grads)
            self.comm_ms_sum += d.last_sync_ms
            self.async_start_ms_sum += d.last_async_start_ms
            if not getattr(m, "handles_sync", False):
                with nvtx_range("adam_update", self.run.profile):
                    m.update(grad_scale=1.0 / d.world_size if d.defer_gradient_average else 1.0)
            self.steps += 1
            return
        accum = len(tokens)
        d.begin_step()
        m.zero_grad()
        for i, (x, y) in enumerate(zip(tokens, targets)):
            last = i == accum - 1
            with nvtx_range("forward", self.run.profile):
                m.forward(x, y)
            if last and self.use_overlap:
                with nvtx_range("backward_bucketed", self.run.profile):
                    m.backward(bucket_callback=self._bucket_ready, buckets=self.buckets, scale=1.0 / accum)
                    d.finish_async_gradient_syncs()
            else:
                with nvtx_range("backward", self.run.profile):
                    m.backward(scale=1.0 / accum)
                if last and d.world_size > 1:
                    with nvtx_range("gradient_sync", self.run.profile):
                        d.sync_gradients(m.grads)
        self.comm_ms_sum += d.last_sync_ms
        self.async_start_ms_sum += d.last_async_start_ms
        grad_scale = 1.0 / d.world_size if d.defer_gradient_average else 1.0
        with nvtx_range("adam_update", self.run.profile):
            m.update(grad_scale=grad_scale)
        self.steps += 1

    def check_device_status(self) -> None:
        """Read the status words of the GEMM, attention and synchronisation kernels (each synchronises the device)
        and raise if a bounded device-side wait ran out since the last check: the step that contained it did not
        compute, or did not distribute, what it should have.  The training driver calls this at every logging
        point and at the end of an epoch."""
        m = self.model
        if getattr(m, "device", None) is None or torch.device(m.device).type != "cuda" or not hasattr(m, "lib"):
            return
        from . import ops
        with torch.cuda.device(m.device):
            bad = {"gemm": ops.gemm_check_status(), "attention": ops.attention_check_status(),
                   "gradient sync": m.fused.check_status() if getattr(m, "fused", None) is not None else 0}
        bad = {k: v for k, v in bad.items() if v}
        if bad:
            raise RuntimeError("device-side wait ran out (status " + ", ".join(f"{k}={v}" for k, v in bad.items())
                               + f") on rank {self.dist.rank} by step {self.steps}; parameters are not trustworthy")

    def reset_timers(self) -> None:
        self.comm_ms_sum = 0.0
        self.async_start_ms_sum = 0.0
        self.steps = 0
