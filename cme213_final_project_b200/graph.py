"""Whole-step CUDA graph: capture ``forward + backward + synchronisation + optimizer`` once, replay per step.

The reference captures ``zero_grad + forward_no_sync + backward + update_adam`` after three eager warm-up
steps, reading tokens from fixed staging buffers refreshed by a device-to-device copy before each replay,
and only on one GPU (``FINAL_CLEAN_CODE_/src/main.cu:299-355``).  Same scheme here, with two differences:
the optimizer's step counter and learning rate live in device memory, so replays apply the right bias
correction (the reference bakes the host-computed corrections of the captured step into the graph); and the
captured region may contain the fused peer-memory synchronisation kernels, so multi-GPU steps are graphs too.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch


class GraphedStep:
    """Wraps ``step_fn(tokens_list, targets_list)``; after ``warmup`` eager calls the next call captures."""

    def __init__(self, step_fn: Callable[[List[torch.Tensor], List[torch.Tensor]], None], tokens_per_step: int,
                 accum: int, device: torch.device, warmup: int = 3) -> None:
        self.step_fn = step_fn
        self.warmup = warmup
        self.calls = 0
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.static_x = torch.zeros(accum, tokens_per_step, dtype=torch.int32, device=device)
        self.static_y = torch.zeros(accum, tokens_per_step, dtype=torch.int32, device=device)
        self.captured_launches = 0

    def __call__(self, tokens: Sequence[torch.Tensor], targets: Sequence[torch.Tensor]) -> None:
        for i, (x, y) in enumerate(zip(tokens, targets)):
            self.static_x[i].copy_(x, non_blocking=True)
            self.static_y[i].copy_(y, non_blocking=True)
        xs = [self.static_x[i] for i in range(self.static_x.shape[0])]
        ys = [self.static_y[i] for i in range(self.static_y.shape[0])]
        self.calls += 1
        if self.calls <= self.warmup:
            self.step_fn(xs, ys)
            return
        if self.graph is None:
            from . import ops
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            with torch.cuda.graph(g):
                self.step_fn(xs, ys)
            self.captured_launches = ops.launch_count() - before
            self.graph = g
        self.graph.replay()
