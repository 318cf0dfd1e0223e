"""Device timers (CUDA events) and an L2 flush helper for micro-benchmarks.

``GpuTimer`` has the role of the reference's cudaEvent timer (``FINAL_CLEAN_CODE_/include/common.h:64-82``)."""
from __future__ import annotations

import time
from typing import Callable, List, Optional

import torch


class GpuTimer:
    """``tic()`` / ``toc()`` on the current stream; ``elapsed_ms()`` synchronises on the stop event."""

    def __init__(self) -> None:
        self.cuda = torch.cuda.is_available()
        if self.cuda:
            self.start = torch.cuda.Event(enable_timing=True)
            self.stop = torch.cuda.Event(enable_timing=True)
        self._t0 = self._t1 = 0.0

    def tic(self) -> None:
        if self.cuda:
            self.start.record()
        else:
            self._t0 = time.perf_counter()

    def toc(self) -> None:
        if self.cuda:
            self.stop.record()
            self.stop.synchronize()
        else:
            self._t1 = time.perf_counter()

    def elapsed_ms(self) -> float:
        return self.start.elapsed_time(self.stop) if self.cuda else (self._t1 - self._t0) * 1e3


class L2Flusher:
    """Writes a buffer larger than the 126 MB L2 so that the next timed launch starts cold."""

    def __init__(self, device, nbytes: int = 256 << 20) -> None:
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def flush(self) -> None:
        self.buf.zero_()


def time_kernel(fn: Callable[[], None], warmup: int = 3, iters: int = 10, flusher: Optional[L2Flusher] = None
                ) -> List[float]:
    """Per-iteration device times in ms: warm-up, then each iteration bracketed by events on the
    launching stream with an optional L2 flush before it."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if flusher is not None:
            flusher.flush()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        out.append(s.elapsed_time(e))
    return out
