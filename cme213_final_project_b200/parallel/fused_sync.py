"""Device-side gradient synchronisation: the per-bucket fused reduce-scatter + AdamW + all-gather kernel and the
peer-memory all-reduce kernels, their symmetric buffers, flags, status word and launch policy.

What the reference does with an OpenMP communication thread issuing ``MPI_Allreduce`` per bucket while
backward continues, a scale kernel per bucket and a separate Adam pass
(``FINAL_CLEAN_CODE_/src/model/distributed.cpp:260-278,407-479``, ``FINAL_CLEAN_CODE_/src/main.cu:385-394``) is
here one kernel per bucket on a communication stream, launched as soon as backward has produced the bucket,
with the next step's forward joined on it.  No host thread, no library collective, and the whole step
(including these kernels) can be captured in one CUDA graph.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import ops
from ..arena import Bucket
from ..config import RunConfig, min_bucket_elems
from .symm import LocalPeers, SymmetricBuffer

ALGOS = {"one_shot": 0, "two_shot": 1, "nvls": 2}


class PeerComm:
    """Flags, control words and status shared by every in-kernel collective of one process."""

    def __init__(self, device: torch.device, max_buckets: int = 256, group=None, budget_ms: float = 2000.0,
                 single: bool = False) -> None:
        self.lib = ops.lib()
        self.device = device
        self.max_buckets = max_buckets
        self.budget_ms = budget_ms
        words = int(self.lib.cme_comm_flag_words(max_buckets))
        if single or not dist.is_initialized() or dist.get_world_size() == 1:
            self.flags = LocalPeers(torch.zeros(words, dtype=torch.int32, device=device))
        else:
            self.flags = SymmetricBuffer(words, torch.int32, device, group)
        self.world, self.rank = self.flags.world, self.flags.rank
        self.ctl = torch.zeros(int(self.lib.cme_comm_ctl_words(max_buckets)), dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.flags.barrier()

    def allreduce(self, src, dst, n: int, offset: int = 0, algo: str = "two_shot", scale: float = 1.0,
                  bucket: int = 0, ctas: int = 64, stream: Optional[torch.cuda.Stream] = None) -> None:
        """``dst[offset:offset+n] = scale * sum_ranks src[offset:offset+n]`` (``src`` / ``dst``: symmetric buffers)."""
        st = stream or torch.cuda.current_stream()
        ops._check(self.lib.cme_comm_allreduce(
            ops._dt(src.tensor), self.world, self.rank, src.c_ptrs, dst.c_ptrs, self.flags.c_ptrs,
            ctypes.c_void_p(src.multicast_ptr), ctypes.c_void_p(dst.multicast_ptr), ctypes.c_longlong(offset),
            ctypes.c_longlong(n), ALGOS[algo], ctypes.c_float(scale), bucket, ctas, ops._p(self.ctl),
            ops._p(self.status), ctypes.c_double(self.budget_ms), ctypes.c_void_p(st.cuda_stream)))

    def check_status(self) -> int:
        """Read and clear the status word (non-zero: a bounded wait on a peer ran out)."""
        v = int(self.status.item())
        if v:
            self.status.zero_()
        return v


def choose_algo(nbytes: int, world: int, has_multicast: bool, table: Optional[dict] = None) -> str:
    """Collective variant for a message size: one-shot below the latency crossover, NVLS above it when the
    fabric offers multicast, else two-shot.  ``table`` (``{"one_shot_max_bytes": ..}``) comes from a measured
    sweep (``benchmarks/bench_allreduce.py``); the defaults are that sweep's crossover on 8 x B200."""
    t = table or {}
    if nbytes <= t.get("one_shot_max_bytes", 256 * 1024):
        return "one_shot"
    if has_multicast and t.get("use_nvls", True):
        return "nvls"
    return "two_shot"


class FusedSync:
    """Owns the symmetric gradient / parameter arenas of an engine and launches the fused kernel per bucket."""

    def __init__(self, model, ctx, run: RunConfig, ctas: int = 296, use_nvls: Optional[bool] = None,
                 budget_ms: float = 5000.0) -> None:
        if model.strict:
            raise ops.NativeError("the fused synchronisation path needs bf16 gradients (--compute-dtype bf16)")
        if model.optim.clip_norm > 0:
            raise ops.NativeError("global-norm clipping needs the whole gradient before any update; "
                                  "use the all-reduce path (comm backend nccl) for that optimizer setting")
        self.model, self.ctx = model, ctx
        dev = model.device
        n = model.layout.total
        self.world = ctx.world_size
        single = self.world == 1
        if single:
            self.grads = LocalPeers(torch.zeros(n, dtype=torch.bfloat16, device=dev))
            self.params = LocalPeers(model.params.clone())
        else:
            self.grads = SymmetricBuffer(n, torch.bfloat16, dev)
            self.params = SymmetricBuffer(n, torch.bfloat16, dev)
            self.params.tensor.copy_(model.params)
        model.rebind(self.params.tensor, self.grads.tensor)
        elem = 2
        self.buckets: List[Bucket] = model.layout.coalesced_buckets(min_bucket_elems(run.bucket_kb, elem))
        self.comm = PeerComm(dev, max_buckets=max(len(self.buckets), 1), budget_ms=budget_ms, single=single)
        import os
        # SM budget: one small CTA per SM while backward is still running (they share SMs with the compute
        # kernels); the last bucket has the GPU to itself and gets four per SM
        self.ctas = int(os.environ.get("CME213_COMM_CTAS", ctas))
        self.tail_ctas = int(os.environ.get("CME213_COMM_TAIL_CTAS", 4 * 148))
        mc = self.grads.multicast_ptr != 0 and self.params.multicast_ptr != 0
        self.use_nvls = mc if use_nvls is None else (use_nvls and mc)
        if os.environ.get("CME213_COMM_NVLS") is not None:
            self.use_nvls = mc and os.environ["CME213_COMM_NVLS"] != "0"
        self.stream = torch.cuda.Stream(device=dev)
        self.grad_scale = 1.0 / self.world
        self.lib = ops.lib()
        self.launched = 0
        self.measure_exposed = False
        self._exposed = []

    def launch_bucket(self, b: Bucket) -> None:
        """Called on the host as soon as backward has enqueued the last kernel of bucket ``b``."""
        m, o = self.model, self.model.optim
        cur = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(cur)
        self.stream.wait_event(ev)
        nd = m.nodecay if o.weight_decay > 0 else None
        ops._check(self.lib.cme_comm_fused_adamw(
            self.world, self.comm.rank, self.grads.c_ptrs, self.params.c_ptrs, self.comm.flags.c_ptrs,
            ctypes.c_void_p(self.grads.multicast_ptr), ctypes.c_void_p(self.params.multicast_ptr),
            ctypes.c_longlong(b.start), ctypes.c_longlong(b.numel), ops._p(m.master), ops._p(m.adam_m),
            ops._p(m.adam_v), ops._p(m.step_dev), ops._p(m.lr_dev), ctypes.c_float(o.beta1), ctypes.c_float(o.beta2),
            ctypes.c_float(o.eps), ctypes.c_float(o.weight_decay), ctypes.c_float(self.grad_scale), ops._p(nd),
            0 if nd is None else nd.shape[0], int(self.use_nvls), b.index,
            self.tail_ctas if b.index == len(self.buckets) - 1 else self.ctas, ops._p(self.comm.ctl),
            ops._p(self.comm.status), ctypes.c_double(self.comm.budget_ms), ctypes.c_void_p(self.stream.cuda_stream)))
        self.launched += 1

    def join(self) -> None:
        """Make the compute stream wait for every bucket kernel (parameters are then final on this rank).  With
        ``measure_exposed`` set (eager steps only) the wait is bracketed by timing events: the time the compute
        stream sits idle behind the last bucket kernels is the step's exposed synchronisation time."""
        ev = torch.cuda.Event()
        ev.record(self.stream)
        cur = torch.cuda.current_stream()
        if self.measure_exposed and not torch.cuda.is_current_stream_capturing():
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(cur)
            cur.wait_event(ev)
            e1.record(cur)
            self._exposed.append((e0, e1))
        else:
            cur.wait_event(ev)

    def exposed_ms(self) -> List[float]:
        """Exposed synchronisation time of every step since ``measure_exposed`` was set (synchronises)."""
        torch.cuda.synchronize(self.model.device)
        out = [a.elapsed_time(b) for a, b in self._exposed]
        self._exposed = []
        return out

    def owned_mask(self) -> torch.Tensor:
        """1.0 where this rank owns the optimizer state (slice ``rank`` of every bucket), else 0.0."""
        mask = torch.zeros(self.model.layout.total, dtype=torch.float32, device=self.model.device)
        for b in self.buckets:
            per = b.numel // self.world
            s0 = b.start + per * self.comm.rank
            mask[s0:s0 + per] = 1.0
        return mask

    def gather_state(self):
        """Full fp32 master / moment arenas on every rank (checkpointing): owned slices summed over ranks."""
        m = self.model
        mask = self.owned_mask()
        out = []
        for t in (m.master, m.adam_m, m.adam_v):
            full = t * mask
            dist.all_reduce(full)
            out.append(full)
        return out[0], out[1], out[2], int(m.step_dev.item())

    def train_step(self, tokens: Sequence[torch.Tensor], targets: Sequence[torch.Tensor]) -> None:
        m = self.model
        ops._check(self.lib.cme_step_inc(ops._p(m.step_dev), ops._stream()))
        m.step_count += 1
        m.train_step_raw(tokens, targets, self.launch_bucket, self.buckets)
        self.join()


def attach_fused_sync(model, ctx, run: RunConfig, **kw) -> FusedSync:
    """Switch an engine to the fused path: symmetric arenas, per-bucket fused kernels, no separate optimizer pass."""
    fs = FusedSync(model, ctx, run, **kw)
    model.fused = fs
    model.handles_sync = True
    return fs
