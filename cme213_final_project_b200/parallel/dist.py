"""Data-parallel context: rendezvous, gradient synchronisation paths, scalar reductions.

Role of the reference's ``DistributedContext`` (``FINAL_CLEAN_CODE_/include/distributed.h:17-90``,
``FINAL_CLEAN_CODE_/src/model/distributed.cpp``) with ``torch.distributed`` as the control plane
instead of MPI.  Gradient collectives are in-place sums over the whole world followed by a
``1/world`` scale per bucket unless averaging is deferred to the optimizer
(``distributed.cpp:71-73,232,352,393``).

Synchronisation paths (reference -> here):

* blocking whole-buffer all-reduce (``distributed.cpp:183-242``)            -> :meth:`sync_gradients`
* per-bucket asynchronous all-reduce on a side stream, NCCL (``:285-298``)  -> ``backend="nccl"``
  (or ``"gloo"`` on CPU tensors)
* per-bucket all-reduce staged through a grow-only pool of pinned host buffers
  (``:19-30,311-331,386-391``)                                              -> ``backend="host"``
* a communication worker thread fed through a condition-variable queue, batching small buckets and
  issuing blocking collectives while backward continues (``:260-278,407-479``) -> ``comm_thread=True``
* (new) the fused peer-memory device path lives in :mod:`.fused_sync`; this class only hands out the
  process group and the rank / world facts it needs.

Timers: ``last_async_start_ms`` accumulates host time spent enqueueing buckets in one step,
``last_sync_ms`` is host time spent in :meth:`finish_async_gradient_syncs` or in the blocking sync —
the reference's definition of exposed communication (``distributed.cpp:254,274-276,343,364-366``).
"""
from __future__ import annotations

import datetime
import os
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional

import torch
import torch.distributed as dist

SMALL_BUCKET_BYTES = 128 * 1024      # worker batches buckets below this ...
SMALL_BATCH_BYTES = 256 * 1024       # ... up to this many bytes per wake-up (distributed.cpp:417-462)


@dataclass
class _Pending:
    tensor: torch.Tensor
    work: Optional[object] = None
    host: Optional[torch.Tensor] = None
    event: Optional[object] = None
    done: threading.Event = field(default_factory=threading.Event)
    error: Optional[BaseException] = None


class DistributedContext:
    def __init__(self) -> None:
        self.world_size = 1
        self.rank = 0
        self.local_rank = 0
        self.device = torch.device("cpu")
        self.backend = "none"               # gradient backend: none | fused | nccl | gloo | host
        self.backend_note = ""              # why the effective backend differs from the requested one
        self.use_comm_thread = False
        self.defer_gradient_average = False
        self.last_allreduce_ms = 0.0
        self.last_sync_ms = 0.0
        self.last_async_start_ms = 0.0
        self.group = None
        self._owns_pg = False
        self._pending: List[_Pending] = []
        self._host_pool: List[torch.Tensor] = []
        self._next_host = 0
        self._comm_stream = None
        self._queue: Deque[_Pending] = deque()
        self._cv = threading.Condition()
        self._shutdown = False
        self._worker: Optional[threading.Thread] = None
        self.drop_next_bucket = False       # host-side fault injection: the next reduced bucket is lost on this rank

    # -- life cycle --------------------------------------------------------------------------------
    def init(self, backend: str = "auto", device: str = "auto", comm_thread: bool = False,
             defer_grad_avg: bool = False, timeout_s: float = 600.0) -> "DistributedContext":
        """Join the job described by ``RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT``;
        a process started without them is a world of one (the reference's non-MPI build,
        ``distributed.cpp:146-150``).  Device choice is ``rank % num_devices`` (``:47``)."""
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
        use_cuda = (device == "cuda") or (device == "auto" and torch.cuda.is_available())
        if use_cuda:
            ndev = torch.cuda.device_count()
            self.device = torch.device("cuda", self.local_rank % max(ndev, 1))
            torch.cuda.set_device(self.device)
        self.world_size, self.rank = world, rank
        if world > 1:
            if not dist.is_initialized():
                pg_backend = "cpu:gloo,cuda:nccl" if use_cuda else "gloo"
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                kw = {"device_id": self.device} if use_cuda else {}
                dist.init_process_group(pg_backend, rank=rank, world_size=world,
                                        timeout=datetime.timedelta(seconds=timeout_s), **kw)
                self._owns_pg = True
            self.group = dist.group.WORLD
        # "auto" on GPUs is the fused device path (parallel/fused_sync.py: peer-memory kernels, no library
        # collective on the gradient path); torch.distributed stays the control plane (rendezvous, handle exchange,
        # scalar reductions).  The training driver attaches the fused path to the model and calls
        # `fall_back` with the reason when the model or the options cannot use it.
        if backend == "auto":
            backend = "none" if world == 1 else ("fused" if use_cuda else "gloo")
        if backend == "fused" and not use_cuda:
            backend, self.backend_note = "gloo", "the fused device path needs GPUs"
        self.backend = backend if world > 1 else "none"
        self.defer_gradient_average = defer_grad_avg and world > 1
        self.use_comm_thread = comm_thread and world > 1
        if use_cuda and world > 1:
            self._comm_stream = torch.cuda.Stream(device=self.device)
        if self.use_comm_thread:
            self._worker = threading.Thread(target=self.comm_worker_loop, name="comm-worker", daemon=True)
            self._worker.start()
        return self

    def fall_back(self, reason: str) -> None:
        """The fused device path cannot serve this run: host-issued NCCL all-reduces take over."""
        if self.backend == "fused":
            self.backend, self.backend_note = "nccl", reason

    def banner(self) -> List[str]:
        """Rank-0 description of the effective mode (``distributed.cpp:128-145``)."""
        return [f"DP: world_size={self.world_size} rank={self.rank} device={self.device}",
                f"DP gradient backend: {self.backend}" + (f" ({self.backend_note})" if self.backend_note else ""),
                f"DP gradient averaging: {'deferred_to_adam' if self.defer_gradient_average else 'post_allreduce'}",
                f"DP comm thread: {'enabled' if self.use_comm_thread else 'disabled'}"]

    def finalize(self) -> None:
        self.request_comm_worker_shutdown()
        if self._worker is not None:
            self._worker.join(timeout=10)
            self._worker = None
        if self._owns_pg and dist.is_initialized():
            dist.destroy_process_group()
        self._owns_pg = False

    def is_root(self) -> bool:
        return self.rank == 0

    # -- collectives -------------------------------------------------------------------------------
    def _host_buffer(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """Grow-only pool of pinned host buffers reused by index each step (``distributed.cpp:19-30``)."""
        i = self._next_host
        self._next_host += 1
        if i >= len(self._host_pool):
            self._host_pool.append(torch.empty(0, dtype=dtype))
        buf = self._host_pool[i]
        if buf.numel() < numel or buf.dtype != dtype:
            buf = torch.empty(numel, dtype=dtype, pin_memory=torch.cuda.is_available())
            self._host_pool[i] = buf
        return buf[:numel]

    def allreduce_sum(self, buf: torch.Tensor) -> None:
        """Blocking in-place sum over all ranks (``distributed.cpp:183-224``)."""
        if self.world_size == 1:
            self.last_allreduce_ms = 0.0
            return
        t0 = time.perf_counter()
        if buf.is_cuda:
            torch.cuda.synchronize(buf.device)
        if self.backend == "host" and buf.is_cuda:
            h = self._host_buffer(buf.numel(), buf.dtype)
            h.copy_(buf.view(-1))
            dist.all_reduce(h, group=self.group)
            buf.view(-1).copy_(h)
        else:
            dist.all_reduce(buf, group=self.group)
        if buf.is_cuda:
            torch.cuda.synchronize(buf.device)
        self.last_allreduce_ms = (time.perf_counter() - t0) * 1e3

    def sync_gradients(self, buf: torch.Tensor) -> None:
        """Blocking whole-buffer gradient sync + averaging (``distributed.cpp:226-242``)."""
        t0 = time.perf_counter()
        self._next_host = 0
        self.last_async_start_ms = 0.0
        if self.world_size > 1:
            self.allreduce_sum(buf)
            if not self.defer_gradient_average:
                buf.mul_(1.0 / self.world_size)
                if buf.is_cuda:
                    torch.cuda.synchronize(buf.device)
        self.last_sync_ms = (time.perf_counter() - t0) * 1e3

    def begin_step(self) -> None:
        self._next_host = 0
        self.last_async_start_ms = 0.0
        self.last_sync_ms = 0.0

    def start_async_gradient_sync(self, buf: torch.Tensor) -> None:
        """Hand one finished gradient bucket to the communication path and return immediately
        (``distributed.cpp:244-335``)."""
        if self.world_size == 1:
            return
        t0 = time.perf_counter()
        if self.drop_next_bucket:
            # injected fault: this rank takes part in the collective (its peers must not be left waiting) but the
            # reduced bucket never reaches its gradient arena
            self.drop_next_bucket = False
            buf = buf.clone()
        p = _Pending(buf)
        if self.use_comm_thread:
            if buf.is_cuda:
                p.event = torch.cuda.Event()
                p.event.record(torch.cuda.current_stream(buf.device))
            with self._cv:
                self._queue.append(p)
                self._cv.notify()
        elif self.backend == "host" and buf.is_cuda:
            p.host = self._host_buffer(buf.numel(), buf.dtype)
            p.host.copy_(buf.view(-1), non_blocking=True)
            torch.cuda.current_stream(buf.device).synchronize()
            p.work = dist.all_reduce(p.host, group=self.group, async_op=True)
        elif buf.is_cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(buf.device))
            self._comm_stream.wait_event(ev)
            with torch.cuda.stream(self._comm_stream):
                p.work = dist.all_reduce(buf, group=self.group, async_op=True)
        else:
            p.work = dist.all_reduce(buf, group=self.group, async_op=True)
        self._pending.append(p)
        self.last_async_start_ms += (time.perf_counter() - t0) * 1e3

    def finish_async_gradient_syncs(self, timeout_s: float = 60.0) -> None:
        """Wait for every bucket started this step, then average each (``distributed.cpp:337-405``)."""
        t0 = time.perf_counter()
        scale = 1.0 / self.world_size
        for p in self._pending:
            if self.use_comm_thread:
                if not p.done.wait(timeout_s):
                    self._pending.clear()
                    raise TimeoutError("gradient bucket was not reduced in time (comm worker stalled?)")
                if p.error is not None:
                    self._pending.clear()
                    raise p.error
            elif p.work is not None:
                p.work.wait()
                if p.host is not None:
                    p.tensor.view(-1).copy_(p.host, non_blocking=True)
            if not self.defer_gradient_average:
                p.tensor.mul_(scale)
        if self._pending and self._pending[0].tensor.is_cuda:
            torch.cuda.synchronize(self._pending[0].tensor.device)
        self._pending.clear()
        self.last_sync_ms = (time.perf_counter() - t0) * 1e3

    # -- communication worker ----------------------------------------------------------------------
    def request_comm_worker_shutdown(self) -> None:
        with self._cv:
            self._shutdown = True
            self._cv.notify_all()

    def comm_worker_loop(self) -> None:
        """Worker: wait for buckets, take one large bucket or a batch of small ones per wake-up, wait
        for the producer's event, reduce in place, publish completion (``distributed.cpp:407-479``)."""
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        while True:
            with self._cv:
                while not self._queue and not self._shutdown:
                    self._cv.wait()
                if not self._queue and self._shutdown:
                    return
                batch = [self._queue.popleft()]
                size = batch[0].tensor.numel() * batch[0].tensor.element_size()
                if size < SMALL_BUCKET_BYTES:
                    while self._queue:
                        nxt = self._queue[0].tensor
                        nb = nxt.numel() * nxt.element_size()
                        if nb >= SMALL_BUCKET_BYTES or size + nb > SMALL_BATCH_BYTES:
                            break
                        batch.append(self._queue.popleft())
                        size += nb
            for p in batch:
                try:
                    if p.event is not None:
                        p.event.synchronize()
                    if p.tensor.is_cuda:
                        with torch.cuda.stream(self._comm_stream):
                            dist.all_reduce(p.tensor, group=self.group)
                        self._comm_stream.synchronize()
                    else:
                        dist.all_reduce(p.tensor, group=self.group)
                except BaseException as e:      # surfaced to the trainer in finish_async_gradient_syncs
                    p.error = e
                p.done.set()

    # -- scalar reductions -------------------------------------------------------------------------
    def _reduce_scalar(self, value: float, op) -> float:
        if self.world_size == 1:
            return float(value)
        t = torch.tensor([value], dtype=torch.float64)
        if self.device.type == "cuda" and not _has_cpu_backend():
            t = t.to(self.device)
        dist.all_reduce(t, op=op, group=self.group)
        return float(t.item())

    def max_double(self, value: float) -> float:
        return self._reduce_scalar(value, dist.ReduceOp.MAX)

    def min_double(self, value: float) -> float:
        return self._reduce_scalar(value, dist.ReduceOp.MIN)

    def barrier(self) -> None:
        if self.world_size > 1:
            if self.device.type == "cuda":
                dist.barrier(group=self.group, device_ids=[self.device.index])
            else:
                dist.barrier(group=self.group)


def _has_cpu_backend() -> bool:
    try:
        return "gloo" in str(dist.get_backend_config()) or dist.get_backend() == "gloo"
    except Exception:
        return False
