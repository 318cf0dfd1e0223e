"""Device-side gradient synchronisation: the per-bucket fused reduce-scatter + AdamW + all-gather kernel and the
peer-memory all-reduce kernels, their symmetric buffers, flags, status word and launch policy.

What the reference does with an OpenMP communication thread issuing ``MPI_Allreduce`` per bucket while
backward continues, a scale kernel per bucket and a separate Adam pass
(``FINAL_CLEAN_CODE_/src/model/distributed.cpp:260-278,407-479``, ``FINAL_CLEAN_CODE_/src/main.cu:385-394``) is
here one kernel per bucket on a communication stream, launched as soon as backward has produced the bucket,
with the next step's forward joined on it.  No host thread, no library collective, and the whole step
(including these kernels) can be captured in one CUDA graph.

With global-norm clipping (the reference's optimizer, ``FINAL_CLEAN_CODE_/src/model/transformer.cu:618-636``) the
update cannot start before the last gradient is reduced, so the step runs in two phases: the per-bucket kernels
only reduce (keeping fp32 sums of this rank's slices and their sums of squares), and one kernel after the last
bucket exchanges the partial norms, clips, applies the optimizer and distributes the parameters.
"""
from __future__ import annotations

import ctypes
import json
import math
import os
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import ops
from ..arena import Bucket
from ..config import RunConfig, min_bucket_elems
from ..utils.nvtx import nvtx_range
from .symm import LocalPeers, SymmetricBuffer

ALGOS = {"one_shot": 0, "two_shot": 1, "nvls": 2}
MAX_CTAS = 740
TABLE_PATH = Path(__file__).with_name("comm_table.json")


def shard_align(world: int, base: int = 64) -> int:
    """Arena alignment (elements) under which every bucket splits into ``world`` slices of whole 16-byte bf16
    vectors: a common multiple of the tensor alignment and ``8 * world``.  Worlds of 3, 5, 6 or 7 ranks need more
    than the default 64 (the reference validates a 3-rank run, ``scripts/run_edge_case_validation.sh:90-97``)."""
    return base * (8 * world) // math.gcd(base, 8 * world)


def load_table(path: Optional[str] = None) -> Dict[str, dict]:
    """Measured algorithm table: ``{"<world>": {"one_shot_max_bytes": .., "nvls_min_bytes": ..}, ..}`` as written
    by ``benchmarks/bench_allreduce.py --table``.  ``path`` (or ``CME213_COMM_TABLE``) overrides the table shipped
    with the package, which holds the sweeps measured on 2 and 8 B200s."""
    p = path or os.environ.get("CME213_COMM_TABLE") or TABLE_PATH
    try:
        with open(p) as f:
            return json.load(f)
    except OSError:
        return {}


def table_for_world(table: Dict[str, dict], world: int) -> dict:
    """The entry measured at ``world`` ranks, else the one of the nearest measured world size."""
    sizes = sorted(int(k) for k in table if str(k).isdigit())
    if not sizes:
        return {}
    return table[str(min(sizes, key=lambda s: (abs(s - world), -s)))]


def choose_algo(nbytes: int, world: int, has_multicast: bool, table: Optional[dict] = None) -> str:
    """Collective variant for one message: one-shot up to the measured latency crossover, NVLS from the size at
    which the in-switch reduction was measured faster than peer loads (when the fabric offers multicast), else
    two-shot.  ``table`` is one world size's entry of :func:`load_table`."""
    t = table or {}
    if world > 1 and nbytes <= t.get("one_shot_max_bytes", 0):
        return "one_shot"
    if has_multicast and t.get("use_nvls", True) and nbytes >= t.get("nvls_min_bytes", 0):
        return "nvls"
    return "two_shot"


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
            ctypes.c_longlong(n), ALGOS[algo], ctypes.c_float(scale), bucket, self.max_buckets, ctas,
            ops._p(self.ctl), ops._p(self.status), ctypes.c_double(self.budget_ms),
            ctypes.c_void_p(st.cuda_stream)))

    def check_status(self) -> int:
        """Read and clear the status word (non-zero: a bounded wait on a peer ran out)."""
        v = int(self.status.item())
        if v:
            self.status.zero_()
        return v


class FusedSync:
    """Owns the symmetric gradient / parameter arenas of an engine and launches the fused kernel per bucket."""

    def __init__(self, model, ctx, run: RunConfig, ctas: int = 296, use_nvls: Optional[bool] = None,
                 budget_ms: float = 5000.0, algo: Optional[str] = None, table: Optional[dict] = None) -> None:
        if model.strict:
            raise ops.NativeError("the fused synchronisation path needs bf16 gradients (--compute-dtype bf16)")
        self.model, self.ctx = model, ctx
        dev = model.device
        n = model.layout.total
        self.world = ctx.world_size
        single = self.world == 1
        elem = 2
        # CME213_COMM_MERGE_TAIL=0 keeps the plain rule (the embeddings as a bucket of their own behind the last
        # layer bucket)
        self.buckets: List[Bucket] = model.layout.coalesced_buckets(
            min_bucket_elems(run.bucket_kb, elem), merge_tail=os.environ.get("CME213_COMM_MERGE_TAIL", "1") != "0")
        grad_mb = n * elem / (1024.0 * 1024.0)
        self.overlap = run.sync_mode == "overlap" or (run.sync_mode == "auto" and grad_mb <= run.auto_overlap_max_mb)
        if not self.overlap:
            # --sync-mode blocking (or auto above its size limit): one call over the whole arena after backward, the
            # reference's blocking whole-buffer synchronisation (FINAL_CLEAN_CODE_/src/main.cu:373-374)
            self.buckets = [Bucket(0, 0, n, tuple(s.name for s in model.layout.specs))]
        bad = [b for b in self.buckets if b.numel % (8 * self.world) or b.start % 8]
        if bad:
            raise ops.NativeError(
                f"bucket {bad[0].index} ({bad[0].numel} elements) does not split into {self.world} slices of whole "
                f"16-byte vectors; build the engine with align=shard_align({self.world}) = {shard_align(self.world)}")
        if single:
            self.grads = LocalPeers(torch.zeros(n, dtype=torch.bfloat16, device=dev))
            self.params = LocalPeers(model.params.clone())
        else:
            self.grads = SymmetricBuffer(n, torch.bfloat16, dev)
            self.params = SymmetricBuffer(n, torch.bfloat16, dev)
            self.params.tensor.copy_(model.params)
        model.rebind(self.params.tensor, self.grads.tensor)
        # flag / control indices past the gradient buckets: two serve the clip kernel (barrier, norm exchange), one the
        # start-up measurement
        self.comm = PeerComm(dev, max_buckets=len(self.buckets) + 3, budget_ms=budget_ms, single=single)
        # SM budget: one small CTA per SM while backward is still running (they share SMs with the compute
        # kernels); the last bucket has the GPU to itself and gets four per SM
        self.ctas = min(int(os.environ.get("CME213_COMM_CTAS", ctas)), MAX_CTAS)
        self.tail_ctas = min(int(os.environ.get("CME213_COMM_TAIL_CTAS", 4 * 148)), MAX_CTAS)
        mc = self.grads.multicast_ptr != 0 and self.params.multicast_ptr != 0
        if os.environ.get("CME213_COMM_NVLS") is not None:
            use_nvls = os.environ["CME213_COMM_NVLS"] != "0"
        self.has_multicast = mc and use_nvls is not False
        self.use_nvls = self.has_multicast            # kept for callers that print the mode
        self.clip = model.optim.clip_norm > 0
        forced = algo or getattr(run, "comm_algo", "auto")
        if forced == "nvls" and not self.has_multicast:
            raise ops.NativeError("comm algorithm 'nvls' requested but the buffers have no multicast mapping")
        tab = table if table is not None else table_for_world(load_table(getattr(run, "comm_table", None)), self.world)
        # Which variant synchronises which bucket: forced by the caller, else measured right here on this machine's
        # fabric (a few all-reduces per distinct bucket size, a few tens of milliseconds), else from the shipped table
        # of earlier sweeps.  The measurement is the reference's alpha-beta sweep idea moved to start-up
        # (FINAL_CLEAN_CODE_/tests/benchmark_allreduce_alpha_beta.cu): the fastest variant differs between world sizes
        # and machines (at 2 ranks peer loads beat the in-switch reduction at every size, at 8 it is the reverse).
        self.calibration: Dict[int, Dict[str, float]] = {}
        measured: Dict[int, str] = {}
        if (forced == "auto" and table is None and not single and self.has_multicast
                and os.environ.get("CME213_COMM_CALIBRATE", "1") != "0"):
            measured = self._calibrate()
        self.algos: List[str] = []
        for b in self.buckets:
            a = forced if forced != "auto" else measured.get(b.numel) or \
                choose_algo(b.numel * elem, self.world, self.has_multicast, tab)
            if a == "one_shot" and (self.clip or single):
                a = "two_shot"                       # the reduce-only form keeps slices; a world of one has one slice
            self.algos.append(a)
        self.stream = torch.cuda.Stream(device=dev)
        self.grad_scale = 1.0 / self.world
        self.lib = ops.lib()
        self.launched = 0
        self.profile = bool(getattr(run, "profile", False))      # NVTX range around every bucket launch
        self.measure_exposed = False
        self._exposed = []
        # device-side time log (ns, %globaltimer): [2b] / [2b + 1] = start / end of bucket b's kernel (index
        # len(buckets): the clip kernel); the last two words = end of backward on the compute stream, end of the
        # last synchronisation kernel.  Written by every step, eager or replayed; read with `timeline()`.
        self.tlog = torch.zeros(2 * (len(self.buckets) + 2), dtype=torch.int64, device=dev)
        if self.clip:
            self.gred = torch.zeros(n, dtype=torch.float32, device=dev)
            self.norm_part = torch.zeros(MAX_CTAS, dtype=torch.float32, device=dev)
            self.norm_bucket = torch.zeros(len(self.buckets), dtype=torch.float32, device=dev)
            self.ranges = torch.tensor([[b.start, b.numel] for b in self.buckets], dtype=torch.int64, device=dev)
        else:
            self.gred = self.norm_part = self.norm_bucket = self.ranges = None

    def _calibrate(self) -> Dict[int, str]:
        """Time the all-reduce variants on every distinct bucket size (same NVLink traffic pattern as the fused kernel:
        reduce-scatter, then all-gather) with the CTA count that bucket will run with; the max over ranks decides, so
        every rank picks the same variant.  Returns ``{bucket elements: variant}``."""
        dev = self.model.device
        sizes = sorted({b.numel for b in self.buckets})
        tmp = SymmetricBuffer(max(sizes), torch.bfloat16, dev)
        spare = len(self.buckets) + 2
        out: Dict[int, str] = {}
        for n in sizes:
            last = self.buckets[-1].numel == n
            ctas = self.tail_ctas if last else self.ctas
            times: Dict[str, float] = {}
            for algo in (("one_shot",) if (n * 2 <= (1 << 20) and not self.clip) else ()) + ("two_shot", "nvls"):
                for _ in range(2):
                    self.comm.allreduce(self.grads, tmp, n, algo=algo, bucket=spare, ctas=ctas)
                dist.barrier(device_ids=[dev.index])
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(5):
                    self.comm.allreduce(self.grads, tmp, n, algo=algo, bucket=spare, ctas=ctas)
                e1.record()
                e1.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / 5], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                times[algo] = t.item()
            self.calibration[n] = times
            out[n] = min(times, key=times.get)
        if self.comm.check_status():
            raise ops.NativeError("a peer did not arrive during the start-up measurement of the synchronisation kernels")
        tmp.barrier()
        del tmp
        return out

    def describe(self) -> str:
        """One line for the training banner: which kernels synchronise which buckets."""
        kinds = sorted(set(self.algos))
        per = ", ".join(f"{k} x{self.algos.count(k)}" for k in kinds)
        form = "reduce per bucket + one clip/AdamW/all-gather kernel" if self.clip else \
               "reduce-scatter + AdamW + all-gather per bucket"
        when = "overlapped with backward" if self.overlap else "after backward"
        how = ""
        if self.calibration:
            how = "; measured at start-up (ms): " + ", ".join(
                f"{n * 2 / 2 ** 20:.0f} MB " + "/".join(f"{k} {v:.3f}" for k, v in t.items())
                for n, t in sorted(self.calibration.items()))
        return f"fused device kernels ({form}), {when}; {len(self.buckets)} buckets: {per}{how}"

    def _opt_args(self):
        m, o = self.model, self.model.optim
        nd = m.nodecay if o.weight_decay > 0 else None
        return (ops._p(m.master), ops._p(m.adam_m), ops._p(m.adam_v), ops._p(m.step_dev), ops._p(m.lr_dev),
                ctypes.c_float(o.beta1), ctypes.c_float(o.beta2), ctypes.c_float(o.eps), ctypes.c_float(o.weight_decay)), \
               (ops._p(nd), 0 if nd is None else nd.shape[0])

    def launch_bucket(self, b: Bucket) -> None:
        """Called on the host as soon as backward has enqueued the last kernel of bucket ``b``."""
        last = b.index == len(self.buckets) - 1
        if last:
            # End of backward on the compute stream.  Recorded before the fence, so the last synchronisation kernel is
            # ordered behind this timestamp: a node beside it in a captured graph could be run after it.
            nlog = self.tlog.numel()
            ops._check(self.lib.cme_record_time(ctypes.c_void_p(self.tlog.data_ptr() + 8 * (nlog - 2)), ops._stream()))
        self.model.fence(self.stream)                 # the bucket's producers, on either of the engine's streams
        opt, nd = self._opt_args()
        with nvtx_range(f"fused_sync_bucket_{b.index}", self.profile):
            self._launch_bucket_kernel(b, opt, nd, last)
        self.launched += 1
        if last and self.clip:
            with nvtx_range("fused_sync_clip_adamw", self.profile):
                self._launch_clip()

    def _launch_bucket_kernel(self, b: Bucket, opt, nd, last: bool) -> None:
        ops._check(self.lib.cme_comm_fused_adamw(
            self.world, self.comm.rank, self.grads.c_ptrs, self.params.c_ptrs, self.comm.flags.c_ptrs,
            ctypes.c_void_p(self.grads.multicast_ptr), ctypes.c_void_p(self.params.multicast_ptr),
            ctypes.c_longlong(b.start), ctypes.c_longlong(b.numel), *opt, ctypes.c_float(self.grad_scale), *nd,
            ALGOS[self.algos[b.index]], b.index, self.comm.max_buckets, self.tail_ctas if last else self.ctas,
            ops._p(self.comm.ctl), ops._p(self.comm.status), ctypes.c_double(self.comm.budget_ms),
            ops._p(self.gred), ops._p(self.norm_part), ops._p(self.norm_bucket), ops._p(self.tlog),
            ctypes.c_void_p(self.stream.cuda_stream)))

    def _launch_clip(self) -> None:
        """Second phase under clipping: global norm across ranks, clip, AdamW on the owned slices, all-gather."""
        opt, nd = self._opt_args()
        nb = len(self.buckets)
        ops._check(self.lib.cme_comm_clip_adamw(
            self.world, self.comm.rank, self.params.c_ptrs, self.comm.flags.c_ptrs,
            ctypes.c_void_p(self.params.multicast_ptr), ops._p(self.ranges), nb, ops._p(self.gred),
            ops._p(self.norm_bucket), *opt[:5], *opt[5:], ctypes.c_float(self.model.optim.clip_norm), *nd,
            int(self.has_multicast), nb, 2 * (nb + 1), self.comm.max_buckets, self.tail_ctas,
            ops._p(self.comm.ctl), ops._p(self.comm.status), ctypes.c_double(self.comm.budget_ms), ops._p(self.tlog),
            ctypes.c_void_p(self.stream.cuda_stream)))
        self.launched += 1

    def join(self) -> None:
        """Make the compute stream wait for every bucket kernel (parameters are then final on this rank).  With
        ``measure_exposed`` set (eager steps only) the wait is bracketed by timing events: the time the compute
        stream sits idle behind the last bucket kernels is the step's exposed synchronisation time."""
        cur = torch.cuda.current_stream()
        nlog = self.tlog.numel()
        ops._check(self.lib.cme_record_time(ctypes.c_void_p(self.tlog.data_ptr() + 8 * (nlog - 1)),
                                            ctypes.c_void_p(self.stream.cuda_stream)))
        ev = torch.cuda.Event()
        ev.record(self.stream)
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

    def timeline(self) -> dict:
        """Device timestamps of the most recent step (synchronises): per bucket the start and end of its kernel
        relative to the end of backward on the compute stream, in ms, and the exposed synchronisation time -- how
        long after the last backward kernel the last synchronisation kernel ended (0 if it ended earlier).  Works
        for replayed CUDA graphs, where host-side events cannot bracket the wait."""
        torch.cuda.synchronize(self.model.device)
        t = self.tlog.tolist()
        bwd_end, comm_end = t[-2], t[-1]
        nb = len(self.buckets) + (1 if self.clip else 0)
        rel = lambda x: (x - bwd_end) / 1e6
        return {"exposed_ms": max(0.0, rel(comm_end)),
                "buckets": [[round(rel(t[2 * b]), 4), round(rel(t[2 * b + 1]), 4)] for b in range(nb)],
                "bucket_mb": [round(b.numel * 2 / 2 ** 20, 2) for b in self.buckets]}

    def check_status(self) -> int:
        """Non-zero when a bounded wait of a synchronisation kernel ran out since the last check: some rank did not
        arrive, the step's parameters are not trustworthy."""
        return self.comm.check_status()

    def owned_mask(self) -> torch.Tensor:
        """1.0 where this rank owns the optimizer state (slice ``rank`` of every bucket), else 0.0.  Buckets
        synchronised one-shot are updated on every rank with identical results; the same slice is taken there."""
        mask = torch.zeros(self.model.layout.total, dtype=torch.float32, device=self.model.device)
        for b in self.buckets:
            per = b.numel // self.world
            s0 = b.start + per * self.comm.rank
            mask[s0:s0 + per] = 1.0
        return mask

    def gather_state(self):
        """Full fp32 master / moment arenas on every rank (checkpointing): owned slices summed over ranks.
        Collective: every rank must call it."""
        m = self.model
        mask = self.owned_mask()
        out = []
        for t in (m.master, m.adam_m, m.adam_v):
            full = t * mask
            if self.world > 1:
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
