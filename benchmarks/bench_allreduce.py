"""Gradient all-reduce micro-benchmark: this library's peer-memory kernels (one-shot, two-shot, NVLS) and the fused
reduce-scatter + AdamW + all-gather kernel against NCCL, 1 KB - 1 GB, bf16 and fp32, with an alpha-beta fit.

Role of the reference's collective benchmarks (FINAL_CLEAN_CODE_/tests/benchmark_allreduce_alpha_beta.cu: 4 KB - 32 MB
sweep over device / host-pinned / nccl backends; FINAL_CLEAN_CODE_/scripts/predict_comm_model.py: t = alpha + beta *
bytes).  Every time is device-timed with CUDA events and is the max over ranks; bus bandwidth = bytes * 2 (W-1)/W / t.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        benchmarks/bench_allreduce.py [--max-mb 1024] [--iters 10] [--json out.json]
"""
import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from cme213_final_project_b200.parallel.comm_model import fit_alpha_beta          # noqa: E402
from cme213_final_project_b200.parallel.dist import DistributedContext            # noqa: E402
from cme213_final_project_b200.parallel.fused_sync import PeerComm                # noqa: E402
from cme213_final_project_b200.parallel.symm import LocalPeers, SymmetricBuffer   # noqa: E402


def timed(fn, iters, dev, sync):
    for _ in range(3):
        fn()
    sync()
    ts = []
    multi = dist.is_initialized() and dist.get_world_size() > 1
    for _ in range(iters):
        if multi:
            dist.barrier(device_ids=[dev.index])
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        t = torch.tensor([s.elapsed_time(e)], device=dev)
        if multi:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ts.append(t.item())
    return statistics.median(ts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-kb", type=int, default=1)
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--factor", type=int, default=4)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ctas", type=int, default=296)
    ap.add_argument("--json")
    a = ap.parse_args()
    ctx = DistributedContext().init(backend="nccl", device="cuda")
    dev, W, R = ctx.device, ctx.world_size, ctx.rank
    comm = PeerComm(dev, max_buckets=4, budget_ms=2000.0)
    multi = dist.is_initialized() and W > 1
    sync = lambda: (torch.cuda.synchronize(), dist.barrier(device_ids=[dev.index]) if multi else None)
    # one rank (a single GPU): plain buffers stand in for the symmetric ones; the kernels run their world-of-one case
    mkbuf = (lambda n, dt: SymmetricBuffer(n, dt, dev)) if multi else \
            (lambda n, dt: LocalPeers(torch.zeros(n, dtype=dt, device=dev)))
    rows = []
    for dtype, es in ((torch.bfloat16, 2), (torch.float32, 4)):
        max_n = a.max_mb * (1 << 20) // es
        src, dst = mkbuf(max_n, dtype), mkbuf(max_n, dtype)
        src.tensor.normal_(generator=torch.Generator(device=dev).manual_seed(1000 + R))
        nccl_buf = src.tensor.clone()
        algos = ["one_shot", "two_shot"] + (["nvls"] if src.multicast_ptr else [])
        fused = None
        if dtype == torch.bfloat16:
            # the training path's kernel: reduce-scatter + scale + AdamW on this rank's fp32 shard + all-gather of the
            # bf16 parameters (src = gradient arena, dst = parameter arena)
            import ctypes
            from cme213_final_project_b200 import ops
            master = torch.zeros(max_n, dtype=torch.float32, device=dev)
            am, av = torch.zeros_like(master), torch.zeros_like(master)
            step = torch.ones(1, dtype=torch.int32, device=dev)
            lr = torch.full((1,), 1e-4, dtype=torch.float32, device=dev)
            has_mc = bool(src.multicast_ptr and dst.multicast_ptr)
            fused_algo = [1]                       # 1 two-shot over peer loads, 2 NVLS; set per measurement below

            def fused(n, ctas):
                ops._check(comm.lib.cme_comm_fused_adamw(
                    W, R, src.c_ptrs, dst.c_ptrs, comm.flags.c_ptrs, ctypes.c_void_p(src.multicast_ptr),
                    ctypes.c_void_p(dst.multicast_ptr), ctypes.c_longlong(0), ctypes.c_longlong(n), ops._p(master),
                    ops._p(am), ops._p(av), ops._p(step), ops._p(lr), ctypes.c_float(0.9), ctypes.c_float(0.95),
                    ctypes.c_float(1e-8), ctypes.c_float(0.1), ctypes.c_float(1.0 / W), None, 0, fused_algo[0], 3,
                    comm.max_buckets, ctas, ops._p(comm.ctl), ops._p(comm.status), ctypes.c_double(comm.budget_ms),
                    None, None, None, None, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        nbytes = a.min_kb * 1024
        while nbytes <= a.max_mb * (1 << 20):
            n = max(nbytes // es, (16 // es) * W)
            n -= n % ((16 // es) * W)
            rec = {"dtype": str(dtype).split(".")[-1], "bytes": n * es, "world": W}
            rec["nccl_ms"] = timed(lambda: dist.all_reduce(nccl_buf[:n]) if multi else None, a.iters, dev, sync)
            for i, algo in enumerate(algos):
                if algo == "one_shot" and n * es > (32 << 20):
                    continue
                ctas = min(a.ctas, max(1, n * es // 4096))
                rec[algo + "_ms"] = timed(lambda: comm.allreduce(src, dst, n, algo=algo, bucket=i, ctas=ctas), a.iters,
                                          dev, sync)
            if fused is not None:
                fc = min(4 * 148, max(1, n * es // 4096))
                for name, code in (("two_shot", 1), ("nvls", 2)):
                    if code == 2 and not has_mc:
                        continue
                    fused_algo[0] = code
                    rec[f"fused_{name}_ms"] = timed(lambda: fused(n, fc), a.iters, dev, sync)
                rec["fused_adamw_ms"] = min(rec[k] for k in ("fused_two_shot_ms", "fused_nvls_ms") if k in rec)
                # bytes over NVLink per GPU and direction: (W-1)/W of the gradients in, the same of the parameters out
                rec["fused_adamw_link_gbs"] = n * es * (W - 1) / W / (rec["fused_adamw_ms"] * 1e-3) / 1e9
            assert comm.check_status() == 0
            best = min((rec[k], k) for k in rec if k.endswith("_ms") and k != "nccl_ms" and not k.startswith("fused_"))
            rec["best"] = best[1][:-3]
            bus = lambda ms: rec["bytes"] * 2 * (W - 1) / W / (ms * 1e-3) / 1e9
            rec["best_busbw_gbs"], rec["nccl_busbw_gbs"] = bus(best[0]), bus(rec["nccl_ms"])
            rec["frac_of_770"] = rec["best_busbw_gbs"] / 770.0
            rows.append(rec)
            if R == 0:
                print(json.dumps(rec), flush=True)
            nbytes *= a.factor
        del src, dst
    fits = {}
    for algo in ("nccl", "one_shot", "two_shot", "nvls"):
        pts = [(r["bytes"], r[algo + "_ms"]) for r in rows if algo + "_ms" in r and r["dtype"] == "bfloat16"]
        if len(pts) >= 3:
            al, be = fit_alpha_beta(pts)
            fits[algo] = {"alpha_ms": al, "beta_ms_per_mb": be * (1 << 20)}
    # The table the training path consumes (parallel/fused_sync.py::choose_algo), from the fused kernel's own timings
    # where it has both variants: one-shot up to the largest size it won; NVLS from the smallest size after which it
    # stays ahead of peer loads.
    bf = [r for r in rows if r["dtype"] == "bfloat16"]
    cross = [r["bytes"] for r in bf if r.get("best") == "one_shot"]
    nvls_min, use_nvls = 0, False
    for r in sorted(bf, key=lambda r: -r["bytes"]):
        two, nv = r.get("fused_two_shot_ms", r.get("two_shot_ms")), r.get("fused_nvls_ms", r.get("nvls_ms"))
        if nv is None or two is None or nv > two:
            break
        nvls_min, use_nvls = r["bytes"], True
    table = {str(W): {"one_shot_max_bytes": max(cross) if cross else 0, "use_nvls": use_nvls,
                      "nvls_min_bytes": nvls_min, "measured": True}}
    if R == 0:
        print("FIT " + json.dumps(fits))
        print("TABLE " + json.dumps(table))
        if a.json:
            json.dump({"rows": rows, "fits": fits, "table": table}, open(a.json, "w"), indent=1)
    ctx.finalize()


if __name__ == "__main__":
    main()
