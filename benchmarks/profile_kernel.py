"""Profile ONE kernel of a command with Nsight Compute and write a short markdown summary; fall back to the command's
own CUDA-event timings when the profiler is missing, refused or closed.

Role of the reference's profiler drivers (FINAL_CLEAN_CODE_/scripts/profile_fusion_kernels.sh:69-81 falls back to
CUDA-event timing when ncu is refused; profile_training_hotspots.sh:50-58 wraps ncu around a dedicated driver;
summarize_fusion_profiles.py / roofline_fusion_analysis.py turn the raw CSV into roofline rows).

    python benchmarks/profile_kernel.py --kernel attn_fwd_tc --skip 2 --count 1 --out prof_attn_fwd \
        -- python benchmarks/bench_attention.py --iters 2

Rules this wrapper enforces, because a profiler run that goes wrong can take a shared GPU down with it:
  * the command first runs WITHOUT the profiler and must exit 0 -- a program that faults is never profiled;
  * one kernel (`-k regex:`), a few launches (`--count`, at most 3), sections instead of `--set full` unless asked;
  * `--clock-control none` always: the profiler must not lock the GPU's clocks;
  * the profiler process is never given a timeout -- killing it in mid-capture is what leaves GPUs hung; size the
    command (small case, few warm-up launches) so the capture ends by itself.
Output: <out>.ncu-rep (if profiled), <out>.md with the figures used for roofline reading, <out>.json with the same.
"""
import argparse
import csv
import io
import json
import os
import shutil
import subprocess
import sys
import time

METRICS = {
    "gpu__time_duration.sum": "duration",
    "launch__grid_size": "grid",
    "launch__block_size": "block",
    "launch__registers_per_thread": "registers per thread",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active": "tensor pipe active %",
    "sm__warps_active.avg.pct_of_peak_sustained_active": "achieved occupancy %",
    "dram__bytes_read.sum": "DRAM read",
    "dram__bytes_write.sum": "DRAM write",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed": "DRAM throughput %",
    "lts__throughput.avg.pct_of_peak_sustained_elapsed": "L2 throughput %",
    "sm__inst_executed.sum": "warp instructions",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed": "SM throughput %",
}


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        return json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))
    except OSError:
        return {}


def summarize(rep, out, kernel, cmd, flops, nbytes):
    r = subprocess.run(["ncu", "-i", rep, "--page", "raw", "--csv"], capture_output=True, text=True)
    rows = list(csv.reader(io.StringIO(r.stdout)))
    if len(rows) < 3:
        return None
    head, units = rows[0], rows[1]
    launches = []
    for row in rows[2:]:
        rec = {}
        for name, unit, val in zip(head, units, row):
            if name in METRICS or name == "Kernel Name":
                rec[name] = (val, unit)
        launches.append(rec)
    pk = peaks()
    lines = [f"# `{kernel}`: Nsight Compute summary", "", "Command (one GPU; the same command had exited 0 without the profiler):", "",
             "    " + " ".join(cmd), ""]
    res = {"kernel": kernel, "launches": []}
    for i, rec in enumerate(launches):
        lines += [f"Launch {i + 1}: `{rec.get('Kernel Name', ('?', ''))[0][:100]}`", "", "| metric | value |", "|---|---|"]
        vals = {}
        for m, label in METRICS.items():
            if m in rec:
                v, u = rec[m]
                lines.append(f"| {label} | {v} {u} |")
                vals[label] = [v, u]
        try:
            dur_ns = float(rec["gpu__time_duration.sum"][0].replace(",", ""))
            if rec["gpu__time_duration.sum"][1] in ("us", "usecond"):
                dur_ns *= 1e3
            elif rec["gpu__time_duration.sum"][1] in ("ms", "msecond"):
                dur_ns *= 1e6
            if flops:
                tf = flops / dur_ns / 1e3
                frac = f" = {tf / pk['bf16_tflops']:.2f} of measured burst peak" if pk.get("bf16_tflops") else ""
                lines.append(f"| achieved TFLOP/s (algorithmic) | {tf:.0f}{frac} |")
                vals["tflops"] = tf
            if nbytes:
                gbs = nbytes / dur_ns
                frac = f" = {gbs / pk['hbm_gbs']:.2f} of measured copy bandwidth" if pk.get("hbm_gbs") else ""
                lines.append(f"| achieved GB/s (algorithmic) | {gbs:.0f}{frac} |")
                vals["gbs"] = gbs
        except (KeyError, ValueError):
            pass
        lines.append("")
        res["launches"].append(vals)
    open(out + ".md", "w").write("\n".join(lines))
    json.dump(res, open(out + ".json", "w"), indent=1)
    return res


def summarize_light(rep, out, kernel, cmd, flops, nbytes):
    """One row per distinct kernel name: launches seen, mean duration, DRAM / L2 / SM throughput of the first one."""
    r = subprocess.run(["ncu", "-i", rep, "--page", "raw", "--csv"], capture_output=True, text=True)
    rows = list(csv.reader(io.StringIO(r.stdout)))
    if len(rows) < 3:
        return None
    head = rows[0]
    col = {n: i for i, n in enumerate(head)}
    want = ["gpu__time_duration.sum", "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
            "lts__throughput.avg.pct_of_peak_sustained_elapsed", "sm__throughput.avg.pct_of_peak_sustained_elapsed",
            "launch__grid_size", "launch__block_size", "launch__registers_per_thread"]
    unit = {n: rows[1][col[n]] for n in want if n in col}
    agg = {}
    for row in rows[2:]:
        name = row[col["Kernel Name"]].split("(")[0][:70]
        rec = agg.setdefault(name, {"n": 0, "dur": 0.0, "first": None})
        try:
            d = float(row[col["gpu__time_duration.sum"]].replace(",", ""))
        except (KeyError, ValueError):
            d = float("nan")
        d *= {"ns": 1e-3, "nsecond": 1e-3, "us": 1.0, "usecond": 1.0, "ms": 1e3, "msecond": 1e3}.get(unit.get("gpu__time_duration.sum", "us"), 1.0)
        rec["n"] += 1
        rec["dur"] += d
        if rec["first"] is None:
            rec["first"] = {n: row[col[n]] for n in want if n in col}
    lines = [f"# Kernels matching `{kernel}`: Nsight Compute SpeedOfLight summary", "",
             "Command (one GPU, small case; the same command had exited 0 without the profiler):", "", "    " + " ".join(cmd), "",
             "| kernel | launches | mean us | DRAM % of peak | L2 % | SM % | grid | block | regs |", "|---|---|---|---|---|---|---|---|---|"]
    res = {"kernel": kernel, "kernels": {}}
    for name, rec in agg.items():
        f = rec["first"] or {}
        g = lambda k: f.get(k, "")
        lines.append(f"| `{name}` | {rec['n']} | {rec['dur'] / rec['n']:.1f} | {g(want[1])} | {g(want[2])} | {g(want[3])} | "
                     f"{g(want[4])} | {g(want[5])} | {g(want[6])} |")
        res["kernels"][name] = {"launches": rec["n"], "mean_us": rec["dur"] / rec["n"], **f}
    open(out + ".md", "w").write("\n".join(lines) + "\n")
    json.dump(res, open(out + ".json", "w"), indent=1)
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True, help="regular expression matched against kernel names")
    ap.add_argument("--skip", type=int, default=0, help="matching launches to skip first (warm-up)")
    ap.add_argument("--count", type=int, default=1, help="launches to capture (1-3)")
    ap.add_argument("--full", action="store_true", help="--set full (about 40 passes per launch) instead of four sections")
    ap.add_argument("--light", action="store_true",
                    help="many short kernels of a small case: the SpeedOfLight section only, up to 80 launches, one "
                         "table row per distinct kernel name")
    ap.add_argument("--flops", type=float, default=0, help="algorithmic FLOPs of one launch, for the roofline line")
    ap.add_argument("--bytes", type=float, default=0, help="algorithmic bytes of one launch")
    ap.add_argument("--out", required=True)
    ap.add_argument("cmd", nargs=argparse.REMAINDER)
    a = ap.parse_args()
    cmd = [c for c in a.cmd if c != "--"]
    if not cmd:
        ap.error("give the command after --")
    a.count = max(1, min(a.count, 80 if a.light else 3))
    os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
    t0 = time.time()
    plain = subprocess.run(cmd, capture_output=True, text=True)
    open(a.out + ".plain.log", "w").write(plain.stdout + plain.stderr)
    if plain.returncode != 0:
        print(f"[profile] the command exits {plain.returncode} without the profiler: not profiled", file=sys.stderr)
        return 86
    print(f"[profile] plain run ok in {time.time() - t0:.1f} s")
    why = None
    if shutil.which("ncu") is None:
        why = "ncu is not installed"
    else:
        sel = ["--set", "full"] if a.full else ["--section", "SpeedOfLight", "--section", "LaunchStats"] if a.light else \
              ["--section", "SpeedOfLight", "--section", "MemoryWorkloadAnalysis", "--section", "LaunchStats",
               "--section", "Occupancy", "--section", "ComputeWorkloadAnalysis"]
        ncu = ["ncu", "--clock-control", "none", "-k", "regex:" + a.kernel, "-s", str(a.skip), "-c", str(a.count),
               *sel, "-f", "-o", a.out] + cmd
        t1 = time.time()
        r = subprocess.run(ncu, capture_output=True, text=True)          # no timeout: never kill a capture
        open(a.out + ".ncu.log", "w").write(r.stdout + r.stderr)
        txt = (r.stdout + r.stderr).lower()
        if r.returncode != 0 or "closed on this pool" in txt or "not profiled" in txt or not os.path.exists(a.out + ".ncu-rep"):
            why = f"ncu exited {r.returncode}: " + (r.stdout + r.stderr).strip().splitlines()[-1][:160] if (r.stdout + r.stderr).strip() else "no output"
        else:
            print(f"[profile] captured in {time.time() - t1:.1f} s")
            res = (summarize_light if a.light else summarize)(a.out + ".ncu-rep", a.out, a.kernel, ncu, a.flops, a.bytes)
            if res is None:
                why = "the report holds no matching launch"
    if why:
        # event-timing fallback: the benchmark commands print their own CUDA-event timings; keep those as the record
        print(f"[profile] profiler unavailable ({why}); keeping the command's CUDA-event timings")
        open(a.out + ".md", "w").write(
            f"# `{a.kernel}`: CUDA-event timings (profiler unavailable: {why})\n\nCommand:\n\n    " + " ".join(cmd) +
            "\n\nOutput of the command (its own CUDA-event timings):\n\n" +
            "\n".join("    " + l for l in plain.stdout.strip().splitlines()[-40:]) + "\n")
        json.dump({"kernel": a.kernel, "profiler": None, "reason": why, "stdout_tail": plain.stdout.strip().splitlines()[-40:]},
                  open(a.out + ".json", "w"), indent=1)
    print(f"[profile] wrote {a.out}.md")
    return 0


if __name__ == "__main__":
    sys.exit(main())
