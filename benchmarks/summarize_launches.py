"""Per-kernel table of one training step from a profiler launch list.

Input: the CSV that `ncu --metrics gpu__time_duration.sum --csv --log-file launches.csv <command>` writes (one row per
launch and metric; profiler banner lines before the header are skipped).  The launches between the last two
occurrences of a marker kernel (default: the embedding forward, the first kernel of a step) are taken as one step and
grouped by kernel name: launches, total and mean device time, share of the step.

Role of the reference's timeline extractors, which do the same from an nsys export
(FINAL_CLEAN_CODE_/scripts/extract_nsys_top_kernels.py, extract_nsys_profile_summary.py); nsys is not part of this
tool chain, the launch list of ncu (one pass per kernel) is.

    ncu --metrics gpu__time_duration.sum --clock-control none -c 1300 --csv --log-file launches.csv \
        python bench.py --no-graph --steps 1 --warmup 1
    python benchmarks/summarize_launches.py launches.csv [--marker embed_fwd] [--json out.json]
"""
import argparse
import collections
import csv
import json
import re
import sys
from typing import Dict, List, Tuple

_UNIT_TO_US = {"nsecond": 1e-3, "ns": 1e-3, "usecond": 1.0, "us": 1.0, "msecond": 1e3, "ms": 1e3, "second": 1e6, "s": 1e6}


def read_launches(path: str, metric: str = "gpu__time_duration.sum") -> List[Tuple[int, str, float]]:
    """(launch id, kernel name, microseconds) per launch, in launch order."""
    with open(path) as f:
        lines = [l for l in f if l.startswith('"')]
    out = []
    for d in csv.DictReader(lines):
        if d.get("Metric Name") != metric:
            continue
        scale = _UNIT_TO_US.get(d.get("Metric Unit", "ns"), 1e-3)
        out.append((int(d["ID"]), d["Kernel Name"], float(d["Metric Value"].replace(",", "")) * scale))
    out.sort(key=lambda r: r[0])
    return out


def short_name(kernel: str) -> str:
    """Function name with its template arguments, without return type, namespaces of this library and parameters."""
    k = re.sub(r"^void ", "", kernel)
    depth, cut = 0, len(k)
    for i, ch in enumerate(k):                      # cut at the parameter list: the first '(' outside <...>
        if ch == "<":
            depth += 1
        elif ch == ">":
            depth -= 1
        elif ch == "(" and depth == 0:
            cut = i
            break
    k = k[:cut]
    for junk in ("<unnamed>::", "(anonymous namespace)::", "gemm_tc::", "(int)"):
        k = k.replace(junk, "")
    return k.replace(", ", ",")


def last_step(rows: List[Tuple[int, str, float]], marker: str) -> List[Tuple[int, str, float]]:
    marks = [i for i, (_, k, _) in enumerate(rows) if marker in k]
    if len(marks) < 2:
        raise SystemExit(f"fewer than two launches of a kernel matching '{marker}': cannot delimit a step")
    return rows[marks[-2]:marks[-1]]


def summarize(step: List[Tuple[int, str, float]]) -> Dict:
    agg: Dict[str, List[float]] = collections.OrderedDict()
    for _, k, us in step:
        a = agg.setdefault(short_name(k), [0, 0.0])
        a[0] += 1
        a[1] += us
    total = sum(us for _, _, us in step)
    rows = [{"kernel": k, "launches": int(n), "total_us": t, "mean_us": t / n, "share": t / total if total else 0.0}
            for k, (n, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])]
    return {"launches": len(step), "total_us": total, "kernels": rows}


def to_markdown(s: Dict) -> str:
    lines = [f"{s['launches']} launches, {s['total_us'] / 1e3:.2f} ms of device time.", "",
             "| kernel | launches | total us | mean us | share |", "|---|---|---|---|---|"]
    for r in s["kernels"]:
        lines.append(f"| `{r['kernel']}` | {r['launches']} | {r['total_us']:.0f} | {r['mean_us']:.1f} | {100 * r['share']:.1f} % |")
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("csv")
    ap.add_argument("--marker", default="embed_fwd", help="substring of the kernel that starts a step")
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    s = summarize(last_step(read_launches(a.csv), a.marker))
    print(to_markdown(s))
    if a.json:
        with open(a.json, "w") as f:
            json.dump(s, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
