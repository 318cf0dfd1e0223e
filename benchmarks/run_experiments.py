"""Experiment harness around the training driver: repeated benchmarks with warm-up drop and validity checks,
bucket-size sweeps, weak / strong scaling over 1/2/4/8 GPUs, trajectory validation of every synchronisation mode
against the blocking one, a correctness matrix, and an artifact check.

Role of the reference's SLURM scripts and Python summarisers (FINAL_CLEAN_CODE_/scripts/: run_correctness_matrix.sh,
run_full_validation.sh, run_single_gpu_repeated_bench.sh, run_training_bucket_sweep.sh, run_strong_scaling.sh,
run_weak_scaling.sh, run_trajectory_validation.sh, run_edge_case_validation.sh, check_artifacts.py).  One Python
entry point instead of a script per experiment; every run goes through the same CLI a user would call, every child
runs under a timeout, results land in one JSON file per experiment under --out.

    python benchmarks/run_experiments.py repeated  --preset parity-h256 --repeats 4 --steps 100
    python benchmarks/run_experiments.py buckets   --preset gpt2-small --gpus 4 --bucket-kb 1024 8192 25600
    python benchmarks/run_experiments.py scaling   --preset gpt2-small --gpus 1 2 4 8 [--strong]
    python benchmarks/run_experiments.py trajectory --preset parity-h128 --gpus 2 --steps 12
    python benchmarks/run_experiments.py edge      --gpus 3            # non-power-of-two ranks, odd batch
    python benchmarks/run_experiments.py matrix                        # pytest groups -> markdown table
    python benchmarks/run_experiments.py check --out results           # artifact audit
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from cme213_final_project_b200.utils.logparse import (compare_trajectories, parse_run, parse_trajectory,  # noqa: E402
                                                      summarize_repeats)

_PORT = [29850]


def clean_env():
    """Environment without inherited CME213_* toggles (the reference's cme213_clean_env, common_env.sh:22-40)."""
    return {k: v for k, v in os.environ.items() if not k.startswith("CME213_")}


def train_cmd(gpus, args):
    if gpus <= 1:
        return [sys.executable, "-m", "cme213_final_project_b200.train"] + args
    _PORT[0] += 1
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}",
            "--master-addr", "127.0.0.1", "--master-port", str(_PORT[0]), "-m",
            "cme213_final_project_b200.train"] + args


def run(gpus, args, timeout=1800):
    t0 = time.time()
    try:
        r = subprocess.run(train_cmd(gpus, args), capture_output=True, text=True, timeout=timeout, env=clean_env(),
                           cwd=ROOT)
        out, rc = r.stdout + "\n" + r.stderr[-2000:], r.returncode
    except subprocess.TimeoutExpired as e:
        out, rc = (e.stdout or "") + "\nTIMEOUT", 124
    return out, rc, time.time() - t0


def base_args(a):
    args = ["--preset", a.preset, "--epochs", str(a.epochs), "--max-steps", str(a.steps), "--synthetic" if a.synthetic
            else a.data, "--log-every", str(max(a.steps, 1))]
    if a.cuda_graph:
        args.append("--cuda-graph")
    return args


def save(a, name, obj):
    os.makedirs(a.out, exist_ok=True)
    path = os.path.join(a.out, name + ".json")
    json.dump(obj, open(path, "w"), indent=1)
    print(f"[harness] wrote {path}")


def cmd_repeated(a):
    toks, valid, rows = [], [], []
    for rep in range(1, a.repeats + 1):
        out, rc, wall = run(a.gpus[0], base_args(a) + a.extra)
        s = parse_run(out)
        ok = s.valid and rc == 0
        toks.append(s.last.tok_s if s.last else float("nan"))
        valid.append(ok)
        rows.append({"repeat": rep, "rc": rc, "valid": ok, "reason": s.reason, "tok_s": toks[-1],
                     "loss": s.last.loss if s.last else None, "wall_s": wall})
        print(f"[repeated] {rep}/{a.repeats} tok/s={toks[-1]:.0f} valid={ok}")
    save(a, f"repeated_{a.preset}_g{a.gpus[0]}", {"runs": rows, "summary": summarize_repeats(toks, valid, a.min_repeat)})


def cmd_buckets(a):
    res = []
    for mode, kb in [("blocking", 0)] + [("overlap", k) for k in a.bucket_kb]:
        out, rc, _ = run(a.gpus[0], base_args(a) + ["--sync-mode", mode, "--bucket-kb", str(kb)] + a.extra)
        s = parse_run(out)
        res.append({"sync_mode": mode, "bucket_kb": kb, "valid": s.valid and rc == 0,
                    "tok_s": s.last.tok_s if s.last else None,
                    "grad_sync_ms": s.last.grad_sync_ms if s.last else None,
                    "grad_finish_ms": s.last.grad_finish_ms if s.last else None,
                    "checksum_span": s.last.checksum_span if s.last else None})
        print(f"[buckets] {mode} kb={kb} -> {res[-1]['tok_s']}")
    base = res[0]["tok_s"] or float("nan")
    for r in res:
        r["speedup_vs_blocking"] = (r["tok_s"] / base) if r["tok_s"] else None
    save(a, f"buckets_{a.preset}_g{a.gpus[0]}", res)


def cmd_scaling(a):
    res = []
    for g in a.gpus:
        extra = list(a.extra)
        if a.strong:                                   # total batch fixed: per-rank batch shrinks
            extra += ["--batch-size", str(max(1, a.total_batch // g))]
        out, rc, _ = run(g, base_args(a) + ["--sync-mode", "overlap" if g > 1 else "blocking"] + extra)
        s = parse_run(out)
        res.append({"gpus": g, "valid": s.valid and rc == 0, "tok_s": s.last.tok_s if s.last else None})
        print(f"[scaling] {g} GPUs -> {res[-1]['tok_s']}")
    one = next((r["tok_s"] for r in res if r["gpus"] == 1), None)
    for r in res:
        if one and r["tok_s"]:
            r["efficiency"] = r["tok_s"] / (one * (1 if a.strong else r["gpus"]))
    save(a, f"{'strong' if a.strong else 'weak'}_scaling_{a.preset}", res)


def cmd_trajectory(a):
    modes = {"blocking": ["--sync-mode", "blocking"], "overlap": ["--sync-mode", "overlap", "--bucket-kb", "256"],
             "comm_thread": ["--sync-mode", "overlap", "--comm-thread", "--bucket-kb", "256"],
             "deferred": ["--sync-mode", "blocking", "--defer-grad-avg"]}
    traj = {}
    for name, flags in modes.items():
        out, rc, _ = run(a.gpus[0], base_args(a) + ["--trace-trajectory"] + flags + a.extra)
        traj[name] = parse_trajectory(out)
        print(f"[trajectory] {name}: {len(traj[name])} steps rc={rc}")
    res = {name: compare_trajectories(traj["blocking"], t) for name, t in traj.items() if name != "blocking"}
    save(a, f"trajectory_{a.preset}_g{a.gpus[0]}", {"comparisons": res, "all_ok": all(r["ok"] for r in res.values())})


def cmd_edge(a):
    cases = [("ranks", a.gpus[0], []), ("batch31", a.gpus[0], ["--batch-size", "31"])]
    res = []
    for name, g, flags in cases:
        for mode in ("blocking", "overlap"):
            out, rc, _ = run(g, base_args(a) + ["--sync-mode", mode] + flags + a.extra)
            s = parse_run(out)
            res.append({"case": name, "gpus": g, "sync_mode": mode, "valid": s.valid and rc == 0, "reason": s.reason,
                        "tok_s": s.last.tok_s if s.last else None})
            print(f"[edge] {name} {mode}: valid={res[-1]['valid']}")
    save(a, "edge_cases", res)


def cmd_matrix(a):
    groups = {"gemm": "tests/test_gemm_gpu.py", "kernels": "tests/test_kernels_gpu.py",
              "attention": "tests/test_attention_tc_gpu.py", "model": "tests/test_model_gpu.py",
              "multi_gpu": "tests/test_multi_gpu.py", "cpu": "-m not gpu"}
    rows = []
    for name, sel in groups.items():
        args = [sys.executable, "-m", "pytest", "-q"] + (sel.split() if sel.startswith("-m") else [sel, "-m", "gpu"])
        if sel.startswith("-m"):
            args += ["tests"]
        t0 = time.time()
        r = subprocess.run(args, capture_output=True, text=True, cwd=ROOT, timeout=3600)
        tail = r.stdout.strip().splitlines()[-1] if r.stdout.strip() else ""
        rows.append({"group": name, "rc": r.returncode, "summary": tail, "seconds": round(time.time() - t0, 1)})
        print(f"[matrix] {name}: {tail}")
    os.makedirs(a.out, exist_ok=True)
    with open(os.path.join(a.out, "correctness_matrix.md"), "w") as f:
        f.write("| group | result | seconds |\n|---|---|---|\n")
        for r in rows:
            f.write(f"| {r['group']} | {'PASS' if r['rc'] == 0 else 'FAIL'}: {r['summary']} | {r['seconds']} |\n")
    save(a, "correctness_matrix", rows)


def cmd_check(a):
    """Artifact audit: every result file parses, is non-empty and has no non-finite number."""
    bad = []
    for fn in sorted(os.listdir(a.out)) if os.path.isdir(a.out) else []:
        if not fn.endswith(".json"):
            continue
        try:
            txt = open(os.path.join(a.out, fn)).read()
            obj = json.loads(txt)
            if not obj or "NaN" in txt or "Infinity" in txt:
                bad.append(fn)
        except Exception:
            bad.append(fn)
    print(f"[check] {'OK' if not bad else 'BAD: ' + ', '.join(bad)}")
    return 1 if bad else 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("experiment", choices=["repeated", "buckets", "scaling", "trajectory", "edge", "matrix", "check"])
    ap.add_argument("--preset", default="parity-h256")
    ap.add_argument("--gpus", type=int, nargs="+", default=[1])
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--repeats", type=int, default=4)
    ap.add_argument("--min-repeat", type=int, default=2)
    ap.add_argument("--bucket-kb", type=int, nargs="+", default=[256, 1024, 4096])
    ap.add_argument("--total-batch", type=int, default=32)
    ap.add_argument("--strong", action="store_true")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--cuda-graph", action="store_true")
    from cme213_final_project_b200.data import reference_corpus_path
    ap.add_argument("--data", default=reference_corpus_path())
    ap.add_argument("--out", default="results")
    a, extra = ap.parse_known_args()          # anything not recognised here is passed to the trainer
    a.extra = [e for e in extra if e != "--"]
    if not a.synthetic and not os.path.exists(a.data):
        a.synthetic = True
    fn = {"repeated": cmd_repeated, "buckets": cmd_buckets, "scaling": cmd_scaling, "trajectory": cmd_trajectory,
          "edge": cmd_edge, "matrix": cmd_matrix, "check": cmd_check}[a.experiment]
    sys.exit(fn(a) or 0)


if __name__ == "__main__":
    main()
