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
    python benchmarks/run_experiments.py fusion    --preset gpt2-small --steps 30      # fusion ablation of the step
    python benchmarks/run_experiments.py graph     --preset parity-h256 --steps 200    # CUDA graph vs eager
    python benchmarks/run_experiments.py null      --preset parity-h256 --repeats 6    # run-to-run noise floor
    python benchmarks/run_experiments.py lr        --preset parity-h512 --lrs 2e-5 5e-5 1e-4 3e-4
    python benchmarks/run_experiments.py ucurve    --preset gpt2-small --gpus 8 --bucket-kb 1024 8192 25600 102400 \
                                                   --fits allreduce_8gpu.json      # bucket U-curve + alpha-beta prediction
    python benchmarks/run_experiments.py precision                                 # GEMM error per backend / precision
    python benchmarks/run_experiments.py check --out results           # artifact audit

Further reference scripts covered here: run_fusion_ablation.sh, cuda_graph_bench.sh, run_null_variance_bench.sh,
run_h512_lr_sweep.sh, summarize_bucket_ucurve.py + predict_comm_model.py, run_gemm_precision_validation.sh.
Every experiment leaves one JSON file and one markdown table under --out.
"""
import argparse
import json
import os
import re
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


def run(gpus, args, timeout=1800, env_extra=None):
    t0 = time.time()
    env = clean_env()
    env.update(env_extra or {})
    try:
        r = subprocess.run(train_cmd(gpus, args), capture_output=True, text=True, timeout=timeout, env=env,
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


def save(a, name, obj, table=None):
    """One JSON file per experiment and, when `table` = (header, rows) is given, the same numbers as markdown."""
    os.makedirs(a.out, exist_ok=True)
    path = os.path.join(a.out, name + ".json")
    json.dump(obj, open(path, "w"), indent=1)
    print(f"[harness] wrote {path}")
    if table:
        head, rows = table
        with open(os.path.join(a.out, name + ".md"), "w") as f:
            f.write("| " + " | ".join(head) + " |\n|" + "---|" * len(head) + "\n")
            for r in rows:
                f.write("| " + " | ".join("" if v is None else (f"{v:.4g}" if isinstance(v, float) else str(v))
                                          for v in r) + " |\n")


def sync_timeline(text):
    """The `SYNC_TIMELINE {json}` line the trainer prints after an epoch on the fused path (device timestamps of the
    last step's bucket kernels), or None."""
    for line in reversed(text.splitlines()):
        if line.startswith("SYNC_TIMELINE "):
            try:
                return json.loads(line[len("SYNC_TIMELINE "):])
            except ValueError:
                return None
    return None


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
    # the host-issued NCCL modes (blocking is the yardstick, as in the reference) and the fused device path, eager
    # and as one CUDA graph per step
    nccl = ["--comm-backend", "nccl"]
    modes = {"blocking": ["--sync-mode", "blocking"] + nccl,
             "overlap": ["--sync-mode", "overlap", "--bucket-kb", "256"] + nccl,
             "comm_thread": ["--sync-mode", "overlap", "--comm-thread", "--bucket-kb", "256"] + nccl,
             "deferred": ["--sync-mode", "blocking", "--defer-grad-avg"] + nccl,
             "fused": ["--sync-mode", "overlap", "--bucket-kb", "256", "--comm-backend", "fused"],
             "fused_graph": ["--sync-mode", "overlap", "--bucket-kb", "256", "--comm-backend", "fused", "--cuda-graph"]}
    traj, n_params = {}, 0
    for name, flags in modes.items():
        out, rc, _ = run(a.gpus[0], base_args(a) + ["--trace-trajectory"] + flags + a.extra)
        traj[name] = parse_trajectory(out)
        m = re.search(r"^Parameters: (\d+)", out, re.M)
        n_params = int(m.group(1)) if m else n_params
        print(f"[trajectory] {name}: {len(traj[name])} steps rc={rc}")
    res = {name: compare_trajectories(traj["blocking"], t, n_params=n_params) for name, t in traj.items()
           if name != "blocking"}
    spans = {name: max([max(abs(s["sum_span"]), abs(s["sumsq_span"]), abs(s["maxabs_span"])) for s in t] or [float("nan")])
             for name, t in traj.items()}
    g = lambda name, key: res[name][key] if name in res else 0.0
    rows = [[name, len(traj[name]), res[name]["ok"] if name in res else True,
             res[name]["identical_path"] if name in res else True, g(name, "max_loss_diff"),
             g(name, "max_rel_sumsq_diff"), g(name, "max_rel_sum_diff"),
             res[name].get("max_sum_diff_per_param", float("nan")) if name in res else 0.0, spans[name]]
            for name in modes]
    save(a, f"trajectory_{a.preset}_g{a.gpus[0]}",
         {"comparisons": res, "cross_rank_span": spans, "all_ok": all(r["ok"] for r in res.values())},
         (["mode", "steps", "within tolerance of blocking", "same sums as blocking", "max loss diff",
           "max rel diff of sum of squares", "max rel diff of sum", "max diff of sum per parameter",
           "largest cross-rank span"], rows))


def cmd_edge(a):
    cases = [("ranks", a.gpus[0], []), ("batch31", a.gpus[0], ["--batch-size", "31"])]
    res = []
    for name, g, flags in cases:
        for mode, backend in (("blocking", "nccl"), ("overlap", "nccl"), ("overlap", "fused")):
            out, rc, _ = run(g, base_args(a) + ["--sync-mode", mode, "--comm-backend", backend] + flags + a.extra)
            s = parse_run(out)
            res.append({"case": name, "gpus": g, "sync_mode": mode, "backend": backend,
                        "valid": s.valid and rc == 0, "reason": s.reason,
                        "tok_s": s.last.tok_s if s.last else None,
                        "checksum_span": s.last.checksum_span if s.last else None})
            print(f"[edge] {name} {mode}/{backend}: valid={res[-1]['valid']}")
    save(a, "edge_cases", res, (["case", "gpus", "sync", "backend", "valid", "tok/s", "checksum span"],
                                [[r["case"], r["gpus"], r["sync_mode"], r["backend"], r["valid"], r["tok_s"],
                                  r["checksum_span"]] for r in res]))


def _one(a, label, flags=(), env=None, gpus=None):
    out, rc, wall = run(gpus or a.gpus[0], base_args(a) + list(flags) + a.extra, env_extra=env)
    s = parse_run(out)
    row = {"variant": label, "rc": rc, "valid": s.valid and rc == 0, "reason": s.reason,
           "tok_s": s.last.tok_s if s.last else None, "loss": s.last.loss if s.last else None,
           "ms_per_step": (s.last.ms / max(s.last.steps, 1)) if s.last else None, "wall_s": round(wall, 1)}
    print(f"[{a.experiment}] {label}: tok/s={row['tok_s']} valid={row['valid']}")
    return row, out


def cmd_fusion(a):
    """Fusion ablation of the training step (the reference's run_fusion_ablation.sh: the same run with and without
    its epilogue fusion).  Variants: everything on; bias / activation / residual / activation-derivative as separate
    kernels after plain products; the GELU derivative re-evaluated in backward with the bias gradient as its own
    kernel; weight-gradient products on the main stream instead of the second one."""
    variants = [("all fusions", [], {}),
                ("no epilogue fusion", ["--no-epilogue-fusion"], {}),
                ("derivative recomputed, separate bias gradient", [], {"CME213_FFN_DERIV": "0"}),
                ("weight gradients on the main stream", [], {"CME213_WGRAD_STREAM": "0"})]
    graph = ["--cuda-graph"] if a.cuda_graph else []
    rows = [_one(a, label, graph + flags, env)[0] for label, flags, env in variants]
    base = rows[0]["tok_s"]
    for r in rows:
        r["relative_to_all"] = (r["tok_s"] / base) if (r["tok_s"] and base) else None
    save(a, f"fusion_ablation_{a.preset}_g{a.gpus[0]}", rows,
         (["variant", "valid", "tok/s", "ms/step", "vs all fusions"],
          [[r["variant"], r["valid"], r["tok_s"], r["ms_per_step"], r["relative_to_all"]] for r in rows]))


def cmd_graph(a):
    """Whole-step CUDA graph against eager launches (the reference's cuda_graph_bench.sh / CME213_USE_CUDA_GRAPH)."""
    rows = []
    for label, flags in (("eager", []), ("cuda graph", ["--cuda-graph"])):
        toks = []
        for _ in range(a.repeats):
            r, _ = _one(a, label, flags)
            toks.append(r["tok_s"] if r["valid"] else float("nan"))
        rows.append({"mode": label, **summarize_repeats(toks, [t == t for t in toks], a.min_repeat)})
    e, g = rows[0].get("mean"), rows[1].get("mean")
    speed = (g / e) if (e and g) else None
    save(a, f"graph_vs_eager_{a.preset}_g{a.gpus[0]}", {"rows": rows, "graph_speedup": speed},
         (["mode", "runs", "mean tok/s", "cv"], [[r["mode"], r.get("runs"), r.get("mean"), r.get("cv")] for r in rows]))


def cmd_null(a):
    """Null-variance run: the same configuration repeated; what differs between identical runs is the noise floor any
    claimed speed-up has to clear (the reference's run_null_variance_bench.sh)."""
    toks, valid = [], []
    for rep in range(a.repeats):
        r, _ = _one(a, f"repeat {rep + 1}", ["--cuda-graph"] if a.cuda_graph else [])
        toks.append(r["tok_s"] if r["tok_s"] else float("nan"))
        valid.append(bool(r["valid"]))
    summ = summarize_repeats(toks, valid, a.min_repeat)
    warm = [t for t, v in list(zip(toks, valid))[a.min_repeat - 1:] if v]
    spread = (max(warm) - min(warm)) / (sum(warm) / len(warm)) if len(warm) > 1 else None
    save(a, f"null_variance_{a.preset}_g{a.gpus[0]}", {"tok_s": toks, "valid": valid, "summary": summ,
                                                        "max_minus_min_over_mean": spread},
         (["repeat", "tok/s", "valid"], [[i + 1, t, v] for i, (t, v) in enumerate(zip(toks, valid))]))


def cmd_lr(a):
    """Learning-rate sweep: final logged loss per rate (the reference's run_h512_lr_sweep.sh)."""
    rows = []
    for lr in a.lrs:
        r, _ = _one(a, f"lr={lr:g}", ["--lr", str(lr)])
        rows.append({"lr": lr, **r})
    ok = [r for r in rows if r["valid"] and r["loss"] is not None]
    best = min(ok, key=lambda r: r["loss"])["lr"] if ok else None
    save(a, f"lr_sweep_{a.preset}_g{a.gpus[0]}", {"rows": rows, "best_lr": best},
         (["lr", "valid", "final loss", "tok/s"], [[r["lr"], r["valid"], r["loss"], r["tok_s"]] for r in rows]))


def cmd_ucurve(a):
    """Bucket-size U-curve on the fused path with the alpha-beta prediction beside the measurement (the reference's
    summarize_bucket_ucurve.py and predict_comm_model.py:109-139).  Measured: throughput, exposed synchronisation time
    and summed device time of the bucket kernels of the last step (from the trainer's SYNC_TIMELINE line).
    Predicted: sum over buckets of alpha + beta * bytes with the fit of --fits (bench_allreduce.py --json)."""
    from cme213_final_project_b200.parallel.comm_model import predict_bucketed
    fits = None
    if a.fits and os.path.exists(a.fits):
        f = json.load(open(a.fits)).get("fits", {})
        fits = f.get("nvls") if (a.gpus[0] > 2 and f.get("nvls")) else f.get("two_shot")
    elif a.fits:
        print(f"[ucurve] fit file {a.fits} not found: no prediction column")
    rows = []
    for kb in a.bucket_kb:
        r, out = _one(a, f"bucket_kb={kb}", ["--sync-mode", "overlap", "--bucket-kb", str(kb), "--comm-backend", "fused"]
                      + (["--cuda-graph"] if a.cuda_graph else []))
        tl = sync_timeline(out)
        row = {"bucket_kb": kb, **r, "buckets": len(tl["buckets"]) if tl else None,
               "exposed_ms": tl["exposed_ms"] if tl else None,
               "kernel_ms_sum": sum(e - s for s, e in tl["buckets"]) if tl else None, "predicted_ms": None}
        if tl and fits:
            row["predicted_ms"] = predict_bucketed(fits["alpha_ms"], fits["beta_ms_per_mb"] / (1 << 20),
                                                   [mb * (1 << 20) for mb in tl["bucket_mb"]])
        rows.append(row)
    save(a, f"bucket_ucurve_{a.preset}_g{a.gpus[0]}", rows,
         (["bucket KB", "buckets", "tok/s", "exposed ms", "bucket kernels ms (sum)", "alpha-beta prediction ms"],
          [[r["bucket_kb"], r["buckets"], r["tok_s"], r["exposed_ms"], r["kernel_ms_sum"], r["predicted_ms"]]
           for r in rows]))


def cmd_precision(a):
    """GEMM error per backend and precision at the reference's test sizes (64^3 ... 512^3), against an fp64 product
    (run_gemm_precision_validation.sh reruns test_gemm under its three precision settings; tolerances there:
    custom 1e-5, cuBLAS strict 1e-3, tensor cores 5e-3, FINAL_CLEAN_CODE_/tests/test_gemm.cu:28-105)."""
    r = subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", "gemm_precision.py")], capture_output=True,
                       text=True, cwd=ROOT, timeout=1800, env=clean_env())
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    print(r.stdout[-2000:] + r.stderr[-1000:])
    save(a, "gemm_precision", {"rc": r.returncode, "rows": rows, "all_pass": bool(rows) and all(x["pass"] for x in rows)},
         (["backend", "storage", "size", "max rel err", "tolerance", "pass"],
          [[x["backend"], x["storage"], x["size"], x["max_rel_err"], x["tol"], x["pass"]] for x in rows]))
    return 0 if r.returncode == 0 and rows and all(x["pass"] for x in rows) else 1


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


def _numbers(obj):
    if isinstance(obj, bool) or obj is None:
        return
    if isinstance(obj, (int, float)):
        yield obj
    elif isinstance(obj, dict):
        for v in obj.values():
            yield from _numbers(v)
    elif isinstance(obj, (list, tuple)):
        for v in obj:
            yield from _numbers(v)


# what each kind of result file must contain: (key that every row has, name of its validity flag or None)
_RESULT_RULES = {"repeated_": ("runs", "valid"), "buckets_": (None, "valid"), "weak_scaling_": (None, "valid"),
                 "strong_scaling_": (None, "valid"), "trajectory_": ("comparisons", None), "edge_cases": (None, "valid"),
                 "fusion_ablation_": (None, "valid"), "graph_vs_eager_": ("rows", None), "null_variance_": ("tok_s", None),
                 "lr_sweep_": ("rows", "valid"), "bucket_ucurve_": (None, "valid"), "gemm_precision": ("rows", "pass"),
                 "correctness_matrix": (None, None)}


def cmd_check(a):
    """Artifact audit (the reference's check_artifacts.py): every result file parses, is non-empty, holds only finite
    numbers, has the rows its experiment produces, every row's validity flag is true, and its markdown twin exists
    where the experiment writes one.  Prints one line per file and a summary; exit status 1 if anything is wrong."""
    import math
    problems, seen = [], 0
    for fn in sorted(os.listdir(a.out)) if os.path.isdir(a.out) else []:
        if not fn.endswith(".json"):
            continue
        seen += 1
        why = []
        try:
            txt = open(os.path.join(a.out, fn)).read()
            obj = json.loads(txt)
        except Exception as e:
            problems.append((fn, [f"unreadable: {e}"]))
            continue
        if not obj:
            why.append("empty")
        if any(isinstance(x, float) and not math.isfinite(x) for x in _numbers(obj)):
            why.append("non-finite number")
        rule = next((r for k, r in _RESULT_RULES.items() if fn.startswith(k)), None)
        if rule is None:
            why.append("unknown experiment")
        else:
            key, flag = rule
            rows = obj.get(key) if (key and isinstance(obj, dict)) else obj
            if key and isinstance(obj, dict) and key not in obj:
                why.append(f"missing '{key}'")
            if isinstance(rows, dict) and isinstance(rows.get("rows"), list):
                rows = rows["rows"]
            if flag and isinstance(rows, list):
                bad = [i for i, r in enumerate(rows) if isinstance(r, dict) and not r.get(flag, False)]
                if not rows:
                    why.append("no rows")
                if bad:
                    why.append(f"rows not {flag}: {bad}")
            if isinstance(obj, dict) and obj.get("all_ok") is False:
                why.append("a comparison is outside its tolerance")
        if fn.startswith(("trajectory_", "edge_cases", "fusion_", "graph_", "null_", "lr_", "bucket_ucurve", "gemm_prec")) \
                and not os.path.exists(os.path.join(a.out, fn[:-5] + ".md")):
            why.append("markdown table missing")
        print(f"[check] {fn}: {'OK' if not why else '; '.join(why)}")
        if why:
            problems.append((fn, why))
    print(f"[check] {seen} result files, {len(problems)} with problems")
    return 1 if problems or not seen else 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("experiment", choices=["repeated", "buckets", "scaling", "trajectory", "edge", "matrix", "check",
                                           "fusion", "graph", "null", "lr", "ucurve", "precision"])
    ap.add_argument("--lrs", type=float, nargs="+", default=[2e-5, 5e-5, 1e-4, 3e-4])
    ap.add_argument("--fits", default=None, help="bench_allreduce.py --json output holding the alpha-beta fits")
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
    if a.experiment in ("fusion", "graph", "null", "ucurve", "buckets", "scaling") and a.epochs < 2:
        a.epochs = 2          # the first epoch carries start-up, warm-up steps and graph capture; the last one is reported
    fn = {"repeated": cmd_repeated, "buckets": cmd_buckets, "scaling": cmd_scaling, "trajectory": cmd_trajectory,
          "edge": cmd_edge, "matrix": cmd_matrix, "check": cmd_check, "fusion": cmd_fusion, "graph": cmd_graph,
          "null": cmd_null, "lr": cmd_lr, "ucurve": cmd_ucurve, "precision": cmd_precision}[a.experiment]
    sys.exit(fn(a) or 0)


if __name__ == "__main__":
    main()
