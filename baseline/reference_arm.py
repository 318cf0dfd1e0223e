"""Reference arm of bench.py: runs the UNMODIFIED reference trainer through its own command line.

The reference (prince71753/CME213-Final-Project) is a Makefile project, not a Python package:
``pip install --no-index --target baseline/_ref <reference checkout>`` fails with "Neither 'setup.py' nor
'pyproject.toml' found".  Instead ``baseline/build_reference.sh`` copies its sources (``Makefile include/ src/
inp.txt``, untouched) into ``baseline/_ref`` and runs its own ``make`` with ``CUDA_ARCH=-arch=sm_100`` once per
hidden size (the model shape is a compile-time macro there).  Only the single-process binary can be built: the
data-parallel binary needs ``mpicxx`` / ``mpirun``, which this image does not have.

What the reference can express: ONE transformer block, 4 heads, context 64, vocabulary from its corpus (65),
batch 32, fp32 storage -- the ``parity-h128 / h256 / h512`` presets.  It cannot express the GPT-2-small
configuration (12 blocks, vocabulary 50304, context 1024, causal, GELU, tied embeddings), so for that
configuration this arm reports ``unavailable``.

Metric of the reference arm: the reference's own epoch line (``Epoch N: ... <ms>ms <tok/s> tok/s``), i.e. host
wall clock between barriers around K steps (``FINAL_CLEAN_CODE_/src/main.cu:322-323,429-450``); epoch 1 (K steps,
at least W) is warm-up, epoch 2 is reported.

``--ref-graph`` sets the reference's own ``CME213_USE_CUDA_GRAPH=1`` (its fastest single-GPU mode: three eager
steps, then the whole step replayed as one CUDA graph, ``FINAL_CLEAN_CODE_/src/main.cu:299-355``); every other
``CME213_*`` variable of the caller's environment is dropped so the reference runs its stock defaults.
"""
from __future__ import annotations

import json
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SHAPES = {"parity-h128": 128, "parity-h256": 256, "parity-h512": 512}
LR = {128: "3e-4", 256: "1e-4", 512: "5e-5"}


def _unavailable(why: str, a) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why, "n_gpus": a.gpus,
                      "config": {"model": a.config}}), flush=True)
    return 0


def run_reference(a) -> int:
    if a.config not in SHAPES:
        return _unavailable(
            f"the reference is a compile-time single-block model (4 heads, context 64, vocabulary 65, ReLU, non-causal); "
            f"it cannot express '{a.config}' (12+ blocks, vocabulary 50304, context 1024); its parity-h128/h256/h512 "
            f"shapes run with --config", a)
    if a.gpus != 1:
        return _unavailable("the reference's data-parallel binary needs an MPI toolchain (mpicxx, mpirun); "
                            "this image has none, only its single-GPU binary builds", a)
    H = SHAPES[a.config]
    exe = os.path.join(REF, f"build_h{H}", "train")
    if not os.path.exists(exe):
        return _unavailable(f"reference binary {os.path.relpath(exe, os.path.dirname(HERE))} not built "
                            f"(run baseline/build_reference.sh)", a)
    steps = max(a.steps, a.warmup)
    env = {k: v for k, v in os.environ.items() if not k.startswith("CME213_")}
    ref_graph = bool(getattr(a, "ref_graph", False))
    if ref_graph:
        env["CME213_USE_CUDA_GRAPH"] = "1"
    cmd = [exe, os.path.join(REF, "inp.txt"), "--epochs", "2", "--max-steps", str(steps), "--lr", LR[H]]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=1800, env=env, cwd=REF)
    if r.returncode != 0:
        return _unavailable(f"reference trainer exited {r.returncode}: {(r.stderr or r.stdout)[-200:]!r}", a)
    m = None
    for line in r.stdout.splitlines():
        mm = re.match(r"Epoch 2: avg_logged_loss=([\d.naif+-]+)\s+steps/rank=(\d+)\s+(\d+)ms\s+(\d+) tok/s", line)
        if mm:
            m = mm
    if m is None:
        return _unavailable("could not parse the reference's epoch line", a)
    loss, nsteps, ms, toks = float(m.group(1)), int(m.group(2)), float(m.group(3)), float(m.group(4))
    # the epoch line prints whole milliseconds; recompute tokens/s from steps for short runs
    tokens = nsteps * 32 * 64
    table = {128: 2.494e6, 256: 1.596e6, 512: 0.732e6}
    out = {"impl": "reference", "metric": "train tokens/sec (reference's own epoch line: host wall clock)",
           "value": toks, "unit": "tokens/s", "n_gpus": 1, "steps": nsteps, "warmup": nsteps,
           "ms_per_step": ms / max(nsteps, 1), "higher_is_better": True, "scaling": "weak",
           "vs_baseline": toks / table[H], "dtype": "fp32 storage, cuBLAS fp16 tensor-core math (its auto backend)",
           "data": "tiny-Shakespeare inp.txt (the reference takes no synthetic input)",
           "config": {"model": a.config, "global_batch": 32, "seq_len": 64, "parallelism": "dp1",
                      "tokens_per_epoch": tokens, "cuda_graph": ref_graph},
           "e2e": {"value": toks, "unit": "tokens/s",
                   "note": "the reference preloads every batch to the device before the loop; its number has no per-step copies"},
           "loss": loss}
    print(json.dumps(out), flush=True)
    return 0
