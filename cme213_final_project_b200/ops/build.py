"""In-tree build of the native library: every ``csrc/*.cu`` compiled by ``nvcc`` for sm_100a into one
shared object with a C ABI (``libcme213_b200.so`` next to this file).

The reference builds with a Makefile (``FINAL_CLEAN_CODE_/Makefile``: ``-arch=sm_75``, every source through
``nvcc``, separate object files, per-thread default stream).  Here: one arch (``sm_100a``), objects cached
by source hash under ``build/`` next to the sources, parallel compile, no link-time dependency on the
driver library (the tensor-map encoder is looked up at run time).
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path
from typing import List

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "libcme213_b200.so"
BUILD = HERE / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(src: Path, headers: List[Path]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for p in [src] + headers:
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile what changed, link, return the path of the shared object."""
    nvcc = _nvcc()
    BUILD.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    jobs = []
    objs = []
    for src in sources:
        obj = BUILD / f"{src.stem}.{_digest(src, headers)}.o"
        objs.append(obj)
        if force or not obj.exists():
            for old in BUILD.glob(f"{src.stem}.*.o"):
                old.unlink()
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = BUILD / f"{src.stem}.ptxas.log"
        log.write_text(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        return src.name

    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for name in ex.map(compile_one, jobs):
                if verbose:
                    print(f"[build] compiled {name}", file=sys.stderr)
    if jobs or not OUT.exists() or force:
        cmd = [nvcc, "-shared", "-o", str(OUT), *map(str, objs), "-lcudart", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(f"[build] linked {OUT}", file=sys.stderr)
    return OUT


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv))
