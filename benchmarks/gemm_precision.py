"""GEMM error per backend and storage precision at the reference's unit-test sizes.

The reference reruns its GEMM test (CPU triple loop vs the dispatched kernel at 64^3 ... 512^3) under three
precision settings with backend-dependent tolerances: custom kernels 1e-5, cuBLAS strict fp32 1e-3, tensor cores 5e-3
(FINAL_CLEAN_CODE_/tests/test_gemm.cu:28-105, FINAL_CLEAN_CODE_/scripts/run_gemm_precision_validation.sh:63-68).  Here the
same sweep over this library's GEMM paths: the SIMT kernel on fp32 (exact-order fp32 accumulation), the tcgen05 kernel
on fp32 storage with tf32 tensor-core math, and the tcgen05 kernel on bf16 storage.  The oracle is an fp64 product of
the stored operands; the error is relative to the largest output magnitude.  One JSON line per case on stdout.

    python benchmarks/gemm_precision.py
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from cme213_final_project_b200 import ops  # noqa: E402

CASES = [("simt", torch.float32, 1e-5), ("tcgen05", torch.float32, 1e-3), ("tcgen05", torch.bfloat16, 5e-3)]


def main() -> int:
    ok = True
    g = torch.Generator(device="cuda").manual_seed(0)
    for backend, dtype, tol in CASES:
        for n in (64, 128, 256, 512):
            a = (torch.randn(n, n, generator=g, device="cuda") * 0.5).to(dtype)
            b = (torch.randn(n, n, generator=g, device="cuda") * 0.5).to(dtype)
            ref = a.double() @ b.double()
            row = {"backend": backend, "storage": str(dtype).split(".")[-1], "size": f"{n}^3", "tol": tol}
            try:
                out = ops.gemm(a, b, backend=backend, out_dtype=torch.float32)
                torch.cuda.synchronize()
                err = (out.double() - ref).abs().max().item() / ref.abs().max().item()
                row.update(max_rel_err=err, **{"pass": bool(err <= tol and ops.gemm_check_status() == 0)})
            except ops.NativeError as e:
                row.update(max_rel_err=None, error=str(e)[:120], **{"pass": False})
            ok = ok and row["pass"]
            print(json.dumps(row), flush=True)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
