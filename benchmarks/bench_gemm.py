"""Device-timed throughput of the tcgen05 GEMM on the training shapes, against torch.matmul (cuBLAS)
on the same device and against the measured bf16 peak.

Role of the reference's GEMM micro-benchmarks (FINAL_CLEAN_CODE_/tests/benchmark_all.cu, gemm_tune.cu).
Each product is timed with CUDA events after warm-up, with an L2 flush before every timed launch.

    python benchmarks/bench_gemm.py [--preset gpt2-small] [--iters 10] [--json out.json]
"""
import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from cme213_final_project_b200 import ops                      # noqa: E402
from cme213_final_project_b200.config import preset            # noqa: E402
from cme213_final_project_b200.utils.timers import L2Flusher, time_kernel  # noqa: E402


def sites(m):
    BT, D, FF, V = m.tokens_per_step, m.hidden, m.ff, m.vocab_size
    tied = m.tied_embeddings
    return [
        # name, M, N, K, a_trans, b_trans, batch
        ("qkv_fwd", BT, D, D, False, False, 3),
        ("attn_out_fwd", BT, D, D, False, False, 1),
        ("ffn1_fwd", BT, FF, D, False, False, 1),
        ("ffn2_fwd", BT, D, FF, False, False, 1),
        ("lm_head_fwd", BT, V, D, False, tied, 1),
        ("ffn2_dgrad", BT, FF, D, False, True, 1),
        ("ffn1_dgrad", BT, D, FF, False, True, 1),
        ("lm_head_dgrad", BT, D, V, False, not tied, 1),
        ("ffn1_wgrad", D, FF, BT, True, False, 1),
        ("ffn2_wgrad", FF, D, BT, True, False, 1),
        ("attn_out_wgrad", D, D, BT, True, False, 1),
        ("qkv_wgrad", D, D, BT, True, False, 3),
    ]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="gpt2-small")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json")
    a = ap.parse_args()
    m, _ = preset(a.preset)
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peaks = json.load(open(p))
    peak = peaks.get("bf16_tflops", 1590.0)
    fl = L2Flusher("cuda")
    rows = []
    for name, M, N, K, at, bt, batch in sites(m):
        if N % 8 or K % 8 or M % 8:
            continue
        ash = ((K, M) if at else (M, K))
        bsh = ((N, K) if bt else (K, N))
        if batch > 1:
            bsh = (batch,) + bsh
            if name == "qkv_wgrad":
                pass
        A = torch.randn(ash, device="cuda").to(torch.bfloat16)
        B = torch.randn(bsh, device="cuda").to(torch.bfloat16)
        if name == "qkv_wgrad":                       # A shared (x^T), B = [3, BT, D] gradients
            pass
        out = ops.gemm(A, B, a_trans=at, b_trans=bt)
        Af = A.t() if at else A
        Bf = B.transpose(-1, -2) if bt else B
        ref = torch.matmul(Af, Bf)
        err = (out.float() - ref.float()).abs().max().item() / (ref.float().abs().max().item() + 1e-6)
        mine = time_kernel(lambda: ops.gemm(A, B, a_trans=at, b_trans=bt, out=out), 3, a.iters, fl)
        cub = time_kernel(lambda: torch.matmul(Af, Bf, out=ref), 3, a.iters, fl)
        flops = 2.0 * M * N * K * batch
        t_me, t_cu = statistics.median(mine), statistics.median(cub)
        rows.append({"site": name, "M": M, "N": N, "K": K, "batch": batch, "a_trans": at, "b_trans": bt,
                     "ms": t_me, "tflops": flops / t_me / 1e9, "frac_of_measured_peak": flops / t_me / 1e9 / peak,
                     "cublas_ms": t_cu, "cublas_tflops": flops / t_cu / 1e9, "vs_cublas": t_cu / t_me, "rel_err": err})
        r = rows[-1]
        print(f"{name:16s} M={M:6d} N={N:6d} K={K:6d} b={batch}  {r['ms']:8.4f} ms {r['tflops']:7.1f} TF "
              f"({r['frac_of_measured_peak']*100:5.1f}% of measured {peak:.0f})  cuBLAS {r['cublas_ms']:8.4f} ms "
              f"{r['cublas_tflops']:7.1f} TF  x{r['vs_cublas']:.2f}  err {err:.1e}", flush=True)
    assert ops.gemm_check_status() == 0
    if a.json:
        json.dump(rows, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
