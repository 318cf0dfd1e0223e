"""Device-timed attention forward / backward (tcgen05 kernels) against torch SDPA on the same device.

Role of the attention rows of the reference's micro-benchmarks (FINAL_CLEAN_CODE_/tests/benchmark_all.cu;
FINAL_CLEAN_CODE/results/correctness_matrix_87896.md:16-19).  FLOPs are counted for the causal half.

    python benchmarks/bench_attention.py [--B 16 --H 12 --T 1024] [--iters 10]
"""
import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from cme213_final_project_b200 import ops                                   # noqa: E402
from cme213_final_project_b200.utils.timers import L2Flusher, time_kernel   # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--B", type=int, default=16)
    ap.add_argument("--H", type=int, default=12)
    ap.add_argument("--T", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--non-causal", action="store_true")
    a = ap.parse_args()
    B, H, T, HD = a.B, a.H, a.T, 64
    causal = not a.non_causal
    D = H * HD
    q, k, v, do = (torch.randn(B * T, D, device="cuda").to(torch.bfloat16) for _ in range(4))
    fl = L2Flusher("cuda")
    out, lse = ops.attention_fwd(q, k, v, B, H, T, "split", causal, backend="tc")
    f = time_kernel(lambda: ops.attention_fwd(q, k, v, B, H, T, "split", causal, backend="tc"), 3, a.iters, fl)
    bw = time_kernel(lambda: ops.attention_bwd(q, k, v, out, lse, do, B, H, T, "split", causal, backend="tc"), 3,
                     a.iters, fl)
    q4, k4, v4 = (t.view(B, T, H, HD).transpose(1, 2).contiguous().requires_grad_(True) for t in (q, k, v))
    do4 = do.view(B, T, H, HD).transpose(1, 2).contiguous()
    sd = lambda: torch.nn.functional.scaled_dot_product_attention(q4, k4, v4, is_causal=causal)
    o4 = sd()
    tf = time_kernel(lambda: sd(), 3, a.iters, fl)
    tb = time_kernel(lambda: torch.autograd.grad(o4, (q4, k4, v4), do4, retain_graph=True), 3, a.iters, fl)
    flops_f = 4.0 * B * H * T * T * HD * (0.5 if causal else 1.0)
    mf, mb, sf, sb = (statistics.median(x) for x in (f, bw, tf, tb))
    res = {"B": B, "H": H, "T": T, "HD": HD, "causal": causal, "fwd_ms": mf, "bwd_ms": mb,
           "fwd_tflops": flops_f / mf / 1e9, "bwd_tflops": 2.5 * flops_f / mb / 1e9, "sdpa_fwd_ms": sf, "sdpa_bwd_ms": sb,
           "status": ops.attention_check_status()}
    print(json.dumps(res))


if __name__ == "__main__":
    main()
