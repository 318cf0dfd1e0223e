"""Device-timed throughput of the tcgen05 GEMM on the training shapes, against torch.matmul (cuBLAS)
on the same device and against the measured bf16 peak.

Role of the reference's GEMM micro-benchmarks (FINAL_CLEAN_CODE_/tests/benchmark_all.cu, gemm_tune.cu).
Each product is timed with CUDA events after warm-up, with an L2 flush before every timed launch.

    python benchmarks/bench_gemm.py [--preset gpt2-small] [--iters 10] [--site ffn1_fwd] [--plain] [--json out.json]
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
    """Every GEMM of one training step of the preset, with the epilogue the engine fuses into it."""
    BT, D, FF, V = m.tokens_per_step, m.hidden, m.ff, m.vocab_size
    tied = m.tied_embeddings
    act = "gelu" if m.activation == "gelu" else "relu"
    qkv = [("qkv_fwd", BT, 3 * D, D, False, False, 1, None), ("qkv_dgrad", BT, D, 3 * D, False, True, 1, None),
           ("qkv_wgrad", D, 3 * D, BT, True, False, 1, None)] if m.mode == "gpt" else \
          [("qkv_fwd", BT, D, D, False, False, 3, None), ("qkv_wgrad", D, D, BT, True, False, 3, None)]
    return qkv + [
        # name, M, N, K, a_trans, b_trans, batch, epilogue
        ("attn_out_fwd", BT, D, D, False, False, 1, "res"),
        ("ffn1_fwd", BT, FF, D, False, False, 1, "bias_" + act + ("_auxd" if act == "gelu" else "")),
        ("ffn2_fwd", BT, D, FF, False, False, 1, "bias_res"),
        ("lm_head_fwd", BT, V, D, False, tied, 1, None),
        ("ffn2_dgrad", BT, FF, D, False, True, 1, ("dmul" if act == "gelu" else "drelu") + "_colsum"),
        ("ffn1_dgrad", BT, D, FF, False, True, 1, None),
        ("attn_out_dgrad", BT, D, D, False, True, 1, None),
        ("lm_head_dgrad", BT, D, V, False, not tied, 1, None),
        ("ffn1_wgrad", D, FF, BT, True, False, 1, None),
        ("ffn2_wgrad", FF, D, BT, True, False, 1, None),
        ("attn_out_wgrad", D, D, BT, True, False, 1, None),
        ("lm_head_wgrad", V, D, BT, True, False, 1, None),
    ]


def epilogue_args(kind, M, N, dev="cuda"):
    """Keyword arguments of ``ops.gemm`` for an epilogue name, and a PyTorch function applying the same to a product."""
    if kind is None:
        return {}, lambda y: y
    bf = torch.bfloat16
    bias = torch.randn(N, device=dev).to(bf)
    res = torch.randn(M, N, device=dev).to(bf)
    pre = torch.randn(M, N, device=dev).to(bf)
    gelu = lambda x: torch.nn.functional.gelu(x, approximate="tanh")
    if kind == "res":
        return {"residual": res}, lambda y: y + res.float()
    if kind == "bias_res":
        return {"bias": bias, "residual": res}, lambda y: y + bias.float() + res.float()
    if kind == "bias_gelu_aux":
        return {"bias": bias, "act": "gelu", "aux_out": torch.empty(M, N, device=dev, dtype=bf)}, \
            lambda y: gelu(y + bias.float())
    if kind == "bias_gelu_auxd":          # what the engine runs: the epilogue also leaves GELU'(pre-activation)
        return {"bias": bias, "act": "gelu", "aux_out": torch.empty(M, N, device=dev, dtype=bf), "aux_deriv": True}, \
            lambda y: gelu(y + bias.float())
    if kind == "dmul_colsum":             # ... and multiplies by it in backward, summing the bias gradient on the way
        return {"dact": "gelu", "aux_in": pre, "aux_deriv": True, "dbias": torch.empty(N, device=dev, dtype=bf)}, \
            lambda y: y * pre.float()
    if kind == "drelu_colsum":
        return {"dact": "relu", "aux_in": pre, "dbias": torch.empty(N, device=dev, dtype=bf)}, \
            lambda y: y * (pre.float() > 0)
    if kind == "bias_relu":
        return {"bias": bias, "act": "relu"}, lambda y: torch.relu(y + bias.float())
    if kind == "dgelu":
        def f(y):
            x = pre.float().requires_grad_(True)
            gelu(x).backward(torch.ones_like(x))
            return y * x.grad
        return {"dact": "gelu", "aux_in": pre}, f
    if kind == "drelu":
        return {"dact": "relu", "aux_in": pre}, lambda y: y * (pre.float() > 0)
    raise ValueError(kind)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="gpt2-small")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--site", help="run only this site (see sites())")
    ap.add_argument("--only-ours", action="store_true", help="skip the cuBLAS timing and the error check (profiling)")
    ap.add_argument("--plain", action="store_true", help="time every site without its fused epilogue")
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
    for name, M, N, K, at, bt, batch, epi in sites(m):
        if N % 8 or K % 8 or M % 8 or (a.site and name != a.site):
            continue
        if a.plain or batch > 1:
            epi = None
        ash = ((K, M) if at else (M, K))
        bsh = ((N, K) if bt else (K, N))
        if batch > 1:
            bsh = (batch,) + bsh
        A = torch.randn(ash, device="cuda").to(torch.bfloat16)
        B = torch.randn(bsh, device="cuda").to(torch.bfloat16)
        kw, ref_fn = epilogue_args(epi, M, N)
        out = ops.gemm(A, B, a_trans=at, b_trans=bt, **kw)
        mine = time_kernel(lambda: ops.gemm(A, B, a_trans=at, b_trans=bt, out=out, **kw), 3, a.iters, fl)
        flops = 2.0 * M * N * K * batch
        t_me = statistics.median(mine)
        row = {"site": name, "epilogue": epi or "none", "M": M, "N": N, "K": K, "batch": batch, "a_trans": at,
               "b_trans": bt, "ms": t_me, "tflops": flops / t_me / 1e9,
               "frac_of_measured_peak": flops / t_me / 1e9 / peak}
        line = (f"{name:16s} {row['epilogue']:14s} M={M:6d} N={N:6d} K={K:6d} b={batch}  {t_me:8.4f} ms "
                f"{row['tflops']:7.1f} TF ({row['frac_of_measured_peak']*100:5.1f}% of measured {peak:.0f})")
        if not a.only_ours:
            Af = A.t() if at else A
            Bf = B.transpose(-1, -2) if bt else B
            ref = torch.matmul(Af, Bf)
            # plain cuBLAS product: the fused work (bias, activation, residual) would be further kernels on top
            cub = time_kernel(lambda: torch.matmul(Af, Bf, out=ref), 3, a.iters, fl)
            t_cu = statistics.median(cub)
            want = ref_fn(torch.matmul(Af.float(), Bf.float()))
            err = (out.float() - want).abs().max().item() / (want.abs().max().item() + 1e-6)
            row.update({"cublas_plain_ms": t_cu, "cublas_plain_tflops": flops / t_cu / 1e9, "vs_cublas_plain": t_cu / t_me,
                        "rel_err": err})
            line += f"  cuBLAS(plain) {t_cu:8.4f} ms {row['cublas_plain_tflops']:7.1f} TF  x{row['vs_cublas_plain']:.2f}  err {err:.1e}"
        rows.append(row)
        print(line, flush=True)
    assert ops.gemm_check_status() == 0
    if a.json:
        json.dump(rows, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
