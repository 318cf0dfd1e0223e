"""Fused vs unfused pipelines, device-timed: bias + activation, residual + LayerNorm forward, LayerNorm backward +
residual-gradient add, activation backward + bias gradient, plus achieved DRAM bandwidth against the measured peak.

Role of the reference's fusion A/B benchmark (FINAL_CLEAN_CODE_/tests/test_fusion_benchmark.cu:54-296 and
profile_fusion_kernels.cu; numbers in FINAL_CLEAN_CODE/results/final_clean_main_table.csv:57-65 and
roofline_fusion.csv).  Inputs are sized above the 126 MB L2 by default so the DRAM figures mean something;
`--reference-shapes` uses the reference's 2048 x {128, 512} matrices instead (L2-resident on a B200).

    python benchmarks/bench_fusion.py [--rows 65536 --cols 3072] [--reference-shapes] [--json out.json]
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
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--cols", type=int, default=3072)
    ap.add_argument("--ln-cols", type=int, default=768)
    ap.add_argument("--reference-shapes", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json")
    a = ap.parse_args()
    rows, cols, lnc = (2048, 512, 128) if a.reference_shapes else (a.rows, a.cols, a.ln_cols)
    peak = 6536.4
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = json.load(open(pk)).get("hbm_gbs", peak)
    fl = L2Flusher("cuda")
    bf = torch.bfloat16
    out = []

    def rec(name, fused, unfused, nbytes):
        f, u = statistics.median(fused), statistics.median(unfused)
        r = {"op": name, "fused_ms": f, "unfused_ms": u, "speedup": u / f, "fused_gbs": nbytes / f / 1e6,
             "frac_of_measured_hbm": nbytes / f / 1e6 / peak}
        out.append(r)
        print(json.dumps(r), flush=True)

    x, res = torch.randn(rows, cols, device="cuda").to(bf), torch.randn(rows, cols, device="cuda").to(bf)
    bias = torch.randn(cols, device="cuda").to(bf)
    fused = time_kernel(lambda: ops.bias_act_residual(x, bias, "relu"), 3, a.iters, fl)

    def unf():
        t, _ = ops.bias_act_residual(x, bias, None)
        ops.bias_act_residual(t, None, "relu")
    rec("bias+relu", fused, time_kernel(unf, 3, a.iters, fl), 2 * x.numel() * 2)
    fused = time_kernel(lambda: ops.bias_act_residual(x, bias, "gelu", res), 3, a.iters, fl)

    def unf2():
        t, _ = ops.bias_act_residual(x, bias, None)
        t, _ = ops.bias_act_residual(t, None, "gelu")
        ops.add(t, res)
    rec("bias+gelu+residual", fused, time_kernel(unf2, 3, a.iters, fl), 3 * x.numel() * 2)
    dout = torch.randn(rows, cols, device="cuda").to(bf)
    fused = time_kernel(lambda: ops.dact_colsum(dout, x, "relu"), 3, a.iters, fl)

    def unf3():
        g = ops.relu_bwd(x, dout)
        ops.dact_colsum(g)
    rec("relu-bwd+bias-bwd", fused, time_kernel(unf3, 3, a.iters, fl), 3 * x.numel() * 2)

    h, r2 = torch.randn(rows, lnc, device="cuda").to(bf), torch.randn(rows, lnc, device="cuda").to(bf)
    g, b = torch.ones(lnc, device="cuda").to(bf), torch.zeros(lnc, device="cuda").to(bf)
    fused = time_kernel(lambda: ops.layernorm_fwd(h, g, b, 1e-5, residual=r2, save_sum=True), 3, a.iters, fl)

    def unf4():
        s = ops.add(h, r2)
        ops.layernorm_fwd(s, g, b, 1e-5)
    rec("residual+layernorm fwd", fused, time_kernel(unf4, 3, a.iters, fl), 4 * h.numel() * 2)
    y, mean, rstd, s = ops.layernorm_fwd(h, g, b, 1e-5, residual=r2, save_sum=True)
    dy = torch.randn(rows, lnc, device="cuda").to(bf)
    fused = time_kernel(lambda: ops.layernorm_bwd(dy, s, g, mean, rstd, dres=r2), 3, a.iters, fl)

    def unf5():
        dx, _, _ = ops.layernorm_bwd(dy, s, g, mean, rstd)
        ops.add(dx, r2)
    rec("layernorm-bwd+residual", fused, time_kernel(unf5, 3, a.iters, fl), 4 * h.numel() * 2)
    fused = time_kernel(lambda: ops.layernorm_fwd(h, g, b, 1e-5), 3, a.iters, fl)
    rec("layernorm fwd", fused, fused, 2 * h.numel() * 2)
    # Softmax-cross-entropy forward + backward in one kernel against PyTorch (forward, then autograd backward), and the
    # fused AdamW step (bf16 gradients in, fp32 master / moments, bf16 parameters out) against torch's fused AdamW.
    ce_rows = min(rows, 4096) if not a.reference_shapes else rows
    V = 65 if a.reference_shapes else 50304
    lg = torch.randn(ce_rows, V, device="cuda").to(bf)
    tg = torch.randint(0, V, (ce_rows,), device="cuda", dtype=torch.int32)
    fused = time_kernel(lambda: ops.cross_entropy(lg, tg), 3, a.iters, fl)
    lg32 = lg.clone().requires_grad_(True)
    tg64 = tg.long()

    def unf6():
        lg32.grad = None
        torch.nn.functional.cross_entropy(lg32.float(), tg64).backward()
    rec("softmax-cross-entropy fwd+bwd (vs torch)", fused, time_kernel(unf6, 3, a.iters, fl), 2 * lg.numel() * 2)

    n = 2048 * 512 if a.reference_shapes else 124 * 1000 * 1000
    master = torch.randn(n, device="cuda") * 0.02
    grads = (torch.randn(n, device="cuda") * 1e-3).to(bf)
    m1, v1 = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    comp = master.to(bf)
    step = torch.ones(1, dtype=torch.int32, device="cuda")
    lr = torch.full((1,), 3e-4, device="cuda")
    fused = time_kernel(lambda: ops.adam_step(master, grads, m1, v1, step, lr, compute=comp, beta2=0.95,
                                              weight_decay=0.1), 3, a.iters, fl)
    pt = torch.nn.Parameter(master.clone())
    pt.grad = grads.float()
    opt = torch.optim.AdamW([pt], lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

    def unf7():
        pt.grad = grads.float()            # torch's optimizer wants the gradient in the parameter's dtype
        opt.step()
        comp.copy_(pt.detach())            # and the bf16 copy of the parameters is one more pass
    rec("adamw step (vs torch fused AdamW + casts)", fused, time_kernel(unf7, 3, a.iters, fl), n * 30)

    # token + position embedding, forward and backward (tied-table scatter with atomics), GPT-2 small sizes, against
    # torch.nn.functional.embedding and its index_add backward
    V, T, D, B = 50304, 1024, 768, 16
    tok_w, pos_w = torch.randn(V, D, device="cuda").to(bf), torch.randn(T, D, device="cuda").to(bf)
    ids = torch.randint(0, V, (B * T,), device="cuda", dtype=torch.int32)
    ids64 = ids.long()
    pos_ids = torch.arange(T, device="cuda").repeat(B)
    dout = torch.randn(B * T, D, device="cuda").to(bf)
    fused = time_kernel(lambda: ops.embedding_fwd(ids, tok_w, pos_w), 3, a.iters, fl)
    unf8 = lambda: torch.nn.functional.embedding(ids64, tok_w) + torch.nn.functional.embedding(pos_ids, pos_w)
    rec("embedding fwd, token + position (vs torch)", fused, time_kernel(unf8, 3, a.iters, fl), B * T * D * 2 * 2)
    dtok, dpos = torch.zeros(V, D, device="cuda", dtype=bf), torch.zeros(T, D, device="cuda", dtype=bf)
    fused = time_kernel(lambda: ops.embedding_bwd(ids, dout, V, T, dtok=dtok, dpos=dpos, accumulate=True), 3, a.iters, fl)
    gt, gp = torch.zeros(V, D, device="cuda", dtype=bf), torch.zeros(T, D, device="cuda", dtype=bf)

    def unf9():
        gt.index_add_(0, ids64, dout)
        gp.index_add_(0, pos_ids, dout)
    rec("embedding bwd, scatter-add into both tables (vs torch index_add)", fused, time_kernel(unf9, 3, a.iters, fl),
        B * T * D * 2 * 3)
    if a.json:
        json.dump(out, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
