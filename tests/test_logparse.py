"""Log-line parsing, run validity and repeat statistics
(FINAL_CLEAN_CODE_/scripts/summarize_single_gpu_bench.py:17-68)."""
from cme213_final_project_b200 import checkpoint as ckpt
from cme213_final_project_b200.utils import logfmt
from cme213_final_project_b200.utils.logparse import (compare_trajectories, parse_run, parse_trajectory,
                                                      summarize_repeats)


def test_epoch_line_round_trip_and_validity():
    text = "\n".join([logfmt.epoch_line(1, 3.19, 100, 82.0, 2494000.0, 1, False, 0, 0, 0),
                      logfmt.epoch_line(2, 3.01, 100, 80.0, 2560000.0, 4, True, 0.011, 2.64, 1.5e-5)])
    r = parse_run(text)
    assert r.valid and len(r.epochs) == 2 and r.last.tok_s == 2560000 and r.last.grad_finish_ms == 2.64
    assert r.last.checksum_span == 1.5e-5 and r.epochs[0].grad_sync_ms is None
    assert not parse_run("nothing here").valid
    bad = parse_run(logfmt.epoch_line(1, float("nan"), 10, 5.0, 1.0, 1, False, 0, 0, 0))
    assert not bad.valid and bad.reason == "non-finite loss"
    assert not parse_run(text + "\nloss went to inf at step 3").valid
    assert parse_run(text + "\ninfo: training finished").valid


def test_repeat_statistics_drop_the_cold_run():
    s = summarize_repeats([600e3, 3.8e6, 3.9e6, 4.0e6], [True, True, True, True])
    assert s["warm_runs"] == 3 and abs(s["mean"] - 3.9e6) < 1 and s["all_valid"] and s["cv"] < 0.03
    s = summarize_repeats([1.0, 2.0, 3.0], [True, False, True])
    assert s["valid_runs"] == 2 and s["warm_runs"] == 1 and not s["all_valid"]


def test_trajectory_parse_and_compare():
    st = ckpt.ParamStats(1.5, 2.5, 0.5, 0x1234)
    a = "\n".join(ckpt.trajectory_line(1, i + 1, 4.0 - 0.1 * i, st, (0.0, 0.0, 0.0)) for i in range(3))
    b = "\n".join(ckpt.trajectory_line(1, i + 1, 4.0 - 0.1 * i + 1e-4, st, (1e-6, 0.0, 0.0)) for i in range(3))
    ta, tb = parse_trajectory(a), parse_trajectory(b)
    assert len(ta) == 3 and ta[0]["hash"] == "0000000000001234" and ta[2]["step"] == 3
    c = compare_trajectories(ta, tb)
    assert c["ok"] and c["max_sum_span"] == 1e-6
    assert not compare_trajectories(ta, tb[:2])["ok"]


def test_trajectory_comparison_has_two_levels():
    """Same arithmetic in another schedule must reproduce the sums; different arithmetic (bf16 gradient sums taken in
    another order, amplified by Adam on near-zero gradients) may move the plain sum -- a residual of cancelling
    values -- while loss, sum of squares and largest magnitude agree."""
    mk = lambda s, sq, mx, loss: "\n".join(
        ckpt.trajectory_line(1, i + 1, loss, ckpt.ParamStats(s, sq, mx, 0x1), (0.0, 0.0, 0.0)) for i in range(2))
    base = parse_trajectory(mk(-0.14, 812.0, 0.25, 3.9))
    same = compare_trajectories(base, parse_trajectory(mk(-0.14, 812.0, 0.25, 3.9)), n_params=222592)
    assert same["identical_path"] and same["ok"] and same["max_sum_diff_per_param"] == 0.0
    moved = compare_trajectories(base, parse_trajectory(mk(-0.17, 812.9, 0.2501, 3.9004)), n_params=222592)
    assert moved["ok"] and not moved["identical_path"]
    assert abs(moved["max_sum_diff_per_param"] - 0.03 / 222592) < 1e-12
    off = compare_trajectories(base, parse_trajectory(mk(-0.14, 840.0, 0.25, 3.9)))
    assert not off["ok"] and "max_sum_diff_per_param" not in off


def test_launch_list_summary(tmp_path):
    """Profiler launch list -> per-kernel table of the last complete step (banner lines skipped, units converted,
    template arguments kept, parameter lists dropped)."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location(
        "summarize_launches", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks",
                                           "summarize_launches.py"))
    sl = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sl)
    hdr = '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"'
    row = lambda i, k, v, unit="ns": f'"{i}","1","python","h","{k}","1","7","(128, 1, 1)","(1, 1, 1)","0","10.0","s","gpu__time_duration.sum","{unit}","{v}"'
    names = ["void <unnamed>::embed_fwd_kernel<__nv_bfloat16>(int const*, T1*)",
             "void gemm_tc::gemm_tc_kernel<256, 0, 1, 0, 1, 545>(CUtensorMap_st, gemm_tc::EpiParams)",
             "<unnamed>::attn_fwd_tc_kernel(CUtensorMap_st, <unnamed>::FwdParams)",
             "void gemm_tc::gemm_tc_kernel<256, 0, 1, 0, 1, 545>(CUtensorMap_st, gemm_tc::EpiParams)"]
    lines = ["==PROF== Connected to process 1", hdr]
    i = 0
    for step in range(3):
        for k, v in zip(names, ("12,000", "60000", "80", "40000")):
            lines.append(row(i, k, v, "us" if v == "80" else "ns"))
            i += 1
    p = tmp_path / "launches.csv"
    p.write_text("\n".join(lines) + "\n")
    s = sl.summarize(sl.last_step(sl.read_launches(str(p)), "embed_fwd"))
    assert s["launches"] == 4 and abs(s["total_us"] - (12 + 60 + 80 + 40)) < 1e-9
    top = s["kernels"][0]
    assert top["kernel"] == "gemm_tc_kernel<256,0,1,0,1,545>" and top["launches"] == 2 and abs(top["total_us"] - 100) < 1e-9
    assert s["kernels"][1]["kernel"] == "attn_fwd_tc_kernel" and "| `attn_fwd_tc_kernel` | 1 | 80 |" in sl.to_markdown(s)
