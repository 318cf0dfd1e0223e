"""Configuration, presets, flag parsing and the --validate-config contract
(FINAL_CLEAN_CODE_/src/main.cu:91-132,148-195)."""
import subprocess
import sys

import pytest

from cme213_final_project_b200 import config as C
from cme213_final_project_b200.utils import logfmt


def test_presets_match_named_configs():
    m, o = C.preset("gpt2-small")
    assert (m.vocab_size, m.seq_len, m.hidden, m.heads, m.layers, m.ff, m.batch_size) == (50304, 1024, 768, 12, 12, 3072, 16)
    assert (o.beta1, o.beta2, o.weight_decay) == (0.9, 0.95, 0.1)
    m, o = C.preset("parity-h256")
    assert (m.hidden, m.ff, m.heads, m.seq_len, m.vocab_size, m.batch_size, m.layers) == (256, 1024, 4, 64, 65, 32, 1)
    assert o.clip_norm == 1.0 and o.weight_decay == 0.0
    assert not m.validate()
    m, _ = C.preset("tiny-gpt")
    assert (m.layers, m.hidden, m.heads, m.batch_size, m.tied_embeddings) == (2, 128, 4, 8, True)


def test_flag_parsing_reference_names():
    m, o, r = C.parse_args(["corpus.txt", "--epochs", "3", "--max-steps", "20", "--lr", "1e-4", "--sync-mode", "auto",
                            "--bucket-kb", "1024", "--auto-overlap-max-mb", "4", "--trace-trajectory"])
    assert r.data_path == "corpus.txt" and r.epochs == 3 and r.max_steps == 20 and o.lr == 1e-4
    assert r.sync_mode == "auto" and r.bucket_kb == 1024 and r.auto_overlap_max_mb == 4 and r.trace_trajectory
    assert C.parse_args(["--overlap"])[2].sync_mode == "overlap"
    assert C.parse_args(["--auto-sync"])[2].sync_mode == "auto"
    m, _, _ = C.parse_args(["--hidden", "256"])
    assert m.ff == 1024


def test_auto_policy_and_bucket_floor():
    r = C.RunConfig(sync_mode="auto", auto_overlap_max_mb=8.0)
    assert C.effective_overlap(r, 3.2, 4) and not C.effective_overlap(r, 12.4, 4) and not C.effective_overlap(r, 1.0, 1)
    assert C.min_bucket_elems(256) == 65536 and C.min_bucket_elems(0) == 0 and C.min_bucket_elems(1, 2) == 512


def test_environment_rules():
    errs, _ = C.validate_environment(1, {"CME213_MIXED_PRECISION": "1"})
    assert any("planned but not implemented" in e for e in errs)
    errs, _ = C.validate_environment(1, {"CME213_FFN_FP16": "1", "CME213_LT_FUSION": "1"})
    assert any("must not be combined" in e for e in errs)
    errs, _ = C.validate_environment(4, {"CME213_FP16_STORAGE_ONLY": "1"})
    assert any("single-GPU" in e for e in errs)
    errs, _ = C.validate_environment(1, {"CME213_FFN_FP16": "1", "CME213_USE_CUDA_GRAPH": "1"})
    assert any("CUDA_GRAPH" in e for e in errs)
    errs, warns = C.validate_environment(1, {"CME213_USE_NCCL": "1"})
    assert not errs and warns
    assert C.validate_environment(1, {"CME213_USE_CUDA_GRAPH": "0"}) == ([], [])
    run = C.apply_environment(C.RunConfig(), {"CME213_USE_CUDA_GRAPH": "1", "CME213_GEMM_BACKEND": "custom",
                                              "CME213_DEFER_GRAD_AVG_TO_ADAM": "1"})
    assert run.cuda_graph and run.gemm_backend == "simt" and run.defer_grad_avg
    # the reduced-precision feed-forward experiments act on fp32 storage
    run = C.apply_environment(C.RunConfig(), {"CME213_FFN_FP16": "1"})
    assert run.ffn_precision == "bf16" and run.compute_dtype == "tf32"
    run = C.apply_environment(C.RunConfig(), {"CME213_FP16_STORAGE_ONLY": "1", "CME213_STRICT_FP32": "1"})
    assert run.ffn_precision == "store" and run.compute_dtype == "fp32"
    m, _ = C.preset("parity-h128")
    assert any("ffn-precision" in e for e in C.validate_run(m, C.RunConfig(ffn_precision="bf16"), 1))
    assert not C.validate_run(m, C.RunConfig(ffn_precision="bf16", compute_dtype="tf32"), 1)


def _run(args, env=None):
    import os
    e = dict(os.environ)
    e = {k: v for k, v in e.items() if not k.startswith("CME213_")}
    e.update(env or {})
    return subprocess.run([sys.executable, "-m", "cme213_final_project_b200.train", *args], capture_output=True,
                          text=True, env=e, timeout=120)


def test_validate_config_exit_codes():
    r = _run(["--validate-config", "--device", "cpu"])
    assert r.returncode == 0 and "Configuration validation: PASS" in r.stdout and "CME213 environment:" in r.stdout
    r = _run(["--validate-config", "--device", "cpu"], {"CME213_MIXED_PRECISION": "1"})
    assert r.returncode == 2 and "Invalid CME213 configuration" in r.stderr
    r = _run(["--validate-config", "--device", "cpu", "--sync-mode", "bogus"])
    assert r.returncode == 2 and "Unknown sync mode" in r.stderr


def test_log_line_formats():
    m, _ = C.preset("parity-h128")
    assert logfmt.model_line(m) == "Model: vocab=65 seq=64 hidden=128 heads=4 ff=512 batch=32"
    assert logfmt.params_line(222592) == "Parameters: 222592 (869.50 KB)"
    assert logfmt.training_line(1, 3e-4, 20, 4, "auto", True, 256, 8.0) == (
        "Training: epochs=1 lr=3.00e-04 max_steps=20 world_size=4 sync_mode=auto effective_sync=overlap "
        "bucket_kb=256 auto_overlap_max_mb=8.0")
    assert logfmt.step_line(1, 20, 20, 3.19234) == "  epoch 1 | step   20/20 | loss 3.1923"
    line = logfmt.epoch_line(1, 3.2, 100, 82.0, 2494000.0, 4, True, 0.011, 2.64, 1.5e-5)
    assert line.startswith("Epoch 1: avg_logged_loss=3.2000  steps/rank=100  82ms  2494000 tok/s")
    assert "avg_grad_start=0.011ms  avg_grad_finish=2.640ms  checksum_span=1.500e-05" in line
    assert "avg_grad_sync=" in logfmt.epoch_line(1, 3.2, 100, 82.0, 1.0, 4, False, 0, 4.52, 0)
    assert "checksum" not in logfmt.epoch_line(1, 3.2, 100, 82.0, 1.0, 1, False, 0, 0, 0)
