"""alpha-beta fit and bucket arithmetic (FINAL_CLEAN_CODE_/scripts/predict_comm_model.py:14-18,109-139)."""
from cme213_final_project_b200.parallel import comm_model as cm


def test_fit_recovers_line():
    pts = [(b, 0.02 + 3e-9 * b) for b in (4096, 65536, 1 << 20, 1 << 25)]
    a, b = cm.fit_alpha_beta(pts)
    assert abs(a - 0.02) < 1e-9 and abs(b - 3e-9) < 1e-15
    assert abs(cm.predict_bucketed(a, b, [1 << 20] * 8) - (8 * 0.02 + 3e-9 * (8 << 20))) < 1e-9


def test_reference_gradient_sizes():
    assert cm.gradient_floats(128, 512, 65, 64) == 222592
    assert cm.gradient_floats(256, 1024, 65, 64) == 838400
    assert cm.gradient_floats(512, 2048, 65, 64) == 3249664


def test_bucket_count_trades_latency_for_overlap():
    assert cm.best_bucket_count(alpha=1.0, beta=1e-9, total_bytes=1e6, backward_time=1.0) == 1
    assert cm.best_bucket_count(alpha=1e-3, beta=1e-6, total_bytes=1e6, backward_time=2.0) > 4
