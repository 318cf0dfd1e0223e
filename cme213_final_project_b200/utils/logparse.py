"""Parsers and summaries for the trainer's log lines.

The reference's experiment scripts regex-parse ``Epoch N: ...`` and ``TRAJECTORY ...`` lines, mark a run valid
only if an epoch line was found, the loss is finite, the checksum is not NaN and the log has no ``nan`` / ``inf``
token, drop the first (cold) repeat, and report mean / median / std / CV and speed-ups
(``FINAL_CLEAN_CODE_/scripts/summarize_single_gpu_bench.py:17-68``, ``summarize_training_bucket_sweep.py:67-70``,
``summarize_trajectory_validation.py:110-232``).  Same contract here.
"""
from __future__ import annotations

import math
import re
import statistics
from dataclasses import dataclass, field
from typing import Dict, List, Optional

EPOCH_RE = re.compile(
    r"Epoch (\d+): avg_logged_loss=(\S+)\s+steps/rank=(\d+)\s+(\d+)ms\s+(\d+) tok/s"
    r"(?:\s+avg_grad_sync=([\d.]+)ms)?(?:\s+avg_grad_start=([\d.]+)ms\s+avg_grad_finish=([\d.]+)ms)?"
    r"(?:\s+checksum_span=(\S+))?")
TRAJ_RE = re.compile(
    r"TRAJECTORY epoch=(\d+) step=(\d+) loss=(\S+) param_sum=(\S+) param_sumsq=(\S+) param_maxabs=(\S+) "
    r"param_hash=([0-9a-f]{16}) sum_span=(\S+) sumsq_span=(\S+) maxabs_span=(\S+)")
BAD_TOKEN_RE = re.compile(r"(?<![A-Za-z_])(nan|inf)(?![A-Za-z_])", re.IGNORECASE)


@dataclass
class EpochLine:
    epoch: int
    loss: float
    steps: int
    ms: float
    tok_s: float
    grad_sync_ms: Optional[float] = None
    grad_start_ms: Optional[float] = None
    grad_finish_ms: Optional[float] = None
    checksum_span: Optional[float] = None


@dataclass
class RunSummary:
    epochs: List[EpochLine] = field(default_factory=list)
    valid: bool = False
    reason: str = ""

    @property
    def last(self) -> Optional[EpochLine]:
        return self.epochs[-1] if self.epochs else None


def _f(s: Optional[str]) -> Optional[float]:
    if s is None:
        return None
    try:
        return float(s)
    except ValueError:
        return float("nan")


def parse_run(text: str) -> RunSummary:
    r = RunSummary()
    for m in EPOCH_RE.finditer(text):
        r.epochs.append(EpochLine(int(m.group(1)), _f(m.group(2)), int(m.group(3)), float(m.group(4)), float(m.group(5)),
                                  _f(m.group(6)), _f(m.group(7)), _f(m.group(8)), _f(m.group(9))))
    if not r.epochs:
        r.reason = "no epoch line"
    elif not math.isfinite(r.epochs[-1].loss):
        r.reason = "non-finite loss"
    elif r.epochs[-1].checksum_span is not None and math.isnan(r.epochs[-1].checksum_span):
        r.reason = "checksum is nan"
    elif BAD_TOKEN_RE.search(text) or "FAIL" in text:
        r.reason = "nan/inf/FAIL token in log"
    else:
        r.valid = True
    return r


def parse_trajectory(text: str) -> List[Dict]:
    out = []
    for m in TRAJ_RE.finditer(text):
        out.append({"epoch": int(m.group(1)), "step": int(m.group(2)), "loss": float(m.group(3)),
                    "sum": float(m.group(4)), "sumsq": float(m.group(5)), "maxabs": float(m.group(6)),
                    "hash": m.group(7), "sum_span": float(m.group(8)), "sumsq_span": float(m.group(9)),
                    "maxabs_span": float(m.group(10))})
    return out


def summarize_repeats(tok_s: List[float], valid: List[bool], min_repeat: int = 2) -> Dict:
    """Statistics over repeats ``min_repeat..`` (1-based: the first repeat is the cold one and is dropped)."""
    warm = [t for i, (t, v) in enumerate(zip(tok_s, valid), start=1) if i >= min_repeat and v]
    n = len(warm)
    mean = statistics.fmean(warm) if n else float("nan")
    std = statistics.stdev(warm) if n > 1 else 0.0
    return {"runs": len(tok_s), "valid_runs": sum(valid), "all_valid": all(valid) and bool(valid), "warm_runs": n,
            "mean": mean, "median": statistics.median(warm) if n else float("nan"), "std": std,
            "cv": (std / mean) if n and mean else float("nan")}


def compare_trajectories(base: List[Dict], other: List[Dict], loss_tol: float = 5e-3, sum_rtol: float = 1e-4,
                         sumsq_rtol: float = 1e-2, maxabs_rtol: float = 1e-2, n_params: int = 0) -> Dict:
    """Per-step comparison of a synchronisation mode against the blocking baseline; hashes need not match
    (floating-point reorder), statistics must agree within the tolerances.

    Two levels, as in the reference's summariser, which takes its tolerances per statistic
    (``summarize_trajectory_validation.py:110-232``).  ``identical_path``: loss and parameter sum agree to
    ``loss_tol`` / ``sum_rtol`` -- what modes that run the same arithmetic in a different schedule must meet (here
    they agree bit for bit).  ``ok``: loss, sum of squares and largest magnitude agree -- what a mode with different
    arithmetic has to meet (the fused path reduces bf16 gradients in fp32, the library all-reduce in bf16): under
    Adam a near-zero gradient that changes sign moves its parameter by a whole step the other way, so the plain sum,
    a residual of cancelling signed values, drifts by many parameters' worth of lr while the magnitudes agree.
    The library's own bucketed bf16 all-reduce deviates from its whole-arena all-reduce by the same amounts (measured
    at 4 ranks), so the second level is the tolerance of the gradient precision, not of one implementation.
    With ``n_params`` the absolute differences of sum and sum of squares are also given per parameter, the
    normalisation the reference's summariser applies (``summarize_trajectory_validation.py:162-166``)."""
    n = min(len(base), len(other))
    rel = lambda key, floor: max((abs(base[i][key] - other[i][key]) / max(floor, abs(base[i][key])) for i in range(n)),
                                 default=float("nan"))
    worst_loss = max((abs(base[i]["loss"] - other[i]["loss"]) for i in range(n)), default=float("nan"))
    worst_sum, worst_sumsq, worst_maxabs = rel("sum", 1.0), rel("sumsq", 1e-12), rel("maxabs", 1e-12)
    span = max((o["sum_span"] for o in other), default=0.0)
    same_len = n > 0 and len(base) == len(other)
    out = {}
    if n_params > 0:
        absd = lambda key: max((abs(base[i][key] - other[i][key]) for i in range(n)), default=float("nan"))
        out = {"max_sum_diff_per_param": absd("sum") / n_params, "max_sumsq_diff_per_param": absd("sumsq") / n_params}
    return {**out,
            "steps": n, "max_loss_diff": worst_loss, "max_rel_sum_diff": worst_sum, "max_rel_sumsq_diff": worst_sumsq,
            "max_rel_maxabs_diff": worst_maxabs, "max_sum_span": span,
            "identical_path": same_len and worst_loss <= loss_tol and worst_sum <= sum_rtol,
            "ok": same_len and worst_loss <= loss_tol and worst_sumsq <= sumsq_rtol and worst_maxabs <= maxabs_rtol}
