"""alpha-beta model of collective cost and its use for bucket sizing.

The reference fits ``t = alpha + beta * bytes`` to an all-reduce sweep and predicts the cost of a bucketed
gradient sync as ``buckets * alpha + beta * total_bytes`` against the measured one
(``FINAL_CLEAN_CODE_/scripts/predict_comm_model.py:14-18,109-139``, ``summarize_allreduce_alpha_beta.py``).
"""
from __future__ import annotations

from typing import Iterable, List, Sequence, Tuple


def fit_alpha_beta(points: Iterable[Tuple[float, float]]) -> Tuple[float, float]:
    """Least-squares ``t = alpha + beta * bytes`` over ``(bytes, time)`` points; returns ``(alpha, beta)``."""
    pts = list(points)
    n = len(pts)
    if n < 2:
        raise ValueError("need at least two points")
    sx = sum(p[0] for p in pts)
    sy = sum(p[1] for p in pts)
    sxx = sum(p[0] * p[0] for p in pts)
    sxy = sum(p[0] * p[1] for p in pts)
    den = n * sxx - sx * sx
    beta = (n * sxy - sx * sy) / den if den else 0.0
    alpha = (sy - beta * sx) / n
    return alpha, beta


def predict_bucketed(alpha: float, beta: float, bucket_bytes: Sequence[float]) -> float:
    """Predicted time of one synchronisation made of the given bucket messages (no overlap)."""
    return sum(alpha + beta * b for b in bucket_bytes)


def gradient_floats(hidden: int, ff: int, vocab: int, seq_len: int) -> int:
    """Parameter count of the reference's one-block model (H128 -> 222,592; H256 -> 838,400; H512 -> 3,249,664)."""
    d = hidden
    return d * vocab + (ff * d + d) + (d * ff + ff) + 2 * d + d * d + 3 * d * d + 2 * d + vocab * d + seq_len * d
