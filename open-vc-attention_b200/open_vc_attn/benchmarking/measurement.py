"""Statistics over timing samples; no CUDA import (src/open_vc_attn/benchmarking/measurement.py of the reference)."""

import math
import statistics


def _checked(samples):
    values = list(samples)
    if not values or not all(math.isfinite(x) and x > 0 for x in values):
        raise ValueError("Timing samples must be finite and positive")
    return values


def summarize(samples):
    """Median, mean, extremes and coefficient of variation of a list of millisecond samples."""
    values = _checked(samples)
    mean = statistics.fmean(values)
    return {
        "median_ms": statistics.median(values),
        "mean_ms": mean,
        "min_ms": min(values),
        "max_ms": max(values),
        "cv_percent": 100.0 * statistics.pstdev(values) / mean,
        "samples_ms": values,
    }


def speedup(baseline, candidate):
    """Paired comparison: samples i of both lists were taken in the same round."""
    base, cand = _checked(baseline) if baseline else [], _checked(candidate) if candidate else []
    if not base or len(base) != len(cand):
        raise ValueError("Paired samples must have equal nonzero length")
    ratios = [b / c for b, c in zip(base, cand)]
    median_base, median_cand = statistics.median(base), statistics.median(cand)
    return {
        "ratio_of_medians": median_base / median_cand,
        "median_paired_ratio": statistics.median(ratios),
        "paired_ratios": ratios,
        "latency_reduction_percent": 100.0 * (1.0 - median_cand / median_base),
    }


def parse_shape(text):
    """'SxHx128' (or with commas) -> (S, H, 128)."""
    parts = text.replace(",", "x").split("x")
    try:
        dims = tuple(int(part) for part in parts)
    except ValueError:
        raise ValueError("Shape must be SxHx128") from None
    if len(dims) != 3 or min(dims) < 1 or dims[2] != 128:
        raise ValueError("Shape must be SxHx128 with positive dimensions")
    return dims
