"""Summary statistics of a sample list, as the reference reports them
(src/bench/stats.rs:10-101): count, mean, sample standard deviation and
variance (n - 1), min, max, and percentiles by linear interpolation between
the two nearest ranks."""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Optional, Sequence


@dataclass(frozen=True)
class Summary:
    count: int
    mean: float
    stdev: float
    variance: float
    min: float
    max: float
    p10: float
    p25: float
    p50: float
    p75: float
    p90: float
    p95: float
    p99: float

    def to_json(self) -> dict:
        return asdict(self)


def percentile(sorted_values: Sequence[float], fraction: float) -> float:
    rank = fraction * (len(sorted_values) - 1)
    lo, hi = math.floor(rank), math.ceil(rank)
    w = rank - lo
    return sorted_values[lo] * (1.0 - w) + sorted_values[hi] * w


def summarize(values: Sequence[float]) -> Optional[Summary]:
    if not values:
        return None
    v = sorted(float(x) for x in values)
    n = len(v)
    mean = sum(v) / n
    variance = sum((x - mean) ** 2 for x in v) / (n - 1) if n > 1 else 0.0
    return Summary(n, mean, math.sqrt(variance), variance, v[0], v[-1],
                   *(percentile(v, p) for p in (0.10, 0.25, 0.50, 0.75, 0.90, 0.95, 0.99)))
