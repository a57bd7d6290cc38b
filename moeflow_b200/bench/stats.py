"""Summary statistics and the paired A/B decision rule of the benchmark harness.

A change counts as a gain only if (1) the 95 % confidence interval of the paired differences
``b[i] - a[i]`` excludes zero **and** (2) the median gain is larger than the larger of the two arms'
own standard deviations.  Counterpart of the reference's ``scripts/bench/stats.py:44-118``.
"""

from __future__ import annotations

import math
import statistics
from dataclasses import asdict, dataclass


def _betacf(a: float, b: float, x: float) -> float:
    """Continued fraction of the incomplete beta function (Lentz)."""
    tiny = 1e-300
    qab, qap, qam = a + b, a + 1.0, a - 1.0
    c, d = 1.0, 1.0 - qab * x / qap
    d = 1.0 / (d if abs(d) > tiny else tiny)
    h = d
    for m in range(1, 400):
        m2 = 2 * m
        aa = m * (b - m) * x / ((qam + m2) * (a + m2))
        d = 1.0 + aa * d
        d = 1.0 / (d if abs(d) > tiny else tiny)
        c = 1.0 + aa / c
        c = c if abs(c) > tiny else tiny
        h *= d * c
        aa = -(a + m) * (qab + m) * x / ((a + m2) * (qap + m2))
        d = 1.0 + aa * d
        d = 1.0 / (d if abs(d) > tiny else tiny)
        c = 1.0 + aa / c
        c = c if abs(c) > tiny else tiny
        delta = d * c
        h *= delta
        if abs(delta - 1.0) < 1e-14:
            break
    return h


def _betainc(a: float, b: float, x: float) -> float:
    if x <= 0.0:
        return 0.0
    if x >= 1.0:
        return 1.0
    front = math.exp(math.lgamma(a + b) - math.lgamma(a) - math.lgamma(b) + a * math.log(x) + b * math.log1p(-x))
    if x < (a + 1.0) / (a + b + 2.0):
        return front * _betacf(a, b, x) / a
    return 1.0 - front * _betacf(b, a, 1.0 - x) / b


def _t_two_sided_tail(t: float, df: int) -> float:
    return _betainc(df / 2.0, 0.5, df / (df + t * t))


def t95(df: int) -> float:
    """Two-sided 95 % critical value of Student's t (bisection on the exact tail probability)."""
    if df < 1:
        raise ValueError("need at least 2 samples")
    lo, hi = 0.0, 100.0
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        if _t_two_sided_tail(mid, df) > 0.05:
            lo = mid
        else:
            hi = mid
    return 0.5 * (lo + hi)


def percentile(xs: list[float], q: float) -> float:
    """Percentile with linear interpolation between order statistics, ``q`` in [0, 100]."""
    if not xs:
        raise ValueError("empty sample")
    ordered = sorted(xs)
    where = (len(ordered) - 1) * q / 100.0
    below = int(math.floor(where))
    above = min(below + 1, len(ordered) - 1)
    return ordered[below] + (ordered[above] - ordered[below]) * (where - below)


@dataclass
class Summary:
    n: int
    median: float
    p95: float
    mean: float
    std: float
    min: float
    max: float

    def to_dict(self) -> dict:
        return asdict(self)


def summarize(xs: list[float]) -> Summary:
    return Summary(
        n=len(xs),
        median=statistics.median(xs),
        p95=percentile(xs, 95.0),
        mean=statistics.fmean(xs),
        std=statistics.stdev(xs) if len(xs) > 1 else 0.0,
        min=min(xs),
        max=max(xs),
    )


@dataclass
class PairedResult:
    n: int
    mean_diff: float  # mean(b - a); negative means B is faster
    ci95: tuple[float, float]
    median_improvement: float  # median(a) - median(b)
    pooled_std: float  # the larger of the two arms' standard deviations
    significant: bool

    @property
    def beneficial(self) -> bool:
        return self.significant and self.median_improvement > 0

    def to_dict(self) -> dict:
        d = asdict(self)
        d["ci95"] = list(self.ci95)
        d["beneficial"] = self.beneficial
        return d


def paired_ab(a: list[float], b: list[float]) -> PairedResult:
    """Paired comparison of alternating repetitions (``a[i]`` and ``b[i]`` measured back to back)."""
    if len(a) != len(b) or len(a) < 2:
        raise ValueError("need equal-length samples with n >= 2")
    diffs = [after - before for before, after in zip(a, b)]
    n = len(diffs)
    mean_diff = statistics.fmean(diffs)
    half_width = t95(n - 1) * statistics.stdev(diffs) / math.sqrt(n)
    ci = (mean_diff - half_width, mean_diff + half_width)
    gain = statistics.median(a) - statistics.median(b)
    noise = max(statistics.stdev(a), statistics.stdev(b))
    excludes_zero = ci[0] > 0.0 or ci[1] < 0.0
    return PairedResult(n, mean_diff, ci, gain, noise, excludes_zero and abs(gain) > noise)
