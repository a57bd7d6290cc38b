"""Summary statistics and the paired A/B decision rule of the benchmark harness.

A change counts as a gain only if (1) the 95 % confidence interval of the paired differences
``b[i] - a[i]`` excludes zero **and** (2) the median gain is larger than the larger of the two arms'
own standard deviations.  Counterpart of the reference's ``scripts/bench/stats.py:44-118``.
"""

from __future__ import annotations

import math
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


class Sample:
    """Order statistics and moments of a list of measurements (values kept sorted)."""

    def __init__(self, values):
        self.sorted = sorted(float(v) for v in values)
        if not self.sorted:
            raise ValueError("empty sample")

    def __len__(self) -> int:
        return len(self.sorted)

    def quantile(self, q: float) -> float:
        """Linear interpolation between the two nearest order statistics, ``q`` in [0, 100]."""
        rank = (len(self) - 1) * (q / 100.0)
        floor = min(int(rank), len(self) - 1)
        ceil = min(floor + 1, len(self) - 1)
        lower, upper = self.sorted[floor], self.sorted[ceil]
        return lower + (upper - lower) * (rank - floor)

    @property
    def mean(self) -> float:
        return math.fsum(self.sorted) / len(self)

    @property
    def std(self) -> float:
        """Sample standard deviation (n - 1 in the denominator); 0 for a single value."""
        if len(self) < 2:
            return 0.0
        centre = self.mean
        return math.sqrt(math.fsum((v - centre) ** 2 for v in self.sorted) / (len(self) - 1))


def percentile(xs: list[float], q: float) -> float:
    return Sample(xs).quantile(q)


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
    s = Sample(xs)
    return Summary(n=len(s), median=s.quantile(50.0), p95=s.quantile(95.0), mean=s.mean, std=s.std,
                   min=s.sorted[0], max=s.sorted[-1])


@dataclass
class PairedResult:
    n: int
    mean_diff: float           # mean of b[i] - a[i]; negative when B is the faster arm
    ci95: tuple[float, float]  # 95 % confidence interval of that mean (Student t, n - 1 degrees of freedom)
    median_improvement: float  # median(a) - median(b); positive when B is the faster arm
    pooled_std: float          # the noisier arm's own standard deviation
    significant: bool          # both conditions of the rule hold

    @property
    def beneficial(self) -> bool:
        return self.significant and self.median_improvement > 0.0

    def to_dict(self) -> dict:
        return {**asdict(self), "ci95": list(self.ci95), "beneficial": self.beneficial}


def paired_ab(a: list[float], b: list[float]) -> PairedResult:
    """Decision for two arms measured in alternation (``a[i]`` and ``b[i]`` back to back)."""
    if len(a) != len(b) or len(a) < 2:
        raise ValueError("need equal-length samples with n >= 2")
    arm_a, arm_b = Sample(a), Sample(b)
    change = Sample(after - before for before, after in zip(a, b))
    reach = t95(len(change) - 1) * change.std / math.sqrt(len(change))
    interval = (change.mean - reach, change.mean + reach)
    gain = arm_a.quantile(50.0) - arm_b.quantile(50.0)
    noise = max(arm_a.std, arm_b.std)
    clear_of_zero = interval[0] > 0.0 or interval[1] < 0.0
    return PairedResult(n=len(change), mean_diff=change.mean, ci95=interval, median_improvement=gain,
                        pooled_std=noise, significant=clear_of_zero and abs(gain) > noise)
