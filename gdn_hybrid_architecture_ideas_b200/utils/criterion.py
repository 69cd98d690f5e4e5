"""Acceptance rule for numeric comparisons: a candidate's error against a ground truth is judged against the error a
trusted path makes against the same truth, not against a bare tolerance.

A `Rule` turns the trusted path's error `ref` into an allowance

    form "sum":  factor * ref + floor          form "max":  max(factor * ref, floor)

clipped from above by `ceil` when given and multiplied by `scale` when the check is relative to a magnitude. A `Reading`
is one judged comparison; besides pass / fail it tells apart a pass earned by the ratio (err <= factor * ref) from one
that only the floor allowed, because a check that passes through its floor alone says little about the candidate. NaN
never passes, on either side. No torch import at module level: tools that only judge numbers load this without it
(reference: ced/utils/criterion.py:64-334).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

ONLY_FLOOR = "PASS ONLY THROUGH THE FLOOR"
BY_RATIO = "ok (ratio alone)"
_FORMS = ("sum", "max")


def over(err: float, bound: float) -> bool:
    """err > bound, with NaN on either side counting as over."""
    return not (err <= bound)


def nan_max(values, default: float = math.nan) -> float:
    """Largest value, NaN if any value is NaN (the built-in max silently drops a NaN unless it comes first)."""
    best, seen = -math.inf, False
    for v in values:
        x = float(v)
        if x != x:
            return math.nan
        best, seen = (x if x > best else best), True
    return best if seen else default


@dataclass(frozen=True)
class Rule:
    factor: float
    floor: float
    form: str = "sum"
    ceil: float | None = None
    source: str = ""        # where the numbers come from (a measurement, a file), for reports

    def __post_init__(self):
        if self.form not in _FORMS:
            raise ValueError(f"Rule.form {self.form!r}: 'sum' or 'max'")

    # -- the allowance
    def ratio_part(self, ref: float, scale: float | None = None) -> float:
        """The allowance the trusted path's error alone gives: factor * ref (times scale)."""
        return self.factor * ref * (1.0 if scale is None else scale)

    def bound(self, ref: float, scale: float | None = None) -> float:
        if ref != ref:
            return math.nan
        scaled = self.factor * ref
        allowance = scaled + self.floor if self.form == "sum" else (scaled if scaled > self.floor else self.floor)
        if self.ceil is not None and allowance > self.ceil:
            allowance = self.ceil
        return allowance * (1.0 if scale is None else scale)

    def passes(self, err: float, ref: float, scale: float | None = None) -> bool:
        return not over(err, self.bound(ref, scale))

    def read(self, label: str, err: float, ref: float, scale: float | None = None) -> "Reading":
        return Reading(label, float(err), float(ref), self, scale)

    @property
    def no_floor(self) -> bool:
        return self.form == "sum" and self.floor == 0.0

    def formula(self) -> str:
        ratio = f"{self.factor:g} x ref"
        if self.no_floor:
            return ratio + " (no floor)"
        return f"{ratio} + floor {self.floor:g}" if self.form == "sum" else f"max({ratio}, floor {self.floor:g})"


@dataclass(frozen=True)
class Reading:
    label: str
    err: float
    ref: float
    rule: Rule
    scale: float | None = None

    @property
    def bound(self) -> float:
        return self.rule.bound(self.ref, self.scale)

    @property
    def ok(self) -> bool:
        return not over(self.err, self.bound)

    @property
    def by_ratio(self) -> bool:
        return not over(self.err, self.rule.ratio_part(self.ref, self.scale))

    @property
    def only_floor(self) -> bool:
        return self.ok and not self.by_ratio

    @property
    def verdict(self) -> str:
        if not self.ok:
            return "FAIL"
        return BY_RATIO if self.by_ratio else ONLY_FLOOR

    def line(self) -> str:
        return (f"{self.label}: err {self.err:.3e} ref {self.ref:.3e} bound {self.bound:.3e} "
                f"[{self.rule.formula()}] {self.verdict}")


@dataclass
class Tally:
    """Running counts over the readings of one check run; keeps the failed readings for the report."""
    passed: int = 0
    failed: int = 0
    floor_only: int = 0
    failures: list = field(default_factory=list)

    def add(self, reading: Reading) -> Reading:
        if reading.ok:
            self.passed += 1
            self.floor_only += reading.only_floor
        else:
            self.failed += 1
            self.failures.append(reading)
        return reading

    @property
    def ok(self) -> bool:
        return self.failed == 0

    def summary(self) -> str:
        return f"{self.passed} passed ({self.floor_only} only through the floor), {self.failed} failed"


def tensor_errors(candidate, reference, truth) -> tuple[float, float]:
    """(candidate's, trusted path's) largest absolute deviation from `truth`, all three tensors, compared in float64."""
    t = truth.double()
    return float((candidate.double() - t).abs().max()), float((reference.double() - t).abs().max())
