"""Pass/fail rule of a numeric check: a candidate's error against a ground truth is compared with the error a reference
path makes against the same ground truth.

    "sum":  err <= factor * err_ref + floor        "max":  err <= max(factor * err_ref, floor)

optionally capped (`ceil`) and scaled (`scale`, e.g. by |value|). A reading records whether it passed by the ratio
alone (err <= factor * err_ref) or only through the floor; a NaN error or bound never passes. Pure Python, so tools and
tests can import it without torch (reference: ced/utils/criterion.py:64-334).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

ONLY_FLOOR = "PASS ONLY THROUGH THE FLOOR"
BY_RATIO = "ok (ratio alone)"


def over(err: float, bound: float) -> bool:
    """True when err exceeds the bound or either is NaN."""
    return not (err <= bound)


def nan_max(values, default: float = math.nan) -> float:
    """max() that keeps a NaN (Python's max drops a NaN that is not first)."""
    xs = [float(v) for v in values]
    if not xs:
        return default
    return math.nan if any(math.isnan(x) for x in xs) else max(xs)


@dataclass(frozen=True)
class Rule:
    factor: float
    floor: float
    form: str = "sum"
    ceil: float | None = None
    source: str = ""

    def __post_init__(self):
        if self.form not in ("sum", "max"):
            raise ValueError(f"Rule.form {self.form!r}: 'sum' or 'max'")

    def bound(self, ref: float, scale: float | None = None) -> float:
        if math.isnan(ref):
            return math.nan
        b = self.factor * ref + self.floor if self.form == "sum" else max(self.factor * ref, self.floor)
        if self.ceil is not None:
            b = min(b, self.ceil)
        return b if scale is None else b * scale

    def passes(self, err: float, ref: float, scale: float | None = None) -> bool:
        return bool(err <= self.bound(ref, scale))

    def read(self, label: str, err: float, ref: float, scale: float | None = None) -> "Reading":
        return Reading(label, float(err), float(ref), self, scale)

    @property
    def no_floor(self) -> bool:
        return self.form == "sum" and self.floor == 0.0

    def formula(self) -> str:
        if self.no_floor:
            return f"{self.factor:g} x ref (no floor)"
        joiner = " + floor " if self.form == "sum" else ", floor "
        body = f"{self.factor:g} x ref{joiner}{self.floor:g}"
        return body if self.form == "sum" else f"max({body})"


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
        return self.rule.passes(self.err, self.ref, self.scale)

    @property
    def by_ratio(self) -> bool:
        rb = self.rule.factor * self.ref * (1.0 if self.scale is None else self.scale)
        return bool(self.err <= rb)

    @property
    def only_floor(self) -> bool:
        return self.ok and not self.by_ratio

    def line(self) -> str:
        verdict = "FAIL" if not self.ok else (BY_RATIO if self.by_ratio else ONLY_FLOOR)
        return f"{self.label}: err {self.err:.3e} ref {self.ref:.3e} bound {self.bound:.3e} [{self.rule.formula()}] {verdict}"


@dataclass
class Tally:
    """Counts over the readings of one check run."""
    passed: int = 0
    failed: int = 0
    floor_only: int = 0

    def add(self, r: Reading) -> Reading:
        if not r.ok:
            self.failed += 1
        else:
            self.passed += 1
            self.floor_only += int(r.only_floor)
        return r

    @property
    def ok(self) -> bool:
        return self.failed == 0

    def summary(self) -> str:
        return f"{self.passed} passed ({self.floor_only} only through the floor), {self.failed} failed"


def tensor_errors(candidate, reference, truth) -> tuple[float, float]:
    """(err, err_ref): max-abs error of candidate and of reference against a ground truth (tensors or nested lists of
    numbers; torch is imported only if tensors are passed)."""
    import torch
    t = truth.double()
    return float((candidate.double() - t).abs().max()), float((reference.double() - t).abs().max())
