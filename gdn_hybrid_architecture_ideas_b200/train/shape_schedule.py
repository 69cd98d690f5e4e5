"""Batch-shape schedule: rows per optimizer step and row length by phases of a run's tokens (batch warm-up and
short-to-long rows).

`phases` lists the phases before the config's own shape, each (until, rows, seq_len) with `until` a fraction of the
run; the config's own (B rows of L tokens) runs last. One reference step = B * L tokens, and a run reads
`steps * B * L` tokens with or without a schedule. A phase ends at reference step floor(until * steps + 0.5). Inside a
phase an optimizer step reads rows_p * len_p tokens, so per_ref = B L / (rows_p len_p) optimizer steps make one
reference step (must be whole). The token clock of optimizer step k (j-th of its phase) is start_p + j / per_ref;
learning-rate schedules read the clock ("clock" mode) or the reference step divided by per_ref ("rows": the linear
scaling rule, LR summed over the run unchanged) (reference: ced/train/shape_schedule.py:80-231).
"""

from __future__ import annotations

import bisect
import math
from dataclasses import dataclass

SHAPE_LR_MODES = ("clock", "rows")


@dataclass(frozen=True)
class Phase:
    start: int          # first reference step
    end: int            # one past the last reference step
    rows: int
    seq_len: int
    per_ref: int        # optimizer steps per reference step
    first_step: int     # first optimizer step of the phase

    @property
    def steps(self) -> int:
        return (self.end - self.start) * self.per_ref


@dataclass(frozen=True)
class StepShape:
    phase: int
    rows: int
    seq_len: int
    first_row: int      # index of the step's first row, in rows of seq_len tokens of the packed stream
    clock: float        # reference steps of tokens read before this step
    lr_scale: float     # 1 / per_ref under "rows", else 1


class ShapeSchedule:
    def __init__(self, phases, steps: int, batch_rows: int, seq_len: int, micro_rows: int | None = None, lr_mode: str = "clock"):
        if lr_mode not in SHAPE_LR_MODES:
            raise ValueError(f"train.shape_lr {lr_mode!r}: one of {SHAPE_LR_MODES}")
        self.batch_rows, self.seq_len, self.ref_steps, self.lr_mode = batch_rows, seq_len, steps, lr_mode
        self.micro_rows = micro_rows or batch_rows
        tokens = batch_rows * seq_len
        out, start, first = [], 0, 0
        listed = [tuple(p) for p in phases] + [(1.0, batch_rows, seq_len)]
        prev_until = 0.0
        for until, rows, length in listed:
            if not (prev_until <= until <= 1.0):
                raise ValueError(f"train.shape_schedule: phase ends must rise within [0, 1], got {until}")
            prev_until = until
            end = min(steps, int(math.floor(until * steps + 0.5)))
            if rows <= 0 or length <= 0 or tokens % (rows * length):
                raise ValueError(f"train.shape_schedule: {rows} rows of {length} must divide the step's {tokens} tokens")
            if seq_len % length:
                raise ValueError(f"train.shape_schedule: row length {length} must divide data.seq_len {seq_len}")
            per_ref = tokens // (rows * length)
            micro = self.micro_rows * seq_len // length
            if rows % micro and micro % rows:
                raise ValueError(f"train.shape_schedule: {rows} rows against a micro-batch of {micro} rows of {length}")
            ph = Phase(start, max(end, start), rows, length, per_ref, first)
            out.append(ph)
            first += ph.steps
            start = ph.end
        self.phases = out
        self.total_steps = first
        self._firsts = [p.first_step for p in out]

    def micro_rows_at(self, phase: Phase) -> int:
        """Rows per forward/backward: the config's tokens per micro-batch."""
        return max(1, min(phase.rows, self.micro_rows * self.seq_len // phase.seq_len))

    def at(self, k: int) -> StepShape:
        if not 0 <= k < self.total_steps:
            raise IndexError(f"optimizer step {k} outside the schedule's {self.total_steps}")
        i = bisect.bisect_right(self._firsts, k) - 1
        while self.phases[i].steps == 0:
            i += 1
        p = self.phases[i]
        j = k - p.first_step
        first_row = p.start * self.batch_rows * self.seq_len // p.seq_len + j * p.rows
        clock = p.start + j / p.per_ref
        if self.lr_mode == "rows":
            clock = float(p.start + j // p.per_ref)
        return StepShape(i, p.rows, p.seq_len, first_row, clock, 1.0 / p.per_ref if self.lr_mode == "rows" else 1.0)


def reference_walk(phases, steps: int, batch_rows: int, seq_len: int):
    """The slow definition: walk optimizer steps counting tokens; yields (rows, seq_len, first_token) per step."""
    tokens = batch_rows * seq_len
    listed = [tuple(p) for p in phases] + [(1.0, batch_rows, seq_len)]
    read, out = 0, []
    for until, rows, length in listed:
        end_tokens = min(steps, int(math.floor(until * steps + 0.5))) * tokens
        while read < end_tokens:
            out.append((rows, length, read))
            read += rows * length
    return out
