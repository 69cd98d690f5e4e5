"""Larger multi-key item sets: the plan of a rerun with enough items that the sampling error is small next to the
seed spread. Pure functions, no torch, no data files.

A cell is (probe, n_keys, length): the multi-key needle probe of `eval/probes.py` with n keys in a sequence of that
length, scored by exact match. An item is a pure function of (seed, kind, index), so a larger set is the old set with
items appended: items 0 .. n_old - 1 are the ones already scored.

The plan cuts the work (every cell's items 0 .. n - 1) into scoring groups of at most a budget of modelled seconds,
the dearest cells first, a cell cut at a multiple of SPLIT_STEP items when it does not fit; deterministic, so the
builder and the scoring runs agree on which group scores which items. The time model is tokens / throughput per item
plus a start cost per process and per distinct row shape. The common values file of a run is
{"run", "family": "items", "cells": {"items|<probe>_n<k>|<length>|exact": accuracy}, "n_items": {...}, "excluded": [...]}
(reference: ced/eval/recall_items.py:1-60, 116-232, 271-357; its cell list, old-item counts and per-length seconds are
those of one cluster's runs and are parameters here).
"""

from __future__ import annotations

import json
import math
import re
from dataclasses import dataclass
from pathlib import Path

FAMILY = "items"
ID_RE = re.compile(r"^([a-z_]+)/len=(\d+)/n=(\d+)/(\d{4,})$")
START_SECONDS = 60.0        # a scoring process's start: model load, extension load, first batch
SHAPE_SECONDS = 5.0         # the first batch of a row shape (graph capture, allocator growth)
GROUP_BUDGET_S = 3000.0
DEADLINE_MAX_S, DEADLINE_STEP_S, DEADLINE_FACTOR = 3600, 300, 1.2
SPLIT_STEP = 50
TOKENS_PER_SECOND = 500_000.0   # forward-only scoring throughput the default time model assumes


@dataclass(frozen=True)
class Cell:
    probe: str
    n_keys: int
    length: int

    @property
    def key(self) -> str:
        return f"{self.probe}_n{self.n_keys}|{self.length}"

    @property
    def item_prefix(self) -> str:
        return f"{self.probe}/len={self.length}/n={self.n_keys}/"


def cells_of(probe: str = "multikey", n_keys=(4, 16), lengths=(8192, 16384, 32768, 65536, 131072)) -> list[Cell]:
    return [Cell(probe, n, L) for n in n_keys for L in lengths]


def item_id(cell: Cell, index: int) -> str:
    return f"{cell.item_prefix}{index:04d}"


def parse_item_id(text: str) -> tuple[Cell, int]:
    m = ID_RE.match(text)
    if not m:
        raise ValueError(f"not a multi-key item id: {text!r}")
    return Cell(m.group(1), int(m.group(3)), int(m.group(2))), int(m.group(4))


def cell_of_key(key: str) -> Cell:
    name, length = key.split("|")
    probe, n = name.rsplit("_n", 1)
    return Cell(probe, int(n), int(length))


def item_seconds(cell: Cell, tokens_per_second: float = TOKENS_PER_SECOND) -> float:
    return cell.length / tokens_per_second


@dataclass(frozen=True)
class Part:
    cell: str
    start: int
    stop: int

    def to_json(self) -> dict:
        return {"cell": self.cell, "start": self.start, "stop": self.stop}


def parts_seconds(parts: list[Part], tokens_per_second: float = TOKENS_PER_SECOND) -> float:
    shapes = {cell_of_key(p.cell).length for p in parts if p.stop > p.start}
    return START_SECONDS + SHAPE_SECONDS * len(shapes) + math.fsum(
        (p.stop - p.start) * item_seconds(cell_of_key(p.cell), tokens_per_second) for p in parts)


def deadline_for(modelled_s: float) -> int:
    d = int(math.ceil(DEADLINE_FACTOR * modelled_s / DEADLINE_STEP_S) * DEADLINE_STEP_S)
    return min(DEADLINE_MAX_S, max(DEADLINE_STEP_S, d))


@dataclass
class Group:
    name: str
    parts: list[Part]
    tokens_per_second: float = TOKENS_PER_SECOND

    @property
    def modelled_s(self) -> float:
        return parts_seconds(self.parts, self.tokens_per_second)

    @property
    def items(self) -> int:
        return sum(p.stop - p.start for p in self.parts)

    def to_json(self) -> dict:
        return {"name": self.name, "modelled_s": round(self.modelled_s, 1), "deadline_s": deadline_for(self.modelled_s), "items": self.items,
                "parts": [p.to_json() for p in self.parts]}


def assign_groups(cell_n: dict[str, int], budget_s: float = GROUP_BUDGET_S, tokens_per_second: float = TOKENS_PER_SECOND,
                  prefix: str = "g") -> list[Group]:
    sec = lambda c: item_seconds(c, tokens_per_second)
    order = sorted((cell_of_key(k) for k in cell_n), key=lambda c: (-sec(c), c.probe, c.n_keys, c.length))
    todo = [(c, 0, cell_n[c.key]) for c in order if cell_n[c.key] > 0]
    groups, cur = [], []
    close = lambda: groups.append(Group(f"{prefix}{len(groups) + 1}", list(cur), tokens_per_second))
    while todo:
        c, a, b = todo.pop(0)
        if parts_seconds(cur + [Part(c.key, a, b)], tokens_per_second) <= budget_s:
            cur.append(Part(c.key, a, b))
            continue
        fixed = parts_seconds(cur + [Part(c.key, a, a + 1)], tokens_per_second) - sec(c)
        k = int((budget_s - fixed) // sec(c))
        stop = min(a + (k // SPLIT_STEP) * SPLIT_STEP if k >= SPLIT_STEP else a, b)
        if stop > a:
            cur.append(Part(c.key, a, stop))
            todo.insert(0, (c, stop, b))
            close()
            cur = []
        elif cur:
            close()
            cur = []
            todo.insert(0, (c, a, b))
        else:
            raise ValueError(f"cell {c.key}: not even {SPLIT_STEP} items fit a group of {budget_s:.0f} s")
    if cur:
        close()
    return groups


def make_plan(cell_n: dict[str, int], n_old: dict[str, int] | None = None, rule: str = "", budget_s: float = GROUP_BUDGET_S,
              tokens_per_second: float = TOKENS_PER_SECOND) -> dict:
    n_old = n_old or {}
    for k, n in cell_n.items():
        if n < n_old.get(k, 0):
            raise ValueError(f"{k}: {n} items is fewer than the {n_old[k]} already scored (the old items are the first block)")
    groups = assign_groups(cell_n, budget_s, tokens_per_second)
    total = math.fsum(g.modelled_s for g in groups)
    return {"version": 1, "rule": rule, "tokens_per_second": tokens_per_second,
            "cells": [{"key": k, "probe": c.probe, "n_keys": c.n_keys, "length": c.length, "n_old": n_old.get(k, 0), "n": cell_n[k]}
                      for k, c in ((k, cell_of_key(k)) for k in cell_n)],
            "groups": [g.to_json() for g in groups],
            "total": {"modelled_s": round(total, 1), "groups": len(groups), "gpu_hours_modelled": round(total / 3600, 3),
                      "gpu_hours_bound": round(math.fsum(deadline_for(g.modelled_s) for g in groups) / 3600, 3)}}


def validate_plan(plan: dict) -> None:
    """Every item of every cell is in exactly one part, parts lie inside their cell, and no group is over its deadline."""
    want = {c["key"]: c["n"] for c in plan["cells"]}
    seen = {k: [] for k in want}
    for g in plan["groups"]:
        if g["modelled_s"] > g["deadline_s"]:
            raise ValueError(f"group {g['name']}: modelled {g['modelled_s']} s over its deadline {g['deadline_s']} s")
        for p in g["parts"]:
            if p["cell"] not in want or not 0 <= p["start"] < p["stop"] <= want[p["cell"]]:
                raise ValueError(f"group {g['name']}: part {p} lies outside its cell")
            seen[p["cell"]].append((p["start"], p["stop"]))
    for k, spans in seen.items():
        at = 0
        for a, b in sorted(spans):
            if a != at:
                raise ValueError(f"cell {k}: items {at} .. {a - 1} are in no group or in two")
            at = b
        if at != want[k]:
            raise ValueError(f"cell {k}: items {at} .. {want[k] - 1} are in no group")


def load_plan(path) -> dict:
    plan = json.loads(Path(path).read_text())
    validate_plan(plan)
    return plan


def values_for_run(run: str, plan: dict, results: list[dict], exclude: set[str] | None = None) -> dict:
    """The common values file from per-item results [{"id", "exact"}]: accuracy per cell over the plan's items, the
    excluded ids left out and listed; an item missing from the results is an error."""
    exclude = exclude or set()
    by_id = {r["id"]: bool(r["exact"]) for r in results}
    cells, counts = {}, {}
    for c in plan["cells"]:
        cell = cell_of_key(c["key"])
        ids = [item_id(cell, i) for i in range(c["n"])]
        missing = [i for i in ids if i not in by_id and i not in exclude]
        if missing:
            raise ValueError(f"run {run}: {len(missing)} items of {c['key']} were not scored (first {missing[0]})")
        kept = [i for i in ids if i not in exclude]
        name = f"{FAMILY}|{c['key']}|exact"
        cells[name] = sum(by_id[i] for i in kept) / len(kept) if kept else None
        counts[name] = len(kept)
    return {"run": run, "family": FAMILY, "cells": cells, "n_items": counts, "excluded": sorted(exclude)}


def binomial_se(p: float, n: int) -> float:
    return math.sqrt(max(p * (1 - p), 0.0) / n) if n > 0 else float("nan")


def items_for_se(p: float, se: float) -> int:
    """Items a cell needs for a standard error of at most `se` at accuracy p."""
    return int(math.ceil(p * (1 - p) / se ** 2))
