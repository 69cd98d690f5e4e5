"""A RULER subset inside the training length: multi-key, multi-value and multi-query needle retrieval and variable
tracking, scored by string-match recall on greedy generations.

The task statements, needle sentences, noise sentence, variable-tracking chains and the string-match metric follow RULER
(Hsieh et al. 2024, https://github.com/NVIDIA/RULER, Apache-2.0); this is a re-implementation (no file of RULER is used).
As in the reference's build (ced/eval/recall_ruler.py:1-99) the tasks whose haystack is essays in RULER take held-out
documents instead ("open" haystack, given as a pool of texts), so numbers compare between models, not with published
RULER tables.

    task              haystack   keys     values   keys  values/key  queried  tokens to generate
    niah_multikey_1   open       words    numbers    4        1         1         128
    niah_multikey_2   needle     words    numbers    1        1         1         128
    niah_multikey_3   needle     uuids    uuids      1        1         1         128
    niah_multivalue   open       words    numbers    1        4         1         128
    niah_multiquery   open       words    numbers    4        1         4         128
    vt                noise      variables numbers   one chain of 4 hops (5 variables)   30

An item is a pure function of (seed, task, length, index) and the pool; it is fitted to `length` tokens (prompt plus
the tokens to generate) under the caller's token counter by growing the haystack. Pure text and arithmetic: the model
side is `scripts/recall_ruler_score.py` with `eval.generate`.
"""

from __future__ import annotations

import hashlib
import re
import uuid
from dataclasses import dataclass, field
from typing import Callable

import numpy as np

BASE_SEED = 20241
LENGTHS = (2048, 4096, 8192)
SPEC = {
    "niah_multikey_1": dict(kind="niah", haystack="open", type_k="words", type_v="numbers", n_k=4, n_v=1, n_q=1, gen=128),
    "niah_multikey_2": dict(kind="niah", haystack="needle", type_k="words", type_v="numbers", n_k=1, n_v=1, n_q=1, gen=128),
    "niah_multikey_3": dict(kind="niah", haystack="needle", type_k="uuids", type_v="uuids", n_k=1, n_v=1, n_q=1, gen=128),
    "niah_multivalue": dict(kind="niah", haystack="open", type_k="words", type_v="numbers", n_k=1, n_v=4, n_q=1, gen=128),
    "niah_multiquery": dict(kind="niah", haystack="open", type_k="words", type_v="numbers", n_k=4, n_v=1, n_q=4, gen=128),
    "vt": dict(kind="vt", haystack="noise", hops=4, gen=30),
}
TASKS = tuple(SPEC)
MULTI_REF = ("niah_multivalue", "niah_multiquery", "vt")

_A = ("brisk calm dusty eager faded gentle hollow icy jagged keen lively mellow nimble odd plush quiet rugged silent tidy "
      "upbeat vivid woven young zesty amber bold crisp dim early frail grand humble ivory jolly kind lean misty neat opal "
      "pale quick rosy sly tall urban vast warm yellow").split()
_N = ("anchor basket candle dagger ember falcon garden hammer island jacket kettle ladder magnet needle orchard pillow "
      "quarry ribbon saddle tunnel umbrella valley walnut yacht zipper acorn bridge comet dune engine fossil glacier "
      "harbor inlet jewel kayak lantern meadow nest otter pebble quill raven spire timber violin wagon").split()
NEEDLE = "One of the special magic {type_v} for {key} is: {value}."
NOISE = "The grass is green. The sky is blue. The sun is yellow. Here we go. There and back again."
NIAH_TEMPLATE = ("Some special magic {type_v} are hidden within the following text. Make sure to memorize it. I will quiz you about the "
                 "{type_v} afterwards.\n{context}\nWhat are all the special magic {type_v} for {query} mentioned in the provided text?")
NIAH_ANSWER = " The special magic {type_v} for {query} mentioned in the provided text are"
VT_TEMPLATE = ("Memorize and track the chain(s) of variable assignment hidden in the following text.\n\n{context}\nQuestion: Find all "
               "variables that are assigned the value {value} in the text above.")
VT_ANSWER = " Answer: According to the chain(s) of variable assignment in the text above, {n} variables are assigned the value {value}, they are:"

Count = Callable[[str], int]


class NoFitError(RuntimeError):
    """No haystack size puts the item within the tolerance of the asked length."""


@dataclass
class RulerItem:
    task: str
    length: int
    index: int
    prompt: str
    refs: list[str]
    gen_tokens: int
    tokens: int = 0
    meta: dict = field(default_factory=dict)

    @property
    def id(self) -> str:
        return f"{self.task}/len={self.length}/{self.index:04d}"


def rng_for(task: str, length: int, index: int, stream: int = 0) -> np.random.Generator:
    h = hashlib.blake2b(f"{BASE_SEED}:{task}:{length}:{index}:{stream}".encode(), digest_size=8).digest()
    return np.random.default_rng(int.from_bytes(h, "little"))


def _number(rng, digits: int = 7) -> str:
    return str(int(rng.integers(10 ** (digits - 1), 10 ** digits)))


def _uuid(rng) -> str:
    return str(uuid.UUID(bytes=bytes(rng.integers(0, 256, 16, dtype=np.uint8).tolist()), version=4))


def draw_keys(rng, kind: str, n: int, exclude: set | None = None) -> list[str]:
    """n distinct keys, none in `exclude`: "adjective-noun" words or uuids."""
    seen, out = set(exclude or ()), []
    while len(out) < n:
        k = _uuid(rng) if kind == "uuids" else f"{_A[int(rng.integers(len(_A)))]}-{_N[int(rng.integers(len(_N)))]}"
        if k not in seen:
            seen.add(k)
            out.append(k)
    return out


def draw_values(rng, kind: str, n: int, exclude: set | None = None) -> list[str]:
    seen, out = set(exclude or ()), []
    while len(out) < n:
        v = _uuid(rng) if kind == "uuids" else _number(rng)
        if v not in seen:
            seen.add(v)
            out.append(v)
    return out


def query_string(keys: list[str]) -> str:
    return keys[0] if len(keys) == 1 else ", ".join(keys[:-1]) + ", and " + keys[-1]


def render_niah(task: str, context: str, keys: list[str]) -> str:
    s = SPEC[task]
    tv = s["type_v"]
    text = NIAH_TEMPLATE + NIAH_ANSWER
    if s["n_q"] * s["n_v"] == 1:        # one answer: singular wording, as RULER's niah.py edits its template
        text = text.replace("Some", "A").replace("are all", "is").replace("are", "is").replace("{type_v}", tv[:-1], 4)
    return text.format(type_v=tv, context=context, query=query_string(keys))


def _insert_at_fractions(units: list[str], inserts: list[str], fracs: list[float], sep: str) -> str:
    """`inserts` placed among `units` at the given depth fractions (stable for equal fractions)."""
    slots = sorted(zip((int(round(f * len(units))) for f in fracs), range(len(inserts))))
    out, at = [], 0
    for pos, j in slots:
        out.extend(units[at:pos])
        out.append(inserts[j])
        at = pos
    out.extend(units[at:])
    return sep.join(out)


def fit_units(make: Callable[[int], str], count: Count, total: int, lo: int, hi: int, tol: float) -> tuple[str, int, int]:
    """Largest n in [lo, hi] with count(make(n)) <= total, by bisection (count grows with n). Returns (text, n, tokens);
    NoFitError if even make(lo) is too long or the best fit is below (1 - tol) total."""
    if count(make(lo)) > total:
        raise NoFitError(f"the smallest haystack already exceeds {total} tokens")
    while lo < hi:
        mid = (lo + hi + 1) // 2
        if count(make(mid)) <= total:
            lo = mid
        else:
            hi = mid - 1
    text = make(lo)
    got = count(text)
    if got < (1 - tol) * total:
        raise NoFitError(f"best fit {got} tokens is below the tolerance of {total}")
    return text, lo, got


def _needles(rng, task: str):
    s = SPEC[task]
    keys = draw_keys(rng, s["type_k"], s["n_k"])
    values = [draw_values(rng, s["type_v"], s["n_v"]) for _ in keys]
    sentences = [NEEDLE.format(type_v=s["type_v"], key=k, value=v) for k, vs in zip(keys, values) for v in vs]
    q = keys[:s["n_q"]]
    refs = [v for k, vs in zip(keys, values) if k in q for v in vs]
    return keys, sentences, q, refs


def niah_item(task: str, length: int, index: int, count: Count, pool: list[str] | None = None, tol: float = 0.05) -> RulerItem:
    s = SPEC[task]
    rng = rng_for(task, length, index)
    keys, sentences, q, refs = _needles(rng, task)
    fracs = sorted(rng.choice(np.linspace(0, 1, 40), size=len(sentences), replace=False).tolist())
    budget = length - s["gen"]
    if s["haystack"] == "needle":       # the haystack is itself needles with other keys and values
        def make(n):
            r = rng_for(task, length, index, 1)
            ks = draw_keys(r, s["type_k"], n, exclude=set(keys))
            vs = draw_values(r, s["type_v"], n, exclude=set(refs))
            hay = [NEEDLE.format(type_v=s["type_v"], key=k, value=v) for k, v in zip(ks, vs)]
            return render_niah(task, _insert_at_fractions(hay, sentences, fracs, " "), q)
        prompt, n, got = fit_units(make, count, budget, 1, max(8, budget), tol)
    else:
        if not pool:
            raise ValueError(f"task {task} has an open haystack: give a pool of held-out documents")
        order = rng_for(task, length, index, 2).permutation(len(pool))
        words = " ".join(pool[int(i)] for i in order).split()
        def make(n):
            body = " ".join(words[:n])
            units = re.split(r"(?<=[.!?])\s+", body) if body else [""]
            return render_niah(task, _insert_at_fractions(units, sentences, fracs, " "), q)
        prompt, n, got = fit_units(make, count, budget, 0, len(words), tol)
    return RulerItem(task, length, index, prompt, refs, s["gen"], got + s["gen"], {"keys": keys, "units": n})


def vt_item(length: int, index: int, count: Count, tol: float = 0.05) -> RulerItem:
    s = SPEC["vt"]
    rng = rng_for("vt", length, index)
    names, seen = [], set()
    while len(names) < s["hops"] + 1:
        nm = "".join(chr(65 + int(c)) for c in rng.integers(0, 26, 5))
        if nm not in seen:
            seen.add(nm)
            names.append(nm)
    value = _number(rng, 5)
    chain = [f"VAR {names[0]} = {value}"] + [f"VAR {names[i + 1]} = VAR {names[i]} " for i in range(s["hops"])]
    fracs = sorted(rng.random(len(chain)).tolist())
    def make(n):
        ctx = _insert_at_fractions([NOISE] * n, chain, fracs, "\n")
        return VT_TEMPLATE.format(context=ctx, value=value) + VT_ANSWER.format(n=len(names), value=value)
    budget = length - s["gen"]
    prompt, n, got = fit_units(make, count, budget, 1, max(8, budget), tol)
    return RulerItem("vt", length, index, prompt, names, s["gen"], got + s["gen"], {"value": value, "units": n})


def make_item(task: str, length: int, index: int, count: Count, pool: list[str] | None = None) -> RulerItem:
    if task not in SPEC:
        raise ValueError(f"unknown task {task!r}: one of {TASKS}")
    return vt_item(length, index, count) if SPEC[task]["kind"] == "vt" else niah_item(task, length, index, count, pool)


# ------------------------------------------------------------------------------------------------------------ scoring

def postprocess_pred(text: str) -> str:
    return re.sub(r"[\x00-\x1f]", "\n", text.strip()).strip()


def recall(pred: str, refs: list[str]) -> float:
    """RULER's string_match_all: the share of reference strings found, lower-cased, in the generation."""
    p = postprocess_pred(pred).lower()
    return sum(r.lower() in p for r in refs) / len(refs)


def all_found(pred: str, refs: list[str]) -> float:
    return float(recall(pred, refs) == 1.0)


def cell_key(task: str, length, metric: str) -> str:
    return f"ruler|{task}|{length}|{metric}"


def values_file(run: str, results: list[dict], code_sha: str = "local", excluded: list[str] | None = None) -> dict:
    """results: [{"task", "length", "id", "recall", "all_found"}]. Cells: per (task, length) recall (also under RULER's name
    string_match_all) and all_found for multi-reference tasks, per task over all lengths, and the task mean per length."""
    skip = set(excluded or ())
    rows = [r for r in results if r["id"] not in skip]
    cells: dict[str, float] = {}
    def mean(xs):
        return float(sum(xs) / len(xs))
    for task in sorted({r["task"] for r in rows}):
        of_task = [r for r in rows if r["task"] == task]
        for length in sorted({r["length"] for r in of_task}):
            sel = [r for r in of_task if r["length"] == length]
            cells[cell_key(task, length, "recall")] = cells[cell_key(task, length, "string_match_all")] = mean([r["recall"] for r in sel])
            if task in MULTI_REF:
                cells[cell_key(task, length, "all_found")] = mean([r["all_found"] for r in sel])
        cells[cell_key(task, "all", "recall")] = mean([r["recall"] for r in of_task])
    for length in sorted({r["length"] for r in rows}):
        per_task = [cells[cell_key(t, length, "recall")] for t in sorted({r["task"] for r in rows}) if cell_key(t, length, "recall") in cells]
        cells[cell_key("mean", length, "recall")] = mean(per_task)
    return {"run": run, "family": "ruler", "code_sha": code_sha, "cells": cells, "n_items": len(rows), "excluded": sorted(skip)}
