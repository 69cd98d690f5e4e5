"""The exact-match readout inside training: a fixed sample of stored probe items scored along a run.

Off by default (`eval.readout_every` 0). Every `eval.readout_every` optimizer steps and at the run's last step the
sample is scored teacher-forced and one record goes to the run's metrics.jsonl:

    {"event": "readout", "step": s, "items": n, "seconds": ..., "exact": ..., "logp": ...,      pooled over the rows
     "rows": {"<set>/<cell>": {"n", "exact", "logp"}}, "sample": "<hash of the items>"}

A row's value is the mean over its items; the pooled value is the mean over the rows. `logp` is the mean log probability
of an answer token.

A model with a looped middle or a gated second pass is scored at one pass and at two on the same items, and the record is

    {"event": "readout", "step": s, "passes": [1, 2], "items": n, "exact": {"1": ..., "2": ...}, "logp": {"1": ..., "2": ...},
     "gap": {"mean": ..., "se": ...}, "gap_logp": {"mean": ..., "se": ...},                T = 2 minus T = 1, paired by item
     "rows": {"<set>/<cell>": {"n", "exact": [T1, T2], "logp": [T1, T2], "gap": {...}, "gap_logp": {...}}}, "sample": ...}

A row's gap is the mean of the per-item differences (exact as 0 / 1; logp as the item's mean log probability of an answer
token) with the standard error of that mean (sample deviation over sqrt(n); 0 for one item); the pooled gap is the mean
of the rows' gaps, its error the root of the rows' summed squared errors over the number of rows (rows hold different
items). Such a run is also scored at its `loop_switch_step`, the last step before the second pass joins.

The sample (`eval.readout_sets`): a list of [stored probe file, cells, items per cell]. The file is what
`scripts/build_probes.py` or `scripts/build_text_probes.py` wrote; `cells` is "*" or a list of kind names / cell names;
of each cell the FIRST `items per cell` items are taken, in file order: no random draw, so `scripts/eval_probes.py --set`
on a checkpoint scores a superset of the same items. The files are read when the run starts: a missing file, a cell with
too few items or a set built for a larger vocabulary stops the run there, before it trains.

Training is the same with the readout on or off: forward only, under no_grad, on the training model put in eval mode and
back; the RNG states are saved and put back; nothing is written to the model and the data stream is not touched. Its
time is not a step's time (it runs in fit() between two steps). An error while scoring is recorded as
{"event": "readout_failed"} and switches the readout off for the rest of the process: it never stops training. A step
whose record is already in metrics.jsonl is not scored again, so a resumed run that repeats steps writes no readout
twice. Only the lead rank scores (the sample is small).
Reference: ced/train/readout.py:84-434 (there the sample is scored on a scoring twin that shares the trainer's parameter
tensors; there is no compiled graph to protect here, so the training model itself is read).
"""

from __future__ import annotations

import hashlib
import json
import time
from pathlib import Path

import torch

from ..eval import probes
from . import periodic_eval

EVENT, FAILED = "readout", "readout_failed"


def parse_sets(value) -> list[dict]:
    out = []
    for entry in value or []:
        if not (isinstance(entry, (list, tuple)) and len(entry) == 3):
            raise ValueError(f"eval.readout_sets entry {entry!r}: [stored probe file, cells ('*' or a list of names), items per cell]")
        path, cells, per = entry
        if not (cells == "*" or (isinstance(cells, (list, tuple)) and cells and all(isinstance(c, str) for c in cells))):
            raise ValueError(f"eval.readout_sets entry {entry!r}: cells is '*' or a non-empty list of kind / cell names")
        if type(per) is not int or per < 1:
            raise ValueError(f"eval.readout_sets entry {entry!r}: items per cell is an integer >= 1")
        out.append({"path": Path(str(path)), "cells": cells if cells == "*" else list(cells), "per_cell": per})
    return out


def check_readout_config(cfg) -> None:
    e = cfg.eval
    if type(e.readout_every) is not int or e.readout_every < 0:
        raise ValueError(f"eval.readout_every {e.readout_every!r}: an integer >= 0 (0: off)")
    sets = parse_sets(e.readout_sets)
    if e.readout_every and not sets:
        raise ValueError("eval.readout_every is set and eval.readout_sets is empty: the readout has nothing to score")
    if type(e.readout_batch_tokens) is not int or e.readout_batch_tokens < 1:
        raise ValueError(f"eval.readout_batch_tokens {e.readout_batch_tokens!r}: a positive integer")


def readout_due(cfg, step: int, total_steps: int | None = None) -> bool:
    r = cfg.eval.readout_every
    last = cfg.steps if total_steps is None else total_steps
    return bool(r) and step > 0 and (step % r == 0 or step == last or step == cfg.loop_switch_step)


def passes_of(model) -> tuple:
    """(1, 2) for a model that can run a second pass (a looped middle, a gated second pass), (1,) otherwise."""
    looped = bool(model.cfg.loop.recur_layers) or model.cfg.loop.pass2_gate != "none"
    return (1, 2) if looped else (1,)


def paired_gap(later: list, first: list) -> dict:
    """The mean of the per-item differences later - first and the standard error of that mean."""
    d = torch.tensor(later, dtype=torch.float64) - torch.tensor(first, dtype=torch.float64)
    se = float(d.std(unbiased=True) / len(d) ** 0.5) if len(d) > 1 else 0.0
    return {"mean": round(float(d.mean()), 6), "se": round(se, 6)}


def pooled_gap(gaps: list) -> dict:
    n = max(len(gaps), 1)
    return {"mean": round(sum(g["mean"] for g in gaps) / n, 6), "se": round(sum(g["se"] ** 2 for g in gaps) ** 0.5 / n, 6)}


def load_sample(sets: list[dict], vocab_size: int) -> list[dict]:
    """[{"row": "<set>/<cell>", "probes": [Probe, ...]}] in the order of the entries and of the file."""
    rows = []
    for s in sets:
        if not s["path"].is_file():
            raise FileNotFoundError(f"eval.readout_sets: no file {s['path']}")
        blob = torch.load(s["path"], map_location="cpu", weights_only=False)
        if int(blob.get("vocab", 0)) > vocab_size:
            raise ValueError(f"{s['path']} was built for a vocabulary of {blob['vocab']}, the model has {vocab_size}")
        label = s["path"].parent.name + "/" + s["path"].stem if s["path"].parent.name else s["path"].stem
        cells: dict[str, list] = {}
        for p in blob["probes"]:
            cell = f"{p['kind']}@{p.get('cell', p.get('length'))}"
            if s["cells"] != "*" and p["kind"] not in s["cells"] and cell not in s["cells"] and str(p.get("cell")) not in s["cells"]:
                continue
            cells.setdefault(cell, [])
            if len(cells[cell]) < s["per_cell"]:
                cells[cell].append(probes.Probe(p["kind"], list(p["ids"]), p["answer_start"], p["answer_len"], tuple(map(tuple, p.get("pieces", ()))),
                                                p.get("group", ""), tuple(map(tuple, p.get("candidates", ()))), p.get("gold", -1)))
        if not cells:
            raise ValueError(f"{s['path']}: no item of cells {s['cells']}")
        short = {c: len(v) for c, v in cells.items() if len(v) < s["per_cell"]}
        if short:
            raise ValueError(f"{s['path']}: cells with fewer than {s['per_cell']} items: {short}")
        rows += [{"row": f"{label}/{c}", "probes": v} for c, v in cells.items()]
    return rows


def sample_hash(rows: list[dict]) -> str:
    h = hashlib.sha256()
    for r in rows:
        h.update(r["row"].encode())
        for p in r["probes"]:
            h.update(json.dumps([p.ids, p.answer_start, p.answer_len]).encode())
    return h.hexdigest()[:16]


def recorded_steps(run_dir) -> set:
    """Steps whose readout record is already in the run's metrics.jsonl."""
    path = Path(run_dir) / "metrics.jsonl" if run_dir is not None else None
    done = set()
    if path is not None and path.is_file():
        for line in path.read_text().splitlines():
            if f'"event": "{EVENT}"' in line:
                try:
                    done.add(int(json.loads(line)["step"]))
                except (ValueError, KeyError):
                    pass
    return done


def batches_by_tokens(items: list, budget: int) -> list[list]:
    """Consecutive items whose padded size (count x longest) stays within `budget` tokens; a single longer item goes alone."""
    out, cur, longest = [], [], 0
    for p in items:
        n = len(p.ids)
        if cur and (len(cur) + 1) * max(longest, n) > budget:
            out.append(cur)
            cur, longest = [], 0
        cur.append(p)
        longest = max(longest, n)
    if cur:
        out.append(cur)
    return out


def score_sample(model, rows: list[dict], batch_tokens: int, autocast_dtype=None, passes: tuple = (1,)) -> dict:
    """{row: {"n", "exact", "logp"}}; with two pass counts the values are [T1, T2] lists and the row carries its gaps."""
    table = {}
    for r in rows:
        per_pass = []
        for t in passes:
            hits, logps, nats, tokens = [], [], 0.0, 0
            for group in batches_by_tokens(r["probes"], batch_tokens):
                res = probes.score_probes(model, group, batch_size=len(group), autocast_dtype=autocast_dtype, passes=t if len(passes) > 1 else None)
                hits += [float(it["exact"]) for it in res["items"]]
                logps += [-it["ce"] for it in res["items"]]
                nats += sum(it["ce"] * p.answer_len for it, p in zip(res["items"], group))
                tokens += sum(p.answer_len for p in group)
            per_pass.append({"hits": hits, "logps": logps, "exact": round(sum(hits) / len(hits), 6), "logp": round(-nats / max(tokens, 1), 6)})
        n = len(r["probes"])
        if len(passes) == 1:
            table[r["row"]] = {"n": n, "exact": per_pass[0]["exact"], "logp": per_pass[0]["logp"]}
        else:
            table[r["row"]] = {"n": n, "exact": [p["exact"] for p in per_pass], "logp": [p["logp"] for p in per_pass],
                               "gap": paired_gap(per_pass[-1]["hits"], per_pass[0]["hits"]), "gap_logp": paired_gap(per_pass[-1]["logps"], per_pass[0]["logps"])}
    return table


class Readout:
    """State of a run's readout: the sample (read once), the steps already recorded, on / off."""

    def __init__(self, trainer):
        cfg = trainer.cfg
        check_readout_config(cfg)
        self.rows = load_sample(parse_sets(cfg.eval.readout_sets), cfg.model.vocab_size)
        self.sample = sample_hash(self.rows)
        self.done = recorded_steps(trainer.run_dir)
        self.off = False

    def run(self, trainer, log=print) -> dict | None:
        step = trainer.step
        if self.off or step in self.done or not trainer.lead:
            return None
        t0 = time.perf_counter()
        saved = periodic_eval.rng_states(trainer.device)
        was_training = trainer.model.training
        try:
            trainer.model.eval()
            ac = torch.bfloat16 if trainer.cfg.autocast == "bfloat16" and trainer.device.type == "cuda" else None
            passes = passes_of(trainer.model)
            table = score_sample(trainer.model, self.rows, trainer.cfg.eval.readout_batch_tokens, ac, passes)
        except Exception as err:          # never stops training
            self.off = True
            record = {"event": FAILED, "step": step, "error": f"{type(err).__name__}: {err}"[:500]}
            log(f"readout failed at step {step} and is switched off: {record['error']}")
            return record
        finally:
            trainer.model.train(was_training)
            periodic_eval.rng_restore(saved, trainer.device)
        self.done.add(step)
        n_rows = max(len(table), 1)
        head = {"event": EVENT, "step": step, "passes": list(passes), "items": sum(v["n"] for v in table.values()), "seconds": round(time.perf_counter() - t0, 3)}
        if len(passes) == 1:
            pooled = {k: round(sum(v[k] for v in table.values()) / n_rows, 6) for k in ("exact", "logp")}
        else:
            pooled = {k: {str(t): round(sum(v[k][i] for v in table.values()) / n_rows, 6) for i, t in enumerate(passes)} for k in ("exact", "logp")}
            pooled.update(gap=pooled_gap([v["gap"] for v in table.values()]), gap_logp=pooled_gap([v["gap_logp"] for v in table.values()]))
        return {**head, **pooled, "rows": table, "sample": self.sample}
