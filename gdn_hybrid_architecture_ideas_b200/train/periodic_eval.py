"""In-loop evaluation: every `eval.every_steps` steps the configured eval sets are scored and written to
`<run_dir>/eval/step_<n>.json`. An evaluation never changes training: the model's mode and every RNG stream
(Python, NumPy, torch CPU and device) are saved before and restored after, and nothing here touches the optimizer
(reference: ced/train/periodic_eval.py:116-217 eval sets, :480-497 RNG save/restore).

An eval set is a `.pt` file holding {"docs": [{"ids": [...], "byte_lens": [...], "scored": [...] or None}, ...]}, or
the literal "synthetic:<n>" (n held-out rows of the run's synthetic data, one byte per token), which needs no file.
"""

from __future__ import annotations

import json
import random
from pathlib import Path

import numpy as np
import torch

from ..eval import span_bpb
from ..eval.units import write_atomic
from .sharded_eval import evaluate_sharded

HELD_OUT_STEP = 1 << 40      # synthetic eval rows come from a step no run reaches


def rng_states(device: torch.device) -> dict:
    s = {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state()}
    if device.type == "cuda":
        s["cuda"] = torch.cuda.get_rng_state(device)
    return s


def rng_restore(saved: dict, device: torch.device) -> None:
    random.setstate(saved["python"])
    np.random.set_state(saved["numpy"])
    torch.set_rng_state(saved["torch"])
    if "cuda" in saved:
        torch.cuda.set_rng_state(saved["cuda"], device)


def load_set(spec: str, trainer) -> list[span_bpb.TokenizedDoc]:
    if spec.startswith("synthetic:"):
        n = int(spec.split(":", 1)[1])
        b = trainer.data.batch(HELD_OUT_STEP, 0, n)
        docs = []
        for r in range(n):
            ids = b.tokens[r].tolist() + [int(b.targets[r, -1])]
            docs.append(span_bpb.TokenizedDoc(ids, [1] * len(ids)))
        return docs
    blob = torch.load(spec, map_location="cpu", weights_only=False)
    return [span_bpb.TokenizedDoc(d["ids"], d["byte_lens"], d.get("scored"), d.get("name", "")) for d in blob["docs"]]


def due(cfg, step: int) -> bool:
    return cfg.eval.every_steps > 0 and bool(cfg.eval.sets) and step > 0 and step % cfg.eval.every_steps == 0


def run_eval_sets(trainer, periodic: bool = True) -> dict:
    """Scores every set of `eval.sets`; returns {name: {...}} (rank 0 writes the step file)."""
    cfg, device = trainer.cfg, trainer.device
    saved = rng_states(device)
    was_training = trainer.model.training
    results = {}
    try:
        seq_len = cfg.data.seq_len
        for name, spec in cfg.eval.sets.items():
            docs = load_set(spec, trainer)
            rows = span_bpb.build_eval_rows(docs, seq_len + 1)
            if periodic and cfg.eval.periodic_max_rows and rows.tokens.shape[0] > cfg.eval.periodic_max_rows:
                keep = slice(0, cfg.eval.periodic_max_rows)
                rows = span_bpb.EvalRows(*(getattr(rows, f)[keep] for f in ("tokens", "targets", "doc_ids", "scored", "target_bytes", "doc_index")),
                                         n_docs=rows.n_docs, skipped=rows.skipped)
            ac = torch.bfloat16 if cfg.autocast == "bfloat16" else None
            ev = evaluate_sharded(trainer.model, rows, trainer.dp, max(cfg.eval.batch_size, 1), autocast_dtype=ac)
            if ev is not None:
                results[name] = {"bpb": ev.bpb, "ce": ev.ce, "rows": int(rows.tokens.shape[0]), "tokens": int(ev.row_tokens.sum()),
                                 "bpb_se": span_bpb.bpb_se(ev, by="row")}
    finally:
        trainer.model.train(was_training)
        rng_restore(saved, device)
    lead = trainer.dp is None or trainer.dp.lead
    if lead and trainer.run_dir is not None:
        write_atomic(Path(trainer.run_dir) / "eval" / f"step_{trainer.step}.json", json.dumps({"step": trainer.step, "sets": results}, indent=1))
    return results
