"""Multiple choice by likelihood: each (context, choice) pair is a document whose choice tokens are scored; the
predicted choice has the lowest summed CE (also reported normalised by bytes)
(reference: ced/eval/multiple_choice.py:36-240)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .span_bpb import TokenizedDoc, build_eval_rows, evaluate


@dataclass
class Item:
    context: list[int]
    choices: list[list[int]]
    answer: int
    choice_bytes: list[int] | None = None


def build_documents(items: list[Item]) -> tuple[list[TokenizedDoc], list[tuple[int, int]]]:
    """One document per (item, choice); index[d] = (item, choice)."""
    docs, index = [], []
    for i, it in enumerate(items):
        for c, ch in enumerate(it.choices):
            ids = it.context + ch
            scored = [False] * len(it.context) + [True] * len(ch)
            nb = (it.choice_bytes[c] if it.choice_bytes else len(ch))
            per = max(nb // max(len(ch), 1), 1)
            docs.append(TokenizedDoc(ids, [1] * len(it.context) + [per] * len(ch), scored))
            index.append((i, c))
    return docs, index


def score_items(model, items: list[Item], seq_len: int = 8192, batch_size: int = 1, autocast_dtype=None) -> dict:
    docs, index = build_documents(items)
    rows = build_eval_rows(docs, seq_len)
    ev = evaluate(model, rows, batch_size, autocast_dtype)
    correct = correct_norm = 0
    for i, it in enumerate(items):
        ds = [d for d, (ii, _) in enumerate(index) if ii == i]
        nats = torch.stack([ev.doc_nats[d] for d in ds])
        norm = nats / torch.stack([ev.doc_bytes[d] for d in ds]).clamp_min(1)
        correct += int(int(nats.argmin()) == it.answer)
        correct_norm += int(int(norm.argmin()) == it.answer)
    n = max(len(items), 1)
    return {"acc": correct / n, "acc_norm": correct_norm / n, "n": len(items), "skipped_docs": len(rows.skipped)}


# ---------------------------------------------------------------------------------------------------------- text-level tasks
# The small general regression set: ARC-Easy, PIQA, WinoGrande, BoolQ by log-likelihood and LAMBADA by target-word bits per
# byte and greedy accuracy. Prompt formats follow the common conventions of public evaluation harnesses. Every (item,
# choice) pair is one document, context tokens then choice tokens, packed WHOLE into rows (no document is cut, so every
# choice is scored with its full context); per task: acc (argmax of the summed log-likelihood), acc_norm (per UTF-8 byte of
# the choice), gold_bpb (bits per byte of the gold choice given its context) and for cloze tasks greedy_acc (every target
# token is the argmax). Rows can be scored on several ranks and joined (reference: ced/eval/multiple_choice.py:36-240).
import math

TASKS = ("arc-easy", "piqa", "boolq", "winogrande", "lambada")


@dataclass
class TextItem:
    task: str
    id: str
    contexts: list[str]          # one per choice (most tasks repeat the same context)
    choices: list[str]
    gold: int
    kind: str = "mc"             # "mc", or "cloze" (one choice: the target)


def format_item(task: str, row: dict, index: int) -> TextItem:
    """A dataset row of `task` (the field names of its public release) as contexts and continuations."""
    if task == "arc-easy":
        texts, labels = list(row["choices"]["text"]), list(row["choices"]["label"])
        ctx = f"Question: {row['question']}\nAnswer:"
        return TextItem(task, str(row.get("id", index)), [ctx] * len(texts), [" " + t for t in texts], labels.index(row["answerKey"]))
    if task == "piqa":
        ctx = f"Question: {row['goal']}\nAnswer:"
        return TextItem(task, str(index), [ctx, ctx], [" " + row["sol1"], " " + row["sol2"]], int(row["label"]))
    if task == "boolq":
        ctx = f"{row['passage']}\nQuestion: {row['question']}?\nAnswer:"
        return TextItem(task, str(index), [ctx, ctx], [" no", " yes"], int(bool(row["answer"])))
    if task == "winogrande":        # partial scoring: the option fills the blank in the context, the text after the blank is scored
        cut = row["sentence"].index("_")
        tail = " " + row["sentence"][cut + 1:].strip()
        head = row["sentence"][:cut]
        return TextItem(task, str(index), [head + row["option1"], head + row["option2"]], [tail, tail], int(row["answer"]) - 1)
    if task == "lambada":
        ctx, _, word = row["text"].rpartition(" ")
        return TextItem(task, str(index), [ctx], [" " + word], 0, kind="cloze")
    raise ValueError(f"unknown task {task!r}: one of {TASKS}")


def encode_items(items: list[TextItem], encode) -> tuple[list[TokenizedDoc], list[tuple[int, int, int]]]:
    """Documents for every (item, choice) and their (item index, choice index, choice bytes). encode: str -> token ids;
    a choice's bytes are spread over its tokens so that document sums give the choice's UTF-8 length."""
    docs, index = [], []
    for i, it in enumerate(items):
        for c, (ctx, ch) in enumerate(zip(it.contexts, it.choices)):
            a, b = list(encode(ctx)), list(encode(ch))
            if not a or not b:
                raise ValueError(f"{it.task} item {it.id}: an empty context or choice after tokenization")
            nb = len(ch.encode("utf-8"))
            per = [nb // len(b)] * len(b)
            per[-1] += nb - sum(per)
            docs.append(TokenizedDoc(a + b, [1] * len(a) + per, [False] * len(a) + [True] * len(b), f"{it.task}/{it.id}/{c}"))
            index.append((i, c, nb))
    return docs, index


@torch.no_grad()
def score_choice_rows(model, rows, batch_size: int = 1, autocast_dtype=None, row_indices=None) -> dict:
    """Per document: summed nats, bytes, tokens over its scored targets and whether every one of them is the argmax."""
    from .span_bpb import token_cross_entropy

    dev = next(model.parameters()).device
    was_training = model.training
    model.eval()
    n = rows.n_docs
    out = {k: torch.zeros(n, dtype=torch.float64) for k in ("nats", "bytes", "tokens", "misses")}
    idx = list(range(len(rows))) if row_indices is None else list(row_indices)
    for s in range(0, len(idx), batch_size):
        sel = torch.tensor(idx[s:s + batch_size], dtype=torch.long)
        tok, tgt, doc = (t[sel].to(dev) for t in (rows.tokens, rows.targets, rows.doc_ids))
        with torch.autocast(dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
            logits = model(tok, doc).logits
        ce = token_cross_entropy(logits, tgt).double().cpu()
        wrong = (logits.argmax(-1) != tgt).cpu()
        sc, di = rows.scored[sel], rows.doc_index[sel]
        keep = sc & (di >= 0)
        out["nats"].index_add_(0, di[keep], ce[keep])
        out["bytes"].index_add_(0, di[keep], rows.target_bytes[sel][keep].double())
        out["tokens"].index_add_(0, di[keep], torch.ones(int(keep.sum()), dtype=torch.float64))
        out["misses"].index_add_(0, di[keep], wrong[keep].double())
    model.train(was_training)
    return out


def join_choice_rows(parts: list[dict]) -> dict:
    """Sum of partial results over disjoint row sets."""
    return {k: sum(p[k] for p in parts) for k in parts[0]}


def choice_results(items: list[TextItem], index, scores: dict) -> tuple[dict, list[dict]]:
    """({task: {"n", "acc", "acc_norm", "gold_bpb"[, "greedy_acc"]}}, one record per item)."""
    by_item: dict[int, list[tuple[int, int, int]]] = {}
    for d, (i, c, nb) in enumerate(index):
        by_item.setdefault(i, []).append((c, d, nb))
    records, tasks = [], {}
    for i, it in enumerate(items):
        entries = sorted(by_item[i])
        nats = torch.stack([scores["nats"][d] for _, d, _ in entries])
        nbytes = torch.tensor([float(nb) for _, _, nb in entries], dtype=torch.float64)
        gold_d = entries[it.gold][1]
        rec = {"task": it.task, "id": it.id, "gold": it.gold, "pred": int(nats.argmin()), "pred_norm": int((nats / nbytes.clamp_min(1)).argmin()),
               "gold_nats": float(scores["nats"][gold_d]), "gold_bytes": float(nbytes[it.gold]), "greedy": bool(scores["misses"][gold_d] == 0)}
        records.append(rec)
        t = tasks.setdefault(it.task, {"n": 0, "acc": 0.0, "acc_norm": 0.0, "nats": 0.0, "bytes": 0.0, "greedy": 0.0, "cloze": it.kind == "cloze"})
        t["n"] += 1
        t["acc"] += rec["pred"] == it.gold
        t["acc_norm"] += rec["pred_norm"] == it.gold
        t["nats"] += rec["gold_nats"]
        t["bytes"] += rec["gold_bytes"]
        t["greedy"] += rec["greedy"]
    table = {}
    for name, t in tasks.items():
        row = {"n": t["n"], "acc": t["acc"] / t["n"], "acc_norm": t["acc_norm"] / t["n"], "gold_bpb": t["nats"] / (max(t["bytes"], 1.0) * math.log(2.0))}
        if t["cloze"]:
            row["greedy_acc"] = t["greedy"] / t["n"]
        table[name] = row
    return table, records


def score_text_items(model, items: list[TextItem], encode, seq_len: int = 8192, batch_size: int = 1, autocast_dtype=None) -> tuple[dict, list[dict]]:
    docs, index = encode_items(items, encode)
    rows = build_eval_rows(docs, seq_len)
    if rows.skipped:
        raise ValueError(f"{len(rows.skipped)} (item, choice) documents are longer than a row of {seq_len}")
    return choice_results(items, index, score_choice_rows(model, rows, batch_size, autocast_dtype))
