"""Long-context grounded-QA probe: items in gold / swap pairs that differ only in whether the context holds what the
answer needs.

One item is ids = [context][question][a_1 .. a_m], the three tokenized apart and concatenated. The model reads ids[:-1]
and predicts ids[1:]; the m positions that predict answer tokens are the scored ones. Batches are left-padded: the
padding is a document of its own (doc 0, the item doc 1), and the model isolates documents exactly, so a padded row
scores like the item alone; left padding puts every row's answer in the same last columns and ends every prompt in
the same column, so greedy generation runs batched.

Per item: answer bpb (bits of the answer tokens / UTF-8 bytes of the answer string), exact match (greedy decoding
from the prompt reproduces the answer's ids; gold items) and tf_greedy (the teacher-forced argmax equals the answer
at every answer position: for a fixed answer length the same event as exact match, so a disagreement means the cached
path and the teacher-forced path differ, and the summary counts them). Per (kind, bin) and per source / depth inside
a bin: mean answer bpb with its standard error, exact match, and the context gain bpb(gold) - bpb(swap) over pairs
with its paired SE; negative = the gold context lowered the answer's loss (reference: ced/eval/qa_probe.py:1-58,
378-460; its looped-model scoring at decoder positions is not built, this is its control-model path).

    python -m gdn_hybrid_architecture_ideas_b200.eval.qa_probe --checkpoint RUN --probe DIR_OR_JSONL --out a.json
    python -m gdn_hybrid_architecture_ideas_b200.eval.qa_probe --compare a.json b.json
"""

from __future__ import annotations

import argparse
import hashlib
import json
import math
from collections import defaultdict
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Callable, Iterable

import torch

from .generate import generate_greedy_batched
from .span_bpb import TokenizedDoc, token_cross_entropy
from .tokenized import byte_tokenize

Tokenize = Callable[[str], TokenizedDoc]
KINDS = ("copy", "kv", "passage_qa")
GROUP_FIELDS = ("source", "depth_target")


@dataclass
class ProbeItem:
    kind: str
    context: str
    question: str
    answer: str
    meta: dict = field(default_factory=dict)


@dataclass
class EncodedItem:
    item: ProbeItem
    ids: list[int]
    n_answer: int
    answer_bytes: int

    @property
    def prompt(self) -> list[int]:
        return self.ids[:len(self.ids) - self.n_answer]

    @property
    def fingerprint(self) -> str:
        """What was scored: two evaluations compare only on the same tokens."""
        return hashlib.sha256(json.dumps([self.ids, self.n_answer]).encode()).hexdigest()[:16]


@dataclass
class ItemScore:
    id: str
    pair_id: str
    kind: str
    bin: str
    condition: str
    group: dict
    n_tokens: int
    n_answer: int
    answer_nats: float
    bpb: float
    tf_greedy: bool
    exact_match: bool | None
    fingerprint: str


def load_items(path, kinds: Iterable[str] = KINDS, max_pairs_per_bin: int | None = None) -> list[ProbeItem]:
    """Items of one JSON-lines file, or of <dir>/<kind>.jsonl; max_pairs_per_bin keeps the first pairs of every
    (kind, bin) in file order."""
    path, kinds = Path(path), tuple(kinds)
    files = [path] if path.is_file() else [path / f"{k}.jsonl" for k in kinds if (path / f"{k}.jsonl").exists()]
    items, seen = [], defaultdict(list)
    for f in files:
        for line in f.read_text(encoding="utf-8").splitlines():
            if not line.strip():
                continue
            r = json.loads(line)
            item = ProbeItem(r["kind"], r["context"], r["question"], r["answer"], r.get("meta", {}))
            if item.kind not in kinds:
                continue
            if max_pairs_per_bin is not None:
                pairs, pair = seen[(item.kind, item.meta.get("bin"))], item.meta.get("pair_id", item.meta.get("id"))
                if pair not in pairs:
                    if len(pairs) >= max_pairs_per_bin:
                        continue
                    pairs.append(pair)
            items.append(item)
    return items


def encode_item(item: ProbeItem, tokenize: Tokenize = byte_tokenize) -> EncodedItem:
    c, q, a = tokenize(item.context), tokenize(item.question), tokenize(item.answer)
    if not len(a.ids) or not len(c.ids) + len(q.ids):
        raise ValueError(f"item {item.meta.get('id')}: an empty answer or an empty prompt")
    return EncodedItem(item, list(c.ids) + list(q.ids) + list(a.ids), len(a.ids), max(1, len(item.answer.encode("utf-8"))))


def left_pad(rows: list[list[int]], pad_id: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """(tokens, doc ids): rows right-aligned, the padding document 0 and the row document 1."""
    width = max(len(r) for r in rows)
    tok = torch.full((len(rows), width), pad_id, dtype=torch.long)
    doc = torch.ones(len(rows), width, dtype=torch.long)
    for b, r in enumerate(rows):
        tok[b, width - len(r):] = torch.tensor(r, dtype=torch.long)
        doc[b, :width - len(r)] = 0
    return tok, doc


def batches_by_length(lengths: list[int], batch_size: int, max_batch_tokens: int | None = None) -> list[list[int]]:
    """Indices grouped in order of length, at most batch_size rows and (rows x longest row) <= max_batch_tokens."""
    order, out, cur = sorted(range(len(lengths)), key=lambda i: lengths[i]), [], []
    for i in order:
        if cur and (len(cur) >= batch_size or (max_batch_tokens and (len(cur) + 1) * lengths[i] > max_batch_tokens)):
            out.append(cur)
            cur = []
        cur.append(i)
    if cur:
        out.append(cur)
    return out


@torch.no_grad()
def score_batch(model, encoded: list[EncodedItem], pad_id: int = 0, autocast_dtype=None):
    """Teacher-forced: per item (answer nats, every answer token is the argmax)."""
    dev = next(model.parameters()).device
    tok, doc = left_pad([e.ids for e in encoded], pad_id)
    with torch.autocast(dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
        logits = model(tok[:, :-1].to(dev), doc[:, :-1].to(dev)).logits
    tgt = tok[:, 1:].to(dev)
    ce = token_cross_entropy(logits, tgt).cpu()
    hit = (logits.argmax(-1) == tgt).cpu()
    out = []
    for b, e in enumerate(encoded):
        out.append((float(ce[b, -e.n_answer:].sum()), bool(hit[b, -e.n_answer:].all())))
    return out


def score_items(model, encoded: list[EncodedItem], batch_size: int = 8, max_batch_tokens: int | None = None,
                exact_match: str = "generate", pad_id: int = 0, autocast_dtype=None) -> list[ItemScore]:
    """exact_match: "generate" (greedy decoding on the caches, gold items), "teacher_forced" (tf_greedy stands in, no
    extra cost) or "none"."""
    if exact_match not in ("generate", "teacher_forced", "none"):
        raise ValueError(f"exact_match {exact_match!r}: generate | teacher_forced | none")
    was_training = model.training
    model.eval()
    scores: list[ItemScore | None] = [None] * len(encoded)
    for idx in batches_by_length([len(e.ids) for e in encoded], batch_size, max_batch_tokens):
        group = [encoded[i] for i in idx]
        tf = score_batch(model, group, pad_id, autocast_dtype)
        em: list[bool | None] = [None] * len(group)
        gold = [k for k, e in enumerate(group) if e.item.meta.get("condition", "gold") != "swap"]
        if exact_match == "teacher_forced":
            for k in gold:
                em[k] = tf[k][1]
        elif exact_match == "generate" and gold:
            new = max(group[k].n_answer for k in gold)
            gen = generate_greedy_batched(model, [group[k].prompt for k in gold], new, pad_id=pad_id, autocast_dtype=autocast_dtype)
            for k, g in zip(gold, gen):
                e = group[k]
                em[k] = list(g[:e.n_answer]) == e.ids[-e.n_answer:]
        for k, (i, e) in enumerate(zip(idx, group)):
            m = e.item.meta
            nats = tf[k][0]
            scores[i] = ItemScore(
                id=str(m.get("id", i)), pair_id=str(m.get("pair_id", m.get("id", i))), kind=e.item.kind, bin=str(m.get("bin", "all")),
                condition=m.get("condition", "gold"), group={f: m[f] for f in GROUP_FIELDS if f in m}, n_tokens=len(e.ids),
                n_answer=e.n_answer, answer_nats=nats, bpb=nats / math.log(2) / e.answer_bytes, tf_greedy=tf[k][1],
                exact_match=em[k], fingerprint=e.fingerprint)
    model.train(was_training)
    return scores


def mean_se(values: list[float]):
    """Mean and standard error (sample standard deviation / sqrt(n)); None where undefined."""
    n = len(values)
    if n == 0:
        return None, None
    mean = sum(values) / n
    if n == 1:
        return mean, None
    return mean, math.sqrt(sum((v - mean) ** 2 for v in values) / (n - 1) / n)


def group_keys(s: ItemScore) -> list[str]:
    return [f"{s.kind}/all", f"{s.kind}/{s.bin}"] + [f"{s.kind}/{s.bin}/{k}={v}" for k, v in sorted(s.group.items())]


def summarize(scores: list[ItemScore]) -> dict:
    groups = defaultdict(list)
    for s in scores:
        for key in group_keys(s):
            groups[key].append(s)
    out = {}
    for key in sorted(groups):
        gold = [s for s in groups[key] if s.condition != "swap"]
        swap = {s.pair_id: s for s in groups[key] if s.condition == "swap"}
        bpb, bpb_se = mean_se([s.bpb for s in gold])
        sw, sw_se = mean_se([s.bpb for s in swap.values()])
        gains = [s.bpb - swap[s.pair_id].bpb for s in gold if s.pair_id in swap]
        gain, gain_se = mean_se(gains)
        ems = [float(s.exact_match) for s in gold if s.exact_match is not None]
        em, em_se = mean_se(ems)
        out[key] = {
            "n": len(gold), "mean_tokens": sum(s.n_tokens for s in gold) / len(gold) if gold else None,
            "answer_bpb": bpb, "answer_bpb_se": bpb_se,
            "answer_nats_per_token": sum(s.answer_nats for s in gold) / sum(s.n_answer for s in gold) if gold else None,
            "exact_match": em, "exact_match_se": em_se, "n_exact_match": len(ems),
            "tf_greedy": mean_se([float(s.tf_greedy) for s in gold])[0],
            "em_tf_disagreements": sum(1 for s in gold if s.exact_match is not None and s.exact_match != s.tf_greedy),
            "swap_answer_bpb": sw, "swap_answer_bpb_se": sw_se, "n_pairs": len(gains), "context_gain": gain, "context_gain_se": gain_se,
        }
    return out


def paired_difference(a: list[ItemScore], b: list[ItemScore]) -> dict:
    """Per group, evaluation a minus evaluation b on the same items (matched by id; the scored tokens must be the same):
    answer bpb of gold items and the context gain."""
    by_id = {s.id: s for s in b}
    pairs = []
    for s in a:
        t = by_id.get(s.id)
        if t is None:
            continue
        if s.fingerprint != t.fingerprint:
            raise ValueError(f"item {s.id} was scored on different tokens in the two evaluations")
        pairs.append((s, t))
    swap_a = {s.pair_id: s for s, _ in pairs if s.condition == "swap"}
    swap_b = {t.pair_id: t for _, t in pairs if t.condition == "swap"}
    groups = defaultdict(list)
    for s, t in pairs:
        if s.condition != "swap":
            for key in group_keys(s):
                groups[key].append((s, t))
    out = {}
    for key in sorted(groups):
        d, d_se = mean_se([s.bpb - t.bpb for s, t in groups[key]])
        g, g_se = mean_se([(s.bpb - swap_a[s.pair_id].bpb) - (t.bpb - swap_b[t.pair_id].bpb)
                           for s, t in groups[key] if s.pair_id in swap_a and t.pair_id in swap_b])
        out[key] = {"n": len(groups[key]), "answer_bpb_diff": d, "answer_bpb_diff_se": d_se, "context_gain_diff": g,
                    "context_gain_diff_se": g_se}
    return out


def scores_to_json(scores: list[ItemScore]) -> list[dict]:
    return [asdict(s) for s in scores]


def scores_from_json(rows: list[dict]) -> list[ItemScore]:
    return [ItemScore(**r) for r in rows]


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--checkpoint")
    ap.add_argument("--probe")
    ap.add_argument("--tokenizer", default="bytes")
    ap.add_argument("--kinds", default=",".join(KINDS))
    ap.add_argument("--max-pairs-per-bin", type=int)
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--max-batch-tokens", type=int)
    ap.add_argument("--exact-match", default="generate")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--compare", nargs=2, metavar=("A", "B"))
    ap.add_argument("--out")
    a = ap.parse_args(argv)
    if a.compare:
        sa, sb = (scores_from_json(json.loads(Path(p).read_text())["items"]) for p in a.compare)
        result = {"paired_difference": paired_difference(sa, sb)}
    else:
        if not (a.checkpoint and a.probe):
            ap.error("--checkpoint and --probe, or --compare A B")
        from ..train import checkpoint as ckpt

        model, cfg, step = ckpt.load_model(a.checkpoint, a.device)
        if a.tokenizer == "bytes":
            tokenize = byte_tokenize
        else:
            from ..data.tokenizers import open_tokenizer

            tk = open_tokenizer(a.tokenizer)

            def tokenize(text: str) -> TokenizedDoc:
                ids = list(tk.encode(text))
                return TokenizedDoc(ids, [1] * len(ids))       # answer bytes come from the answer string itself
        items = load_items(a.probe, a.kinds.split(","), a.max_pairs_per_bin)
        enc = [encode_item(i, tokenize) for i in items]
        ac = torch.bfloat16 if a.device.startswith("cuda") else None
        scores = score_items(model, enc, a.batch_size, a.max_batch_tokens, a.exact_match, autocast_dtype=ac)
        result = {"step": step, "summary": summarize(scores), "items": scores_to_json(scores)}
        for key, v in result["summary"].items():
            print(f"{key:32s} n {v['n']:4d}  bpb {v['answer_bpb']}  em {v['exact_match']}  gain {v['context_gain']}")
    if a.out:
        Path(a.out).write_text(json.dumps(result, indent=1))
    return result


if __name__ == "__main__":
    main()
