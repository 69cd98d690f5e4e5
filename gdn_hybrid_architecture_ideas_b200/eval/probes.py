"""Synthetic recall probes scored teacher-forced.

Each probe is a token sequence with an answer span; the score is exact match of the argmax at every answer position
and the mean CE there. Kinds: "needle" (one key -> value pair in filler, queried at the end), "multikey" (n pairs, one
queried), "copy" (repeat a random string after a separator), "twohop" (a -> b and b -> c stated apart, query a)
(reference: ced/eval/probes.py, ced/eval/probe_gen.py; builders there work on tokenizer text, these on token ids so
they run on any vocabulary).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..data.synthetic import counter_generator
from .span_bpb import token_cross_entropy

PROBE_KINDS = ("needle", "multikey", "copy", "twohop")


@dataclass
class Probe:
    kind: str
    ids: list[int]
    answer_start: int        # index in ids of the first answer token
    answer_len: int


def _rand(g, lo, hi, n):
    return torch.randint(lo, hi, (n,), generator=g).tolist()


def build_probe(kind: str, vocab: int, length: int, seed: int, index: int, key_len: int = 4, value_len: int = 4, n_keys: int = 8) -> Probe:
    """Token layout: ids >= 8 are content; 1 = key marker, 2 = value marker, 3 = query marker, 4 = separator."""
    g = counter_generator(seed, index, PROBE_KINDS.index(kind) + 7000)
    body = lambda n: _rand(g, 8, vocab, n)
    if kind == "copy":
        n = min(length // 2 - 1, 64)
        s = body(n)
        ids = s + [4] + s
        return Probe(kind, ids, n + 1, n)
    pairs = [(body(key_len), body(value_len)) for _ in range(1 if kind == "needle" else n_keys)]
    facts = [[1] + k + [2] + v for k, v in pairs]
    q = int(torch.randint(0, len(pairs), (1,), generator=g))
    answer = pairs[q][1]
    query = [3] + pairs[q][0] + [2]
    if kind == "twohop":
        mid = body(key_len)
        facts = [[1] + pairs[q][0] + [2] + mid, [1] + mid + [2] + answer] + [f for i, f in enumerate(facts) if i != q]
    filler_total = max(0, length - sum(len(f) for f in facts) - len(query) - len(answer))
    cuts = sorted(_rand(g, 0, filler_total + 1, len(facts)))
    ids, prev = [], 0
    for f, c in zip(facts, cuts):
        ids += body(c - prev) + f
        prev = c
    ids += body(filler_total - prev) + query
    start = len(ids)
    return Probe(kind, ids + answer, start, len(answer))


@torch.no_grad()
def score_probes(model, probes: list[Probe], batch_size: int = 8, autocast_dtype=None) -> dict:
    """Teacher-forced: exact = every answer token is the argmax given the true prefix."""
    dev = next(model.parameters()).device
    exact, ce_sum, n_tok, per = 0, 0.0, 0, []
    for s in range(0, len(probes), batch_size):
        group = probes[s:s + batch_size]
        width = max(len(p.ids) for p in group) - 1
        tok = torch.zeros(len(group), width, dtype=torch.long)
        tgt = torch.zeros_like(tok)
        doc = torch.ones_like(tok)
        for b, p in enumerate(group):
            n = len(p.ids) - 1
            tok[b, :n], tgt[b, :n] = torch.tensor(p.ids[:-1]), torch.tensor(p.ids[1:])
            doc[b, :n] = 0
        with torch.autocast(dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
            logits = model(tok.to(dev), doc.to(dev)).logits
        ce = token_cross_entropy(logits, tgt.to(dev)).cpu()
        top = logits.argmax(-1).cpu()
        for b, p in enumerate(group):
            sl = slice(p.answer_start - 1, p.answer_start - 1 + p.answer_len)
            hit = bool((top[b, sl] == tgt[b, sl]).all())
            exact += int(hit)
            ce_sum += float(ce[b, sl].sum())
            n_tok += p.answer_len
            per.append({"kind": p.kind, "exact": hit, "ce": float(ce[b, sl].mean())})
    return {"exact": exact / max(len(probes), 1), "ce": ce_sum / max(n_tok, 1), "n": len(probes), "items": per}
