"""Synthetic recall probes scored teacher-forced.

Each probe is a token sequence with an answer span; the score is exact match of the argmax at every answer position
and the mean CE there. Kinds: "needle" (one key -> value pair in filler, queried at the end), "multikey" (n pairs, one
queried), "copy" (repeat a random string after a separator), "twohop" (a -> b and b -> c stated apart, query a),
"pathcopy" (several marked strings in filler, one asked by its key and copied whole), "mf_chain" / "mf_concat" (k facts
at controlled depths and an answer that needs all of them: a chain of k pointers written out, or k values in the
order the question lists them; the answer alternates fact pieces and scaffold pieces and `multifact_metrics` reads
the fact tokens) and "transcode" (a string shown in a raw or an escaped form, asked for in the other one)
(reference: ced/eval/probes.py, ced/eval/probe_gen.py, ced/eval/probe_gen_multifact.py:1-60,
ced/eval/probe_gen_transcode.py:1-40, ced/eval/probe_gen_copy.py; builders there work on tokenizer text, these on
token ids so they run on any vocabulary).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..data.synthetic import counter_generator
from .span_bpb import token_cross_entropy

PROBE_KINDS = ("needle", "multikey", "copy", "twohop", "pathcopy", "mf_chain", "mf_concat", "transcode")
LAYOUTS = ("spread", "front", "back")        # where the facts of a multi-fact item sit; cycles with the item index
ESC, N_SPECIAL = 5, 4                          # transcode: the escape token; content ids 8 .. 8 + N_SPECIAL - 1 need escaping


@dataclass
class Probe:
    kind: str
    ids: list[int]
    answer_start: int        # index in ids of the first answer token
    answer_len: int
    pieces: tuple = ()       # multi-fact answers: (length, is_fact) per piece, in answer order
    group: str = ""          # multi-fact: the layout; transcode: the direction
    candidates: tuple = ()   # multiple choice (text-level depth items): one single-token continuation per candidate
    gold: int = -1           # index of the right candidate


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
    if kind in ("mf_chain", "mf_concat"):
        return _multifact(kind, g, body, length, index, key_len, value_len, k=max(2, min(n_keys, 8)))
    if kind == "transcode":
        return _transcode(g, vocab, length, seed, index)
    if kind == "pathcopy":
        value_len = min(32, max(value_len, length // (4 * n_keys)))
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


def layout_depths(layout: str, k: int, g) -> list[float]:
    """Depths in [0, 1) of the k facts: "spread" = the centres of k equal parts, "front" = inside 5-30 % (the far end
    from the query), "back" = inside 70-95 %; which fact sits at which depth is a random permutation
    (reference: ced/eval/probe_gen_multifact.py `layout_depths`)."""
    if layout == "spread":
        d = [(i + 0.5) / k for i in range(k)]
    else:
        lo = 0.05 if layout == "front" else 0.70
        d = [lo + 0.25 * (i + 0.5) / k for i in range(k)]
    perm = torch.randperm(k, generator=g).tolist()
    return [d[j] for j in perm]


def _multifact(kind, g, body, length, index, key_len, value_len, k):
    layout = LAYOUTS[index % len(LAYOUTS)]
    if kind == "mf_chain":        # name_0 -> name_1 -> ... -> name_k; the answer writes the chain out
        names = [body(key_len) for _ in range(k + 1)]
        facts = [[1] + names[i] + [2] + names[i + 1] for i in range(k)]
        query = [3] + names[0] + [2]
        pieces = []
        for i in range(1, k + 1):
            pieces.append((names[i], True))
            if i < k:
                pieces.append(([4, 1] + names[i] + [2], False))
    else:                          # k names with k values, asked in the order of the question's list
        names, values = [body(key_len) for _ in range(k)], [body(value_len) for _ in range(k)]
        facts = [[1] + n + [2] + v for n, v in zip(names, values)]
        order = torch.randperm(k, generator=g).tolist()
        query = [3] + [t for j in order for t in names[j] + [4]] + [1] + names[order[0]] + [2]
        pieces = []
        for r, j in enumerate(order):
            pieces.append((values[j], True))
            if r + 1 < k:
                pieces.append(([4, 1] + names[order[r + 1]] + [2], False))
    answer = [t for p, _ in pieces for t in p]
    hay = max(0, length - sum(len(f) for f in facts) - len(query) - len(answer))
    at = sorted(zip((int(d * hay) for d in layout_depths(layout, k, g)), range(k)))
    ids, prev = [], 0
    for c, i in at:
        ids += body(c - prev) + facts[i]
        prev = c
    ids += body(hay - prev) + query
    return Probe(kind, ids + answer, len(ids), len(answer), tuple((len(p), f) for p, f in pieces), layout)


def escape_ids(raw: list[int]) -> list[int]:
    """The escaped form: a special token s becomes the pair (ESC, s + N_SPECIAL); every other token stands."""
    out = []
    for t in raw:
        out += [ESC, t + N_SPECIAL] if 8 <= t < 8 + N_SPECIAL else [t]
    return out


def _transcode(g, vocab, length, seed, index):
    """Both directions over the same content: index even = escaped shown, raw asked ("esc2raw"); odd = the reverse.
    The content holds at least one special token, so the answer never occurs in the context as it stands."""
    n = max(4, min(48, length // 6))
    base = index // 2
    gc = counter_generator(seed, base, 7100)           # the content: one stream per base, shared by its two directions
    raw = torch.randint(8 + 2 * N_SPECIAL, vocab, (n,), generator=gc).tolist()
    n_sp = max(1, n // 6)
    for p in torch.randperm(n, generator=gc)[:n_sp].tolist():
        raw[p] = 8 + int(torch.randint(0, N_SPECIAL, (1,), generator=gc))
    esc = escape_ids(raw)
    direction = "esc2raw" if index % 2 == 0 else "raw2esc"
    src, ans = (esc, raw) if direction == "esc2raw" else (raw, esc)
    mark = 6 if direction == "esc2raw" else 7          # which form the query asks for
    fill = max(0, length - len(src) - len(ans) - 4)
    cut = int(torch.randint(0, fill + 1, (1,), generator=g))
    filler = lambda m: torch.randint(8 + 2 * N_SPECIAL, vocab, (m,), generator=g).tolist()
    ids = filler(cut) + [1] + src + [2] + filler(fill - cut) + [3, mark]
    return Probe("transcode", ids + ans, len(ids), len(ans), (), direction)


def copy_floor(p: Probe) -> dict:
    """Transcode floor: the source as it stands taken as the answer; token_acc = share of answer positions with the
    same token, lcs_share = token LCS / answer tokens (reference: ced/eval/probe_gen_transcode.py:34-37)."""
    a = p.ids.index(1) + 1
    src, ans = p.ids[a:p.ids.index(2, a)], p.ids[p.answer_start:p.answer_start + p.answer_len]
    same = sum(1 for x, y in zip(src, ans) if x == y)
    row = [0] * (len(ans) + 1)
    for x in src:
        prev = 0
        for j, y in enumerate(ans, 1):
            cur = row[j]
            row[j] = prev + 1 if x == y else max(row[j], row[j - 1])
            prev = cur
    return {"exact": src == ans, "token_acc": same / len(ans), "lcs_share": row[-1] / len(ans)}


def multifact_metrics(p: Probe, ok: list[bool], nats: list[float]) -> dict:
    """From the per-token record of one item's answer (ok = the token is the argmax, nats = -log p): exact (every token
    of every fact), fact_acc, nats per fact token, first_ok / first_nats (the first token of each fact), rest_nats,
    exact_all (scaffold included), hop_ok per fact in answer order (reference: ced/eval/probe_gen_multifact.py:22-31)."""
    at, facts = 0, []
    for n, is_fact in p.pieces:
        if is_fact:
            facts.append((at, n))
        at += n
    fact_ok = [all(ok[a:a + n]) for a, n in facts]
    ftok = [i for a, n in facts for i in range(a, a + n)]
    rest = [i for a, n in facts for i in range(a + 1, a + n)]
    return {
        "exact": all(fact_ok), "fact_acc": sum(fact_ok) / len(facts), "nats": sum(nats[i] for i in ftok) / len(ftok),
        "first_ok": sum(ok[a] for a, _ in facts) / len(facts), "first_nats": sum(nats[a] for a, _ in facts) / len(facts),
        "rest_nats": sum(nats[i] for i in rest) / max(len(rest), 1), "exact_all": all(ok),
        "hop_ok": [float(x) for x in fact_ok], "group": p.group,
    }


@torch.no_grad()
def score_probes(model, probes: list[Probe], batch_size: int = 8, autocast_dtype=None, keep_tokens: bool = False, passes: int | None = None) -> dict:
    """Teacher-forced: exact = every answer token is the argmax given the true prefix. keep_tokens: every item also
    carries its per-token record ("ok", "nats") and its index, what `eval/probe_analysis.py` reads. passes: the pass count
    of a model with a looped middle or a second pass (None: the model's own evaluation count)."""
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
        extra = {} if passes is None else {"T": passes}
        if model.cfg.arch == "looped_ced":        # the answer's positions run the decoder (their next token is generated); every slot is kept
            dec = torch.zeros_like(tok, dtype=torch.bool)
            for b, p in enumerate(group):
                dec[b, p.answer_start - 1: p.answer_start - 1 + p.answer_len] = True
            extra.update(dec_mask=dec.to(dev), capacity=width)
        with torch.autocast(dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
            logits = model(tok.to(dev), doc.to(dev), **extra).logits
        ce = token_cross_entropy(logits, tgt.to(dev)).cpu()
        top = logits.argmax(-1).cpu()
        for b, p in enumerate(group):
            sl = slice(p.answer_start - 1, p.answer_start - 1 + p.answer_len)
            hit = bool((top[b, sl] == tgt[b, sl]).all())
            ce_sum += float(ce[b, sl].sum())
            n_tok += p.answer_len
            item = {"kind": p.kind, "exact": hit, "ce": float(ce[b, sl].mean())}
            if p.group:
                item["group"] = p.group
            if p.pieces:         # the headline of a multi-fact item counts the fact tokens only
                item.update(multifact_metrics(p, (top[b, sl] == tgt[b, sl]).tolist(), ce[b, sl].tolist()), exact_all=hit)
            if p.candidates:     # multiple choice among single-token continuations: the candidate with the largest logit
                cand = torch.tensor([c[0] for c in p.candidates])
                item["choice_ok"] = int(logits[b, p.answer_start - 1].float().cpu()[cand].argmax()) == p.gold
            if keep_tokens:
                item.update(index=s + b, ok=(top[b, sl] == tgt[b, sl]).tolist(), nats=ce[b, sl].tolist())
            exact += int(item["exact"])
            per.append(item)
    return {"exact": exact / max(len(probes), 1), "ce": ce_sum / max(n_tok, 1), "n": len(probes), "items": per}
