"""Text-level probe items: a context string and the continuation a model has to produce, built from held-out documents.

`eval/probes.py` builds its probes on token ids of any vocabulary; the items here are TEXT, so one set can be tokenized
for several tokenizers and read by people. Eight probes:

  uuid_needle   a haystack of held-out documents of total length T with one sentence "The access code for <name> is
                <uuid>." placed at the sentence start nearest a depth fraction; the question repeats the form and the
                answer is " <uuid>".
  multikey      the same with n such sentences (distinct names and values) at random depths; one is asked.
  path_copy     an index of K lines "class <Name> -> <path>" whose paths share a prefix and differ in one directory (a
                K x 1 x 1 grid) or are near-duplicates one directory, stem or digit apart (g x s x d grids); the question
                is "class <Name> ->" and the answer " <path>".
  depth         Python assignments inside `def main():` forming C chains of h + 1 lines (one asked, the others
                distractors) between filler statements; the question is "    assert <var> == " and the answer the digit
                the chain ends in, scored over the ten digits. The asked literal's rank among the literal lines cycles
                with the item index, so no position heuristic beats 1 / C.
  mf_chain      k pointer sentences "The supervisor of N0 is N1." ... at controlled depths; the answer writes the whole
                chain out, so every fact has to be retrieved.
  mf_concat     k sentences "The access code for Ni is Ci." and a question listing the names in another order; the
                answer gives the codes in the question's order.
  vt            variable tracking: two chains of assignments "VAR <B> = VAR <A>." scattered over the haystack; the answer lists
                the variables that hold one chain's number, in order.
  twohop        a link fact and a value fact per chain; the question asks for the value behind the link without naming
                the bridge, with matched controls (one hop, the link alone, a link to nowhere, links moved one chain on).

An item is a pure function of (seed, probe, cell, index), the document pool and the length measure `count` (a callable
from text to a token count: the build script passes the largest count over its tokenizers, the tests a byte count).
Content (names, values, depths) and haystack (which documents, in which order) come from two separate random streams.
Names are drawn from a synthetic list and checked to be absent from the haystack. Answers begin with a space after a
letter or ">" (or are a single digit), so context and answer tokenize separately as they do together under a
byte-level BPE split pattern; the build script checks that per tokenizer.
Multi-fact answers alternate fact pieces and scaffold pieces, recorded in `meta["pieces"]`.
Reference: ced/eval/probe_gen.py (needles, path_copy, depth), ced/eval/probe_gen_multifact.py (mf_*),
ced/eval/probe_gen_distance.py (needles at a fixed token distance: `needle_at_distance` here).
"""

from __future__ import annotations

import bisect
import keyword
import re
import uuid
from dataclasses import asdict, dataclass, field
from typing import Callable

import numpy as np

SEED = 0x5EED_2026
ROW = 8192
LENGTHS = (ROW, 2 * ROW, 4 * ROW, 8 * ROW)
DEPTHS = (0.1, 0.3, 0.5, 0.7, 0.9)
MULTIKEY_COUNTS = (4, 16)
PATH_CELLS = ((4, (4, 1, 1)), (8, (8, 1, 1)), (16, (16, 1, 1)), (12, (2, 3, 4)))
PATH_PREFIX_DEPTH = {"shallow": 2, "deep": 6}
HOPS = tuple(range(9))
CHAINS = 3
DEPTH_LINES = 32
FACT_COUNTS = (2, 4, 8)
LAYOUTS = ("spread", "front", "back")
LAYOUT_SPAN = {"spread": (0.0, 1.0), "front": (0.05, 0.30), "back": (0.70, 0.95)}
LENGTH_SLACK = 0.03          # an item's total length lies in [(1 - slack) T, T]
JOIN = "\n\n"
PROBES = ("uuid_needle", "multikey", "path_copy", "depth", "mf_chain", "mf_concat", "twohop", "vt")
_CODE = {p: i for i, p in enumerate(PROBES)}


@dataclass
class TextItem:
    id: str
    probe: str
    cell: dict                       # what the scores are averaged over (length; n_keys; k, grid, prefix; hops; ...)
    context: str
    answer: str
    candidates: list | None = None   # multiple choice: the continuations, `gold` the index of the right one
    gold: int | None = None
    group: dict = field(default_factory=dict)      # a finer split inside a cell (the needle's depth, the layout)
    meta: dict = field(default_factory=dict)

    def to_json(self) -> dict:
        return {k: v for k, v in asdict(self).items() if v is not None}

    @classmethod
    def from_json(cls, d: dict) -> "TextItem":
        return cls(**d)


def cell_name(cell: dict) -> str:
    return ",".join(f"{k}={cell[k]}" for k in sorted(cell))


def stream(probe: str, cell: tuple, index: int, purpose: int, seed: int = SEED) -> np.random.Generator:
    """One generator per (probe, cell, item, purpose); purpose 0: content, 1: haystack."""
    words = [seed, _CODE[probe]] + [int(round(x * 1000)) if isinstance(x, float) else int(x) for x in cell] + [index, purpose]
    return np.random.default_rng(np.random.SeedSequence(words))


# ------------------------------------------------------------------------------------------------------------ vocabularies
# Names are assembled from syllables: pronounceable, capitalised, and rare enough in running text that a handful of
# candidates always holds some that the haystack does not.
_ONSET = ("Bal", "Cor", "Dav", "El", "Fen", "Gar", "Hal", "Is", "Jor", "Kel", "Lor", "Mar", "Nev", "Or", "Per", "Quin", "Ros", "Sel", "Tam", "Ul", "Ver", "Wil", "Yar", "Zel")
_CODA = ("adan", "beth", "cia", "dric", "elle", "fiel", "gard", "hild", "ian", "jana", "kin", "lene", "mund", "nor", "olf", "pha", "rik", "sten", "tha", "uin", "vyn", "wen")
_FAMILY_A = ("Ash", "Black", "Cold", "Dun", "East", "Fair", "Grey", "High", "Iron", "Long", "Mill", "North", "Oak", "Pen", "Red", "Stone", "Thorn", "Under", "West", "Wind")
_FAMILY_B = ("bourne", "brook", "combe", "croft", "dale", "field", "ford", "gate", "holm", "hurst", "leigh", "mere", "ridge", "shaw", "stead", "thwaite", "wick", "wood", "worth")
GIVEN = [a + b for a in _ONSET for b in _CODA]
FAMILY = [a + b for a in _FAMILY_A for b in _FAMILY_B]
ROOTS = ("/srv", "/opt", "/var/lib", "/home/build", "/usr/local/share", "/mnt/work")
DIRS = ("app core api internal service worker jobs lib pkg src common shared utils auth storage billing search metrics events cache queue "
        "gateway admin reports sync tasks models views routes hooks tools").split()
STEMS = ("ledger_sync invoice_merge payment_batch refund_queue account_audit token_refresh session_store order_import stock_export "
         "rate_limit mail_digest index_rebuild quota_check lease_renew shard_move").split()
_TINT = "Amber Azure Brisk Cedar Cobalt Crimson Dusky Ember Gilded Hollow Ivory Jade Lunar Mossy Nimble Opal Pale Quiet Russet Silver Tawny Umber Vivid".split()
_BEAST = "Badger Condor Falcon Heron Ibex Jackal Kestrel Lynx Marten Newt Osprey Puffin Quail Raven Stoat Tern Urchin Vole Wren Yak".split()
CLASSES = [a + b for a in _TINT for b in _BEAST]
_LETTERS = "abcdefghijklmnopqrstuvwxyz"
VARS = [a + b for a in _LETTERS for b in _LETTERS if not keyword.iskeyword(a + b) and a + b not in {"as", "if", "in", "is", "or", "id", "io", "os", "re"}]
FILLER = ("None", "True", "False", "[]", "{}", '""')          # right-hand sides of filler statements: never a digit
HEXDIGITS = "0123456789abcdef"
_SENTENCE = re.compile(r"[.!?][\"')\]]? +(?=[A-Z\"'(])|\n(?=\S)")


def fresh_uuid(rng: np.random.Generator) -> str:
    return str(uuid.UUID(bytes=rng.bytes(16), version=4))


def full_names(rng: np.random.Generator, n: int) -> list[str]:
    """n distinct "Given Family" names in a random order."""
    picks = rng.choice(len(GIVEN) * len(FAMILY), size=n, replace=False)
    return [f"{GIVEN[p // len(FAMILY)]} {FAMILY[p % len(FAMILY)]}" for p in picks]


def unseen_names(candidates: list[str], text: str, n: int) -> list[str]:
    """The first n candidates neither of whose words occurs in `text`."""
    out = []
    for name in candidates:
        if all(part not in text for part in name.split()):
            out.append(name)
            if len(out) == n:
                return out
    raise ValueError(f"only {len(out)} of {n} names are absent from the haystack")


# ---------------------------------------------------------------------------------------------------------------- haystack

def usable(text: str) -> bool:
    """A document that can serve as haystack: some length, mostly ordinary characters, no uuid-looking strings."""
    if len(text) < 400 or re.search(r"[0-9a-f]{8}-[0-9a-f]{4}-", text):
        return False
    ordinary = sum(c.isalnum() or c.isspace() or c in ".,;:!?'\"()-" for c in text)
    return ordinary >= 0.9 * len(text)


class DocPool:
    """Held-out documents for haystacks (never training data). `take(rng)` yields them in a random order without repeats."""

    def __init__(self, docs: list[str]):
        self.docs = [d.strip() for d in docs if usable(d)]
        if not self.docs:
            raise ValueError("no usable haystack document")

    def take(self, rng: np.random.Generator):
        for i in rng.permutation(len(self.docs)):
            yield self.docs[i]

    def describe(self) -> dict:
        return {"documents": len(self.docs), "characters": sum(map(len, self.docs))}


def sentence_starts(text: str) -> list[int]:
    return [0] + [m.end() for m in _SENTENCE.finditer(text)]


def nearest_start(starts: list[int], text_len: int, fraction: float) -> int:
    want = fraction * text_len
    i = bisect.bisect_left(starts, want)
    best = min(starts[max(i - 1, 0):i + 1] or [0], key=lambda s: abs(s - want))
    return best


def plant(text: str, sentences: list[tuple[float, str]]) -> tuple[str, list[int]]:
    """`text` with every (fraction, sentence) placed at the sentence start nearest its fraction; returns the new text and
    each sentence's character offset in it (in the order given). Two sentences never share a start: a taken start moves
    the later one to the next free start."""
    starts = sentence_starts(text)
    taken, where = set(), []
    for frac, _ in sentences:
        s = nearest_start(starts, len(text), frac)
        k = starts.index(s)
        while starts[k] in taken and k + 1 < len(starts):
            k += 1
        taken.add(starts[k])
        where.append(starts[k])
    order = sorted(range(len(sentences)), key=lambda i: where[i])
    out, offsets, cursor, shift = [], [0] * len(sentences), 0, 0
    for i in order:
        out.append(text[cursor:where[i]])
        offsets[i] = where[i] + shift
        piece = sentences[i][1] + " "
        out.append(piece)
        shift += len(piece)
        cursor = where[i]
    out.append(text[cursor:])
    return "".join(out), offsets


def haystack_to_length(pool: DocPool, rng: np.random.Generator, total: int, count: Callable[[str], int], finish: Callable[[str], tuple[str, str]]) -> tuple[str, str, dict]:
    """Documents joined until the finished item (`finish(haystack)` -> (context, answer)) is at least `total` long under
    `count`, then cut back sentence by sentence (bisection over the last document's sentence starts) until the item's
    length lies in [(1 - LENGTH_SLACK) total, total]. Returns (context, answer, {"documents", "length"})."""
    def measure(hay: str) -> int:
        c, a = finish(hay)
        return count(c + a)

    docs, approx = [], 0
    for doc in pool.take(rng):
        docs.append(doc)
        approx += count(doc) + 2                   # a running estimate; the finished item is measured only near the target
        if approx >= total and measure(JOIN.join(docs)) >= total:
            break
    else:
        raise ValueError(f"the pool is too small for a haystack of {total}")
    head = JOIN.join(docs[:-1])
    last = docs[-1]
    cuts = sentence_starts(last)[1:] + [len(last)]
    lo, hi = 0, len(cuts) - 1                      # the largest cut whose item still fits
    fit = None
    while lo <= hi:
        mid = (lo + hi) // 2
        hay = (head + JOIN if head else "") + last[:cuts[mid]].rstrip()
        n = measure(hay)
        if n <= total:
            fit, lo = (hay, n), mid + 1
        else:
            hi = mid - 1
    if fit is None:
        if not head:
            raise ValueError("a single sentence exceeds the requested length")
        fit = (head, measure(head))
    hay, n = fit
    if n < (1 - LENGTH_SLACK) * total:
        raise ValueError(f"could not reach {total}: best {n} (a very long sentence at the cut)")
    c, a = finish(hay)
    return c, a, {"documents": len(docs), "length": n}


# ----------------------------------------------------------------------------------------------------------------- needles

def needle_sentence(name: str, value: str) -> str:
    return f"The access code for {name} is {value}."


def needle_question(name: str) -> str:
    return f"What is the access code for {name}? The access code for {name} is"


def _needles(probe: str, cell: tuple, pool: DocPool, count, length: int, fractions: list[float], index: int, asked: int, seed: int):
    content, hay_rng = stream(probe, cell, index, 0, seed), stream(probe, cell, index, 1, seed)
    values = [fresh_uuid(content) for _ in fractions]
    candidates = full_names(content, 4 * len(fractions) + 8)
    state = {}

    def finish(hay: str):
        names = unseen_names(candidates, hay, len(fractions))
        body, offsets = plant(hay, [(f, needle_sentence(n, v)) for f, n, v in zip(fractions, names, values)])
        state.update(names=names, offsets=offsets, body_len=len(body))
        return body + JOIN + needle_question(names[asked]), " " + values[asked]

    context, answer, info = haystack_to_length(pool, hay_rng, length, count, finish)
    info.update(name=state["names"][asked], asked=asked,
                needle_offsets=[o / max(state["body_len"], 1) for o in state["offsets"]], question_chars=len(needle_question(state["names"][asked])))
    return context, answer, info


def uuid_needle(pool: DocPool, count, length: int, depth: float, index: int, seed: int = SEED) -> TextItem:
    context, answer, info = _needles("uuid_needle", (length, depth), pool, count, length, [depth], index, 0, seed)
    return TextItem(f"uuid_needle/len={length}/depth={depth}/{index:04d}", "uuid_needle", {"length": length}, context, answer,
                    group={"depth": depth}, meta=info)


def multikey(pool: DocPool, count, length: int, n_keys: int, index: int, seed: int = SEED) -> TextItem:
    content = stream("multikey", (length, n_keys, 7), index, 0, seed)
    fractions = sorted(float(x) for x in content.uniform(0.03, 0.97, size=n_keys))
    asked = int(content.integers(n_keys))
    context, answer, info = _needles("multikey", (length, n_keys), pool, count, length, fractions, index, asked, seed)
    return TextItem(f"multikey/len={length}/n={n_keys}/{index:04d}", "multikey", {"length": length, "n_keys": n_keys}, context, answer,
                    group={"asked_depth": round(fractions[asked], 1)}, meta=info)


def needle_at_distance(pool: DocPool, count, length: int, distance: int, index: int, n_keys: int = 1, tol: int = 64, seed: int = SEED) -> TextItem:
    """A needle item whose (asked) needle sits `distance` tokens before the end of the context instead of at a depth
    fraction: the depth is searched (bisection on the fraction, the measured distance is monotone in it) until the
    distance from the needle's value to the context's end is within `tol` of the request. The documents, name and value
    of item `index` are the same at every distance of a length."""
    if distance + 512 > (1 - LENGTH_SLACK) * length:
        raise ValueError(f"distance {distance} does not fit a length of {length}")
    probe = "uuid_needle" if n_keys == 1 else "multikey"
    lo, hi, best = 0.0, 1.0, None
    for _ in range(24):
        frac = (lo + hi) / 2
        content = stream(probe, (length, n_keys, 11), index, 0, seed)
        others = sorted(float(x) for x in content.uniform(0.03, 0.97, size=n_keys - 1))
        fractions = others + [frac]
        cell = (length, n_keys, 11)
        context, answer, info = _needles(probe, cell, pool, count, length, fractions, index, n_keys - 1, seed)
        at = context.rfind(answer.strip())
        measured = count(context[at:])
        if best is None or abs(measured - distance) < abs(best[0] - distance):
            best = (measured, context, answer, info, frac)
        if abs(measured - distance) <= tol:
            break
        if measured > distance:
            lo = frac          # the needle is too far from the end: move it deeper
        else:
            hi = frac
    measured, context, answer, info, frac = best
    if abs(measured - distance) > tol:
        raise ValueError(f"no sentence start within {tol} tokens of distance {distance} (closest {measured})")
    info.update(needle_distance=measured)
    return TextItem(f"{probe}/len={length}/dist={distance}/{index:04d}", probe, {"length": length, "distance": distance, **({"n_keys": n_keys} if n_keys > 1 else {})},
                    context, answer, group={"depth": round(1 - distance / length, 3), "distance": distance}, meta=info)


# --------------------------------------------------------------------------------------------------------------- path_copy

def path_copy(k: int, grid: tuple[int, int, int], prefix: str, index: int, seed: int = SEED) -> TextItem:
    """K lines "class <Name> -> <root>/<shared prefix>/<dir>/<stem>_<digit>.py" in a random order, their (dir, stem, digit)
    K distinct points of a g x s x d grid (all of it when K = g s d; a sample of near-duplicates otherwise); one is asked."""
    g, s, d = grid
    if g * s * d < k:
        raise ValueError(f"grid {grid} does not hold {k} paths")
    rng = stream("path_copy", (k, g, s, d, PATH_PREFIX_DEPTH[prefix]), index, 0, seed)
    root = ROOTS[int(rng.integers(len(ROOTS)))]
    shared = [DIRS[i] for i in rng.choice(len(DIRS), size=PATH_PREFIX_DEPTH[prefix], replace=False)]
    free = [w for w in DIRS if w not in shared]
    groups = [free[i] for i in rng.choice(len(free), size=g, replace=False)]
    stems = [STEMS[i] for i in rng.choice(len(STEMS), size=s, replace=False)]
    digits = [int(x) for x in rng.choice(9, size=d, replace=False) + 1]
    points = [(gr, st, dg) for gr in groups for st in stems for dg in digits]
    paths = [f"{root}/{'/'.join(shared)}/{gr}/{st}_{dg}.py" for gr, st, dg in (points[i] for i in rng.choice(len(points), size=k, replace=False))]
    names = [CLASSES[i] for i in rng.choice(len(CLASSES), size=k, replace=False)]
    order = rng.permutation(k)
    lines = [f"class {names[i]} -> {paths[i]}" for i in order]
    asked = int(rng.integers(k))
    context = "# module index\n" + "\n".join(lines) + f"\n\nclass {names[asked]} ->"
    return TextItem(f"path_copy/k={k}/grid={g}x{s}x{d}/{prefix}/{index:04d}", "path_copy", {"k": k, "grid": f"{g}x{s}x{d}", "prefix": prefix},
                    context, " " + paths[asked], meta={"line": int(list(order).index(asked)), "name": names[asked]})


# ------------------------------------------------------------------------------------------------------------------- depth

def depth(hops: int, index: int, chains: int = CHAINS, lines: int = DEPTH_LINES, seed: int = SEED) -> TextItem:
    """`chains` chains of hops + 1 assignments (a literal digit, then each variable copied into the next) shuffled with filler
    inside `def main():`, each chain's lines in order; the question asserts the last variable of chain 0."""
    need = chains * (hops + 1)
    if need > lines:
        raise ValueError(f"{chains} chains of {hops + 1} lines do not fit {lines} statements")
    rng = stream("depth", (hops, chains, lines), index, 0, seed)
    names = [VARS[i] for i in rng.choice(len(VARS), size=need + (lines - need), replace=False)]
    digits = [int(x) for x in rng.choice(10, size=chains, replace=False)]
    chain_vars = [names[c * (hops + 1):(c + 1) * (hops + 1)] for c in range(chains)]
    filler_vars = names[need:]
    stmts = []                                   # (chain or -1, text)
    for c in range(chains):
        stmts.append((c, f"{chain_vars[c][0]} = {digits[c]}"))
        stmts += [(c, f"{chain_vars[c][j]} = {chain_vars[c][j - 1]}") for j in range(1, hops + 1)]
    fill = [(-1, f"{v} = {FILLER[int(rng.integers(len(FILLER)))]}") for v in filler_vars]
    # a random interleave that keeps each chain's order: shuffle slot labels, then deal every chain's lines into its slots
    labels = [c for c, _ in stmts] + [-1] * len(fill)
    rng.shuffle(labels)
    # the asked literal's rank among the literal lines cycles with the index: rotate chain labels until it holds
    want_rank = index % chains
    firsts = [labels.index(c) for c in range(chains)]
    by_pos = sorted(range(chains), key=lambda c: firsts[c])
    swap = by_pos[want_rank]
    labels = [({0: swap, swap: 0}.get(x, x)) for x in labels]
    queues = {c: [t for cc, t in stmts if cc == c] for c in range(chains)}
    queues[-1] = [t for _, t in fill]
    body = [queues[x].pop(0) for x in labels]
    asked = chain_vars[0][hops]
    context = "def main():\n" + "\n".join("    " + s for s in body) + f"\n    assert {asked} == "
    cands = [str(x) for x in range(10)]
    return TextItem(f"depth/hops={hops}/{index:04d}", "depth", {"hops": hops}, context, str(digits[0]), candidates=cands, gold=digits[0],
                    meta={"assigned": digits, "rank": want_rank, "lines_after_asked": len(body) - 1 - max(i for i, s in enumerate(body) if s.startswith(asked + " "))})


# -------------------------------------------------------------------------------------------------------------- multi-fact

def layout_fractions(layout: str, k: int) -> list[float]:
    """Centres of k equal parts of the layout's span of the haystack, increasing."""
    lo, hi = LAYOUT_SPAN[layout]
    return [lo + (hi - lo) * (i + 0.5) / k for i in range(k)]


def _hexcode(rng, first: str) -> str:
    return first + "".join(HEXDIGITS[int(i)] for i in rng.integers(16, size=7))


def multifact(probe: str, pool: DocPool, count, length: int, k: int, index: int, seed: int = SEED) -> TextItem:
    if probe not in ("mf_chain", "mf_concat"):
        raise ValueError(probe)
    layout = LAYOUTS[index % len(LAYOUTS)]
    content, hay_rng = stream(probe, (length, k), index, 0, seed), stream(probe, (length, k), index, 1, seed)
    fractions = layout_fractions(layout, k)
    place = [int(i) for i in content.permutation(k)]          # fact i sits at fractions[place[i]]
    candidates = full_names(content, 4 * k + 12)
    firsts = [HEXDIGITS[int(i)] for i in content.choice(16, size=k, replace=False)] if probe == "mf_concat" else []
    codes = [_hexcode(content, f) for f in firsts]
    ask_order = [int(i) for i in content.permutation(k)]
    state = {}

    def finish(hay: str):
        if probe == "mf_chain":
            names = unseen_names(candidates, hay, k + 1)
            facts = [f"The supervisor of {names[i]} is {names[i + 1]}." for i in range(k)]
            question = f"Who is the supervisor of {names[0]}? The supervisor of {names[0]} is"
            pieces = []
            for i in range(k):
                pieces.append([" " + names[i + 1], True])
                if i + 1 < k:
                    pieces.append([f". The supervisor of {names[i + 1]} is", False])
        else:
            names = unseen_names(candidates, hay, k)
            facts = [f"The access code for {names[i]} is {codes[i]}." for i in range(k)]
            asked = [names[i] for i in ask_order]
            listing = ", ".join(asked[:-1]) + " and " + asked[-1]
            question = f"What are the access codes for {listing}, in that order? The access code for {asked[0]} is"
            pieces = []
            for j, i in enumerate(ask_order):
                pieces.append([" " + codes[i], True])
                if j + 1 < k:
                    pieces.append([f". The access code for {names[ask_order[j + 1]]} is", False])
        body, offsets = plant(hay, [(fractions[place[i]], facts[i]) for i in range(k)])
        state.update(pieces=pieces, question=question, offsets=[o / max(len(body), 1) for o in offsets])
        return body + JOIN + question, "".join(p for p, _ in pieces)

    context, answer, info = haystack_to_length(pool, hay_rng, length, count, finish)
    info.update(pieces=state["pieces"], fact_offsets=state["offsets"], question_chars=len(state["question"]))
    return TextItem(f"{probe}/len={length}/k={k}/{index:04d}", probe, {"length": length, "k": k}, context, answer, group={"layout": layout}, meta=info)


# -------------------------------------------------------------------------------------------------------- variable tracking
# Two chains of VT_HOPS + 1 variables assigned at random places of the haystack, each chain's statements in order:
# "VAR <A> = <number>." then "VAR <B> = VAR <A>." and so on; the chains hold different 5-digit numbers and the variables
# are random 5-letter upper-case names absent from the haystack. The question asks which variables hold one chain's
# number; the answer lists them in the chain's order. Copying every VAR name in order gives eight names, not four: the
# second chain is what makes it tracking. Cell: length. Reference: ced/eval/report_pcr_gen.py (pcr_vt; RULER's VT).
VT_HOPS, VT_CHAINS = 3, 2


def _var_names(rng, n: int, text: str) -> list[str]:
    out = []
    while len(out) < n:
        name = "".join(chr(65 + int(i)) for i in rng.integers(26, size=5))
        if name not in text and name not in out:
            out.append(name)
    return out


def var_track(pool: DocPool, count, length: int, index: int, seed: int = SEED) -> TextItem:
    content, hay_rng = stream("vt", (length,), index, 0, seed), stream("vt", (length,), index, 1, seed)
    numbers = [str(int(x)) for x in content.choice(90000, size=VT_CHAINS, replace=False) + 10000]
    per = VT_HOPS + 1
    fractions = sorted(float(x) for x in content.uniform(0.03, 0.97, size=VT_CHAINS * per))
    owner = [c for c in range(VT_CHAINS) for _ in range(per)]
    content.shuffle(owner)                                     # which chain each place belongs to; a chain fills its places in order
    name_seed = int(content.integers(1 << 31))
    state = {}

    def finish(hay: str):
        names = _var_names(np.random.default_rng(name_seed), VT_CHAINS * per, hay)       # the same candidates at every trial length
        chains = [names[c * per:(c + 1) * per] for c in range(VT_CHAINS)]
        step = [0] * VT_CHAINS
        planted = []
        for f, c in zip(fractions, owner):
            j = step[c]
            step[c] += 1
            rhs = numbers[c] if j == 0 else f"VAR {chains[c][j - 1]}"
            planted.append((f, f"VAR {chains[c][j]} = {rhs}."))
        body, _ = plant(hay, planted)
        q = f"Question: Which variables are assigned the value {numbers[0]}? Answer: The variables assigned the value {numbers[0]} are:"
        state.update(chains=chains, question=q)
        return body + JOIN + q, " " + " ".join(chains[0])

    context, answer, info = haystack_to_length(pool, hay_rng, length, count, finish)
    info.update(chains=state["chains"], numbers=numbers, question_chars=len(state["question"]))
    return TextItem(f"vt/len={length}/{index:04d}", "vt", {"length": length}, context, answer, meta=info)


# ----------------------------------------------------------------------------------------------------------------- two-hop
# A latent two-hop lookup: the answer is reached only by reading one fact (the link, "The supervisor of <head> is
# <bridge>.") and using what it says as the key of a second one (the value, "The access code for <bridge> is <code>.");
# nothing is written between the question and the answer, so the first hop stays unwritten (mf_chain writes it out).
# D + 1 chains of that form are planted; chain 0 is asked. One base item gives five scored variants:
#   twohop    "What is the access code for the supervisor of <head>? ..." -> " <code>"
#   onehop    the value fact asked directly by its key (what the same answer costs without a hop)
#   link      the link fact alone -> " <bridge>"
#   shuffled  the two-hop question on a context whose asked link names a stranger with no code: the ceiling of guessing
#   swapped   every link moved one chain on: each fact where it stood, every bridge still named twice, so whatever does
#             not read the asked link scores as on twohop and a model that follows it gives another chain's code.
#             twohop - swapped is the share of answers that follow the link.
# Cell: length, gap between a chain's two facts ("adjacent", "near": about NEAR_TOKENS apart, "far": half the haystack),
# distractor chains D, value "word" (one common word: the hop has to happen inside one token) or "uuid" (letter-first).
# Group: the order of the two facts in the text, "AB" or "BA". Order and the asked chain's rank among the chains cycle
# with the item index, so "the first code" is right 1 / (D + 1) of the time. Reference: ced/eval/probe_gen_twohop.py.
TWOHOP_VARIANTS = ("twohop", "onehop", "link", "shuffled", "swapped")
GAPS = ("adjacent", "near", "far")
NEAR_TOKENS = 256
CODE_WORDS = ("anchor bridge candle dragon engine forest garden hammer island jacket kitchen ladder marble needle orange pencil quartz "
              "ribbon saddle tunnel umbrella velvet window yellow zipper").split()          # distinct first letters


def _letter_uuid(rng, first: str) -> str:
    u = fresh_uuid(rng)
    return first + u[1:]


def twohop(pool: DocPool, count, length: int, gap: str, distractors: int, value: str, index: int, seed: int = SEED) -> list[TextItem]:
    """The five variants of base item `index` of the cell (same haystack, names, codes and places)."""
    if gap not in GAPS or value not in ("word", "uuid") or distractors < 1:
        raise ValueError(f"two-hop cell gap {gap!r} of {GAPS}, value {value!r} of ('word', 'uuid'), distractors {distractors} >= 1")
    n = distractors + 1
    cell = (length, GAPS.index(gap), distractors, value == "uuid")
    content, hay_rng = stream("twohop", cell, index, 0, seed), stream("twohop", cell, index, 1, seed)
    order = "AB" if index % 2 == 0 else "BA"
    rank = (index // 2) % n                                   # the asked chain's place among the chains, in text order
    candidates = full_names(content, 8 * n + 16)
    if value == "word":
        codes = [CODE_WORDS[i] for i in content.choice(len(CODE_WORDS), size=n, replace=False)]
    else:
        codes = [_letter_uuid(content, "abcdef"[i]) for i in content.choice(6, size=n, replace=False)]
    span = 0.45 if gap == "far" else 0.9
    slots = [0.04 + span * (i + 0.5) / n for i in range(n)]    # anchors of the chains, in text order
    others = [int(i) for i in content.permutation(n - 1) + 1]
    at = others[:rank] + [0] + others[rank:]                    # at[j]: which chain sits at slot j
    slot_of = {c: j for j, c in enumerate(at)}
    state = {}

    def sentences(heads, bridges, linked):
        """linked[c]: the name chain c's link fact gives."""
        link = [f"The supervisor of {heads[c]} is {linked[c]}." for c in range(n)]
        val = [f"The access code for {bridges[c]} is {codes[c]}." for c in range(n)]
        return link, val

    def render(hay, heads, bridges, linked, question):
        link, val = sentences(heads, bridges, linked)
        per_tok = len(hay) / max(count(hay), 1)
        shift = {"adjacent": 0.0, "near": NEAR_TOKENS * per_tok / max(len(hay), 1), "far": 0.5}[gap]
        planted = []
        for c in range(n):
            first, second = (link[c], val[c]) if order == "AB" else (val[c], link[c])
            f = slots[slot_of[c]]
            if gap == "adjacent":
                planted.append((f, first + " " + second))
            else:
                planted += [(f, first), (min(f + shift, 0.98), second)]
        body, _ = plant(hay, planted)
        return body + JOIN + question

    def finish(hay: str):
        names = unseen_names(candidates, hay, 2 * n + 1)
        heads, bridges, stranger = names[:n], names[n:2 * n], names[2 * n]
        state.update(hay=hay, heads=heads, bridges=bridges, stranger=stranger)
        q = f"What is the access code for the supervisor of {heads[0]}? The access code for the supervisor of {heads[0]} is"
        return render(hay, heads, bridges, bridges, q), " " + codes[0]

    _, _, info = haystack_to_length(pool, hay_rng, length, count, finish)
    hay, heads, bridges, stranger = state["hay"], state["heads"], state["bridges"], state["stranger"]
    two = f"What is the access code for the supervisor of {heads[0]}? The access code for the supervisor of {heads[0]} is"
    one = f"What is the access code for {bridges[0]}? The access code for {bridges[0]} is"
    lnk = f"Who is the supervisor of {heads[0]}? The supervisor of {heads[0]} is"
    moved = [bridges[(c + 1) % n] for c in range(n)]
    forms = {
        "twohop": (bridges, two, " " + codes[0]),
        "onehop": (bridges, one, " " + codes[0]),
        "link": (bridges, lnk, " " + bridges[0]),
        "shuffled": ([stranger] + bridges[1:], two, " " + codes[0]),
        "swapped": (moved, two, " " + codes[0]),
    }
    out = []
    for variant, (linked, question, answer) in forms.items():
        context = render(hay, heads, bridges, linked, question)
        meta = dict(info, codes=codes, rank=rank, head=heads[0], bridge=bridges[0], question_chars=len(question),
                    followed=" " + codes[1 % n] if variant == "swapped" else None)
        out.append(TextItem(f"twohop/len={length}/gap={gap}/d={distractors}/{value}/{variant}/{index:04d}", "twohop",
                            {"length": length, "gap": gap, "distractors": distractors, "value": value, "variant": variant},
                            context, answer, group={"order": order}, meta=meta))
    return out


def twohop_summary(scores: dict[str, list[float]]) -> dict:
    """From per-variant lists of exact-match scores over the SAME base items (paired): the means, the share of answers
    that follow the link (twohop - swapped) and what the hop costs (onehop - twohop)."""
    mean = {v: sum(x) / max(len(x), 1) for v, x in scores.items()}
    out = dict(mean)
    if "twohop" in mean and "swapped" in mean:
        out["follows_link"] = mean["twohop"] - mean["swapped"]
    if "twohop" in mean and "onehop" in mean:
        out["hop_cost"] = mean["onehop"] - mean["twohop"]
    return out


def question_text(item: TextItem) -> str:
    """The question of a needle or multi-fact item: the context from the question's first word to its end."""
    n = item.meta.get("question_chars")
    if n is None:
        raise ValueError(f"probe {item.probe!r} has no question")
    return item.context[-n:]


# ------------------------------------------------------------------------------------------------------------------- sets

def build_cells(probe: str, per_cell: int, pool: DocPool | None = None, count=None, lengths=LENGTHS, seed: int = SEED) -> list[TextItem]:
    """Every cell of a probe's standard grid, `per_cell` items each (needles: per depth)."""
    out = []
    if probe == "uuid_needle":
        for T in lengths:
            for d in DEPTHS:
                out += [uuid_needle(pool, count, T, d, i, seed) for i in range(per_cell)]
    elif probe == "multikey":
        for T in lengths:
            for n in MULTIKEY_COUNTS:
                out += [multikey(pool, count, T, n, i, seed) for i in range(per_cell)]
    elif probe == "path_copy":
        for k, grid in PATH_CELLS:
            for prefix in PATH_PREFIX_DEPTH:
                out += [path_copy(k, grid, prefix, i, seed) for i in range(per_cell)]
    elif probe == "depth":
        for h in HOPS:
            out += [depth(h, i, seed=seed) for i in range(per_cell)]
    elif probe in ("mf_chain", "mf_concat"):
        for T in lengths:
            for k in FACT_COUNTS:
                out += [multifact(probe, pool, count, T, k, i, seed) for i in range(per_cell)]
    elif probe == "vt":
        for T in lengths:
            out += [var_track(pool, count, T, i, seed) for i in range(per_cell)]
    elif probe == "twohop":
        for T in lengths:
            for gap in GAPS:
                for d in (1, 3):
                    for value in ("word", "uuid"):
                        for i in range(per_cell):
                            out += twohop(pool, count, T, gap, d, value, i, seed)
    else:
        raise ValueError(f"unknown probe {probe!r}: one of {PROBES}")
    return out


# ---------------------------------------------------------------------------------------------------------------- encoding

def clean_boundary(encode: Callable[[str], list[int]], context: str, answer: str) -> bool:
    """Tokenizing context and answer apart gives the tokens of the whole."""
    return encode(context + answer) == encode(context) + encode(answer)


def occurrences(hay: list[int], needle: list[int]) -> int:
    n, m = len(hay), len(needle)
    return sum(1 for i in range(n - m + 1) if hay[i] == needle[0] and hay[i:i + m] == needle) if m else 0


def encode_item(item: TextItem, encode: Callable[[str], list[int]]) -> dict:
    """The stored form scored by `eval/probes.py`: ids (context + answer), the answer's span, multi-fact pieces as token
    lengths, multiple-choice candidates as token lists, and the per-item checks the build reports."""
    ctx, ans = encode(item.context), encode(item.answer)
    rec = {"id": item.id, "kind": item.probe, "cell": cell_name(item.cell), "group": cell_name(item.group) if item.group else "",
           "ids": ctx + ans, "answer_start": len(ctx), "answer_len": len(ans), "length": len(ctx) + len(ans),
           "checks": {"clean_boundary": clean_boundary(encode, item.context, item.answer)}}
    if item.probe in ("uuid_needle", "multikey", "path_copy"):
        rec["checks"]["answer_once"] = occurrences(ctx, ans) == 1
    if item.probe == "twohop" and "codes" in item.meta:      # the first answer token decides: the codes start with different tokens
        firsts = [encode(" " + c)[0] for c in item.meta["codes"]]
        rec["checks"]["distinct_first_tokens"] = len(set(firsts)) == len(firsts)
    if item.candidates is not None:
        cands = [encode(c) for c in item.candidates]
        rec.update(candidates=cands, gold=item.gold)
        rec["checks"]["single_token_candidates"] = all(len(c) == 1 for c in cands)
    if "pieces" in item.meta:
        lens = [(len(encode(text)), bool(is_fact)) for text, is_fact in item.meta["pieces"]]
        rec["pieces"] = tuple(lens)
        rec["checks"]["pieces_add_up"] = sum(n for n, _ in lens) == len(ans)
    if "question_chars" in item.meta:
        rec["question_tokens"] = len(encode(question_text(item)))
    return rec
