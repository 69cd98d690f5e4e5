"""Probes on synthetic code-like material: copying, line addressing, and moving a string across the JSON-escape boundary.

Nothing here reads a document: files, logs and records are assembled from fixed word lists and statement templates, so
a model cannot know their content and what it has to write is only in the context. Six probes.

Text level (`TextItem`, tokenized like the probes of `eval/probe_text.py`):

  copy            `$ cat <path>` views of synthetic modules, then either "repeat the body of <function>" (form repeat) or the
                  `old_str:` field of a str_replace call (form edit); the answer is the function body, verbatim with its
                  indentation. Cells: span length 8 / 32 / 128 nominal tokens x distance 1024 / 4096 / 8192 tokens from the
                  end of the source span to the instruction x variant plain / near_dup. near_dup puts a decoy function next
                  to the target whose body differs from it in one token of each of 1 / 2 / 3 lines (a digit, an operator,
                  a comparison or a boolean); `meta["diff_chars"]` marks where.
  line_edit       a numbered view (`cat -n`) of a module of 40 / 160 / 480 lines and a question naming one definition; the
                  answer is its line number: "Answer: line" + " <N>" (form number) or "$ sed -i '" + "<N>d" (form sed).
  line_edit_foil  the same contexts with other line numbers as the answer (neighbours at +-1, 2, 4, 8 and other definition
                  lines); `line_choice` turns the log-likelihoods of one question's gold and foil rows into the model's
                  choice and the distance |chosen - gold|.

Chat level (`ChatItem`: the pieces of a conversation in the chat format, a lead-in that is teacher-forced inside the last
text piece, and the answer; encoded piece by piece as the training shards are, `encode_chat_item`):

  copy_span       a source message (a tool result, or an earlier assistant message) holding K = 4 labelled snippets of one
                  type (code / path / ident / random) and length, filler turns (a `view` call with a synthetic file, a `run`
                  call with a log) until the target lies the wanted distance back, then a user message naming one label.
                  The reply opens with a fixed lead-in (a sentence and a code fence) and the answer follows in the same
                  piece. near_dup (code): one look-alike is the target with one token changed per 1 / 2 / 3 lines.
  edit_old        a file view as a tool result and a `str_replace` call for "lines A-B" (1 / 3 / 8 lines, unique in the file);
                  the model is forced up to the start of the old_str value and scored on the old text. Renderings of the
                  same content: json_num / json_plain (arguments as escaped JSON; view with or without line numbers) and
                  raw_num / raw_plain (the same frame with the old text unescaped: a diagnostic of the escaping alone).
  transcode       one multi-line string, two directions: esc2raw (a tool result holds it JSON-escaped, the user wants plain
                  text; lead-in and code fence as above) and raw2esc (a `cat` result shows it raw, the assistant saves it
                  with `write_file`; the answer is the escaped text between the quotes of the `content` argument). Cells:
                  dir x lines 1 / 3 / 8 / 20; group: kind code / text. Every base holds a character besides the line breaks
                  that needs escaping, so source and answer differ; the answer form occurs nowhere in the context.

Floors are stored per item (`floor`): for copy / copy_span a copier that picks one of the W (K) bodies at random (exact
1 / W, nats ln W, token accuracy from the bodies' positionwise agreement), for edit_old a random window of the same
number of lines, for line_edit a random definition line and a random line, for transcode the untranscoded source taken
as the answer (`transcode_floor`: exact 0, token accuracy and the LCS share against the gold tokens).

An item is a pure function of (seed, probe, cell, index, attempt) and the length measure `count`; the build script
retries with the next attempt when a per-tokenizer check fails (a token straddling the lead-in's end, a span that does
not tokenize alone as it does in place). Reference: ced/eval/probe_gen_ext.py:1-60, ced/eval/probe_gen_copy.py:1-75,
ced/eval/probe_gen_transcode.py:1-45 (there also the decoded-argument renderings of a second chat format, which is not
built here: `data/chat_format.py` renders the JSON form only).
"""

from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass, field
from typing import Callable

import numpy as np

from ..data import chat_format as CF
from .probe_text import SEED, TextItem, cell_name

PROBES = ("copy", "line_edit", "line_edit_foil", "copy_span", "edit_old", "transcode")
_CODE = {"copy": 101, "line_edit": 102, "line_edit_foil": 102, "copy_span": 103, "edit_old": 104, "transcode": 105}
COPY_LENGTHS, COPY_DISTANCES, COPY_VARIANTS, COPY_FORMS = (8, 32, 128), (1024, 4096, 8192), ("plain", "near_dup"), ("repeat", "edit")
COPY_DIFFS = {8: 1, 32: 2, 128: 3}
DIST_LO = 0.90
SPAN_TOL = 0.5
FILE_LINES = (40, 160, 480)
FOIL_OFFSETS = (-8, -4, -2, -1, 1, 2, 4, 8)
SPAN_TYPES, SPAN_SOURCES, K_SNIPPETS = ("code", "path", "ident", "random"), ("tool", "assistant"), 4
EDIT_LINES, EDIT_FILES = (1, 3, 8), (40, 200)
RENDERS = ("json_num", "json_plain", "raw_num", "raw_plain")
TC_DIRS, TC_LINES, TC_KINDS = ("esc2raw", "raw2esc"), (1, 3, 8, 20), ("code", "text")
LEADIN_COPY = "Here is the snippet, verbatim:\n```\n"
LEADIN_ESC2RAW = "Here is the decoded text:\n```\n"

VERBS = ("load parse merge flush sync build check clean close count drain emit fetch find group index join keep list map mark "
         "move open pack pick plan poll pull push read scan send sort split store swap tag trim wrap write").split()
NOUNS = ("batch block buffer cache chunk client cursor digest entry event field frame handle header index item job key layer "
         "ledger lock node offset page path queue record region report route row shard slot span stream table task token").split()
ROOTS = ("src", "lib", "app", "pkg", "core", "tools")
LEVELS = ("INFO", "WARN", "DEBUG")
OPERATORS = ("+", "-", "*")
COMPARISONS = ("<", ">", "<=", ">=", "==", "!=")
TOOLS = [{"name": "view", "description": "Show a file.", "parameters": {"type": "object", "properties": {"path": {"type": "string"}}, "required": ["path"]}},
         {"name": "run", "description": "Run a shell command.", "parameters": {"type": "object", "properties": {"cmd": {"type": "string"}}, "required": ["cmd"]}},
         {"name": "str_replace", "description": "Replace text in a file.", "parameters": {"type": "object", "properties": {
             "path": {"type": "string"}, "old_str": {"type": "string"}, "new_str": {"type": "string"}}, "required": ["path", "old_str", "new_str"]}},
         {"name": "write_file", "description": "Write content to a file.", "parameters": {"type": "object", "properties": {
             "path": {"type": "string"}, "content": {"type": "string"}}, "required": ["path", "content"]}}]
SYSTEM = "You are a coding assistant working in a repository."


def stream(probe: str, cell: tuple, index: int, attempt: int = 0, purpose: int = 0, seed: int = SEED) -> np.random.Generator:
    words = [seed, _CODE[probe]] + [int(x) if not isinstance(x, str) else sum(ord(c) * 131 ** i for i, c in enumerate(x)) % (1 << 31) for x in cell]
    return np.random.default_rng(np.random.SeedSequence(words + [index, attempt, purpose]))


def pick(rng, seq):
    return seq[int(rng.integers(len(seq)))]


# ------------------------------------------------------------------------------------------------------------- material

def ident(rng) -> str:
    return f"{pick(rng, VERBS)}_{pick(rng, NOUNS)}"


def path_of(rng, ext: str = "py") -> str:
    return "/".join([pick(rng, ROOTS)] + [pick(rng, NOUNS) for _ in range(int(rng.integers(1, 4)))] + [f"{ident(rng)}.{ext}"])


def statement(rng, names: list[str], indent: str = "    ") -> str:
    """One body line. Every line ends in a letter, digit or underscore or a closing bracket followed by nothing."""
    a, b = pick(rng, names), pick(rng, names)
    kind = int(rng.integers(6))
    if kind == 0:
        return f"{indent}{a} = {b} {pick(rng, OPERATORS)} {int(rng.integers(2, 97))}"
    if kind == 1:
        return f"{indent}{a} = {ident(rng)}({b}, {int(rng.integers(2, 97))})"
    if kind == 2:
        return f"{indent}if {a} {pick(rng, COMPARISONS)} {int(rng.integers(2, 97))}: {b} = {pick(rng, ('True', 'False'))}"
    if kind == 3:
        return f"{indent}{a}.{pick(rng, VERBS)}({b})"
    if kind == 4:
        return f"{indent}{a} = {b}[{int(rng.integers(0, 9))}] {pick(rng, OPERATORS)} {pick(rng, names)}"
    return f"{indent}assert {a} {pick(rng, COMPARISONS)} {b}"


def function(rng, name: str, n_lines: int) -> list[str]:
    names = sorted({pick(rng, NOUNS) for _ in range(4)} | {"value"})
    lines = [f"def {name}({', '.join(names[:2])}):"] + [statement(rng, names) for _ in range(max(1, n_lines - 1))]
    return lines + [f"    return {pick(rng, names)}"]


@dataclass
class Module:
    path: str
    lines: list
    defs: list            # (kind, name, 1-based line number) of every top-level definition
    bodies: dict          # function name -> (first body line index, end index) into `lines`, 0-based, end exclusive

    def text(self, numbered: bool = False) -> str:
        if numbered:
            return "\n".join(f"{i + 1:6d}\t{line}" for i, line in enumerate(self.lines))
        return "\n".join(self.lines)


def module(rng, n_lines: int, body: tuple = (3, 9), names: list | None = None) -> Module:
    """A module of about n_lines lines: constants, functions and a class, separated by blank lines; definition names distinct."""
    lines, defs, bodies, used = [f'"""{ident(rng).replace("_", " ").capitalize()} helpers."""', "", "import os", ""], [], {}, set()
    for _ in range(int(rng.integers(1, 4))):
        name = ident(rng).upper()
        if name not in used:
            used.add(name)
            defs.append(("constant", name, len(lines) + 1))
            lines.append(f"{name} = {int(rng.integers(2, 4096))}")
    lines.append("")
    queue = list(names or [])
    while len(lines) < n_lines or queue:
        name = queue.pop(0) if queue else ident(rng)
        if name in used:
            continue
        used.add(name)
        if not queue and rng.random() < 0.12:
            cls = "".join(w.capitalize() for w in name.split("_"))
            defs.append(("class", cls, len(lines) + 1))
            lines += [f"class {cls}:", f"    limit = {int(rng.integers(2, 512))}", ""]
            continue
        fn = function(rng, name, int(rng.integers(body[0], body[1] + 1)))
        defs.append(("function", name, len(lines) + 1))
        bodies[name] = (len(lines) + 1, len(lines) + len(fn))
        lines += fn + ["", ""]
    while lines and lines[-1] == "":
        lines.pop()
    return Module(path_of(rng), lines, defs, bodies)


def log_lines(rng, n: int) -> str:
    return "\n".join(f"2026-{int(rng.integers(1, 13)):02d}-{int(rng.integers(1, 29)):02d} {int(rng.integers(24)):02d}:{int(rng.integers(60)):02d}:"
                     f"{int(rng.integers(60)):02d} {pick(rng, LEVELS)} {pick(rng, NOUNS)}-{int(rng.integers(1, 17))} {pick(rng, VERBS)} "
                     f"{int(rng.integers(1, 5000))} {pick(rng, NOUNS)}s in {int(rng.integers(1, 900))} ms" for _ in range(n))


def body_of_length(rng, target: int, count: Callable[[str], int], tries: int = 200) -> list[str]:
    """Body lines whose token count lies within SPAN_TOL of `target`."""
    names = sorted({pick(rng, NOUNS) for _ in range(4)} | {"value"})
    lines = [statement(rng, names)]
    for _ in range(tries):
        n = count("\n".join(lines))
        if abs(n - target) <= SPAN_TOL * target:
            return lines
        if n < target:
            lines.append(statement(rng, names))
        else:
            lines = lines[:-1] or [f"    return {pick(rng, names)}"]
            if len(lines) == 1 and count(lines[0]) > (1 + SPAN_TOL) * target:
                lines = [f"    {pick(rng, names)} = {int(rng.integers(2, 9))}"]
    return lines


def near_duplicate(rng, lines: list[str], n_diff: int) -> tuple[list[str], list[tuple[int, int]]]:
    """`lines` with one token changed in each of n_diff lines (a digit, an operator, a comparison or a boolean). Returns the
    decoy and, per change, (line index, character offset in the line)."""
    out, where = list(lines), []
    order = [int(i) for i in rng.permutation(len(lines))]
    for i in order:
        if len(where) == n_diff:
            break
        parts = out[i].split(" ")
        spots = [j for j, p in enumerate(parts) if p in OPERATORS or p in COMPARISONS or p in ("True", "False") or p.rstrip(")],:").isdigit()]
        if not spots:
            continue
        j = spots[int(rng.integers(len(spots)))]
        p = parts[j]
        if p in OPERATORS:
            new = pick(rng, [o for o in OPERATORS if o != p])
        elif p in COMPARISONS:
            new = pick(rng, [o for o in COMPARISONS if o != p])
        elif p in ("True", "False"):
            new = "False" if p == "True" else "True"
        else:
            digits = p.rstrip(")],:")
            new = str(int(digits) + int(rng.integers(1, 9))) + p[len(digits):]
        parts[j] = new
        where.append((i, len(" ".join(parts[:j])) + (1 if j else 0)))
        out[i] = " ".join(parts)
    return out, sorted(where)


def agreement(target: list, other: list) -> float:
    """Positionwise agreement of two token sequences over the target's length."""
    return sum(1 for a, b in zip(target, other) if a == b) / max(len(target), 1)


def copier_floor(target: str, others: list[str], tokens: Callable[[str], list] = list) -> dict:
    """A copier that reproduces one of the W candidates at random, perfectly."""
    W = len(others) + 1
    t = tokens(target)
    return {"exact": 1.0 / W, "token_acc": (1.0 + sum(agreement(t, tokens(o)) for o in others)) / W, "nats": math.log(W), "choices": W}


# -------------------------------------------------------------------------------------------------------- text level: copy

def _views_to_distance(rng, distance: int, count, lo: float = DIST_LO) -> str:
    """`$ cat` views of filler modules, topped up with a log view one line at a time, so that the total lies in
    [lo * distance, distance] tokens."""
    text = ""
    for _ in range(200):
        room = distance - count(text)
        if room < 0.25 * distance or room < 200:
            break
        m = module(rng, max(8, min(80, room // 24)))
        view = f"\n\n$ cat {m.path}\n{m.text()}"
        if count(text + view) > distance - 40:
            break
        text += view
    if count(text) >= lo * distance:
        return text
    head, lines = f"\n\n$ tail -n 200 logs/{ident(rng)}.log", []
    for _ in range(2000):
        lines.append(log_lines(rng, 1))
        n = count(text + head + "\n" + "\n".join(lines))
        if n > distance:
            lines.pop()
            break
        if n >= (lo + 1) / 2 * distance:
            break
    return text + head + "\n" + "\n".join(lines)


def copy(length: int, distance: int, variant: str, form: str, index: int, count: Callable[[str], int], attempt: int = 0, seed: int = SEED) -> TextItem:
    cell = {"len": length, "dist": distance, "variant": variant}
    rng = stream("copy", (length, distance, variant, form), index, attempt, 0, seed)
    fill = stream("copy", (length, distance, variant, form), index, attempt, 1, seed)
    target = ident(rng)
    body = body_of_length(rng, length, count)
    others = []
    for _ in range(int(rng.integers(3, 6))):
        name = ident(rng)
        if name != target and name not in [n for n, _ in others]:
            others.append((name, body_of_length(rng, length, count)))
    decoy, diffs = None, []
    if variant == "near_dup":
        decoy, diffs = near_duplicate(rng, body, COPY_DIFFS[length])
        decoy_name = target + "_v2"
    funcs = [(n, b) for n, b in others]
    at = int(rng.integers(len(funcs) + 1))
    funcs.insert(at, (target, body))
    if decoy is not None:
        funcs.insert(at + 1, (decoy_name, decoy))
    path = path_of(rng)
    source = f"$ cat {path}\n" + "\n\n\n".join(f"def {n}(value):\n" + "\n".join(b) for n, b in funcs)
    answer = "\n".join(body)
    tail = count(source[source.index(answer) + len(answer):])            # the rest of the source file lies between the span and the instruction too
    room = distance - tail - 8
    filler = _views_to_distance(fill, room, count, lo=max(0.0, (0.92 * distance - tail) / room)) if room > 64 else ""
    if form == "repeat":
        ask = f"\n\nRepeat the body of the function `{target}` from {path} exactly, keeping its indentation.\n\ndef {target}(value):\n"
    else:
        ask = f"\n\nReplace the body of `{target}` in {path}.\n\nstr_replace\npath: {path}\nold_str:\n"
    offsets, pos = [], 0
    for i, line in enumerate(body):
        offsets += [pos + c for (li, c) in diffs if li == i]
        pos += len(line) + 1
    floor = copier_floor(answer, ["\n".join(b) for n, b in funcs if n != target])
    context = source + filler + ask
    realised = count(context[context.index(answer) + len(answer):]) - count(ask)
    return TextItem(id=f"copy/{cell_name(cell)}/{form}/{index:04d}", probe="copy", cell=cell, context=context, answer=answer,
                    group={"form": form}, meta={"floor": floor, "diff_chars": offsets, "decoy": None if decoy is None else "\n".join(decoy),
                                                "target": target, "path": path, "attempt": attempt, "distance": realised})


# --------------------------------------------------------------------------------------------------- text level: line edit

def _line_context(n_lines: int, index: int, attempt: int, seed: int):
    rng = stream("line_edit", (n_lines,), index, attempt, 0, seed)
    m = module(rng, n_lines)
    kind, name, line = m.defs[int(rng.integers(len(m.defs)))]
    view = f"$ cat -n {m.path}\n{m.text(numbered=True)}"
    return m, kind, name, line, view


def line_edit(n_lines: int, form: str, index: int, attempt: int = 0, seed: int = SEED, answer_line: int | None = None) -> TextItem:
    m, kind, name, line, view = _line_context(n_lines, index, attempt, seed)
    what = {"constant": "the constant", "class": "the class", "function": "the function"}[kind]
    if form == "number":
        ask, fmt = f"\n\nOn which line of {m.path} is {what} `{name}` defined?\nAnswer: line", " {}"
    else:
        ask, fmt = f"\n\nDelete the line of {m.path} where {what} `{name}` is defined.\n$ sed -i '", "{}d"
    n = line if answer_line is None else answer_line
    cell = {"lines": n_lines}
    probe = "line_edit" if answer_line is None else "line_edit_foil"
    floor = {"definition_line": 1.0 / len(m.defs), "any_line": 1.0 / len(m.lines)}
    return TextItem(id=f"{probe}/{cell_name(cell)}/{form}/{index:04d}" + ("" if answer_line is None else f"/{n}"), probe=probe, cell=cell,
                    context=view + ask, answer=fmt.format(n), group={"form": form},
                    meta={"floor": floor, "gold_line": line, "line": n, "question": f"{n_lines}/{form}/{index}", "file_lines": len(m.lines),
                          "definition_lines": [d[2] for d in m.defs], "attempt": attempt})


def line_edit_foils(n_lines: int, form: str, index: int, attempt: int = 0, seed: int = SEED) -> list[TextItem]:
    """The foil rows of one question: the neighbours at FOIL_OFFSETS and the other definition lines (inside the file, not gold)."""
    gold = line_edit(n_lines, form, index, attempt, seed)
    g, total = gold.meta["gold_line"], gold.meta["file_lines"]
    lines = sorted({g + o for o in FOIL_OFFSETS if 1 <= g + o <= total} | {d for d in gold.meta["definition_lines"] if d != g})
    return [line_edit(n_lines, form, index, attempt, seed, answer_line=n) for n in lines]


def line_choice(rows: list[dict]) -> dict:
    """rows: scored rows of ONE question, each {"line", "gold_line", "logp"} (the answer's total log-likelihood). The model's
    choice is the row with the largest log-likelihood."""
    best = max(rows, key=lambda r: r["logp"])
    gold = rows[0]["gold_line"]
    return {"chosen": best["line"], "gold": gold, "correct": float(best["line"] == gold), "distance": abs(best["line"] - gold), "rows": len(rows)}


def line_choice_table(rows: list[dict]) -> dict:
    """All questions: accuracy of the choice and the histogram of |chosen - gold|."""
    by_q: dict = {}
    for r in rows:
        by_q.setdefault(r["question"], []).append(r)
    picks = [line_choice(v) for v in by_q.values()]
    hist: dict = {}
    for p in picks:
        hist[p["distance"]] = hist.get(p["distance"], 0) + 1
    return {"questions": len(picks), "choice_acc": sum(p["correct"] for p in picks) / max(len(picks), 1), "distance_hist": dict(sorted(hist.items()))}


# ------------------------------------------------------------------------------------------------------------- chat level

@dataclass
class ChatItem:
    id: str
    probe: str
    cell: dict
    conversation: dict               # the context's messages (and tools); the reply that holds the answer is NOT in it
    reply_prefix: list               # pieces (text, control) of the reply before the lead-in: [] or a reasoning / call frame
    leadin: str                      # teacher-forced text in the same piece as the answer ("" for none)
    answer: str
    suffix: str = ""                 # what follows the answer in its piece (fixed context after it; never scored)
    group: dict = field(default_factory=dict)
    floor: dict = field(default_factory=dict)
    meta: dict = field(default_factory=dict)

    def to_json(self) -> dict:
        return asdict(self)

    def context_pieces(self) -> list:
        """The (text, control) pieces before the answer's piece: the conversation, the reply's header and its prefix."""
        ps = [(t, c) for t, _, c in CF.pieces(self.conversation)]
        return ps + [(CF.IM_START, True), ("assistant\n", False)] + list(self.reply_prefix)

    def context_text(self) -> str:
        return "".join(t for t, _ in self.context_pieces()) + self.leadin


def boundary_ok(encode: Callable[[str], list], left: str, answer: str, right: str = "") -> bool:
    """No token straddles the answer's ends inside its piece, and the answer's tokens are its tokens alone."""
    whole, a = encode(left + answer + right), encode(answer)
    return whole == encode(left) + a + encode(right) if right else whole == encode(left) + a


def control_ids(first: int) -> dict:
    """The control tokens' ids, `first` upward (the training shards' convention: right after the text vocabulary)."""
    return {name: first + i for i, name in enumerate(CF.CONTROL_TOKENS)}


def encode_chat_item(item: ChatItem, encode: Callable[[str], list], control: dict) -> dict:
    """The stored form `eval/probes.py` scores: control pieces as their ids, every text piece encoded on its own, the answer
    inside its piece after the lead-in."""
    ids: list = []
    for text, is_control in item.context_pieces():
        ids += [control[text]] if is_control else list(encode(text))
    enc = encode
    lead, ans = list(enc(item.leadin)) if item.leadin else [], list(enc(item.answer))
    ctx = ids + lead
    rec = {"id": item.id, "kind": item.probe, "cell": cell_name(item.cell), "group": cell_name(item.group) if item.group else "",
           "ids": ctx + ans, "answer_start": len(ctx), "answer_len": len(ans), "length": len(ctx) + len(ans), "pieces": (),
           "checks": {"clean_boundary": boundary_ok(enc, item.leadin, item.answer, item.suffix)}, "floor": item.floor}
    text = item.context_text()
    if item.probe == "copy_span":
        rec["checks"]["answer_once"] = text.count(item.answer) == 1
    if item.probe == "transcode":
        rec["checks"]["answer_absent"] = item.answer not in text
        rec["checks"]["source_once"] = text.count(item.meta["source"]) == 1
        rec["floor"] = transcode_floor(list(enc(item.meta["source"])), ans)
    if item.meta.get("diff_chars"):
        marks, out = sorted(item.meta["diff_chars"]), []
        for m in marks:
            out.append(len(enc(item.answer[:m])))
        rec["diff_index"] = out
    return rec


def _conversation(messages: list) -> dict:
    return {"tools": TOOLS, "messages": [{"role": "system", "content": SYSTEM}] + messages}


def _filler_turns(rng, tokens: int, count) -> list:
    """Assistant `view` / `run` calls with their tool results, about `tokens` tokens in all (within DIST_LO)."""
    turns, used = [], 0
    for _ in range(400):
        if used >= DIST_LO * tokens:
            break
        room = tokens - used
        if rng.random() < 0.7:
            m = module(rng, max(8, min(60, room // 14)))
            turn = [{"role": "assistant", "content": "", "tool_calls": [{"name": "view", "arguments": {"path": m.path}}]},
                    {"role": "tool", "content": m.text()}]
        else:
            turn = [{"role": "assistant", "content": "", "tool_calls": [{"name": "run", "arguments": {"cmd": f"tail -n 40 logs/{ident(rng)}.log"}}]},
                    {"role": "tool", "content": log_lines(rng, max(2, min(30, room // 30)))}]
        n = count(CF.render({"messages": turn}))
        if used + n > tokens:
            if room < 60:
                break
            continue
        turns += turn
        used += n
    return turns


def snippet(rng, kind: str, length: int, count) -> str:
    """One snippet of a type and nominal length; starts with a non-space character, ends with a letter, digit or underscore."""
    if kind == "code":
        lines = body_of_length(rng, length, count)
        lines = [line[4:] if i == 0 else line for i, line in enumerate(lines)]
        while lines and not (lines[-1][-1].isalnum() or lines[-1][-1] == "_"):
            lines[-1] = lines[-1] + " or value"
        return "\n".join(lines)
    make = {"path": lambda: path_of(rng, pick(rng, ("py", "rs", "go", "ts"))), "ident": lambda: ident(rng),
            "random": lambda: "".join(pick(rng, "abcdefghijklmnopqrstuvwxyz0123456789") for _ in range(int(rng.integers(5, 11))))}[kind]
    parts = [make()]
    while count(" ".join(parts)) < (1 - SPAN_TOL / 2) * length:
        parts.append(make())
    return " ".join(parts)


def copy_span(kind: str, length: int, distance: int, src: str, variant: str, index: int, count, attempt: int = 0, leadin: str | None = LEADIN_COPY,
              seed: int = SEED) -> ChatItem:
    if variant == "near_dup" and kind != "code":
        raise ValueError("copy_span near_dup is built for type 'code'")
    cell = {"type": kind, "len": length, "dist": distance, "src": src, "variant": variant}
    key = (kind, length, distance, src, variant)
    rng, fill = stream("copy_span", key, index, attempt, 0, seed), stream("copy_span", key, index, attempt, 1, seed)
    labels = [f"{pick(rng, NOUNS)}-{int(rng.integers(100, 1000))}" for _ in range(K_SNIPPETS)]
    while len(set(labels)) < K_SNIPPETS:
        labels = [f"{pick(rng, NOUNS)}-{int(rng.integers(100, 1000))}" for _ in range(K_SNIPPETS)]
    snippets = [snippet(rng, kind, length, count) for _ in range(K_SNIPPETS)]
    t = int(rng.integers(K_SNIPPETS))
    diffs = []
    if variant == "near_dup":
        other = (t + 1) % K_SNIPPETS
        decoy, where = near_duplicate(rng, snippets[t].split("\n"), COPY_DIFFS[length])
        snippets[other] = "\n".join(decoy)
        pos, lines = 0, snippets[t].split("\n")
        for i, line in enumerate(lines):
            diffs += [pos + c for (li, c) in where if li == i]
            pos += len(line) + 1
    block = "\n\n".join(f"[{lab}]\n{s}" for lab, s in zip(labels, snippets))
    if src == "tool":
        head = [{"role": "user", "content": "Show me the saved snippets."},
                {"role": "assistant", "content": "", "tool_calls": [{"name": "run", "arguments": {"cmd": "snippets list --all"}}]},
                {"role": "tool", "content": block}]
    else:
        head = [{"role": "user", "content": "Draft four snippets and label them."}, {"role": "assistant", "content": "Here are four labelled snippets.\n\n" + block}]
    ask = {"role": "user", "content": f"Give me the snippet labelled [{labels[t]}] again, verbatim, and nothing else."}
    after = count(CF.render({"messages": [ask]})) + count(block[block.index(snippets[t]) + len(snippets[t]):]) + 24
    filler = [{"role": "user", "content": "Look around the repository for a while first."}] + _filler_turns(fill, max(0, distance - after), count) if distance > after + 80 else []
    conv = _conversation(head + filler + [ask])
    floor = copier_floor(snippets[t], [s for i, s in enumerate(snippets) if i != t])
    item = ChatItem(id=f"copy_span/{cell_name(cell)}/{index:04d}", probe="copy_span", cell=cell, conversation=conv, reply_prefix=[], leadin=leadin or "",
                    answer=snippets[t], floor=floor, meta={"label": labels[t], "diff_chars": diffs, "attempt": attempt, "k": K_SNIPPETS})
    text = item.context_text()
    item.meta["distance"] = count(text[text.index(snippets[t]) + len(snippets[t]):])      # from the end of the target to the start of the answer
    return item


def edit_old(n_lines: int, file_lines: int, render: str, index: int, attempt: int = 0, seed: int = SEED) -> ChatItem:
    """The same content under every `render`: the stream does not depend on it."""
    if render not in RENDERS:
        raise ValueError(f"render {render!r}: one of {RENDERS}")
    cell = {"lines": n_lines, "file": file_lines, "render": render}
    rng = stream("edit_old", (n_lines, file_lines), index, attempt, 0, seed)
    for _ in range(200):
        m = module(rng, file_lines)
        a = int(rng.integers(1, max(2, len(m.lines) - n_lines)))
        span = m.lines[a - 1:a - 1 + n_lines]
        old = "\n".join(span)
        if len(span) == n_lines and span[0].strip() and span[-1].strip() and m.text().count(old) == 1:
            break
    else:
        raise RuntimeError("no unique span")
    numbered = render.endswith("_num")
    b = a + n_lines - 1
    conv = _conversation([{"role": "user", "content": f"Open {m.path}."},
                          {"role": "assistant", "content": "", "tool_calls": [{"name": "view", "arguments": {"path": m.path}}]},
                          {"role": "tool", "content": m.text(numbered=numbered)},
                          {"role": "user", "content": f"Replace lines {a}-{b} of {m.path} with a single `pass` statement."}])
    frame = json.dumps({"name": "str_replace", "arguments": {"path": m.path, "old_str": "@@OLD@@", "new_str": "pass"}}, ensure_ascii=False)
    before, after = frame.split("@@OLD@@")
    answer = json.dumps(old, ensure_ascii=False)[1:-1] if render.startswith("json") else old
    windows = len(m.lines) - n_lines + 1
    floor = {"exact": 1.0 / windows, "nats": math.log(windows), "choices": windows}
    return ChatItem(id=f"edit_old/{cell_name(cell)}/{index:04d}", probe="edit_old", cell=cell, conversation=conv,
                    reply_prefix=[("\n", False), (CF.TOOL_CALL, True)], leadin="\n" + before, answer=answer, suffix=after + "\n", floor=floor,
                    group={"content": f"{n_lines}/{file_lines}/{index}"}, meta={"first_line": a, "last_line": b, "path": m.path, "attempt": attempt})


def _tc_line(rng, kind: str) -> str:
    """One line that holds at least one of `"`, a backslash or a tab; never starts with a quote or a backslash."""
    w, n = lambda: pick(rng, VERBS + NOUNS), lambda: int(rng.integers(1, 99))
    if kind == "code":
        forms = (lambda: f'print("{w()} {w()}: " + str({w()}))', lambda: f'pattern = re.compile(r"\\d+\\s{w()}\\.{w()}")',
                 lambda: f'path = "C:\\\\{w()}\\\\{w()}\\\\{w()}.txt"', lambda: f'\tif {w()} != "{w()}": return {n()}',
                 lambda: f'echo "{w()}=\\"{w()}\\"" >> {w()}.env', lambda: f"SELECT {w()} FROM {w()} WHERE {w()} = \"{w()}\" LIMIT {n()}",
                 lambda: f'msg = "{w()}\\n{w()}\\t{n()}"')
    else:
        forms = (lambda: f'{w().capitalize()} said "{w()} the {w()} by {n()}" and left', lambda: f"{w()}\t{n()}\t{w()}\t{n()}",
                 lambda: f"Copy it to D:\\{w()}\\{w()} before {n()} o'clock", lambda: f'The sign read "{w()} {w()}" in {w()} letters')
    return pick(rng, forms)()


def transcode(direction: str, n_lines: int, kind: str, index: int, attempt: int = 0, leadin: str | None = LEADIN_ESC2RAW, seed: int = SEED) -> ChatItem:
    """Both directions of one (n_lines, kind, index) share their content."""
    if direction not in TC_DIRS:
        raise ValueError(f"dir {direction!r}: one of {TC_DIRS}")
    cell = {"dir": direction, "lines": n_lines}
    rng = stream("transcode", (n_lines, kind), index, attempt, 0, seed)
    lines = [_tc_line(rng, kind).rstrip() for _ in range(n_lines)]
    lines[0] = lines[0].lstrip()
    raw = "\n".join(lines)
    esc = json.dumps(raw, ensure_ascii=False)[1:-1]
    assert raw != esc, "a base holds a character that needs escaping"
    sid, path = int(rng.integers(100, 1000)), path_of(rng, "txt" if kind == "text" else "py")
    if direction == "esc2raw":
        conv = _conversation([{"role": "user", "content": f"Fetch snippet {sid}."},
                              {"role": "assistant", "content": "", "tool_calls": [{"name": "run", "arguments": {"cmd": f"snippets get {sid} --json"}}]},
                              {"role": "tool", "content": json.dumps({"id": sid, "content": raw}, ensure_ascii=False)},
                              {"role": "user", "content": "Print that content as plain text: decode the escapes (\\n is a line break, \\\" a quote, \\\\ one backslash, "
                                                          "\\t a tab). Only the text."}])
        return ChatItem(id=f"transcode/{cell_name(cell)}/{kind}/{index:04d}", probe="transcode", cell=cell, conversation=conv, reply_prefix=[],
                        leadin=leadin or "", answer=raw, group={"kind": kind}, meta={"source": esc, "base": f"{n_lines}/{kind}/{index}", "attempt": attempt})
    conv = _conversation([{"role": "user", "content": f"Show me {path}."},
                          {"role": "assistant", "content": "", "tool_calls": [{"name": "run", "arguments": {"cmd": f"cat {path}"}}]},
                          {"role": "tool", "content": raw},
                          {"role": "user", "content": f"Save exactly that text to backup/{path} with the write_file tool."}])
    frame = json.dumps({"name": "write_file", "arguments": {"path": f"backup/{path}", "content": "@@TC@@"}}, ensure_ascii=False)
    before, after = frame.split("@@TC@@")
    return ChatItem(id=f"transcode/{cell_name(cell)}/{kind}/{index:04d}", probe="transcode", cell=cell, conversation=conv,
                    reply_prefix=[("\n", False), (CF.TOOL_CALL, True)], leadin="\n" + before, answer=esc, suffix=after + "\n", group={"kind": kind},
                    meta={"source": raw, "base": f"{n_lines}/{kind}/{index}", "attempt": attempt})


def lcs(a: list, b: list) -> int:
    prev = [0] * (len(b) + 1)
    for x in a:
        cur = [0]
        for j, y in enumerate(b):
            cur.append(prev[j] + 1 if x == y else max(prev[j + 1], cur[j]))
        prev = cur
    return prev[-1]


def transcode_floor(source: list, answer: list) -> dict:
    """The untranscoded source taken as the answer: exact 0 (the forms differ), the share of answer positions with the same
    token, and the token LCS over the answer's length."""
    return {"exact": 0.0, "token_acc": agreement(answer, source), "lcs_share": lcs(source, answer) / max(len(answer), 1)}


# ------------------------------------------------------------------------------------------------------------------ cells

def build_cells(probe: str, per_cell: int, count: Callable[[str], int], distances=None, seed: int = SEED, file_lines=None) -> list:
    """Every cell of a probe, `per_cell` items each (distances: the copy probes' cells; file_lines: the line probes')."""
    items: list = []
    if probe == "copy":
        for length in COPY_LENGTHS:
            for dist in distances or COPY_DISTANCES:
                for variant in COPY_VARIANTS:
                    for i in range(per_cell):
                        items.append(copy(length, dist, variant, COPY_FORMS[i % 2], i, count, seed=seed))
    elif probe in ("line_edit", "line_edit_foil"):
        for n in file_lines or FILE_LINES:
            for i in range(per_cell):
                form = ("number", "sed")[i % 2]
                gold = line_edit(n, form, i, seed=seed)
                if probe == "line_edit_foil":          # the gold row leads its foils, so one stored set holds every row of a question
                    gold.probe, gold.id = "line_edit_foil", gold.id.replace("line_edit/", "line_edit_foil/") + f"/{gold.meta['line']}"
                items += [gold] if probe == "line_edit" else [gold] + line_edit_foils(n, form, i, seed=seed)
    elif probe == "copy_span":
        for kind in SPAN_TYPES:
            for length in COPY_LENGTHS:
                for dist in distances or COPY_DISTANCES:
                    for src in SPAN_SOURCES:
                        for variant in (COPY_VARIANTS if kind == "code" else ("plain",)):
                            for i in range(per_cell):
                                items.append(copy_span(kind, length, dist, src, variant, i, count, seed=seed))
    elif probe == "edit_old":
        for n in EDIT_LINES:
            for size in EDIT_FILES:
                for i in range(per_cell):
                    items += [edit_old(n, size, r, i, seed=seed) for r in RENDERS]
    elif probe == "transcode":
        for n in TC_LINES:
            for kind in TC_KINDS:
                for i in range(per_cell):
                    items += [transcode(d, n, kind, i, seed=seed) for d in TC_DIRS]
    else:
        raise ValueError(f"probe {probe!r}: one of {PROBES}")
    return items


# --------------------------------------------------------------------------------------------------------------- analysis

def cell_extras(records: list[dict], scored: list[dict]) -> dict:
    """What a cell of these probes reports beside exact match: `records` are the stored items of the cell, `scored` their
    results from `probes.score_probes(..., keep_tokens=True)`, in the same order.

      floor          the mean of each floor entry over the items (the copier's / the random window's / the untranscoded
                     source's score), to read the model's numbers against
      token_acc, nats_per_token   means over the items
      diff_acc, diff_nats         near-duplicates: accuracy and nats at the answer tokens where target and decoy differ
                                  (a copier that mixes the two up sits at 1/2)
      line_choice    line_edit_foil rows (with their gold rows, when the cell holds both): the choice among each question's
                     rows by total log-likelihood, its accuracy and the histogram of |chosen - gold|"""
    out: dict = {}
    if not records:
        return out
    keys = sorted({k for r in records for k, v in (r.get("floor") or {}).items() if isinstance(v, (int, float))})
    if keys:
        out["floor"] = {k: sum(float(r["floor"][k]) for r in records if k in (r.get("floor") or {})) / sum(1 for r in records if k in (r.get("floor") or {})) for k in keys}
    if all("ok" in s for s in scored):
        out["token_acc"] = sum(sum(s["ok"]) / len(s["ok"]) for s in scored) / len(scored)
        out["nats_per_token"] = sum(sum(s["nats"]) / len(s["nats"]) for s in scored) / len(scored)
        at = [(r["diff_index"], s) for r, s in zip(records, scored) if r.get("diff_index")]
        hits = [float(s["ok"][i]) for idx, s in at for i in idx if i < len(s["ok"])]
        if hits:
            out["diff_acc"] = sum(hits) / len(hits)
            out["diff_nats"] = sum(s["nats"][i] for idx, s in at for i in idx if i < len(s["nats"])) / len(hits)
            out["diff_tokens"] = len(hits)
        rows = [{"question": r["question"], "line": r["line"], "gold_line": r["gold_line"], "logp": -sum(s["nats"])}
                for r, s in zip(records, scored) if "question" in r]
        if rows and any(r["line"] != r["gold_line"] for r in rows):
            out["line_choice"] = line_choice_table(rows)
    return out
