"""Token types of generated (assistant) tokens in agent trajectories, from the token stream alone.

Input: the token ids of a document in the chat rendering of `data/chat_format.py`, the flags saying which tokens the
assistant generates, and the bytes of every vocabulary entry. No model and no text: the labels are a pure function of
those, so a changed rule is a re-run over stored ids.

Every generated token gets one fine type (FINE), rolled up into TYPES:

    scaffold         whitespace between the parts of a message, <think>, </think>, </tool_call> and the call's syntax
                     (JSON braces, quotes, colons, commas, argument names)                              -> other
    call_open        the <tool_call> token                                                               -> other
    turn_end         <|im_end|>                                                                          -> other
    reasoning_think  inside <think> ... </think>                                                         -> reasoning
    reasoning_call   the value of a thought argument (REASONING_KEYS)                                    -> reasoning
    narration        message text of a message that goes on to make a tool call that is not finish-type  -> reasoning
    head_name        the tool name (and an editor tool's sub-command)                                    -> head
    head_path        the value of a path argument (`is_path_key`)                                        -> head
    arg              any other argument value                                                            -> args
    code_arg         the value of an argument that carries code or text to write (CODE_KEYS)             -> code
    copied_arg       a token of an arg / code_arg value inside a window of >= COPY_MIN_TOKENS consecutive tokens of
                     that value whose bytes occur verbatim earlier in the document, wholly before the window starts
                     (JSON escapes of call arguments undone on both sides)                               -> copied
    code_content     the body of a fenced code block in message content                                  -> code
    final_answer     message text of a message without a call (or with finish-type calls only), and the message
                     argument of a finish-type tool                                                      -> final

Precedence for an argument value: head_path > reasoning_call > final_answer > copied_arg > code_arg > arg. A token
that holds bytes of more than one part takes the type of its first value byte; a token with no value byte is
scaffold. Labels depend on the tokens before a token and on the rest of its own message only.

The labeller works on bytes: the document's bytes are laid out with the offset of every token, each assistant message
is parsed on the byte string, bytes get a type, and a token reads the type of its first value byte. A second,
prefix-only labelling gives SEGMENTS (reasoning, content, call_head, call_body, unplaced)
(reference: ced/eval/token_types.py:1-108, 166-192; the version-1 rendering only; line-number prefixes of file views
are compared as they stand).
"""

from __future__ import annotations

import re

import numpy as np

from ..data import chat_format as cf

FINE = ("scaffold", "call_open", "turn_end", "reasoning_think", "reasoning_call", "narration", "head_name", "head_path",
        "arg", "code_arg", "copied_arg", "code_content", "final_answer")
F = {name: i for i, name in enumerate(FINE)}
TYPES = ("reasoning", "head", "args", "copied", "code", "final", "other")
ROLLUP = {"scaffold": "other", "call_open": "other", "turn_end": "other", "reasoning_think": "reasoning",
          "reasoning_call": "reasoning", "narration": "reasoning", "head_name": "head", "head_path": "head", "arg": "args",
          "code_arg": "code", "copied_arg": "copied", "code_content": "code", "final_answer": "final"}
FINE_TO_TYPE = np.array([TYPES.index(ROLLUP[f]) for f in FINE], dtype=np.int8)
SEGMENTS = ("reasoning", "content", "call_head", "call_body", "unplaced")

COPY_MIN_TOKENS = 16
COPY_MIN_BYTES = 8
PATH_KEYS = frozenset({"path", "file_path", "filepath", "file", "filename", "target_file", "notebook_path", "directory",
                       "dir", "old_path", "new_path", "cwd", "root"})
PATH_WORDS = frozenset({"path", "filepath", "file", "filename", "dir", "directory", "folder"})
REASONING_KEYS = frozenset({"thought", "thoughts", "thinking", "reasoning"})
FINAL_KEYS = frozenset({"message", "answer", "result", "final_answer"})
FINISH_TOOLS = frozenset({"finish", "task_complete", "submit", "final_answer", "complete", "done", "stop"})
CODE_KEYS = frozenset({"command", "cmd", "keystrokes", "content", "file_text", "new_str", "old_str", "new_string",
                       "old_string", "code", "script", "patch", "diff", "insert_text", "replacement"})
SUBCOMMAND_TOOLS = ("editor", "str_replace")
_KEY_WORDS = re.compile(r"[A-Z]+(?![a-z])|[A-Z]?[a-z]+|\d+")
_ESC = {ord("n"): 10, ord("t"): 9, ord("r"): 13, ord('"'): 34, ord("\\"): 92, ord("/"): 47, ord("b"): 8, ord("f"): 12}
_WS = b" \t\r\n"
NONE = 255          # a byte that is syntax or whitespace between parts: no value


def is_path_key(key: str) -> bool:
    """An argument name that carries a target file or path: in PATH_KEYS as written, or, split into words at
    underscores, hyphens and capitals, the joined words are in PATH_KEYS or the last word is in PATH_WORDS (filePath,
    FILE_PATH, output_file, repoDir; "profile" and "xpath" are one word each and are not)."""
    if key in PATH_KEYS:
        return True
    words = [w.lower() for w in _KEY_WORDS.findall(key)]
    return bool(words) and ("_".join(words) in PATH_KEYS or "".join(words) in PATH_KEYS or words[-1] in PATH_WORDS)


def classify(tool: str, key: str, is_string: bool) -> int:
    """The fine type of an argument value, copy detection aside."""
    if is_string and is_path_key(key):
        return F["head_path"]
    if key == "command" and is_string and any(w in tool.lower() for w in SUBCOMMAND_TOOLS):
        return F["head_name"]
    if key in REASONING_KEYS and is_string:
        return F["reasoning_call"]
    if tool in FINISH_TOOLS and key in FINAL_KEYS and is_string:
        return F["final_answer"]
    if key in CODE_KEYS:
        return F["code_arg"]
    return F["arg"]


# ------------------------------------------------------------------------------------------------ JSON on bytes
def _skip_ws(s: bytes, i: int) -> int:
    while i < len(s) and s[i] in _WS:
        i += 1
    return i


def _string_end(s: bytes, i: int) -> int:
    """s[i] is the opening quote: the index of the closing one, or -1."""
    i += 1
    while i < len(s):
        if s[i] == 92:
            i += 2
            continue
        if s[i] == 34:
            return i
        i += 1
    return -1


def _value_end(s: bytes, i: int) -> int:
    """One past the JSON value that starts at s[i], or -1."""
    if i >= len(s):
        return -1
    if s[i] == 34:
        e = _string_end(s, i)
        return -1 if e < 0 else e + 1
    if s[i] in b"{[":
        depth = 0
        while i < len(s):
            c = s[i]
            if c == 34:
                i = _string_end(s, i)
                if i < 0:
                    return -1
            elif c in b"{[":
                depth += 1
            elif c in b"}]":
                depth -= 1
                if depth == 0:
                    return i + 1
            i += 1
        return -1
    j = i
    while j < len(s) and s[j] not in b",}] \t\r\n":
        j += 1
    return j if j > i else -1


def _members(s: bytes, i: int):
    """s[i] == '{': yields (key, value_start, value_end) of the object's members; returns at the closing brace.
    Raises ValueError on anything that is not an object of string keys."""
    i = _skip_ws(s, i + 1)
    if i < len(s) and s[i] == 125:
        return
    while True:
        if i >= len(s) or s[i] != 34:
            raise ValueError("key")
        e = _string_end(s, i)
        if e < 0:
            raise ValueError("key end")
        key = unescape(s[i + 1:e])[0].decode("utf-8", "replace")
        i = _skip_ws(s, e + 1)
        if i >= len(s) or s[i] != 58:
            raise ValueError("colon")
        a = _skip_ws(s, i + 1)
        b = _value_end(s, a)
        if b < 0:
            raise ValueError("value")
        yield key, a, b
        i = _skip_ws(s, b)
        if i < len(s) and s[i] == 44:
            i = _skip_ws(s, i + 1)
            continue
        if i < len(s) and s[i] == 125:
            return
        raise ValueError("object end")


def unescape(s: bytes) -> tuple[bytes, np.ndarray]:
    """The bytes of a JSON string's inside with its escapes undone, and for every source byte (plus one past the end)
    the position in the output where its character starts."""
    out, pos, i = bytearray(), np.zeros(len(s) + 1, dtype=np.int64), 0
    while i < len(s):
        pos[i] = len(out)
        if s[i] == 92 and i + 1 < len(s):
            c = s[i + 1]
            if c == ord("u") and i + 6 <= len(s):
                try:
                    out += chr(int(s[i + 2:i + 6], 16)).encode("utf-8", "surrogatepass")
                except ValueError:
                    out += s[i:i + 6]
                pos[i + 1:i + 6] = pos[i]
                i += 6
                continue
            out.append(_ESC.get(c, c))
            pos[i + 1] = pos[i]
            i += 2
            continue
        out.append(s[i])
        i += 1
    pos[len(s)] = len(out)
    return bytes(out), pos


# ------------------------------------------------------------------------------------------------ the labeller
class Layout:
    """The document's bytes with every token's offset, and the control tokens' ids."""

    def __init__(self, ids, table, control: dict[str, int]):
        self.ids = np.asarray(ids, dtype=np.int64)
        parts = [table[int(t)] for t in self.ids]
        self.off = np.zeros(len(parts) + 1, dtype=np.int64)
        np.cumsum([len(p) for p in parts], out=self.off[1:])
        self.raw = b"".join(parts)
        self.control = control
        self.is_control = np.isin(self.ids, list(control.values()))


def _strip(raw: bytes, a: int, b: int) -> tuple[int, int]:
    while a < b and raw[a] in _WS:
        a += 1
    while b > a and raw[b - 1] in _WS:
        b -= 1
    return a, b


def _fences(raw: bytes, a: int, b: int) -> list[tuple[int, int]]:
    """Byte ranges of the bodies of fenced code blocks in raw[a:b]: the opening ``` starts a line, the closing ``` is
    alone on one; an unclosed fence runs to the end."""
    out, body, at = [], None, a
    for line in raw[a:b].split(b"\n"):
        end = at + len(line)
        if body is None and line.lstrip(b" ").startswith(b"```"):
            body = min(end + 1, b)
        elif body is not None and line.strip() == b"```":
            out.append((body, max(body, at)))
            body = None
        at = end + 1
    if body is not None:
        out.append((body, b))
    return out


def _label_call(raw: bytes, a: int, b: int, bl: np.ndarray, values: list, name_end: list) -> str:
    """Types of the bytes of one call's JSON raw[a:b]; appends (start, end, type) of every string argument value that
    copy detection looks at, and the offset one past the tool name. Returns the tool name ("" when unparsed)."""
    s = raw[a:b]
    i = _skip_ws(s, 0)
    try:
        if i >= len(s) or s[i] != 123:
            raise ValueError("object")
        top = {k: (x, y) for k, x, y in _members(s, i)}
        nx, ny = top["name"]
        if s[nx] != 34:
            raise ValueError("name")
        tool = unescape(s[nx + 1:ny - 1])[0].decode("utf-8", "replace")
        bl[a + nx + 1:a + ny - 1] = F["head_name"]
        name_end.append(a + ny)
        if "arguments" in top:
            ax, _ = top["arguments"]
            if s[ax] != 123:
                raise ValueError("arguments")
            for key, x, y in _members(s, ax):
                is_string = s[x] == 34
                kind = classify(tool, key, is_string)
                lo, hi = (x + 1, y - 1) if is_string else (x, y)
                bl[a + lo:a + hi] = kind
                if is_string and kind in (F["arg"], F["code_arg"]):
                    values.append((a + lo, a + hi, kind))
        return tool
    except (ValueError, KeyError):          # not a call in this format: its text counts as an argument
        lo, hi = _strip(raw, a, b)
        bl[lo:hi] = F["arg"]
        return ""


def label_document(ids, assistant, table, control: dict[str, int] | None = None, copy_min: int = COPY_MIN_TOKENS,
                   stats: dict | None = None) -> np.ndarray:
    """(n,) int8 fine types; -1 on tokens the assistant does not generate. `table[id]` = the bytes of a token,
    `control` = name -> id of the control tokens (default: the byte chat tokenizer's)."""
    if control is None:
        control = cf.ChatTokenizer().control
    L = Layout(ids, table, control)
    assistant = np.asarray(assistant, dtype=bool)
    n, raw, off = len(L.ids), L.raw, L.off
    lab = np.full(n, -1, dtype=np.int8)
    bl = np.full(len(raw), NONE, dtype=np.uint8)
    cid = {k: control[k] for k in (cf.IM_START, cf.IM_END, cf.THINK, cf.THINK_END, cf.TOOL_CALL, cf.TOOL_CALL_END)}
    values, calls_bad = [], 0
    t = 0
    while t < n:
        if not assistant[t]:
            t += 1
            continue
        a = t                                   # a generated run: one assistant message body, to its <|im_end|> or the cut
        while t < n and assistant[t] and L.ids[t] != cid[cf.IM_END]:
            t += 1
        b = t
        if t < n and assistant[t]:
            t += 1                              # the <|im_end|> itself
        ctl = [j for j in range(a, b) if L.is_control[j]]
        opens = [j for j in ctl if L.ids[j] == cid[cf.TOOL_CALL]]
        closes = [j for j in ctl if L.ids[j] == cid[cf.TOOL_CALL_END]]
        text_from = a
        if a < b and L.ids[a] == cid[cf.THINK]:
            ends = [j for j in ctl if L.ids[j] == cid[cf.THINK_END]]
            stop = ends[0] if ends else (opens[0] if opens else b)
            lo, hi = _strip(raw, off[a + 1], off[stop])
            bl[lo:hi] = F["reasoning_think"]
            text_from = min(stop + 1, b) if ends else stop
        text_to = opens[0] if opens else b
        tools, name_end = [], []
        for k, o in enumerate(opens):
            close = next((c for c in closes if c > o), b)
            close = min(close, opens[k + 1]) if k + 1 < len(opens) else close
            tools.append(_label_call(raw, int(off[o + 1]), int(off[close]), bl, values, name_end))
            calls_bad += tools[-1] == ""
        acts = any(tool not in FINISH_TOOLS for tool in tools)
        kind = F["narration"] if acts else F["final_answer"]
        lo, hi = _strip(raw, off[text_from], off[text_to])
        bl[lo:hi] = kind
        for x, y in _fences(raw, lo, hi):
            bl[x:y] = F["code_content"]
    # tokens read the type of their first value byte
    for j in np.nonzero(assistant)[0]:
        tid = int(L.ids[j])
        if L.is_control[j]:
            lab[j] = F["call_open"] if tid == cid[cf.TOOL_CALL] else F["turn_end"] if tid == cid[cf.IM_END] else F["scaffold"]
            continue
        seg = bl[off[j]:off[j + 1]]
        hit = np.nonzero(seg != NONE)[0]
        lab[j] = seg[hit[0]] if len(hit) else F["scaffold"]
    copied = _copied(L, lab, values, copy_min)
    lab[copied] = F["copied_arg"]
    if stats is not None:
        stats["unparsed_calls"] = stats.get("unparsed_calls", 0) + calls_bad
        stats["copied_tokens"] = stats.get("copied_tokens", 0) + int(copied.sum())
    return lab


def _compare_bytes(L: Layout, values: list) -> tuple[bytes, np.ndarray]:
    """The document's bytes with the JSON escapes of the argument string values undone, and for every source byte
    (plus one past the end) its position there."""
    out, pos, at = bytearray(), np.zeros(len(L.raw) + 1, dtype=np.int64), 0
    for lo, hi, _ in sorted(values):
        pos[at:lo] = len(out) + np.arange(lo - at)
        out += L.raw[at:lo]
        un, p = unescape(L.raw[lo:hi])
        pos[lo:hi] = len(out) + p[:-1]
        out += un
        at = hi
    pos[at:len(L.raw)] = len(out) + np.arange(len(L.raw) - at)
    out += L.raw[at:]
    pos[len(L.raw)] = len(out)
    return bytes(out), pos


def _copied(L: Layout, lab: np.ndarray, values: list, copy_min: int) -> np.ndarray:
    """Mask of the tokens inside copied spans: greedy from the left, a window of >= copy_min tokens (and >=
    COPY_MIN_BYTES bytes) of one argument value that occurs earlier, wholly before the window's first byte; a window
    found is grown token by token while it still occurs."""
    mask = np.zeros(len(lab), dtype=bool)
    if not values:
        return mask
    cmp, pos = _compare_bytes(L, values)
    for lo, hi, kind in values:
        first = int(np.searchsorted(L.off, lo, side="left"))      # tokens that start inside the value
        last = int(np.searchsorted(L.off, hi, side="left"))
        toks = [j for j in range(first, last) if lab[j] == kind]
        i = 0
        while i + copy_min <= len(toks):
            j = i + copy_min
            if toks[j - 1] - toks[i] != j - 1 - i:                 # not consecutive
                i += 1
                continue
            start = int(pos[L.off[toks[i]]])
            end_of = lambda jj: int(pos[min(L.off[toks[jj - 1] + 1], hi)])
            needle = cmp[start:end_of(j)]
            if len(needle) < COPY_MIN_BYTES or cmp.find(needle, 0, start) < 0:
                i += 1
                continue
            while j < len(toks) and toks[j] == toks[j - 1] + 1 and cmp.find(cmp[start:end_of(j + 1)], 0, start) >= 0:
                j += 1
            mask[toks[i]:toks[j - 1] + 1] = True
            i = j
    return mask


def coarse(lab: np.ndarray) -> np.ndarray:
    """Fine types -> indices into TYPES (-1 stays -1)."""
    out = np.full(lab.shape, -1, dtype=np.int8)
    ok = lab >= 0
    out[ok] = FINE_TO_TYPE[lab[ok]]
    return out


def segment_positions(ids, assistant, table, control: dict[str, int] | None = None) -> np.ndarray:
    """(n,) indices into SEGMENTS, a function of the tokens up to each position only: inside <think> ... </think>
    (both tokens included) = reasoning; from <tool_call> through the token that closes the tool name = call_head; the
    rest of the call through </tool_call> = call_body; other generated tokens = content; not generated = unplaced."""
    if control is None:
        control = cf.ChatTokenizer().control
    ids, assistant = np.asarray(ids), np.asarray(assistant, dtype=bool)
    seg = np.full(len(ids), SEGMENTS.index("unplaced"), dtype=np.int8)
    state, quotes = "content", 0
    for j, tid in enumerate(ids.tolist()):
        if not assistant[j]:
            state = "content"
            continue
        if tid == control[cf.THINK]:
            state = "reasoning"
        elif tid == control[cf.TOOL_CALL]:
            state, quotes = "call_head", 0
        seg[j] = SEGMENTS.index(state)
        if tid == control[cf.THINK_END] or tid == control[cf.TOOL_CALL_END] or tid == control[cf.IM_END]:
            state = "content"
        elif state == "call_head" and tid not in control.values():
            # {"name": "N": the name's closing quote is the fourth unescaped quote of the call
            piece, k = table[tid], 0
            while k < len(piece):
                if piece[k] == 92:
                    k += 2
                    continue
                quotes += piece[k] == 34
                k += 1
            if quotes >= 4:
                state = "call_body"
    return seg


def summarize(labels: list[np.ndarray], byte_lens: list[np.ndarray]) -> dict:
    """Shares of generated tokens and of their bytes by fine type and by rolled-up type."""
    tok, byt = np.zeros(len(FINE)), np.zeros(len(FINE))
    for lab, bl in zip(labels, byte_lens):
        ok = lab >= 0
        tok += np.bincount(lab[ok], minlength=len(FINE))
        byt += np.bincount(lab[ok], weights=np.asarray(bl, dtype=np.float64)[ok], minlength=len(FINE))
    nt, nb = max(tok.sum(), 1.0), max(byt.sum(), 1.0)
    fine = {f: {"tokens": int(tok[i]), "token_share": float(tok[i] / nt), "byte_share": float(byt[i] / nb)} for i, f in enumerate(FINE)}
    types = {}
    for i, name in enumerate(TYPES):
        pick = FINE_TO_TYPE == i
        types[name] = {"tokens": int(tok[pick].sum()), "token_share": float(tok[pick].sum() / nt),
                       "byte_share": float(byt[pick].sum() / nb)}
    return {"tokens": int(tok.sum()), "bytes": int(byt.sum()), "fine": fine, "types": types}


def loss_by_type(labels: list[np.ndarray], losses: list[np.ndarray]) -> dict:
    """Mean per-token loss of every rolled-up type (the token at position i is predicted at i - 1: `losses[d][i]` is
    the loss of predicting token i)."""
    s, c = np.zeros(len(TYPES)), np.zeros(len(TYPES))
    for lab, ls in zip(labels, losses):
        co = coarse(lab)
        ok = co >= 0
        s += np.bincount(co[ok], weights=np.asarray(ls, dtype=np.float64)[ok], minlength=len(TYPES))
        c += np.bincount(co[ok], minlength=len(TYPES))
    return {name: {"loss": float(s[i] / c[i]) if c[i] else None, "tokens": int(c[i])} for i, name in enumerate(TYPES)}
