#!/usr/bin/env python
"""Build an eval-set file ({"docs": [{"ids", "byte_lens", "scored", "name"}]}) for `scripts/rescore.py`, the in-loop evals
and `scripts/eval_long.py` from plain text or JSON-lines (reference: tools/build_probes.py, tools/data/chat_format.py).

    python scripts/build_eval_set.py --input docs.jsonl --out set.pt [--tokenizer spm.model] [--field text]
                                     [--chat] [--max-docs N] [--min-tokens 2]

Without --tokenizer the bytes of the text are the tokens (ids 0..255, one byte each): enough for smoke evaluations on any
vocabulary of at least 256 entries. With --chat each JSON line holds {"messages": [{"role", "content"}, ...]}; the
document is the turns joined as "<role>\\n<content>\\n" and only assistant content is scored. With --agent each JSON
line holds a conversation {"tools", "messages" (with "reasoning" and "tool_calls")} and the document is its ChatML-like
rendering with control tokens at ids 256 upward over byte tokens (`data/chat_format.py`); the set then carries the
vocabulary's byte table, which is what `scripts/token_type_losses.py` labels the generated tokens from.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class ByteTokenizer:
    def encode(self, text: str) -> tuple[list[int], list[int]]:
        b = list(text.encode("utf-8"))
        return b, [1] * len(b)


class SentencePieceTokenizer:
    def __init__(self, path: str):
        import sentencepiece as spm

        self.sp = spm.SentencePieceProcessor(model_file=path)

    def encode(self, text: str) -> tuple[list[int], list[int]]:
        ids = self.sp.encode(text)
        pieces = [self.sp.id_to_piece(i) for i in ids]
        lens = [max(len(p.replace("▁", " ").encode("utf-8")), 1) for p in pieces]
        return ids, lens


def chat_document(messages: list[dict], tok) -> dict:
    ids, lens, scored = [], [], []
    for m in messages:
        head, _ = tok.encode(f"<{m['role']}>\n")
        body, blens = tok.encode(m["content"] + "\n")
        ids += head + body
        lens += [1] * len(head) + blens
        scored += [False] * len(head) + [m["role"] == "assistant"] * len(body)
    return {"ids": ids, "byte_lens": lens, "scored": scored}


def build(lines, tok, field: str, chat: bool, min_tokens: int, max_docs: int | None) -> list[dict]:
    docs = []
    for n, line in enumerate(lines):
        line = line.strip()
        if not line:
            continue
        if chat:
            d = chat_document(json.loads(line)["messages"], tok)
        else:
            text = json.loads(line)[field] if line.startswith("{") else line
            ids, lens = tok.encode(text)
            d = {"ids": ids, "byte_lens": lens, "scored": None}
        if len(d["ids"]) >= min_tokens:
            d["name"] = f"doc{n}"
            docs.append(d)
        if max_docs and len(docs) >= max_docs:
            break
    return docs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--input", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokenizer")
    ap.add_argument("--field", default="text")
    ap.add_argument("--chat", action="store_true")
    ap.add_argument("--agent", action="store_true")
    ap.add_argument("--max-docs", type=int)
    ap.add_argument("--min-tokens", type=int, default=2)
    a = ap.parse_args(argv)
    if a.agent:
        from gdn_hybrid_architecture_ideas_b200.data.chat_format import ChatTokenizer

        if a.tokenizer:
            ap.error("--agent renders over byte tokens: no --tokenizer")
        chat = ChatTokenizer()
        docs = []
        with open(a.input) as f:
            for n, line in enumerate(f):
                if line.strip() and (not a.max_docs or len(docs) < a.max_docs):
                    docs.append({**chat.encode_conversation(json.loads(line)), "name": f"doc{n}"})
        torch.save({"docs": docs, "tokenizer": "bytes+chat", "token_bytes": chat.table, "control": chat.control}, a.out)
        print(f"{len(docs)} conversations, {sum(len(d['ids']) for d in docs)} tokens -> {a.out}")
        return 0
    tok = SentencePieceTokenizer(a.tokenizer) if a.tokenizer else ByteTokenizer()
    with open(a.input) as f:
        docs = build(f, tok, a.field, a.chat, a.min_tokens, a.max_docs)
    torch.save({"docs": docs, "tokenizer": a.tokenizer or "bytes"}, a.out)
    print(f"{len(docs)} documents, {sum(len(d['ids']) for d in docs)} tokens -> {a.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
