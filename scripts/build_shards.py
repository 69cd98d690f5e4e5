#!/usr/bin/env python
"""Tokenize documents into a training shard set (`data/shard_format.py`), the input of `data.kind: shards`.

    python scripts/build_shards.py --out shards/train --tokenizer tokenizer.json|spm.model|bytes --input docs.jsonl[.gz] [--input ...]
        [--field text] [--eos-token "<|endoftext|>"] [--chat] [--first-control ID] [--max-docs N] [--min-tokens 2] [--holdout-every K --holdout-out DIR]

Plain documents: one JSON object a line with the text under --field (or a .txt file: one document per blank-line-separated
block). Each document becomes its tokens plus the end-of-document token (when the tokenizer has one); its byte count
(for bits per byte) is the UTF-8 length of its text.

--chat: each line is a conversation {"tools": [...], "messages": [{"role", "content", "reasoning", "tool_calls"}]}, rendered
by `data/chat_format.py` with every control token at an id of its own (--first-control upward; default: right after the
tokenizer's vocabulary) and text pieces encoded on their own. The shard set then carries, per token, the `generated` flag
(1 where the assistant produced the token: what `data.loss_mask: assistant` trains on) and the loss-span class (0 plain,
1 / 2 the middle / the head and tail of a tool output, 3 always masked: role headers and other harness text), and per
document the chat flag (`data.chat_whole` keeps such documents off the row boundaries).

--holdout-every K: every K-th document goes to --holdout-out instead (a held-out set that is in no training shard), and its
text is also written to <holdout-out>/docs.jsonl.gz for the probe and recall builders (`--docs`).
Prints the set's counts and fingerprint; the invariants a loss mask relies on are checked by opening the set.
"""

from __future__ import annotations

import argparse
import gzip
import io
import json
import os
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.data import chat_format as CF  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.data import shard_format as SF  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.data.tokenizers import open_tokenizer  # noqa: E402

TOOL_EDGE = 32          # tokens at each end of a tool output that form its head and tail (class 2); the rest is its middle (class 1)


def read_records(paths, field: str, chat: bool):
    for p in paths:
        p = str(p)
        opener = gzip.open if p.endswith(".gz") else open
        with opener(p, "rt", encoding="utf-8") as f:
            if p.endswith((".txt", ".txt.gz")):
                for block in f.read().split("\n\n"):
                    if block.strip():
                        yield block.strip()
                continue
            for line in f:
                if line.strip():
                    rec = json.loads(line)
                    yield rec if chat else rec[field]


def chat_document(conv: dict, tok, control: dict):
    """(ids, generated, loss-span classes, bytes) of one conversation."""
    ids, gen, cls, nbytes = [], [], [], 0
    in_tool = False
    for text, generated, is_control in CF.pieces(conv):
        new = [control[text]] if is_control else list(tok.encode(text))
        nbytes += len(text.encode("utf-8"))
        if is_control and text == CF.TOOL_RESPONSE:
            in_tool = True
        if generated:
            c = [0] * len(new)
        elif in_tool and not is_control:         # a tool output: head and tail apart from the middle
            n = len(new)
            c = [2 if (i < TOOL_EDGE or i >= n - TOOL_EDGE) else 1 for i in range(n)]
        else:
            c = [3] * len(new)                   # harness text: role headers, system / user turns, control tokens nobody generated
        if is_control and text == CF.TOOL_RESPONSE_END:
            in_tool = False
        ids += new
        gen += [int(generated)] * len(new)
        cls += c
    return ids, gen, cls, nbytes


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--eos-token", default=CF.EOT)
    ap.add_argument("--input", action="append", required=True)
    ap.add_argument("--field", default="text")
    ap.add_argument("--chat", action="store_true")
    ap.add_argument("--first-control", type=int, default=0)
    ap.add_argument("--max-docs", type=int, default=0)
    ap.add_argument("--min-tokens", type=int, default=2)
    ap.add_argument("--holdout-every", type=int, default=0)
    ap.add_argument("--holdout-out")
    a = ap.parse_args(argv)
    if bool(a.holdout_every) != bool(a.holdout_out):
        ap.error("--holdout-every and --holdout-out go together")
    tok = open_tokenizer(a.tokenizer, a.eos_token)
    control, vocab = {}, tok.vocab_size
    if a.chat:
        first = a.first_control or tok.vocab_size
        control = {name: first + i for i, name in enumerate(CF.CONTROL_TOKENS)}
        vocab = max(vocab, first + len(CF.CONTROL_TOKENS))
    eos = getattr(tok, "eos_id", None)
    if a.chat and eos is None:
        eos = control[CF.EOT]
    writers = {"train": SF.ShardWriter(a.out, vocab)}
    held_text = None
    if a.holdout_every:
        writers["held"] = SF.ShardWriter(a.holdout_out, vocab)
        raw = open(Path(a.holdout_out) / "docs.jsonl.gz", "wb")
        held_text = io.TextIOWrapper(gzip.GzipFile(filename="", mode="wb", fileobj=raw, mtime=0), encoding="utf-8")
    counts = {"train": 0, "held": 0, "short": 0}
    for n, rec in enumerate(read_records(a.input, a.field, a.chat)):
        if a.max_docs and counts["train"] + counts["held"] >= a.max_docs:
            break
        which = "held" if a.holdout_every and n % a.holdout_every == a.holdout_every - 1 else "train"
        if a.chat:
            ids, gen, cls, nbytes = chat_document(rec, tok, control)
            ids, gen, cls = ids + [eos], gen + [0], cls + [3]
            if len(ids) < a.min_tokens:
                counts["short"] += 1
                continue
            writers[which].add_document(np.asarray(ids), n_bytes=nbytes, generated=np.asarray(gen, dtype=np.uint8), loss_spans=np.asarray(cls, dtype=np.uint8), chat=True)
            text = CF.render(rec)
        else:
            ids = list(tok.encode(rec)) + ([eos] if eos is not None else [])
            if len(ids) < a.min_tokens:
                counts["short"] += 1
                continue
            writers[which].add_document(np.asarray(ids), n_bytes=len(rec.encode("utf-8")))
            text = rec
        counts[which] += 1
        if which == "held" and held_text is not None:
            held_text.write(json.dumps({"id": f"doc{n}", "text": text}, ensure_ascii=False) + "\n")
    for w in writers.values():
        w.close()
    if held_text is not None:
        held_text.close()
    report = {"documents": counts, "vocab_size": vocab}
    for name, path in (("train", a.out), ("held", a.holdout_out)):
        if path and counts[name]:
            s = SF.open_shards([path])            # opening checks the side arrays' invariants
            report[name] = {"path": str(path), "tokens": int(s.n_tokens), "documents": len(s), "fingerprint": s.fingerprint()}
    print(json.dumps(report))
    return 0


if __name__ == "__main__":
    sys.exit(main())
