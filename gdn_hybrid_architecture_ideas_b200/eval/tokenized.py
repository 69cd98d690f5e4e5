"""Tokenized evaluation documents: ids plus, per token, the UTF-8 bytes it covers, so bits per byte compares across
tokenizers (reference: ced/eval/tokenized.py:1-59). `byte_tokenize` (one token per byte) serves tests and byte-level
models; `hf_tokenize` wraps a `tokenizers.Tokenizer` and attributes whole characters to the token that ends them."""

from __future__ import annotations

from .span_bpb import TokenizedDoc


def byte_tokenize(text: str) -> TokenizedDoc:
    data = text.encode("utf-8")
    return TokenizedDoc(list(data), [1] * len(data))


def hf_tokenize(tokenizer):
    """text -> TokenizedDoc for anything whose encode() gives .ids and character .offsets. A token's bytes are those of the
    characters from the previous token's end to its own end, so the per-document total equals the text's UTF-8 bytes."""
    def run(text: str) -> TokenizedDoc:
        enc = tokenizer.encode(text, add_special_tokens=False)
        prefix = [0]
        for ch in text:
            prefix.append(prefix[-1] + len(ch.encode("utf-8")))
        lens, last = [], 0
        for (_, end) in enc.offsets:
            end = max(end, last)
            lens.append(prefix[end] - prefix[last])
            last = end
        if lens:
            lens[-1] += prefix[len(text)] - prefix[last]
        return TokenizedDoc(list(enc.ids), lens)
    return run
