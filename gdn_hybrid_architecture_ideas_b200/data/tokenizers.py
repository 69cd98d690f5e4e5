"""Tokenizer identity: evaluation sets record the sha256 of the tokenizer file they were built with, and scoring
refuses a mismatch (reference: ced/data/tokenizers.py:24-42)."""

from __future__ import annotations

import hashlib
from pathlib import Path


def tokenizer_sha256(path: str | Path) -> str:
    return hashlib.sha256(Path(path).read_bytes()).hexdigest()


def check_tokenizer(path: str | Path, expected: str) -> None:
    got = tokenizer_sha256(path)
    if got != expected:
        raise ValueError(f"tokenizer {path} has sha256 {got[:12]}..., the evaluation set was built with {expected[:12]}...")


class ByteTokenizer:
    """UTF-8 bytes as token ids 0..255 (tests, and models trained on bytes)."""

    name = "bytes"
    vocab_size = 256
    eos_id = None

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids) -> str:
        return bytes(int(i) & 255 for i in ids).decode("utf-8", errors="replace")


class FileTokenizer:
    """A tokenizer file: `tokenizer.json` (the `tokenizers` library, through transformers' fast tokenizer) or a
    SentencePiece `.model`. Only encode / decode / vocabulary size / end-of-document id are used."""

    def __init__(self, path: str | Path, eos_token: str | None = None):
        self.path = Path(path)
        self.name = self.path.name
        if self.path.suffix == ".model":
            import sentencepiece as spm

            sp = spm.SentencePieceProcessor(model_file=str(self.path))
            self.encode, self.decode = (lambda t: sp.encode(t)), (lambda ids: sp.decode([int(i) for i in ids]))
            self.vocab_size, self.eos_id = sp.get_piece_size(), (sp.eos_id() if sp.eos_id() >= 0 else None)
        else:
            from tokenizers import Tokenizer

            tk = Tokenizer.from_file(str(self.path))
            self.encode = lambda t: tk.encode(t, add_special_tokens=False).ids
            self.decode = lambda ids: tk.decode([int(i) for i in ids], skip_special_tokens=False)
            self.vocab_size = tk.get_vocab_size()
            self.eos_id = tk.token_to_id(eos_token) if eos_token else None


def open_tokenizer(spec: str, eos_token: str | None = None):
    """"bytes" or a path to a tokenizer file."""
    return ByteTokenizer() if spec == "bytes" else FileTokenizer(spec, eos_token)
