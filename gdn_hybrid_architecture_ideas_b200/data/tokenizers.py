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
