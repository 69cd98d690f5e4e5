"""Token shards on disk: memory-mapped token ids plus a document index, written once and read by many ranks.

A shard set is a directory with `tokens.bin` (little-endian uint16 or uint32 ids, all documents back to back),
`docs.npy` (int64 document end offsets), optional `bytes.npy` (UTF-8 byte length of each document, for bits-per-byte)
and `meta.json` (vocab size, dtype, counts, a sha256 fingerprint over the index and a sample of the tokens). Several
sets can be read as one union (reference: ced/data/shard_format.py:94-593 — same roles, own layout).
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np

FORMAT = "ghb-shards-1"


class ShardWriter:
    def __init__(self, path: str | Path, vocab_size: int):
        self.path = Path(path)
        self.path.mkdir(parents=True, exist_ok=True)
        self.vocab_size = vocab_size
        self.dtype = np.uint16 if vocab_size <= 65536 else np.uint32
        self._file = open(self.path / "tokens.bin", "wb")
        self._ends, self._bytes, self._n = [], [], 0

    def add_document(self, ids, n_bytes: int | None = None) -> None:
        arr = np.asarray(ids)
        if arr.ndim != 1 or arr.size == 0:
            raise ValueError("a document is a non-empty 1-D array of token ids")
        if arr.min() < 0 or arr.max() >= self.vocab_size:
            raise ValueError(f"token id outside [0, {self.vocab_size})")
        self._file.write(arr.astype(self.dtype).tobytes())
        self._n += arr.size
        self._ends.append(self._n)
        self._bytes.append(-1 if n_bytes is None else int(n_bytes))

    def close(self) -> dict:
        self._file.close()
        ends = np.asarray(self._ends, dtype=np.int64)
        np.save(self.path / "docs.npy", ends)
        if any(b >= 0 for b in self._bytes):
            np.save(self.path / "bytes.npy", np.asarray(self._bytes, dtype=np.int64))
        meta = {"format": FORMAT, "vocab_size": self.vocab_size, "dtype": np.dtype(self.dtype).name,
                "n_tokens": int(self._n), "n_docs": int(ends.size)}
        meta["fingerprint"] = _fingerprint(self.path, meta)
        (self.path / "meta.json").write_text(json.dumps(meta, indent=1))
        return meta

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def _fingerprint(path: Path, meta: dict) -> str:
    h = hashlib.sha256(json.dumps({k: meta[k] for k in ("format", "vocab_size", "dtype", "n_tokens", "n_docs")}, sort_keys=True).encode())
    h.update(np.load(path / "docs.npy").tobytes())
    tokens = np.memmap(path / "tokens.bin", dtype=meta["dtype"], mode="r")
    h.update(np.ascontiguousarray(tokens[:: max(1, tokens.size // 65536)]).tobytes())
    return h.hexdigest()


class ShardSet:
    def __init__(self, path: str | Path):
        self.path = Path(path)
        self.meta = json.loads((self.path / "meta.json").read_text())
        if self.meta.get("format") != FORMAT:
            raise ValueError(f"{path}: not a {FORMAT} shard set")
        self.tokens = np.memmap(self.path / "tokens.bin", dtype=self.meta["dtype"], mode="r")
        self.ends = np.load(self.path / "docs.npy")
        self.starts = np.concatenate([[0], self.ends[:-1]])
        b = self.path / "bytes.npy"
        self.byte_lens = np.load(b) if b.exists() else None
        self.vocab_size = self.meta["vocab_size"]

    def __len__(self) -> int:
        return int(self.ends.size)

    def doc(self, i: int) -> np.ndarray:
        return np.asarray(self.tokens[self.starts[i]:self.ends[i]])

    def doc_len(self, i) -> np.ndarray:
        return self.ends[i] - self.starts[i]

    def fingerprint(self) -> str:
        return self.meta["fingerprint"]


class ShardUnion:
    """Several shard sets as one document collection; `order` "permute" mixes their documents in one epoch
    permutation, "sets_in_order" reads the sets one after another."""

    def __init__(self, sets: list[ShardSet], order: str = "permute"):
        if order not in ("permute", "sets_in_order"):
            raise ValueError(f"data.union_order {order!r}")
        if len({s.vocab_size for s in sets}) != 1:
            raise ValueError("shard sets of a union must share a vocabulary size")
        self.sets, self.order = sets, order
        self.offsets = np.cumsum([0] + [len(s) for s in sets])
        self.vocab_size = sets[0].vocab_size

    def __len__(self) -> int:
        return int(self.offsets[-1])

    def _locate(self, i: int):
        s = int(np.searchsorted(self.offsets, i, side="right") - 1)
        return self.sets[s], i - int(self.offsets[s])

    def doc(self, i: int) -> np.ndarray:
        s, j = self._locate(i)
        return s.doc(j)

    def doc_len(self, i):
        i = np.asarray(i)
        out = np.empty(i.shape, dtype=np.int64)
        which = np.searchsorted(self.offsets, i, side="right") - 1
        for s, shard in enumerate(self.sets):
            m = which == s
            out[m] = shard.doc_len(i[m] - self.offsets[s])
        return out

    def fingerprint(self) -> str:
        return hashlib.sha256("|".join([self.order] + [s.fingerprint() for s in self.sets]).encode()).hexdigest()


def open_shards(dirs, order: str = "permute"):
    sets = [ShardSet(d) for d in dirs if d]
    if not sets:
        raise ValueError("data.kind 'shards' needs data.shard_dir")
    return sets[0] if len(sets) == 1 else ShardUnion(sets, order)
