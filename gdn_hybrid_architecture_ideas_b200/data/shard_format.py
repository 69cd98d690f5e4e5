"""Token shards on disk: memory-mapped token ids plus a document index, written once and read by many ranks.

Two on-disk layouts are read through one interface (`len`, `doc(i)`, `doc_len(i)`, `side(name)`, `fingerprint()`):

* this framework's own (`ShardWriter` / `ShardSet`): `tokens.bin` (little-endian uint16 or uint32 ids, all documents
  back to back), `docs.npy` (int64 document end offsets), optional `bytes.npy` (UTF-8 byte length of each document, for
  bits-per-byte), optional per-token side files `generated.bin` / `loss_spans.bin` (uint8) with `chat.npy` (uint8 per
  document), and `meta.json` (vocab size, dtype, counts, a sha256 fingerprint over the index and a sample of the tokens);
* the layout written by the reference's tokenisation tools (`ReferenceLayoutSet`, recognised by its `doc_starts.npy`):
  `tokens.bin` (uint32, or uint16 when meta.json says so), `generated.bin`, optional `byte_lens.bin` and
  `loss_spans.bin` (one uint8 per token), `doc_starts.npy`, `doc_chat.npy`, optional `doc_source.npy`
  (ced/data/shard_format.py:1-60, 216-250), so shard sets tokenised for the reference train here unchanged.

Per-token side arrays: `generated` (1 where the assistant produced the token) and `loss_spans` (a class 0..3 per token:
0 loss everywhere, 1 the middle of a tool output, 2 its first / last 64 content tokens, 3 always masked). They feed the
per-token loss mask (`data.loss_mask`: "all", "assistant", "spans_full" keeps classes 0-2, "spans_head_tail" 0 and 2,
"spans_mask" 0 only); `check_loss_spans` verifies what a mask relies on when a set is opened under one. Several sets can
be read as one union; a union's side arrays are concatenated views (`ConcatView`), never copies.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np

FORMAT = "ghb-shards-1"
LOSS_SPAN_KEEP = {"spans_full": (0, 1, 2), "spans_head_tail": (0, 2), "spans_mask": (0,)}
LOSS_MASK_MODES = ("all", "assistant", *LOSS_SPAN_KEEP)
SIDE_FILES = {"generated": "generated.bin", "loss_spans": "loss_spans.bin"}


def loss_keep_table(mode: str) -> np.ndarray:
    """(256,) bool: whether a target whose loss-span class is the index keeps its loss under span mode `mode`."""
    table = np.zeros(256, dtype=bool)
    table[list(LOSS_SPAN_KEEP[mode])] = True
    return table


class ConcatView:
    """Read-only 1-D concatenation of array-likes (memory maps of several sets) addressed by global offsets, without
    materialising the whole: an integer gives one value, a unit-step slice the concatenated pieces it spans. A missing
    part (None) reads as zeros of its length."""

    def __init__(self, parts: list, lengths: list[int], dtype=np.uint8):
        self.parts, self.dtype = parts, np.dtype(dtype)
        self.bounds = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int64)

    def __len__(self) -> int:
        return int(self.bounds[-1])

    def _piece(self, p: int, a: int, b: int) -> np.ndarray:
        part = self.parts[p]
        return np.zeros(b - a, dtype=self.dtype) if part is None else np.asarray(part[a:b]).astype(self.dtype, copy=False)

    def __getitem__(self, key):
        n = len(self)
        if isinstance(key, (int, np.integer)):
            i = int(key) + (n if key < 0 else 0)
            if not 0 <= i < n:
                raise IndexError(key)
            p = int(np.searchsorted(self.bounds, i, side="right") - 1)
            return self._piece(p, i - int(self.bounds[p]), i - int(self.bounds[p]) + 1)[0]
        a, b, step = key.indices(n)
        if step != 1:
            raise IndexError("ConcatView reads unit-step slices")
        out, p = [], int(np.searchsorted(self.bounds, a, side="right") - 1)
        while a < b:
            lo, hi = int(self.bounds[p]), int(self.bounds[p + 1])
            take = min(b, hi)
            out.append(self._piece(p, a - lo, take - lo))
            a, p = take, p + 1
        return np.concatenate(out) if out else np.zeros(0, dtype=self.dtype)


class ShardWriter:
    def __init__(self, path: str | Path, vocab_size: int):
        self.path = Path(path)
        self.path.mkdir(parents=True, exist_ok=True)
        self.vocab_size = vocab_size
        self.dtype = np.uint16 if vocab_size <= 65536 else np.uint32
        self._file = open(self.path / "tokens.bin", "wb")
        self._ends, self._bytes, self._n = [], [], 0
        self._side, self._chat = {}, []          # per-token side files, opened at the first document that carries one

    def _write_side(self, name: str, values, n: int) -> None:
        f = self._side.get(name)
        if f is None:
            if values is None:
                return
            f = self._side[name] = open(self.path / SIDE_FILES[name], "wb")
            f.write(np.zeros(self._n, dtype=np.uint8).tobytes())        # the documents before carried none: zeros
        arr = np.zeros(n, dtype=np.uint8) if values is None else np.asarray(values)
        if arr.shape != (n,) or arr.min() < 0 or arr.max() > (1 if name == "generated" else 3):
            raise ValueError(f"{name}: one value per token, {'0/1' if name == 'generated' else '0..3'}")
        f.write(arr.astype(np.uint8).tobytes())

    def add_document(self, ids, n_bytes: int | None = None, generated=None, loss_spans=None, chat: bool = False) -> None:
        """generated: 1 per token the assistant produced (chat documents); loss_spans: the loss-span class of every token
        (module docstring). Classes 1 and 2 only in chat documents; no class above 0 on a generated token."""
        arr = np.asarray(ids)
        if arr.ndim != 1 or arr.size == 0:
            raise ValueError("a document is a non-empty 1-D array of token ids")
        if arr.min() < 0 or arr.max() >= self.vocab_size:
            raise ValueError(f"token id outside [0, {self.vocab_size})")
        if loss_spans is not None:
            sp = np.asarray(loss_spans)
            if not chat and bool(((sp == 1) | (sp == 2)).any()):
                raise ValueError("loss-span classes 1 and 2 (tool-output content) outside a chat document")
            if generated is not None and bool(((sp > 0) & (np.asarray(generated) > 0)).any()):
                raise ValueError("a loss-span class above 0 on a generated token")
        if generated is not None and not chat and bool(np.asarray(generated).any()):
            raise ValueError("generated tokens outside a chat document")
        self._write_side("generated", generated, arr.size)
        self._write_side("loss_spans", loss_spans, arr.size)
        self._file.write(arr.astype(self.dtype).tobytes())
        self._n += arr.size
        self._ends.append(self._n)
        self._bytes.append(-1 if n_bytes is None else int(n_bytes))
        self._chat.append(int(bool(chat)))

    def close(self) -> dict:
        self._file.close()
        for f in self._side.values():
            f.close()
        ends = np.asarray(self._ends, dtype=np.int64)
        np.save(self.path / "docs.npy", ends)
        if any(self._chat):
            np.save(self.path / "chat.npy", np.asarray(self._chat, dtype=np.uint8))
        if any(b >= 0 for b in self._bytes):
            np.save(self.path / "bytes.npy", np.asarray(self._bytes, dtype=np.int64))
        meta = {"format": FORMAT, "vocab_size": self.vocab_size, "dtype": np.dtype(self.dtype).name,
                "n_tokens": int(self._n), "n_docs": int(ends.size)}
        if self._side:
            meta["side"] = sorted(self._side)
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
        c = self.path / "chat.npy"
        self.doc_chat = np.load(c) if c.exists() else np.zeros(self.ends.size, dtype=np.uint8)
        self.n_tokens = int(self.ends[-1]) if self.ends.size else 0
        self._sides = {}

    def __len__(self) -> int:
        return int(self.ends.size)

    def side(self, name: str):
        """The per-token side array `name` ("generated", "loss_spans") as a uint8 memory map, or None when the set has none."""
        if name not in self._sides:
            f = self.path / SIDE_FILES[name]
            self._sides[name] = np.memmap(f, dtype=np.uint8, mode="r") if f.exists() and self.n_tokens else None
        return self._sides[name]

    def doc(self, i: int) -> np.ndarray:
        return np.asarray(self.tokens[self.starts[i]:self.ends[i]])

    def doc_len(self, i) -> np.ndarray:
        return self.ends[i] - self.starts[i]

    def fingerprint(self) -> str:
        return self.meta["fingerprint"]


class ReferenceLayoutSet:
    """A shard set in the layout of the reference's tokenisation tools (module docstring), behind the ShardSet interface."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        self.meta = json.loads((self.path / "meta.json").read_text())
        dtype = {"uint32": np.uint32, "uint16": np.uint16}[self.meta.get("token_dtype", "uint32")]
        self.tokens = np.memmap(self.path / "tokens.bin", dtype=dtype, mode="r")
        bounds = np.load(self.path / "doc_starts.npy").astype(np.int64)
        self.starts, self.ends = bounds[:-1], bounds[1:]
        self.n_tokens = int(bounds[-1])
        if len(self.tokens) != self.n_tokens:
            raise ValueError(f"{path}: tokens.bin holds {len(self.tokens)} ids, doc_starts.npy says {self.n_tokens}")
        self.doc_chat = np.load(self.path / "doc_chat.npy")
        src = self.path / "doc_source.npy"
        self.doc_source = np.load(src) if src.exists() else None
        self.sources = self.meta.get("sources", [])
        bl = self.path / "byte_lens.bin"
        self.token_bytes = np.memmap(bl, dtype=np.uint8, mode="r") if bl.exists() else None       # UTF-8 bytes per TOKEN
        self.byte_lens = None if self.token_bytes is None else np.add.reduceat(np.asarray(self.token_bytes, dtype=np.int64), self.starts) \
            if self.n_tokens else np.zeros(0, dtype=np.int64)
        self.vocab_size = int(self.meta.get("vocab_size", 0)) or None
        self._sides = {}

    def __len__(self) -> int:
        return int(self.ends.size)

    def doc(self, i: int) -> np.ndarray:
        return np.asarray(self.tokens[self.starts[i]:self.ends[i]])

    def doc_len(self, i) -> np.ndarray:
        return self.ends[i] - self.starts[i]

    def side(self, name: str):
        if name not in self._sides:
            f = self.path / SIDE_FILES[name]
            self._sides[name] = np.memmap(f, dtype=np.uint8, mode="r") if f.exists() and self.n_tokens else None
        return self._sides[name]

    def fingerprint(self) -> str:
        """The data identity the reference's reader computes for this layout: blake2b-128 over the document index, the chat
        flags and the first and last 65,536 token ids as uint32 (ced/data/shard_format.py:252-268)."""
        h = hashlib.blake2b(digest_size=16)
        h.update(np.concatenate([self.starts, self.ends[-1:]]).astype(np.int64).tobytes())
        h.update(np.asarray(self.doc_chat).tobytes())
        h.update(np.asarray(self.tokens[:65536]).astype("<u4").tobytes())
        h.update(np.asarray(self.tokens[-65536:]).astype("<u4").tobytes())
        return h.hexdigest()


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
        self.n_tokens = sum(s.n_tokens for s in sets)
        self.token_offsets = np.cumsum([0] + [s.n_tokens for s in sets])
        self.doc_chat = np.concatenate([np.asarray(s.doc_chat) for s in sets])
        # document bounds in the union's token numbering (side arrays are addressed by them)
        self.starts = np.concatenate([s.starts + o for s, o in zip(sets, self.token_offsets)])
        self.ends = np.concatenate([s.ends + o for s, o in zip(sets, self.token_offsets)])

    def side(self, name: str):
        parts = [s.side(name) for s in self.sets]
        if all(p is None for p in parts):
            return None
        return ConcatView(parts, [s.n_tokens for s in self.sets])

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


def check_loss_spans(shards, mode: str) -> dict:
    """What a per-token loss mask relies on, verified over a set or a union opened under `mode` ("assistant" or a span
    mode); a ValueError names the token otherwise. `generated` must be 0/1; a span mode needs a `loss_spans` array with
    classes 0..3, classes 1 and 2 only inside chat documents, no class above 0 on a generated token. Returns the identity
    of what was read ({"mode", "class_tokens", "blake2b"}), which a checkpoint keeps so a resume on other span files is
    refused (reference: ced/data/shard_format.py:504-582). One pass in chunks."""
    if mode not in LOSS_MASK_MODES or mode == "all":
        raise ValueError(f"check_loss_spans: mode {mode!r} is one of {LOSS_MASK_MODES[1:]}")
    gen, spans = shards.side("generated"), shards.side("loss_spans")
    span_mode = mode in LOSS_SPAN_KEEP
    if span_mode and spans is None:
        raise ValueError(f"data.loss_mask {mode!r} reads the loss-span classes ({SIDE_FILES['loss_spans']}), and the shard set has none")
    if not span_mode and gen is None:
        raise ValueError(f"data.loss_mask {mode!r} reads the generated flags ({SIDE_FILES['generated']}), and the shard set has none")
    n = shards.n_tokens
    counts, digest = np.zeros(256, dtype=np.int64), hashlib.blake2b(digest_size=16)
    chat_tok = None
    for a in range(0, n, 1 << 22):
        b = min(n, a + (1 << 22))
        g = np.zeros(b - a, dtype=np.uint8) if gen is None else np.asarray(gen[a:b])
        if g.size and int(g.max()) > 1:
            raise ValueError(f"generated flags hold {int(g.max())} at token {a + int(np.argmax(g > 1))}: they must be 0/1 under a loss mask")
        if not span_mode:
            continue
        sp = np.ascontiguousarray(spans[a:b])
        counts += np.bincount(sp, minlength=256)
        digest.update(sp.tobytes())
        if sp.size and int(sp.max()) > 3:
            raise ValueError(f"loss-span class {int(sp.max())} at token {a + int(np.argmax(sp > 3))}: the classes are 0..3")
        clash = (sp > 0) & (g > 0)
        if bool(clash.any()):
            raise ValueError(f"loss-span class {int(sp[np.argmax(clash)])} on a generated token at token {a + int(np.argmax(clash))}")
        inner = (sp == 1) | (sp == 2)
        if bool(inner.any()):
            if chat_tok is None:      # 1 where the token lies in a chat document
                chat_tok = np.repeat(np.asarray(shards.doc_chat).astype(bool), np.asarray(shards.ends - shards.starts))
            outside = inner & ~chat_tok[a:b]
            if bool(outside.any()):
                raise ValueError(f"loss-span class {int(sp[np.argmax(outside)])} at token {a + int(np.argmax(outside))}, outside a chat document")
    out = {"mode": mode}
    if span_mode:
        out.update(class_tokens={str(c): int(counts[c]) for c in range(4)}, blake2b=digest.hexdigest())
    return out


def _open_one(d):
    return ReferenceLayoutSet(d) if (Path(d) / "doc_starts.npy").exists() else ShardSet(d)


def open_shards(dirs, order: str = "permute"):
    sets = [_open_one(d) for d in dirs if d]
    if not sets:
        raise ValueError("data.kind 'shards' needs data.shard_dir")
    return sets[0] if len(sets) == 1 else ShardUnion(sets, order)
