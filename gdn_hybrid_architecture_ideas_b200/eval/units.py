"""Resumable scoring units: results are written one unit at a time with atomic renames, keyed by a hash of the unit's
definition and a fingerprint of what produced them, so an interrupted evaluation continues where it stopped and a
changed input invalidates only its own units (reference: ced/eval/units.py:45-177)."""

from __future__ import annotations

import hashlib
import json
import os
from pathlib import Path


def write_atomic(path, text: str) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(path.name + f".tmp{os.getpid()}")
    with open(tmp, "w") as f:
        f.write(text)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def file_fingerprint(path, edge: int = 1 << 20) -> dict:
    """Size plus sha256 of the first and last `edge` bytes (cheap identity of a large file)."""
    p = Path(path)
    size = p.stat().st_size
    h = hashlib.sha256()
    with open(p, "rb") as f:
        h.update(f.read(edge))
        if size > edge:
            f.seek(max(size - edge, edge))
            h.update(f.read(edge))
    return {"size": size, "sha256_edges": h.hexdigest()}


def key_hash(key) -> str:
    return hashlib.sha256(json.dumps(key, sort_keys=True).encode()).hexdigest()[:16]


class UnitStore:
    def __init__(self, root, fingerprint: dict):
        self.root, self.fp = Path(root), fingerprint
        self.root.mkdir(parents=True, exist_ok=True)

    def path(self, key) -> Path:
        return self.root / f"{key_hash(key)}.json"

    def get(self, key):
        p = self.path(key)
        if not p.exists():
            return None
        rec = json.loads(p.read_text())
        return rec["value"] if rec.get("fingerprint") == self.fp and rec.get("key") == key else None

    def put(self, key, value) -> None:
        write_atomic(self.path(key), json.dumps({"key": key, "fingerprint": self.fp, "value": value}))

    def run(self, key, fn):
        """fn() once per (key, fingerprint); later calls read the stored value."""
        got = self.get(key)
        if got is None:
            got = fn()
            self.put(key, got)
        return got
