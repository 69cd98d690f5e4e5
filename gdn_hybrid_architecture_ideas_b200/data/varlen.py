"""Cumulative sequence lengths of the documents in a flattened batch, in a plain and a fixed-capacity form.

The fixed-capacity form pads the boundary vector to a length that depends only on (rows, seq_len, docs_per_row), with
empty segments and a sentinel, so a CUDA graph captured once replays for any document layout
(reference: ced/train/varlen.py:33-120)."""

from __future__ import annotations

import numpy as np
import torch


def cu_seqlens_host(doc_ids: torch.Tensor) -> np.ndarray:
    d = doc_ids.cpu().numpy()
    B, L = d.shape
    change = np.ones((B, L), dtype=bool)
    change[:, 1:] = d[:, 1:] != d[:, :-1]
    starts = np.nonzero(change.reshape(-1))[0]
    return np.concatenate([starts, [B * L]]).astype(np.int32)


def fixed_capacity(rows: int, docs_per_row: int) -> int:
    return rows * docs_per_row + 2


def fixed_varlen_host(doc_ids: torch.Tensor, docs_per_row: int) -> np.ndarray:
    cu = cu_seqlens_host(doc_ids)
    cap = fixed_capacity(doc_ids.shape[0], docs_per_row)
    if cu.size > cap - 1:
        raise ValueError(f"{cu.size - 1} documents exceed the fixed capacity of {cap - 2} segments")
    total = doc_ids.numel()
    out = np.full(cap, total, dtype=np.int32)
    out[:cu.size] = cu
    return out


def to_device(cu: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(cu)).to(device, non_blocking=True)
