"""CUDA path of causal document-masked attention with the rotary distance cap.

Stage 1 (this file today): rows are processed one at a time through the PyTorch statement of the op under
activation checkpointing, which bounds memory at one row's score matrix. Stage 2 replaces it by the tcgen05
flash-attention kernels in csrc/attention_*.cu behind the same signature.
"""

from __future__ import annotations

import torch
import torch.utils.checkpoint as ckpt

from . import reference as ref


def _row(q, k, v, doc, q_far, k_far, cap):
    L = q.shape[1]
    idx = torch.arange(L, device=q.device)[None]
    return ref.attention(q, k, v, idx, doc, idx, doc, None, q_far, k_far, cap)


def attention(q, k, v, doc, q_far, k_far, cap):
    outs = []
    for b in range(q.shape[0]):
        args = [t[b:b + 1] if t is not None else None for t in (q, k, v, doc, q_far, k_far)]
        if torch.is_grad_enabled() and q.requires_grad:
            outs.append(ckpt.checkpoint(_row, *args, cap, use_reentrant=False))
        else:
            outs.append(_row(*args, cap))
    return torch.cat(outs, dim=0)
