"""CUDA path of the chunked gated delta rule (forward and backward).

Stage 1 (this file today): the chunk-local quantities and the sequential state pass run as batched fp32 PyTorch
kernels on the device (`reference.chunk_local` / `chunk_scan`), value heads sharing key heads by indexing.
Stage 2 replaces both by the hand-written sm_100a kernels in csrc/gdn_*.cu behind the same signature.
"""

from __future__ import annotations

import torch

from . import reference as ref


def delta_rule(q, k, v, g, beta, is_doc_start, S0, chunk_size, need_state):
    rep = v.shape[2] // q.shape[2]
    if rep > 1:
        q, k = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
    if S0 is None:
        S0 = torch.zeros(q.shape[0], v.shape[2], q.shape[-1], v.shape[-1], dtype=torch.float32, device=q.device)
    o, S = ref.chunked_delta_rule(q.float(), k.float(), v.float(), g.float(), beta.float(), is_doc_start, S0.float(), chunk_size)
    return o.to(v.dtype), S
