"""CUDA path of causal document-masked attention with the rotary distance cap: `torch.autograd.Function` over the
tcgen05 flash-attention kernels of csrc/attention.cu (head dimension 64, any query/KV head grouping, optional cap,
optional document ids). Shapes the kernels do not cover (another head dimension) go through the PyTorch statement of
the op one row at a time under activation checkpointing, which bounds memory at one row's score matrix.
"""

from __future__ import annotations

import torch
import torch.utils.checkpoint as ckpt

from . import native
from . import reference as ref

BF16 = torch.bfloat16


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, q_far, k_far, doc32, pos32, cap):
        capped = cap is not None
        qc, kc, vc = (native._bf16(t).contiguous() for t in (q, k, v))
        qf = native._bf16(q_far).contiguous() if capped else None
        kf = native._bf16(k_far).contiguous() if capped else None
        B, L, Hq, hd = qc.shape
        o = torch.empty_like(qc)
        lse = torch.empty(B, Hq, L, dtype=torch.float32, device=q.device)
        native.ext().attention_fwd(qc, qf, kc, kf, vc, o, lse, doc32, pos32, cap if capped else -1, hd ** -0.5, native.err_flag(q.device))
        native._count()
        ctx.save_for_backward(qc, kc, vc, qf, kf, o, lse, pos32)
        ctx.cap, ctx.dtypes = cap, (q.dtype, k.dtype, v.dtype)
        return o

    @staticmethod
    def backward(ctx, dO):
        qc, kc, vc, qf, kf, o, lse, pos32 = ctx.saved_tensors
        capped = ctx.cap is not None
        B, L, Hq, hd = qc.shape
        dq = torch.zeros(qc.shape, dtype=torch.float32, device=qc.device)
        dqf = torch.zeros_like(dq) if capped else None
        dk, dv = torch.empty_like(kc), torch.empty_like(vc)
        dkf = torch.empty_like(kc) if capped else None
        dsum = torch.empty_like(lse)
        native.ext().attention_bwd(qc, qf, kc, kf, vc, o, native._bf16(dO).contiguous(), lse, dsum, dq, dqf, dk, dkf, dv, pos32,
                                   ctx.cap if capped else -1, hd ** -0.5, native.err_flag(qc.device))
        native._count(2)
        qd, kd, vd = ctx.dtypes
        return (dq.to(qd), dk.to(kd), dv.to(vd), dqf.to(qd) if capped else None, dkf.to(kd) if capped else None, None, None, None)


def _row(q, k, v, doc, q_far, k_far, cap):
    L = q.shape[1]
    idx = torch.arange(L, device=q.device)[None]
    return ref.attention(q, k, v, idx, doc, idx, doc, None, q_far, k_far, cap)


def attention(q, k, v, doc, q_far, k_far, cap, pos=None, single_doc=False):
    if q.shape[-1] == 64:
        doc32 = pos32 = None
        if not single_doc:
            doc32 = doc.to(torch.int32).contiguous()
            pos32 = pos.to(torch.int32).contiguous()
        return _Attention.apply(q, k, v, q_far, k_far, doc32, pos32, cap)
    outs = []
    for b in range(q.shape[0]):
        args = [t[b:b + 1] if t is not None else None for t in (q, k, v, doc, q_far, k_far)]
        if torch.is_grad_enabled() and q.requires_grad:
            outs.append(ckpt.checkpoint(_row, *args, cap, use_reentrant=False))
        else:
            outs.append(_row(*args, cap))
    return torch.cat(outs, dim=0)
