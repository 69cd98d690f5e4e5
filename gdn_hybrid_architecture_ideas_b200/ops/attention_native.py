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


# ---------------------------------------------------------------------------------------------------- q / k preparation


class GradSlot:
    """Hands the gate half of the query projection's gradient (written by the output gate's backward, which runs first)
    to the q / k preparation's backward, which fills the query half of the same buffer: the projection gets one dense
    gradient and no slice is ever re-assembled."""

    def __init__(self):
        self.buf = None


class _AttnPrep(torch.autograd.Function):
    """(qg [B, L, Hq * hq_width], k_raw [B, L, Hkv * 64], gains, rotary tables) -> (q, q_far, k, k_far): RMSNorm per head,
    rotation at the token's position, and under the cap the query rotated by the cap and the unrotated normed key."""

    @staticmethod
    def forward(ctx, qg, k_raw, wq, wk, cos, sin, cos_c, sin_c, eps, hq, hkv, interleaved, slot):
        B, L = qg.shape[:2]
        qv = native._bf16(qg).contiguous().view(B, L, hq, 128 if interleaved else 64)[..., :64]
        kv = native._bf16(k_raw).contiguous().view(B, L, hkv, 64)
        dev = qg.device
        capped = cos_c is not None
        qr = torch.empty(B, L, hq, 64, dtype=BF16, device=dev)
        kr = torch.empty(B, L, hkv, 64, dtype=BF16, device=dev)
        qf = torch.empty_like(qr) if capped else None
        kf = torch.empty_like(kr) if capped else None
        wdt = (wq.dtype, wk.dtype)
        wq, wk = wq.detach().float().contiguous(), wk.detach().float().contiguous()
        native.ext().attn_prep_fwd(qv, kv, wq, wk, cos, sin, cos_c, sin_c, eps, qr, qf, kr, kf)
        native._count()
        ctx.save_for_backward(qv, kv, wq, wk, cos, sin, cos_c, sin_c)
        ctx.meta = (eps, interleaved, slot, qg.dtype, k_raw.dtype, qg.shape, k_raw.shape, wdt)
        if not capped:
            qf, kf = qr.new_zeros(0), kr.new_zeros(0)
            ctx.mark_non_differentiable(qf, kf)
        return qr, qf, kr, kf

    @staticmethod
    def backward(ctx, dqr, dqf, dkr, dkf):
        qv, kv, wq, wk, cos, sin, cos_c, sin_c = ctx.saved_tensors
        eps, interleaved, slot, qdt, kdt, qshape, kshape, wdt = ctx.meta
        capped = cos_c is not None
        B, L, hq, _ = qv.shape
        full = slot.buf if (slot is not None and slot.buf is not None) else None
        if full is None:
            full = torch.zeros(B, L, hq * (128 if interleaved else 64), dtype=BF16, device=qv.device) if interleaved else \
                torch.empty(B, L, hq * 64, dtype=BF16, device=qv.device)
        if slot is not None:
            slot.buf = None
        dq_view = full.view(B, L, hq, 128 if interleaved else 64)[..., :64]
        dk = torch.empty(kv.shape, dtype=BF16, device=kv.device)
        dw = torch.zeros(2, 64, dtype=torch.float32, device=qv.device)
        c = lambda t: native._bf16(t).contiguous()
        native.ext().attn_prep_bwd(qv, kv, wq, wk, cos, sin, cos_c, sin_c, eps, c(dqr), c(dqf) if capped else None, c(dkr), c(dkf) if capped else None,
                                   dq_view, dk, dw)
        native._count()
        return (full.view(qshape).to(qdt), dk.view(kshape).to(kdt), dw[0].to(wdt[0]), dw[1].to(wdt[1]), None, None, None, None, None, None, None, None,
                None)


class _GateOut(torch.autograd.Function):
    """y = o * sigmoid(gate), the gate being the second 64 channels of every head of the query projection's output."""

    @staticmethod
    def forward(ctx, o, qg, slot):
        oc, qc = native._bf16(o).contiguous(), native._bf16(qg).contiguous()
        y = torch.empty_like(oc)
        native.ext().gate_out_fwd(oc, qc, y)
        native._count()
        ctx.save_for_backward(oc, qc)
        ctx.slot, ctx.odt, ctx.qdt = slot, o.dtype, qg.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        oc, qc = ctx.saved_tensors
        do = torch.empty_like(oc)
        dqg = torch.empty_like(qc)        # the query half is written by the preparation's backward
        native.ext().gate_out_bwd(native._bf16(dy).contiguous(), oc, qc, do, dqg)
        native._count()
        if ctx.slot is not None:
            ctx.slot.buf = dqg
            return do.to(ctx.odt), None, None
        dqg.view(*qc.shape[:2], -1, 128)[..., :64].zero_()
        return do.to(ctx.odt), dqg.to(ctx.qdt), None


def rotary_tables(pos, r: int, theta: float, cap):
    """cos / sin [tokens, r / 2] fp32 at positions `pos` (angles in float64), and the tables of the cap rotation."""
    inv = theta ** (-torch.arange(0, r, 2, dtype=torch.float64, device=pos.device) / r)
    ang = pos.reshape(-1, 1).to(torch.float64) * inv
    cap_t = (None, None)
    if cap is not None:
        a = float(cap) * inv
        cap_t = (a.cos().float().contiguous(), a.sin().float().contiguous())
    return ang.cos().float().contiguous(), ang.sin().float().contiguous(), cap_t[0], cap_t[1]
