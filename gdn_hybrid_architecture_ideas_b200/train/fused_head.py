"""LM head fused with the cross-entropy: loss = sum_i a_i ce_i + b_i lse_i^2 over positions, where the logits
h W^T of a chunk of positions are formed, reduced to (ce, lse) and overwritten by their gradient
softmax * (a + 2 b lse) - a * onehot(target) before the next chunk starts; dh and dW come from that gradient, so the
full (N, V) logit matrix never exists and the backward only scales (reference: ced/train/fused_head.py:218-296).

On CUDA each chunk is: tcgen05 GEMM (bf16 operands, fp32 accumulate) -> one online-softmax kernel that writes the
bf16 gradient in place of the logits -> two tcgen05 GEMMs (dh = G W, dW += G^T h).
Targets may be bags (N, s) with weights (N, s) (token-superposition training, fused_head.py:299-372).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

CHUNK = 2048


def _ce_grad_chunk(logits, targets, a, b):
    """(ce (n,), lse (n,), dlogits) for one chunk; targets (n, s), a (n, s) per-target weights (0 = ignored),
    b (n,) z-loss weights. dlogits = softmax * (sum_k a_k + 2 b lse) - sum_k a_k onehot(t_k)."""
    lse = torch.logsumexp(logits, dim=-1)
    picked = logits.gather(1, targets.clamp(min=0))
    ce = ((lse[:, None] - picked) * a).sum(1)
    asum = a.sum(1)
    g = torch.softmax(logits, dim=-1) * (asum + 2.0 * b * lse)[:, None]
    g.scatter_add_(1, targets.clamp(min=0), -a)
    return ce, lse, g


class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, a, b, chunk):
        dt = torch.promote_types(hidden.dtype, torch.float32)
        d = hidden.shape[-1]
        with torch.autocast(hidden.device.type, enabled=False):
            h = hidden.reshape(-1, d).to(dt)
            W = weight.to(dt)
            t = targets.reshape(h.shape[0], -1)
            a2 = a.reshape(h.shape[0], -1).to(dt)
            b1 = b.reshape(-1).to(dt)
            n = h.shape[0]
            ce = torch.empty(n, dtype=dt, device=h.device)
            lse = torch.empty_like(ce)
            dh = torch.empty_like(h)
            dW = torch.zeros_like(W)
            for lo in range(0, n, chunk):
                hi = min(n, lo + chunk)
                c, l, g = _ce_grad_chunk(h[lo:hi] @ W.T, t[lo:hi], a2[lo:hi], b1[lo:hi])
                ce[lo:hi], lse[lo:hi] = c, l
                dh[lo:hi] = g @ W
                dW.addmm_(g.T, h[lo:hi])
            loss = ce.sum() + (b1 * lse * lse).sum()
        ctx.save_for_backward(dh, dW)
        ctx.meta = (hidden.dtype, hidden.shape, weight.dtype)
        ctx.mark_non_differentiable(ce, lse)
        return loss, ce, lse

    @staticmethod
    def backward(ctx, g_loss, g_ce, g_lse):
        dh, dW = ctx.saved_tensors
        hd, hs, wd = ctx.meta
        return (dh * g_loss).to(hd).reshape(hs), (dW * g_loss).to(wd), None, None, None, None


def fused_linear_ce(hidden, weight, targets, a, b, chunk: int | None = None, weight_lp=None):
    """hidden (..., d), weight (V, d), targets (...,) or (..., s), a like targets, b (...,) -> (loss, ce, lse) with
    ce, lse per position and without gradient."""
    if hidden.is_cuda:
        from .. import ops

        if ops.use_native(hidden):
            from ..ops import native

            return native.fused_linear_ce(hidden, weight, targets, a, b, chunk or CHUNK, weight_lp)
    return _FusedLinearCE.apply(hidden, weight, targets, a, b, chunk or CHUNK)


def chunked_ce(hidden, weight, targets, a, b, chunk: int = 1024):
    """Unfused head: checkpointed chunks of fp32 logits through autograd (reference: ced/train/chunked_loss.py:33-140)."""
    import torch.utils.checkpoint as ckpt

    d = hidden.shape[-1]
    h = hidden.reshape(-1, d)
    t = targets.reshape(h.shape[0], -1)
    a2, b1 = a.reshape(h.shape[0], -1), b.reshape(-1)

    def piece(hc, W, tc, ac, bc):
        dt = torch.promote_types(hc.dtype, torch.float32)
        logits = F.linear(hc.to(dt), W.to(dt))
        lse = torch.logsumexp(logits, dim=-1)
        ce = ((lse[:, None] - logits.gather(1, tc.clamp(min=0))) * ac.to(dt)).sum(1)
        return torch.stack([ce.sum() + (bc.to(dt) * lse * lse).sum(), ce.sum()])

    total = 0
    for lo in range(0, h.shape[0], chunk):
        hi = min(h.shape[0], lo + chunk)
        total = total + ckpt.checkpoint(piece, h[lo:hi], weight, t[lo:hi], a2[lo:hi], b1[lo:hi], use_reentrant=False)
    return total[0], total[1]
