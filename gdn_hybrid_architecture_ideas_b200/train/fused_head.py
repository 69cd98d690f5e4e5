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
CE_FORMS = ("standard", "fixed")


def check_ce_form(form: str) -> bool:
    """True for "fixed" (reference: ced/train/ce_fix.py:55-90)."""
    if form not in CE_FORMS:
        raise ValueError(f"loss.ce_form {form!r}: one of {CE_FORMS} ('fixed': softplus(LSE_(j != t) z_j - z_t), whose target gradient "
                         "-sigmoid keeps its accuracy where softmax_t - 1 rounds to 0)")
    return form == "fixed"


def sigmoid_stable(x: torch.Tensor) -> torch.Tensor:
    e = torch.exp(-x.abs())
    return torch.where(x < 0, e, torch.ones_like(e)) / (1.0 + e)


def fixed_terms(logits: torch.Tensor, targets: torch.Tensor):
    """(z_t (n, K), L' (n, K), lse (n,)) of the fixed cross-entropy, L'_k = LSE_(j != t_k)(z_j) - z_(t_k). Only the row's
    argmax can have a softmax within rounding of 1, so only its column needs the log-sum-exp without it; every other
    target has p <= 1/2 and L' = (lse - z_t) + log1p(-p) without cancellation (reference: ced/train/ce_fix.py:151-170)."""
    xt = logits.gather(1, targets)
    am = logits.argmax(dim=-1, keepdim=True)
    zam = logits.gather(1, am).squeeze(1)
    lse_am = torch.logsumexp(logits.scatter(1, am, float("-inf")), dim=-1)
    lse = torch.logaddexp(lse_am, zam)
    lp_other = (lse[:, None] - xt) + torch.log1p(-torch.exp(xt - lse[:, None]).clamp(max=0.75))
    return xt, torch.where(targets == am, (lse_am - zam)[:, None], lp_other), lse


def _ce_grad_chunk(logits, targets, a, b, fixed: bool = False):
    """(ce (n,), lse (n,), dlogits) for one chunk; targets (n, s), a (n, s) per-target weights (0 = ignored),
    b (n,) z-loss weights. dlogits = softmax * (sum_k a_k + 2 b lse) - sum_k a_k onehot(t_k); with the fixed form a term's
    loss is softplus(L'_k) and column j of the targets gets (A - A_j + 2 b lse) softmax_j - A_j sigmoid(L'_j), A_j the
    weight of the terms whose target is j (reference: ced/train/ce_fix.py:130-150, 176-190)."""
    if fixed:
        t = targets.clamp(min=0)
        xt, lp, lse = fixed_terms(logits, t)
        ce = (torch.logaddexp(lp, torch.zeros_like(lp)) * a).sum(1)
        asum = a.sum(1)
        g = torch.exp(logits - lse[:, None]) * (asum + 2.0 * b * lse)[:, None]
        a_j = (a[:, None, :] * (t[:, :, None] == t[:, None, :])).sum(-1)
        val = (asum[:, None] - a_j + (2.0 * b * lse)[:, None]) * torch.exp(xt - lse[:, None]) - a_j * sigmoid_stable(lp)
        live = a != 0
        for k in range(t.shape[1]):
            col = t[:, k:k + 1]
            g.scatter_(1, col, torch.where(live[:, k:k + 1], val[:, k:k + 1], g.gather(1, col)))
        return ce, lse, g
    lse = torch.logsumexp(logits, dim=-1)
    picked = logits.gather(1, targets.clamp(min=0))
    ce = ((lse[:, None] - picked) * a).sum(1)
    asum = a.sum(1)
    g = torch.softmax(logits, dim=-1) * (asum + 2.0 * b * lse)[:, None]
    g.scatter_add_(1, targets.clamp(min=0), -a)
    return ce, lse, g


class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, a, b, chunk, fixed=False, precision="fp32"):
        from .head_precision import addmm_acc_, mm_acc

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
                c, l, g = _ce_grad_chunk(mm_acc(h[lo:hi], W.T, precision), t[lo:hi], a2[lo:hi], b1[lo:hi], fixed)
                ce[lo:hi], lse[lo:hi] = c, l
                dh[lo:hi] = mm_acc(g, W, precision)
                addmm_acc_(dW, g.T, h[lo:hi], precision)
            loss = ce.sum() + (b1 * lse * lse).sum()
        ctx.save_for_backward(dh, dW)
        ctx.meta = (hidden.dtype, hidden.shape, weight.dtype)
        ctx.mark_non_differentiable(ce, lse)
        return loss, ce, lse

    @staticmethod
    def backward(ctx, g_loss, g_ce, g_lse):
        dh, dW = ctx.saved_tensors
        hd, hs, wd = ctx.meta
        return (dh * g_loss).to(hd).reshape(hs), (dW * g_loss).to(wd), None, None, None, None, None, None


def fused_linear_ce(hidden, weight, targets, a, b, chunk: int | None = None, weight_lp=None, ce_form: str = "standard", precision: str = "fp32"):
    """hidden (..., d), weight (V, d), targets (...,) or (..., s), a like targets, b (...,) -> (loss, ce, lse) with
    ce, lse per position and without gradient. precision: the form of the PyTorch statements (train/head_precision.py); the
    native kernels are the "bf16" form."""
    from .head_precision import check_head_precision

    fixed = check_ce_form(ce_form)
    check_head_precision(precision)
    if hidden.is_cuda:
        from .. import ops

        if ops.use_native(hidden):
            from ..ops import native

            return native.fused_linear_ce(hidden, weight, targets, a, b, chunk or CHUNK, weight_lp, fixed)
    return _FusedLinearCE.apply(hidden, weight, targets, a, b, chunk or CHUNK, fixed, precision)


def chunked_ce(hidden, weight, targets, a, b, chunk: int = 1024, ce_form: str = "standard", precision: str = "fp32"):
    """Unfused head: checkpointed chunks of fp32 logits through autograd (reference: ced/train/chunked_loss.py:33-140).
    With the fixed form each term masks its own target column out of the log-sum-exp, so autograd's target gradient is
    -sigmoid(L') exactly (reference: ced/train/ce_fix.py:94-120)."""
    import torch.utils.checkpoint as ckpt

    fixed = check_ce_form(ce_form)

    d = hidden.shape[-1]
    h = hidden.reshape(-1, d)
    t = targets.reshape(h.shape[0], -1)
    a2, b1 = a.reshape(h.shape[0], -1), b.reshape(-1)

    def piece(hc, W, tc, ac, bc):
        from .head_precision import head_linear

        dt = torch.promote_types(hc.dtype, torch.float32)
        logits = head_linear(hc.to(dt), W.to(dt), precision)
        if fixed:
            tcl = tc.clamp(min=0)
            ces, lse = [], None
            for k in range(tcl.shape[1]):
                col = tcl[:, k:k + 1]
                zt = logits.gather(1, col).squeeze(1)
                lse_nt = torch.logsumexp(logits.scatter(1, col, float("-inf")), dim=-1)
                ces.append(torch.logaddexp(lse_nt - zt, torch.zeros_like(zt)))
                if lse is None:
                    lse = torch.logaddexp(lse_nt, zt)
            ce = (torch.stack(ces, 1) * ac.to(dt)).sum(1)
            return torch.stack([ce.sum() + (bc.to(dt) * lse * lse).sum(), ce.sum()])
        lse = torch.logsumexp(logits, dim=-1)
        ce = ((lse[:, None] - logits.gather(1, tc.clamp(min=0))) * ac.to(dt)).sum(1)
        return torch.stack([ce.sum() + (bc.to(dt) * lse * lse).sum(), ce.sum()])

    total = 0
    for lo in range(0, h.shape[0], chunk):
        hi = min(h.shape[0], lo + chunk)
        total = total + ckpt.checkpoint(piece, h[lo:hi], weight, t[lo:hi], a2[lo:hi], b1[lo:hi], use_reentrant=False)
    return total[0], total[1]
