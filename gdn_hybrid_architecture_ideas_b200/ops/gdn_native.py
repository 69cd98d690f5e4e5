"""CUDA path of the chunked gated delta rule (forward and backward).

Two stages. The chunk-local stage (cumulative decays, the (I + A)^-1 solve giving U and W, the intra-chunk score
matrix, document masks) is independent across chunks; the sequential stage carries the state across chunks. The
sequential stage is the hand-written tcgen05 kernel pair of csrc/gdn_scan.cu behind `_Scan` (key dimension 128, value
dimension a multiple of 128, chunk 64). The chunk-local stage currently runs as batched fp32 device ops with autograd
(`reference.chunk_local`); its operands are handed to the scan in bfloat16.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import native
from . import reference as ref

BF16 = torch.bfloat16
CHUNK = 64


class _Scan(torch.autograd.Function):
    """(U, W, q_in, Aqk, k_out, carry, S0) -> (o, S_final); tensors [B, H, L, *] bf16, carry [B, H, L/64] fp32."""

    @staticmethod
    def forward(ctx, U, W, Qin, Aqk, Kout, carry, S0, need_state):
        B, H, L, dv = U.shape
        dev = U.device
        needs_grad = any(ctx.needs_input_grad[:7])
        O = torch.empty_like(U)
        Sfinal = torch.empty(B, H, 128, dv, dtype=torch.float32, device=dev) if need_state else None
        Hsave = torch.empty(B, H, L // CHUNK, dv, 128, dtype=BF16, device=dev) if needs_grad else None
        Vnew = torch.empty_like(U) if needs_grad else None
        native.ext().gdn_scan_fwd(W, Qin, Kout, Aqk, U, carry, S0, O, Sfinal, Hsave, Vnew, native.err_flag(dev))
        native._count()
        ctx.save_for_backward(W, Qin, Kout, Aqk, carry, Hsave, Vnew)
        ctx.has_s0 = S0 is not None
        if Sfinal is None:
            Sfinal = torch.zeros(0, device=dev)
            ctx.mark_non_differentiable(Sfinal)
        return O, Sfinal

    @staticmethod
    def backward(ctx, dO, dSfinal):
        W, Qin, Kout, Aqk, carry, Hsave, Vnew = ctx.saved_tensors
        B, H, L, dv = Vnew.shape
        dev = W.device
        nvs = dv // 128
        dO = native._bf16(dO).contiguous()
        dU = torch.empty_like(Vnew)
        parts = torch.empty(3, nvs, B, H, L, 128, dtype=torch.float32, device=dev)
        dcarry = torch.zeros_like(carry)
        dS0 = torch.empty(B, H, 128, dv, dtype=torch.float32, device=dev) if ctx.has_s0 else None
        dSf = dSfinal.float().contiguous() if (dSfinal is not None and dSfinal.numel()) else None
        native.ext().gdn_scan_bwd(W, Qin, Kout, Aqk, Hsave.view(-1, 128), Vnew, dO, carry, dSf, dU, parts[0], parts[1], parts[2], dcarry, dS0,
                                  native.err_flag(dev))
        native._count()
        dW, dQ, dK = (parts[i].sum(0).to(BF16) if nvs > 1 else parts[i, 0].to(BF16) for i in range(3))
        n = L // CHUNK
        dA = torch.matmul(dO.view(B, H, n, CHUNK, dv), Vnew.view(B, H, n, CHUNK, dv).transpose(-1, -2)).view(B, H, L, CHUNK)
        return dU, dW, dQ, dA, dK, dcarry, dS0, None


class _Local(torch.autograd.Function):
    """Chunk-local stage on the device kernels of csrc/gdn_local.cu: (q, k, v, g, beta, starts) -> (U, W, q_in, Aqk, k_out,
    carry), inputs token-major [B, L, H, *] (strided views are fine), outputs [B, Hv, L, *]."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, start_u8):
        B, L, Hv, dv = v.shape
        dev = v.device

        def out(d, dtype=BF16):
            return torch.empty(B, Hv, L, d, dtype=dtype, device=dev)

        U, W, Aqk, Qin, Kout = out(dv), out(128), out(CHUNK), out(128), out(128)
        carry = torch.empty(B, Hv, L // CHUNK, dtype=torch.float32, device=dev)
        native.ext().gdn_local_fwd(q, k, v, g, beta, start_u8, U, W, Aqk, Qin, Kout, carry)
        native._count()
        ctx.save_for_backward(q, k, v, g, beta, start_u8, U, W)
        return U, W, Qin, Aqk, Kout, carry

    @staticmethod
    def backward(ctx, dU, dW, dQin, dAqk, dKout, dcarry):
        q, k, v, g, beta, start_u8, U, W = ctx.saved_tensors
        B, L, Hv, dv = v.shape
        Hk = q.shape[2]
        dev = v.device
        dq = torch.empty(B, L, Hv, 128, dtype=torch.float32, device=dev)
        dk = torch.empty_like(dq)
        dv_ = torch.empty(B, L, Hv, dv, dtype=BF16, device=dev)
        dg = torch.empty(B, L, Hv, dtype=torch.float32, device=dev)
        dbeta = torch.empty_like(dg)
        c = lambda t: native._bf16(t).contiguous()
        native.ext().gdn_local_bwd(q, k, v, g, beta, start_u8, U, W, c(dU), c(dW), c(dQin), c(dKout), c(dAqk), dcarry.float().contiguous(), dq, dk, dv_, dg, dbeta)
        native._count()
        if Hv != Hk:
            dq = dq.view(B, L, Hk, Hv // Hk, 128).sum(3)
            dk = dk.view(B, L, Hk, Hv // Hk, 128).sum(3)
        return dq.to(q.dtype), dk.to(k.dtype), dv_.to(v.dtype), dg, dbeta, None


def _tok_major_ok(t) -> bool:
    return (t.dtype == BF16 and t.stride(3) == 1 and t.stride(2) == t.shape[3] and t.stride(0) == t.stride(1) * t.shape[1]
            and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0)


def supported(q, v) -> bool:
    return q.shape[-1] == 128 and v.shape[-1] % 128 == 0


def delta_rule(q, k, v, g, beta, is_doc_start, S0, chunk_size, need_state):
    """q, k: [B, L, Hk, dk]; v: [B, L, Hv, dv]; g, beta: [B, L, Hv]. Returns (o [B, L, Hv, dv], final state or None)."""
    B, L, Hk, dk = q.shape
    Hv, dv = v.shape[2], v.shape[3]
    if not (dk == 128 and dv in (128, 256) and chunk_size == CHUNK):
        rep = Hv // Hk
        if rep > 1:
            q, k = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
        if S0 is None:
            S0 = torch.zeros(B, Hv, dk, dv, dtype=torch.float32, device=q.device)
        o, S = ref.chunked_delta_rule(q.float(), k.float(), v.float(), g.float(), beta.float(), is_doc_start, S0.float(), chunk_size)
        return o.to(v.dtype), S
    pad = (-L) % CHUNK
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
        g, beta = (F.pad(t, (0, 0, 0, pad)) for t in (g, beta))
        is_doc_start = F.pad(is_doc_start, (0, pad))
    q, k, v = (t if _tok_major_ok(t) else native._bf16(t).contiguous() for t in (q, k, v))
    U, W, Qin, Aqk, Kout, carry = _Local.apply(q, k, v, g.float().contiguous(), beta.float().contiguous(),
                                               is_doc_start.to(torch.uint8).contiguous())
    O, S = _Scan.apply(U, W, Qin, Aqk, Kout, carry, None if S0 is None else S0.float().contiguous(), need_state)
    o = O[:, :, :L].transpose(1, 2)
    return o, (S if need_state else None)
