"""CUDA path of the chunked gated delta rule (forward and backward).

Two stages. The chunk-local stage (cumulative decays, the (I + A)^-1 solve giving U and W, the intra-chunk score
matrix, document masks) is independent across chunks; the sequential stage carries the state across chunks. The
sequential stage is the hand-written tcgen05 kernel pair of csrc/gdn_scan.cu (key dimension 128, value dimension 128 or
256, chunk 64); the chunk-local stage is the kernel pair of csrc/gdn_local.cu. `_DeltaRule` chains the four launches.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import native
from . import reference as ref

BF16 = torch.bfloat16
CHUNK = 64


def _unpack(qkv, hk, hv, dk, dv):
    """Token-major views (q, k, v) of a packed [B, L, hk dk | hk dk | hv dv] tensor."""
    B, L, _ = qkv.shape
    nq = hk * dk
    return (qkv[..., :nq].view(B, L, hk, dk), qkv[..., nq:2 * nq].view(B, L, hk, dk), qkv[..., 2 * nq:].view(B, L, hv, dv))


class _DeltaRule(torch.autograd.Function):
    """(qkv, g, beta, starts, S0) -> (o [B, L, Hv, dv], S_final); qkv packs q | k | v per token ([B, L, C] bf16).
    Forward: the chunk-local kernel writes U, W, q_in, Aqk, k_out [B, Hv, L, *] and the per-chunk carry, the state scan
    consumes them and writes the output token-major. Backward: the state scan's backward leaves dU and fp32 partial
    sums (one per 128-wide value slice) of dW, dq_in, dk_out; the chunk-local backward reads those directly, forms
    dAqk = dO v_new^T itself and writes dq | dk | dv into one packed gradient (fp32 dq, dk and a head-group sum when
    several value heads share a key head)."""

    @staticmethod
    def forward(ctx, qkv, g, beta, start_u8, S0, need_state, hk, hv, dk, dv):
        q, k, v = _unpack(qkv, hk, hv, dk, dv)
        B, L, Hv, _ = v.shape
        dev = v.device
        ex = native.ext()
        needs_grad = any(ctx.needs_input_grad[:5])

        def buf(d, dtype=BF16):
            return torch.empty(B, Hv, L, d, dtype=dtype, device=dev)

        U, W, Aqk, Qin, Kout = buf(dv), buf(128), buf(CHUNK), buf(128), buf(128)
        carry = torch.empty(B, Hv, L // CHUNK, dtype=torch.float32, device=dev)
        ex.gdn_local_fwd(q, k, v, g, beta, start_u8, U, W, Aqk, Qin, Kout, carry)
        O = torch.empty(B, L, Hv, dv, dtype=BF16, device=dev)
        Sfinal = torch.empty(B, Hv, 128, dv, dtype=torch.float32, device=dev) if need_state else None
        Hsave = torch.empty(B, Hv, L // CHUNK, dv, 128, dtype=BF16, device=dev) if needs_grad else None
        Vnew = torch.empty_like(U) if needs_grad else None
        ex.gdn_scan_fwd(W, Qin, Kout, Aqk, U, carry, S0, O, Sfinal, Hsave, Vnew, native.err_flag(dev))
        native._count(2)
        if needs_grad:
            ctx.save_for_backward(qkv, g, beta, start_u8, U, W, Qin, Kout, Aqk, carry, Hsave, Vnew)
        ctx.has_s0, ctx.dims = S0 is not None, (hk, hv, dk, dv)
        if Sfinal is None:
            Sfinal = torch.zeros(0, device=dev)
            ctx.mark_non_differentiable(Sfinal)
        return O, Sfinal

    @staticmethod
    def backward(ctx, dO, dSfinal):
        qkv, g, beta, start_u8, U, W, Qin, Kout, Aqk, carry, Hsave, Vnew = ctx.saved_tensors
        hk, hv, dk_, dv = ctx.dims
        q, k, v = _unpack(qkv, hk, hv, dk_, dv)
        B, L, Hv, _ = v.shape
        dev = v.device
        ex = native.ext()
        nvs = dv // 128
        dO = native._bf16(dO).contiguous()
        dU = torch.empty_like(Vnew)
        parts = torch.empty(3, nvs, B, Hv, L, 128, dtype=torch.float32, device=dev)
        dcarry = torch.zeros_like(carry)
        dS0 = torch.empty(B, Hv, 128, dv, dtype=torch.float32, device=dev) if ctx.has_s0 else None
        dSf = dSfinal.float().contiguous() if (dSfinal is not None and dSfinal.numel()) else None
        ex.gdn_scan_bwd(W, Qin, Kout, Aqk, Hsave.view(-1, 128), Vnew, dO, carry, dSf, dU, parts[0], parts[1], parts[2], dcarry, dS0,
                        native.err_flag(dev))
        dqkv = torch.empty_like(qkv)
        dq, dk, dv_ = _unpack(dqkv, hk, hv, dk_, dv)
        dg = torch.empty(B, L, Hv, dtype=torch.float32, device=dev)
        dbeta = torch.empty_like(dg)
        if hv == hk:
            ex.gdn_local_bwd(q, k, v, g, beta, start_u8, U, W, dU, parts, dO, Vnew, dcarry, dq, dk, dv_, dg, dbeta)
        else:
            dq32 = torch.empty(B, L, Hv, 128, dtype=torch.float32, device=dev)
            dk32 = torch.empty_like(dq32)
            ex.gdn_local_bwd(q, k, v, g, beta, start_u8, U, W, dU, parts, dO, Vnew, dcarry, dq32, dk32, dv_, dg, dbeta)
            dq.copy_(dq32.view(B, L, hk, hv // hk, 128).sum(3))
            dk.copy_(dk32.view(B, L, hk, hv // hk, 128).sum(3))
        native._count(2)
        return dqkv, dg, dbeta, None, dS0, None, None, None, None, None


def _tok_major_ok(t) -> bool:
    return (t.dtype == BF16 and t.stride(3) == 1 and t.stride(2) == t.shape[3] and t.stride(0) == t.stride(1) * t.shape[1]
            and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0)


def supported(q, v) -> bool:
    return q.shape[-1] == 128 and v.shape[-1] % 128 == 0


def packed_ok(qkv, hk, hv, dk, dv, chunk_size) -> bool:
    return (dk == 128 and dv in (128, 256) and chunk_size == CHUNK and qkv.dtype == BF16 and qkv.is_contiguous() and qkv.shape[1] % CHUNK == 0
            and qkv.shape[-1] % 8 == 0)


def delta_rule_packed(qkv, hk, hv, dk, dv, g, beta, is_doc_start, S0, need_state):
    """qkv: [B, L, hk dk | hk dk | hv dv] bf16 (the conv/norm stage's output); g, beta: [B, L, Hv]. Returns
    (o [B, L, Hv, dv], final state or None). One autograd node: its gradient comes back packed the same way."""
    O, S = _DeltaRule.apply(qkv, g.float().contiguous(), beta.float().contiguous(), is_doc_start.to(torch.uint8).contiguous(),
                            None if S0 is None else S0.float().contiguous(), need_state, hk, hv, dk, dv)
    return O, (S if need_state else None)


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
    qkv = torch.cat([native._bf16(t).flatten(2) for t in (q, k, v)], dim=-1)
    O, S = delta_rule_packed(qkv, Hk, Hv, dk, dv, g, beta, is_doc_start, S0, need_state)
    return (O[:, :L] if pad else O), S


def step_ok(q, v, S0) -> bool:
    """One cached token on the fused step kernel: key dim 128, value dim a multiple of 128, an fp32 state, no autograd."""
    return (q.shape[1] == 1 and S0 is not None and S0.dtype == torch.float32 and q.shape[-1] == 128 and v.shape[-1] % 128 == 0
            and not (torch.is_grad_enabled() and any(t.requires_grad for t in (q, v, S0))))


def delta_rule_step(q, k, v, g, beta, is_doc_start, S0, inplace: bool = False):
    """(o [B, 1, Hv, dv], S): one token of the rule per row through `gdn_step_kernel`, which reads and writes the state
    once. inplace: S0 itself is updated and returned (the decode engine's static state buffer); otherwise a copy is."""
    B = q.shape[0]
    f = lambda t: t.reshape(B, *t.shape[2:]).float().contiguous()
    S = S0 if (inplace and S0.is_contiguous()) else S0.clone(memory_format=torch.contiguous_format)
    o = torch.empty(B, v.shape[2], v.shape[3], dtype=torch.float32, device=v.device)
    start = None if is_doc_start is None else is_doc_start.reshape(B).to(torch.bool).contiguous()
    native.ext().gdn_step(S, f(q), f(k), f(v), f(g), f(beta), start, o)
    native._count()
    return o.view(B, 1, *o.shape[1:]).to(v.dtype), S
