"""A separate erase direction in a Gated DeltaNet layer (`gdn.erase.mode: eda`).

    S_t = (I - beta_t k_t k_t^T)(I - gamma_t e_t e_t^T) D_t S_{t-1} + beta_t k_t v_t^T

per token: reset at a document start; the decay (the scalar a_t, or Diag(a_t) with `gdn.kda.decay: channel`); the erase
S <- S - gamma_t e_t (e_t^T S), a delta-rule step with value 0; the delta write; the read S^T q_t. gamma = 0 is the base
layer's rule exactly.

Tensors (`GatedDeltaNet.erase`): e_t = L2norm(W_up W_down x_t), one unit vector per key head (e_down d -> r Hk, e_up
r -> dk on each key head's own rank slice); gamma_t = c(s) sigmoid(W_gamma x_t) per value head with s zero-initialised
and c the inward clamp: clamp(s, 0, 1) forward, and a backward that outside [0, 1] passes only the gradient moving s
back toward it, so a head's erase can always reopen and s does not drift away while it is shut. The tensors are built
without touching the global random stream and drawn by the model's build from a generator of their own, so every
other tensor starts as in the base model of the same seed.

Paths: the token loop (`erase_recurrence`), and the 2T interleave into the chunked rule of the layer's decay: token t
becomes sub-step 2t, the erase (k' = e_t, beta' = gamma_t, v' = 0, q' = 0, g' = g_t, a document start where t starts
one) and sub-step 2t + 1, the write (k_t, beta_t, v_t, q_t, g' = 0); outputs are read on the write sub-steps. Tensor
ops on every device (reference: ced/model/gdn_erase.py:1-75, 162-262, 276-325).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from .linear import Linear

MODES = ("none", "eda")
SEED_OFFSET = 0xE7A5E_2026_1022
STANDALONE_SEED = 0xE7A5E


def is_on(cfg) -> bool:
    return cfg.erase.mode == "eda"


def check_config(cfg) -> None:
    e = cfg.erase
    if e.mode not in MODES:
        raise ValueError(f"gdn.erase.mode {e.mode!r}: one of {MODES}")
    if e.mode == "none":
        if e.rank != type(e)().rank:
            raise ValueError("gdn.erase.rank is read with erase.mode 'eda'; this layer's erase.mode is 'none'")
        return
    if type(e.rank) is not int or not 1 <= e.rank <= cfg.k_head_dim:
        raise ValueError(f"gdn.erase.rank {e.rank!r}: an integer in [1, k_head_dim = {cfg.k_head_dim}]")
    if cfg.negeig.beta_max != 1 or cfg.dprod.n_h != 1:
        raise ValueError("gdn.erase.mode 'eda' is built with negeig.beta_max 1 and dprod.n_h 1 (and with either decay)")


def check_model(cfg) -> None:
    """Model-level refusals: the encoder's GDN layers only, without the GDN write / query mixes, the MTP drafter or
    low-precision linears."""
    if not is_on(cfg.encoder.gdn):
        return
    refused = [(cfg.encoder.gdn_write_mix != "none", f"model.encoder.gdn_write_mix {cfg.encoder.gdn_write_mix!r}"),
               (bool(cfg.mtp.enabled), "model.mtp.enabled"), (cfg.fp8.mode != "none", f"model.fp8.mode {cfg.fp8.mode!r}"),
               (cfg.nvfp4.mode != "none", f"model.nvfp4.mode {cfg.nvfp4.mode!r}")]
    bad = [why for cond, why in refused if cond]
    if bad:
        raise ValueError(f"model.encoder.gdn.erase.mode 'eda' is not built with: {'; '.join(bad)}")


class _InwardClamp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, s):
        ctx.save_for_backward(s)
        return s.clamp(0.0, 1.0)

    @staticmethod
    def backward(ctx, grad):
        (s,) = ctx.saved_tensors
        return torch.where(s < 0, grad.clamp(max=0.0), torch.where(s > 1, grad.clamp(min=0.0), grad))


def inward_clamp(s: torch.Tensor) -> torch.Tensor:
    return _InwardClamp.apply(s)


class EraseGate(nn.Module):
    def __init__(self, d_model: int, cfg):
        super().__init__()
        self.hk, self.hv, self.dk, self.rank = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.erase.rank
        with torch.random.fork_rng(devices=[]):          # nothing of the global stream is consumed
            self.e_down = Linear(d_model, self.rank * self.hk)
            self.e_up = Linear(self.rank, self.hk * self.dk)
            self.in_proj_gamma = Linear(d_model, self.hv)
        for lin in (self.e_down, self.e_up, self.in_proj_gamma):
            lin.own_init = True
        self.scale = nn.Parameter(torch.zeros(self.hv))
        self.reset_own(torch.Generator().manual_seed(STANDALONE_SEED), 0.02)

    @torch.no_grad()
    def reset_own(self, gen: torch.Generator, std: float) -> None:
        for p in (self.e_down.weight, self.e_up.weight, self.in_proj_gamma.weight):
            if not p.is_meta:
                p.copy_((torch.randn(p.shape, generator=gen, dtype=torch.float32) * std).to(device=p.device, dtype=p.dtype))
        if not self.scale.is_meta:
            self.scale.zero_()

    def direction(self, x: torch.Tensor) -> torch.Tensor:
        """e (..., Hk, dk): a unit vector per key head, >= float32."""
        z = self.e_down(x).unflatten(-1, (self.hk, self.rank))
        w = self.e_up.weight.to(z.dtype).view(self.hk, self.dk, self.rank)
        e = torch.einsum("...hr,hdr->...hd", z, w)
        return ops.ref.l2_normalize(e.to(torch.promote_types(e.dtype, torch.float32)))

    def strength(self, x: torch.Tensor) -> torch.Tensor:
        """gamma (..., Hv) in [0, 1]."""
        return inward_clamp(self.scale) * torch.sigmoid(self.in_proj_gamma(x))

    def extra_repr(self) -> str:
        return f"rank={self.rank}, key_heads={self.hk}, value_heads={self.hv}"


def init_own_parameters(model: nn.Module, std: float) -> int:
    """Every EraseGate of the model, in module order, from one generator seeded torch.initial_seed() + SEED_OFFSET."""
    gates = [m for m in model.modules() if isinstance(m, EraseGate)]
    if gates:
        g = torch.Generator().manual_seed((torch.initial_seed() + SEED_OFFSET) % (1 << 63))
        for m in gates:
            m.reset_own(g, std)
    return len(gates)


def erase_recurrence(q, k, v, g, beta, e, gamma, is_doc_start, S):
    """The rule a token at a time. q, k, e (B, L, H, dk) at the value heads; g (B, L, H) or (B, L, H, dk)."""
    per_channel = g.dim() == 4
    outs = []
    for q_t, k_t, v_t, g_t, b_t, e_t, c_t, s_t in zip(q.unbind(1), k.unbind(1), v.unbind(1), g.unbind(1), beta.unbind(1), e.unbind(1),
                                                      gamma.unbind(1), is_doc_start.unbind(1)):
        S = S * (~s_t).to(S.dtype)[:, None, None, None]
        S = S * (torch.exp(g_t)[..., None] if per_channel else torch.exp(g_t)[:, :, None, None])
        S = S - torch.einsum("bhk,bhv->bhkv", e_t, c_t[..., None] * torch.einsum("bhkv,bhk->bhv", S, e_t))
        S = S + torch.einsum("bhk,bhv->bhkv", k_t, b_t[..., None] * (v_t - torch.einsum("bhkv,bhk->bhv", S, k_t)))
        outs.append(torch.einsum("bhkv,bhk->bhv", S, q_t))
    return torch.stack(outs, dim=1), S


def interleave(q, k, v, g, beta, e, gamma, is_doc_start):
    """(q, k, v, g, beta, starts) of length 2L: the erase sub-step, then the write sub-step, of every token."""
    B, L = q.shape[:2]

    def pair(first, second):
        return torch.stack([first, second], dim=2).reshape(B, 2 * L, *first.shape[2:])

    return (pair(torch.zeros_like(q), q), pair(e, k), pair(torch.zeros_like(v), v), pair(g, torch.zeros_like(g)), pair(gamma, beta),
            pair(is_doc_start, torch.zeros_like(is_doc_start)))


def write_substeps(o: torch.Tensor) -> torch.Tensor:
    B, T = o.shape[:2]
    return o.reshape(B, T // 2, 2, *o.shape[2:])[:, :, 1]


def rule(q, k, v, g, beta, e, gamma, is_doc_start, S, kernel: str, chunk_size: int):
    """Outputs and final state by the token loop (kernel "recurrence", or one token) or the interleave into the chunked
    rule of the decay's kind."""
    dt = ops.ref.work_dtype(q)
    q, k, v, g, beta, e, gamma, S = (t.to(dt) for t in (q, k, v, g, beta, e, gamma, S))
    if kernel == "recurrence" or q.shape[1] == 1:
        return erase_recurrence(q, k, v, g, beta, e, gamma, is_doc_start, S)
    qi, ki, vi, gi, bi, si = interleave(q, k, v, g, beta, e, gamma, is_doc_start)
    chunked = ops.ref.kda_chunked if g.dim() == 4 else ops.ref.chunked_delta_rule
    oi, S = chunked(qi, ki, vi, gi, bi, si, S, chunk_size)
    return write_substeps(oi), S
