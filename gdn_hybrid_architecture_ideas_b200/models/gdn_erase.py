"""An erase direction of its own for a Gated DeltaNet layer (`gdn.erase.mode: eda`).

The delta rule erases along the key it is about to write. Here a token may first erase along a SECOND, learned direction:

    S_t = (I - beta_t k_t k_t^T) (I - gamma_t e_t e_t^T) D_t S_{t-1} + beta_t k_t v_t^T

i.e. per token, in this order: reset at a document start, decay (D_t a scalar per head, or per key channel with
`gdn.kda.decay: channel`), erase S <- S - gamma_t e_t (e_t^T S), the usual delta write, read o_t = S^T q_t. With
gamma = 0 the erase factor is the identity and the layer is the base layer exactly.

* e_t: one unit vector per KEY head, e = normalise(U_h (W_down x)_h): a rank-r bottleneck, each head reading its own
  r-slice through its own (dk, r) block (`erase.e_down`: d -> r Hk, `erase.e_up`: r -> dk per head).
* gamma_t in [0, 1] per VALUE head: clamp01(s_h) * sigmoid(w_h . x) with `erase.scale` s starting at 0 (the erase is
  shut at the start) and `erase.in_proj_gamma` w. The clamp is "inward": forward clamp(s, 0, 1); backward, inside
  [0, 1] the gradient passes, outside only the part that would move s back toward the interval passes. A plain clamp
  would leave a shut head (s < 0) without gradient for ever; a straight-through one would let s wander off while shut.

The erase step is itself a delta-rule step with value 0, so the whole rule maps onto the ordinary chunked rule at twice
the length: token t becomes sub-step 2t (key e_t, write strength gamma_t, value 0, query 0, the token's decay and
document start) followed by sub-step 2t + 1 (k_t, beta_t, v_t, q_t, no decay); outputs are taken at the odd sub-steps.
`rule` runs either that interleave (through the scalar or the per-channel chunked rule) or, for one token or on request,
the plain token loop. Tensor ops on every device.

The gate's tensors are drawn from a generator of their own (seeded from the run's seed plus a constant), after and apart
from every other tensor, so a model with the erase starts with the same base weights as the model without it.
Reference: ced/model/gdn_erase.py (gate 162-262, rule 276-325).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from .linear import Linear

MODES = ("none", "eda")
SEED_OFFSET = 0xE7A5E_2026_1022     # added to the run's seed for the erase tensors' generator (shared with the reference: equal starts)
STANDALONE_SEED = 0xE7A5E           # a gate built outside a model


def is_on(cfg) -> bool:
    return cfg.erase.mode == "eda"


def check_config(cfg) -> None:
    section = cfg.erase
    if section.mode not in MODES:
        raise ValueError(f"gdn.erase.mode {section.mode!r}: one of {MODES}")
    if not is_on(cfg):
        if section.rank != type(section)().rank:
            raise ValueError("gdn.erase.rank is read with erase.mode 'eda'; this layer's erase.mode is 'none'")
        return
    if type(section.rank) is not int or not 1 <= section.rank <= cfg.k_head_dim:
        raise ValueError(f"gdn.erase.rank {section.rank!r}: an integer in [1, k_head_dim = {cfg.k_head_dim}]")
    if cfg.negeig.beta_max != 1 or cfg.dprod.n_h != 1:
        raise ValueError("gdn.erase.mode 'eda' is built with negeig.beta_max 1 and dprod.n_h 1 (and with either decay)")


def check_model(cfg) -> None:
    """What the erase is not built together with, named: the GDN write / query mixes, the MTP drafter, low-precision linears."""
    if not is_on(cfg.encoder.gdn):
        return
    clashes = {f"model.encoder.gdn_write_mix {cfg.encoder.gdn_write_mix!r}": cfg.encoder.gdn_write_mix != "none",
               "model.mtp.enabled": bool(cfg.mtp.enabled),
               f"model.fp8.mode {cfg.fp8.mode!r}": cfg.fp8.mode != "none",
               f"model.nvfp4.mode {cfg.nvfp4.mode!r}": cfg.nvfp4.mode != "none"}
    found = [name for name, hit in clashes.items() if hit]
    if found:
        raise ValueError(f"model.encoder.gdn.erase.mode 'eda' is not built with: {'; '.join(found)}")


class _ClampTowardUnitInterval(torch.autograd.Function):
    """clamp(s, 0, 1) whose gradient, outside [0, 1], keeps only the sign that pulls s back in."""

    @staticmethod
    def forward(ctx, s):
        ctx.save_for_backward(s)
        return s.clamp(0.0, 1.0)

    @staticmethod
    def backward(ctx, grad):
        (s,) = ctx.saved_tensors
        # a descent step moves s by -grad: below 0 only grad <= 0 raises s, above 1 only grad >= 0 lowers it
        pull_up = torch.minimum(grad, torch.zeros_like(grad))
        pull_down = torch.maximum(grad, torch.zeros_like(grad))
        return torch.where(s < 0, pull_up, torch.where(s > 1, pull_down, grad))


def inward_clamp(s: torch.Tensor) -> torch.Tensor:
    return _ClampTowardUnitInterval.apply(s)


class EraseGate(nn.Module):
    def __init__(self, d_model: int, cfg):
        super().__init__()
        self.hk, self.hv, self.dk, self.rank = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.erase.rank
        with torch.random.fork_rng(devices=[]):      # building the projections must not advance the global stream
            self.e_down = Linear(d_model, self.rank * self.hk)
            self.e_up = Linear(self.rank, self.hk * self.dk)
            self.in_proj_gamma = Linear(d_model, self.hv)
        self.scale = nn.Parameter(torch.zeros(self.hv))
        for own in self._drawn():
            own.own_init = True                      # the model's general init skips these; `reset_own` draws them
        self.reset_own(torch.Generator().manual_seed(STANDALONE_SEED), 0.02)

    def _drawn(self):
        return (self.e_down, self.e_up, self.in_proj_gamma)

    @torch.no_grad()
    def reset_own(self, gen: torch.Generator, std: float) -> None:
        """N(0, std) on the three projections from `gen` (float32 draws on the CPU, in this order), zeros on the scale."""
        for lin in self._drawn():
            w = lin.weight
            if w.is_meta:
                continue
            w.copy_(torch.randn(w.shape, generator=gen, dtype=torch.float32).mul_(std).to(device=w.device, dtype=w.dtype))
        if not self.scale.is_meta:
            self.scale.zero_()

    def direction(self, x: torch.Tensor) -> torch.Tensor:
        """e (..., Hk, dk): unit vectors, float32 or wider."""
        low = self.e_down(x).unflatten(-1, (self.hk, self.rank))
        blocks = self.e_up.weight.to(low.dtype).view(self.hk, self.dk, self.rank)
        raw = torch.einsum("...hr,hdr->...hd", low, blocks)
        return ops.ref.l2_normalize(raw.to(torch.promote_types(raw.dtype, torch.float32)))

    def strength(self, x: torch.Tensor) -> torch.Tensor:
        """gamma (..., Hv) in [0, 1]."""
        return inward_clamp(self.scale) * torch.sigmoid(self.in_proj_gamma(x))

    def extra_repr(self) -> str:
        return f"rank={self.rank}, key_heads={self.hk}, value_heads={self.hv}"


def init_own_parameters(model: nn.Module, std: float) -> int:
    """Draws every EraseGate of `model`, in module order, from ONE generator seeded with the run's seed + SEED_OFFSET.
    Returns how many gates there were."""
    found = [m for m in model.modules() if isinstance(m, EraseGate)]
    if found:
        gen = torch.Generator().manual_seed((torch.initial_seed() + SEED_OFFSET) % (1 << 63))
        for gate in found:
            gate.reset_own(gen, std)
    return len(found)


# ------------------------------------------------------------------------------------------------------------------ the rule

def _outer(a, b):
    return a[..., :, None] * b[..., None, :]


def _read(S, key):
    """key^T S per head: (B, H, dk) x (B, H, dk, dv) -> (B, H, dv)."""
    return (key[..., None] * S).sum(-2)


def erase_recurrence(q, k, v, g, beta, e, gamma, is_doc_start, S):
    """The rule one token at a time (the definition). q, k, e: (B, L, H, dk) at the value heads; v (B, L, H, dv);
    g (B, L, H) or, per channel, (B, L, H, dk); beta, gamma (B, L, H); S (B, H, dk, dv). Returns (o (B, L, H, dv), S)."""
    outs = []
    for t in range(q.shape[1]):
        keep = (~is_doc_start[:, t]).to(S.dtype)
        decay = torch.exp(g[:, t])
        S = S * keep[:, None, None, None]
        S = S * (decay[..., None] if decay.dim() == 3 else decay[..., None, None])
        S = S - _outer(e[:, t], gamma[:, t, :, None] * _read(S, e[:, t]))
        S = S + _outer(k[:, t], beta[:, t, :, None] * (v[:, t] - _read(S, k[:, t])))
        outs.append(_read(S, q[:, t]))
    return torch.stack(outs, dim=1), S


def _zip_steps(first, second):
    """(B, L, ...) x 2 -> (B, 2L, ...): first[0], second[0], first[1], second[1], ..."""
    B, L = first.shape[:2]
    return torch.stack((first, second), dim=2).reshape(B, 2 * L, *first.shape[2:])


def interleave(q, k, v, g, beta, e, gamma, is_doc_start):
    """The 2L-step inputs (q, k, v, g, beta, starts) of the ordinary rule: per token the erase step then the write step."""
    none_q, none_v, none_g = torch.zeros_like(q), torch.zeros_like(v), torch.zeros_like(g)
    return (_zip_steps(none_q, q), _zip_steps(e, k), _zip_steps(none_v, v), _zip_steps(g, none_g), _zip_steps(gamma, beta),
            _zip_steps(is_doc_start, torch.zeros_like(is_doc_start)))


def write_substeps(o: torch.Tensor) -> torch.Tensor:
    """Outputs of the odd (write) sub-steps of a 2L-step run."""
    return o[:, 1::2]


def rule(q, k, v, g, beta, e, gamma, is_doc_start, S, kernel: str, chunk_size: int):
    """(outputs, final state): the token loop (kernel "recurrence", or a single token) or the interleave through the
    chunked rule that matches the decay's kind."""
    dt = ops.ref.work_dtype(q)
    q, k, v, g, beta, e, gamma, S = (t.to(dt) for t in (q, k, v, g, beta, e, gamma, S))
    if kernel == "recurrence" or q.shape[1] == 1:
        return erase_recurrence(q, k, v, g, beta, e, gamma, is_doc_start, S)
    steps = interleave(q, k, v, g, beta, e, gamma, is_doc_start)
    chunked = ops.ref.kda_chunked if g.dim() == 4 else ops.ref.chunked_delta_rule
    o2, S = chunked(*steps, S, chunk_size)
    return write_substeps(o2), S
