"""Per-channel decay (KDA) and the horizon floor of a Gated DeltaNet layer (`gdn.kda.decay: channel`).

    S_t = (I - beta_t k_t k_t^T) Diag(a_t) S_{t-1} + beta_t k_t v_t^T,   o_t = S_t^T q_t,   a_t = exp(g_t) in (0, 1]^dk

The gate: u = W_up W_down x (+ a per-channel dt_bias, stored flat (Hv dk) so no matrix optimizer takes it);
free channels g = -exp(A_log_h) softplus(u + dt_bias); the first `floor_channels` channels of every value head
g = ln(1 - 1/H_i) sigmoid(u + dt_bias) with H_i log-spaced from floor_min to floor_max tokens, so their decay never
falls below 1 - 1/H_i. The bound is a non-persistent float32 buffer rounded toward zero. The layer holds `kda` where
`in_proj_a` and the per-head `dt_bias` were; beta, the conv, q, k, v and the output gate are the scalar layer's.
proj "shared": W_down d -> rank, W_up rank -> Hv dk (rank 0 = v_head_dim); "per_head": W_down d -> rank x Hv, each
value head's own rank slice through its own (dk, rank) block of W_up (rank 0 = 16). The rule runs as tensor ops
(`ops/reference.py` `kda_recurrence`, `kda_chunked`) on every device
(reference: ced/model/gdn_kda.py:1-80, 101-141, 166-283).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .linear import Linear

DECAYS = ("scalar", "channel")
PROJ_FORMS = ("per_head", "shared")
PER_HEAD_RANK = 16


def is_on(cfg) -> bool:
    return cfg.kda.decay == "channel"


def _number(x) -> bool:
    return not isinstance(x, bool) and isinstance(x, (int, float)) and math.isfinite(float(x))


def check_config(cfg) -> None:
    """gdn.kda checked; with decay "scalar" every other key must be at its default."""
    k = cfg.kda
    if k.decay not in DECAYS:
        raise ValueError(f"gdn.kda.decay {k.decay!r}: one of {DECAYS}")
    if k.decay == "scalar":
        default = type(k)()
        moved = [f"kda.{n}" for n in ("proj", "rank", "floor_channels", "floor_min", "floor_max") if getattr(k, n) != getattr(default, n)]
        if moved:
            raise ValueError(f"gdn {', '.join(moved)}: read with kda.decay 'channel'; this layer's decay is 'scalar'")
        return
    if k.proj not in PROJ_FORMS:
        raise ValueError(f"gdn.kda.proj {k.proj!r}: one of {PROJ_FORMS}")
    if type(k.rank) is not int or k.rank < 0:
        raise ValueError(f"gdn.kda.rank {k.rank!r}: an integer >= 0 (0: per_head {PER_HEAD_RANK}, shared v_head_dim)")
    if type(k.floor_channels) is not int or not 0 <= k.floor_channels < cfg.k_head_dim:
        raise ValueError(f"gdn.kda.floor_channels {k.floor_channels!r}: an integer in [0, k_head_dim = {cfg.k_head_dim})")
    if not (_number(k.floor_min) and _number(k.floor_max) and 1.0 < float(k.floor_min) <= float(k.floor_max)):
        raise ValueError(f"gdn.kda.floor_min / floor_max {k.floor_min!r} / {k.floor_max!r}: horizons in tokens, 1 < floor_min <= floor_max")
    if cfg.negeig.beta_max != 1 or cfg.dprod.n_h != 1:
        raise ValueError("gdn.kda.decay 'channel' is built with negeig.beta_max 1 and dprod.n_h 1 (and with or without the erase)")


def rank_of(cfg) -> int:
    return cfg.kda.rank or (PER_HEAD_RANK if cfg.kda.proj == "per_head" else cfg.v_head_dim)


def floor_horizons(cfg) -> list[float]:
    n = cfg.kda.floor_channels if is_on(cfg) else 0
    lo, hi = float(cfg.kda.floor_min), float(cfg.kda.floor_max)
    if n <= 1:
        return [lo] * n
    r = math.log2(hi / lo)
    return [lo * 2.0 ** (r * i / (n - 1)) for i in range(n)]


def floor_log_values(horizons: list[float], dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """ln(1 - 1/H_i) in `dtype`, rounded toward zero: never below the float64 value, so g >= it means a >= 1 - 1/H_i."""
    exact = torch.tensor([math.log1p(-1.0 / h) for h in horizons], dtype=torch.float64)
    out = exact.to(dtype)
    below = out.to(torch.float64) < exact
    return torch.where(below, torch.nextafter(out, torch.zeros_like(out)), out)


class KDAGate(nn.Module):
    def __init__(self, d_model: int, cfg):
        super().__init__()
        self.hv, self.dk, self.proj, self.rank = cfg.n_v_heads, cfg.k_head_dim, cfg.kda.proj, rank_of(cfg)
        self.n_floor = cfg.kda.floor_channels
        self.horizons = floor_horizons(cfg)
        self.f_down = Linear(d_model, self.rank * (self.hv if self.proj == "per_head" else 1))
        self.f_up = Linear(self.rank, self.hv * self.dk)
        self.dt_bias = nn.Parameter(torch.empty(self.hv * self.dk))
        self.register_buffer("floor_log", floor_log_values(self.horizons), persistent=False)

    @torch.no_grad()
    def reset_dt_bias(self, scheme: str) -> None:
        """The per-head law of the scalar layer, a channel at a time; 0 on the floored channels (sigmoid 1/2)."""
        if scheme == "fla":
            dt = torch.exp(torch.rand(self.hv, self.dk) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3)).clamp(min=1e-4)
            value = dt + torch.log(-torch.expm1(-dt))
        elif scheme == "hf":
            value = torch.ones(self.hv, self.dk)
        else:
            raise ValueError(f"unknown GDN init scheme {scheme!r}")
        value[:, :self.n_floor] = 0.0
        self.dt_bias.copy_(value.flatten())

    def decay_input(self, x: torch.Tensor) -> torch.Tensor:
        """u + dt_bias, (..., Hv, dk)."""
        z = self.f_down(x)
        if self.proj == "shared":
            u = self.f_up(z).unflatten(-1, (self.hv, self.dk))
        else:       # one batched product over the value heads: no per-token copy of W_up is saved for the backward
            w = self.f_up.weight.to(z.dtype).view(self.hv, self.dk, self.rank)
            u = torch.einsum("...hr,hdr->...hd", z.unflatten(-1, (self.hv, self.rank)), w)
        return u + self.dt_bias.view(self.hv, self.dk)

    def extra_repr(self) -> str:
        return f"proj={self.proj}, rank={self.rank}, floor_channels={self.n_floor}"


def gates(layer, x: torch.Tensor):
    """(g (..., Hv, dk) <= 0 in >= float32, beta (..., Hv))."""
    kda = layer.kda
    pre = kda.decay_input(x)
    pre = pre.to(torch.promote_types(pre.dtype, torch.float32))
    nf = kda.n_floor
    g = -torch.exp(layer.A_log.to(pre.dtype))[:, None] * F.softplus(pre[..., nf:])
    if nf:
        g = torch.cat([kda.floor_log.to(pre.dtype) * torch.sigmoid(pre[..., :nf]), g], dim=-1)
    return g, torch.sigmoid(layer.in_proj_b(x))


def added_parameters(cfg, d_model: int) -> int:
    """Parameters a layer gains over the scalar layer (in_proj_a and the per-head dt_bias leave)."""
    r, hv, dk = rank_of(cfg), cfg.n_v_heads, cfg.k_head_dim
    down = d_model * r * (hv if cfg.kda.proj == "per_head" else 1)
    return down + r * hv * dk + hv * dk - (d_model * hv + hv)
