"""Per-channel decay (KDA) of a Gated DeltaNet layer, with an optional horizon floor (`gdn.kda.decay: channel`).

The scalar layer forgets every key channel of a head at one rate; here each of the dk key channels has its own:

    S_t = (I - beta_t k_t k_t^T) Diag(a_t) S_{t-1} + beta_t k_t v_t^T,      a_t = exp(g_t) in (0, 1]^dk,      o_t = S_t^T q_t

What produces g_t (this module): a low-rank projection u = W_up (W_down x) plus a per-channel bias, then

* an ordinary channel of value head h:   g = -exp(A_log_h) * softplus(u + bias)              (any rate)
* a FLOORED channel i (the first `floor_channels` of every head): g = ln(1 - 1/H_i) * sigmoid(u + bias), so its decay
  stays within [1 - 1/H_i, 1]: the channel keeps a memory horizon of at least H_i tokens whatever the input. The H_i
  climb geometrically from floor_min to floor_max.

Two shapes of the projection: "shared" (one W_down: d -> rank, W_up: rank -> Hv dk; default rank = v_head_dim) and
"per_head" (W_down: d -> Hv rank, and each head reads only its own rank-slice through its own (dk, rank) block of
W_up; default rank 16). The layer then has no `in_proj_a` and no per-head `dt_bias`: `kda.f_down`, `kda.f_up` and the
flat `kda.dt_bias` (Hv dk values; flat so that a matrix optimizer never claims it) stand in their place. The rule itself
runs as tensor ops (`ops/reference.py`: `kda_recurrence`, `kda_chunked`).
Reference: ced/model/gdn_kda.py (gate: 101-283).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .linear import Linear

DECAYS = ("scalar", "channel")
PROJ_FORMS = ("per_head", "shared")
PER_HEAD_RANK = 16
_OWN_KEYS = ("proj", "rank", "floor_channels", "floor_min", "floor_max")


def is_on(cfg) -> bool:
    return cfg.kda.decay == "channel"


@dataclass(frozen=True)
class KDAShape:
    """Everything the gate's constructor needs, resolved from a GDN config."""
    heads: int
    key_dim: int
    per_head: bool
    rank: int
    floored: int
    horizon_lo: float
    horizon_hi: float

    @property
    def down_width(self) -> int:
        return self.rank * (self.heads if self.per_head else 1)

    def horizons(self) -> list[float]:
        """H_0 .. H_{floored-1}: geometric from horizon_lo to horizon_hi (a single floored channel sits at horizon_lo)."""
        if self.floored <= 1:
            return [self.horizon_lo] * self.floored
        octaves = math.log2(self.horizon_hi / self.horizon_lo)
        return [self.horizon_lo * 2.0 ** (octaves * i / (self.floored - 1)) for i in range(self.floored)]


def _finite_number(x) -> bool:
    return isinstance(x, (int, float)) and not isinstance(x, bool) and math.isfinite(float(x))


def check_config(cfg) -> None:
    """Refuses, by key name, a `gdn.kda` section that cannot be built. With decay "scalar" the section's other keys are
    not read, so a value away from its default there is a mistake, not a setting."""
    k = cfg.kda
    if k.decay not in DECAYS:
        raise ValueError(f"gdn.kda.decay {k.decay!r}: one of {DECAYS}")
    if not is_on(cfg):
        fresh = type(k)()
        stray = [f"kda.{name}" for name in _OWN_KEYS if getattr(k, name) != getattr(fresh, name)]
        if stray:
            raise ValueError(f"gdn {', '.join(stray)}: read with kda.decay 'channel'; this layer's decay is 'scalar'")
        return
    if k.proj not in PROJ_FORMS:
        raise ValueError(f"gdn.kda.proj {k.proj!r}: one of {PROJ_FORMS}")
    if type(k.rank) is not int or k.rank < 0:
        raise ValueError(f"gdn.kda.rank {k.rank!r}: an integer >= 0 (0: per_head {PER_HEAD_RANK}, shared v_head_dim)")
    if type(k.floor_channels) is not int or not 0 <= k.floor_channels < cfg.k_head_dim:
        raise ValueError(f"gdn.kda.floor_channels {k.floor_channels!r}: an integer in [0, k_head_dim = {cfg.k_head_dim})")
    if not (_finite_number(k.floor_min) and _finite_number(k.floor_max) and 1.0 < float(k.floor_min) <= float(k.floor_max)):
        raise ValueError(f"gdn.kda.floor_min / floor_max {k.floor_min!r} / {k.floor_max!r}: horizons in tokens, 1 < floor_min <= floor_max")
    if cfg.negeig.beta_max != 1 or cfg.dprod.n_h != 1:
        raise ValueError("gdn.kda.decay 'channel' is built with negeig.beta_max 1 and dprod.n_h 1 (and with or without the erase)")


def rank_of(cfg) -> int:
    return cfg.kda.rank or (PER_HEAD_RANK if cfg.kda.proj == "per_head" else cfg.v_head_dim)


def shape_of(cfg) -> KDAShape:
    k = cfg.kda
    return KDAShape(heads=cfg.n_v_heads, key_dim=cfg.k_head_dim, per_head=k.proj == "per_head", rank=rank_of(cfg),
                    floored=k.floor_channels if is_on(cfg) else 0, horizon_lo=float(k.floor_min), horizon_hi=float(k.floor_max))


def floor_horizons(cfg) -> list[float]:
    return shape_of(cfg).horizons()


def floor_log_values(horizons: list[float], dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """ln(1 - 1/H) per horizon in `dtype`, never BELOW the exact value: where rounding to `dtype` landed below, the
    neighbour toward zero is taken instead. The floor promises a >= 1 - 1/H, i.e. g >= ln(1 - 1/H); a table entry that
    rounding pushed further negative would quietly break the promise."""
    exact = torch.tensor([math.log1p(-1.0 / h) for h in horizons], dtype=torch.float64)
    rounded = exact.to(dtype)
    too_low = rounded.double() < exact
    return torch.where(too_low, torch.nextafter(rounded, torch.zeros_like(rounded)), rounded)


class KDAGate(nn.Module):
    """Holds the decay projection of one layer and forms the gate's pre-activation."""

    def __init__(self, d_model: int, cfg):
        super().__init__()
        sh = shape_of(cfg)
        self.shape = sh
        self.hv, self.dk, self.rank, self.n_floor = sh.heads, sh.key_dim, sh.rank, sh.floored
        self.proj = "per_head" if sh.per_head else "shared"
        self.horizons = sh.horizons()
        self.f_down = Linear(d_model, sh.down_width)
        self.f_up = Linear(sh.rank, sh.heads * sh.key_dim)
        self.dt_bias = nn.Parameter(torch.empty(sh.heads * sh.key_dim))
        self.register_buffer("floor_log", floor_log_values(self.horizons), persistent=False)

    @torch.no_grad()
    def reset_dt_bias(self, scheme: str) -> None:
        """The bias start. Ordinary channels follow the scalar layer's law for its per-head bias, drawn per channel:
        "fla": softplus^-1 of a step size log-uniform in [1e-3, 0.1]; "hf": ones. Floored channels start at 0, the middle
        of their sigmoid (decay half way between the floor and 1 in log space)."""
        if scheme == "fla":
            lo, hi = math.log(1e-3), math.log(0.1)
            step = torch.exp(torch.rand(self.hv, self.dk) * (hi - lo) + lo).clamp(min=1e-4)
            start = step + torch.log(-torch.expm1(-step))          # softplus^-1(step)
        elif scheme == "hf":
            start = torch.ones(self.hv, self.dk)
        else:
            raise ValueError(f"unknown GDN init scheme {scheme!r}")
        start[:, : self.n_floor] = 0.0
        self.dt_bias.copy_(start.reshape(-1))

    def decay_input(self, x: torch.Tensor) -> torch.Tensor:
        """u + bias as (..., Hv, dk)."""
        low = self.f_down(x)
        if self.shape.per_head:
            # every head's own slice of `low` through its own (dk, rank) block: one batched contraction, so autograd keeps
            # W_up once and not a per-token expansion of it
            blocks = self.f_up.weight.to(low.dtype).view(self.hv, self.dk, self.rank)
            u = torch.einsum("...hr,hdr->...hd", low.unflatten(-1, (self.hv, self.rank)), blocks)
        else:
            u = self.f_up(low).unflatten(-1, (self.hv, self.dk))
        return u + self.dt_bias.view(self.hv, self.dk)

    def log_decay(self, pre: torch.Tensor, A_log: torch.Tensor) -> torch.Tensor:
        """g <= 0 from the pre-activation (..., Hv, dk) (float32 or wider) and the layer's per-head A_log."""
        nf = self.n_floor
        free = -torch.exp(A_log.to(pre.dtype))[:, None] * F.softplus(pre[..., nf:])
        if not nf:
            return free
        held = self.floor_log.to(pre.dtype) * torch.sigmoid(pre[..., :nf])
        return torch.cat([held, free], dim=-1)

    def extra_repr(self) -> str:
        return f"proj={self.proj}, rank={self.rank}, floor_channels={self.n_floor}"


def gates(layer, x: torch.Tensor):
    """(g (..., Hv, dk) <= 0, computed in float32 or wider; beta (..., Hv)) of a layer that carries a KDAGate."""
    pre = layer.kda.decay_input(x)
    pre = pre.to(torch.promote_types(pre.dtype, torch.float32))
    return layer.kda.log_decay(pre, layer.A_log), torch.sigmoid(layer.in_proj_b(x))


def added_parameters(cfg, d_model: int) -> int:
    """Parameters a layer gains over the scalar layer: the projection and the per-channel bias come, in_proj_a (d x Hv)
    and the per-head bias (Hv) go."""
    sh = shape_of(cfg)
    gained = d_model * sh.down_width + sh.rank * sh.heads * sh.key_dim + sh.heads * sh.key_dim
    return gained - (d_model * sh.heads + sh.heads)
