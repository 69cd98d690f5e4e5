"""Gated softmax attention with grouped or grid-shared keys/values, QK-norm, partial rotary embedding, an optional
rotary distance cap and an optional length-aware temperature.

* q_proj emits the query and (gate "elementwise") a same-sized sigmoid output gate, interleaved per head.
* Distance cap C (rope_max_distance): a key at most C positions back is scored R(pos_q)q . R(pos_k)k; a key further
  back is scored R(C)q . k with the key unrotated, so no relative angle beyond C is ever seen. The cache therefore
  holds both the rotated keys and the unrotated ones (`k_far`) (reference: ced/model/attention.py:436-553, 902-941).
* Grid KV sharing: k_proj / v_proj emit R row components and C column components; head (i, j) uses [row_i ; col_j].
  The cache holds the raw components and the entries' positions; the read assembles, norms and rotates
  (reference: ced/model/attention.py:263-406, 943-1030).
* Temperature "ssmax": q is scaled per head by (1 + w_h) (1 + ln(n / ref) / ln ref), n = position + 1
  (reference: ced/model/attention.py:631-645, 761-790).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import ops
from ..config import AttentionConfig
from .linear import Linear
from .norms import RMSNorm
from .rope import apply_rope, rotary_dims
from .sequence import SeqContext


@dataclass
class KeySet:
    """Cached keys/values plus what the mask needs. k, v: (B, S, Hkv, hd) (grid: (B, S, 1, width) raw components);
    k_far: the unrotated keys under the distance cap; pos: rotary positions of the entries (grid caches only)."""

    k: torch.Tensor
    v: torch.Tensor
    idx: torch.Tensor
    doc: torch.Tensor
    ok: torch.Tensor
    k_far: torch.Tensor | None = None
    pos: torch.Tensor | None = None
    cp_q: torch.Tensor | None = None           # the Copy-Paste pointer's shared head: this chunk's head query and its key head's key
    cp_k: torch.Tensor | None = None           # (B, L, hd) each; set by the shared layer, taken off by the model, not joined by `cat`
    canon_input: torch.Tensor | None = None    # last K - 1 inputs of the layer's Canon convolution and their documents:
    canon_doc: torch.Tensor | None = None      # set by the encoder layer, not joined by `cat`

    @staticmethod
    def cat(*sets: "KeySet | None") -> "KeySet":
        sets = [s for s in sets if s is not None]
        if len(sets) == 1:
            return sets[0]
        def join(name):
            parts = [getattr(s, name) for s in sets]
            if any(p is None for p in parts):
                if not all(p is None for p in parts):
                    raise ValueError(f"KeySet.cat: field {name!r} is present in some key sets and absent in others")
                return None
            return torch.cat(parts, dim=1)
        return KeySet(**{n: join(n) for n in ("k", "v", "idx", "doc", "ok", "k_far", "pos")})

    def __len__(self) -> int:
        return self.k.shape[1]


@dataclass(frozen=True)
class GridSpec:
    rows: int
    cols: int
    row_dim: int
    col_dim: int
    heads_per_cell: int = 1
    depth: int = 0
    depth_dim: int = 0

    @property
    def axes(self):
        return ((self.rows, self.row_dim), (self.cols, self.col_dim)) + (((self.depth, self.depth_dim),) if self.depth else ())

    @property
    def n_heads(self) -> int:
        return math.prod(c for c, _ in self.axes) * self.heads_per_cell

    @property
    def head_dim(self) -> int:
        return sum(d for _, d in self.axes)

    @property
    def width(self) -> int:
        return sum(c * d for c, d in self.axes)


def grid_spec(cfg: AttentionConfig) -> GridSpec | None:
    """The grid of a config, validated by name; None for kv_sharing "gqa" (reference: ced/model/attention.py:331-366)."""
    keys = (cfg.grid_rows, cfg.grid_cols, cfg.row_dim, cfg.col_dim)
    third = (cfg.grid_depth, cfg.depth_dim)
    if cfg.kv_sharing not in ("gqa", "grid"):
        raise ValueError(f"attention.kv_sharing {cfg.kv_sharing!r}: 'gqa' or 'grid'")
    if cfg.kv_sharing == "gqa":
        if any(keys) or any(third) or cfg.heads_per_cell != 1:
            raise ValueError("attention.grid_rows/grid_cols/row_dim/col_dim/grid_depth/depth_dim/heads_per_cell belong to "
                             "kv_sharing 'grid'; with 'gqa' leave them 0 (heads_per_cell 1)")
        return None
    if not all(type(v) is int and v >= 1 for v in (*keys, cfg.heads_per_cell)):
        raise ValueError(f"attention.kv_sharing 'grid': grid_rows, grid_cols, row_dim, col_dim, heads_per_cell must be integers >= 1, got {(*keys, cfg.heads_per_cell)}")
    if (third[0] == 0) != (third[1] == 0) or min(third) < 0:
        raise ValueError("attention.grid_depth and attention.depth_dim are set together (both 0 or both >= 1)")
    g = GridSpec(*keys, cfg.heads_per_cell, *third)
    if cfg.n_q_heads != g.n_heads:
        raise ValueError(f"attention.kv_sharing 'grid': n_q_heads {cfg.n_q_heads} must equal the grid's {g.n_heads} heads")
    if cfg.head_dim != g.head_dim:
        raise ValueError(f"attention.kv_sharing 'grid': head_dim {cfg.head_dim} must equal row_dim + col_dim (+ depth_dim) = {g.head_dim}")
    if cfg.n_kv_heads != 1:
        raise ValueError("attention.kv_sharing 'grid': n_kv_heads must be 1 (the cache is one head of components)")
    return g


def assemble_grid(comp: torch.Tensor, g: GridSpec) -> torch.Tensor:
    """(B, S, 1, width) components -> (B, S, n_heads, head_dim): head of cell (i, j[, k]) = [row i ; col j (; depth k)],
    cells row-major with the last axis fastest, heads_per_cell consecutive heads per cell. Pure indexing."""
    B, S = comp.shape[:2]
    counts = [c for c, _ in g.axes]
    parts, lo = [], 0
    for a, (count, dim) in enumerate(g.axes):
        shape = [B, S] + [1] * len(counts) + [1, dim]
        shape[2 + a] = count
        parts.append(comp[..., lo:lo + count * dim].reshape(shape).expand(B, S, *counts, g.heads_per_cell, dim))
        lo += count * dim
    return torch.cat(parts, dim=-1).reshape(B, S, g.n_heads, g.head_dim)


def rope_cap(cfg: AttentionConfig) -> int | None:
    C = cfg.rope_max_distance
    if C is None:
        return None
    if not (isinstance(C, int) and not isinstance(C, bool) and C >= 1):
        raise ValueError(f"attention.rope_max_distance {C!r}: None or an integer >= 1")
    return C if rotary_dims(cfg.head_dim, cfg.rope_fraction) > 0 else None


class GatedAttention(nn.Module):
    def __init__(self, d_model: int, cfg: AttentionConfig, norm_eps: float):
        super().__init__()
        if cfg.n_q_heads % cfg.n_kv_heads:
            raise ValueError("attention.n_q_heads must be a multiple of attention.n_kv_heads")
        if cfg.temperature not in ("fixed", "learned", "ssmax"):
            raise ValueError(f"attention.temperature {cfg.temperature!r}")
        self.cfg = cfg
        self.grid = grid_spec(cfg)
        hq, hkv, hd = cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim
        kv_width = hkv * hd if self.grid is None else self.grid.width
        self.q_proj = Linear(d_model, hq * hd * (2 if cfg.gate == "elementwise" else 1))
        self.g_proj = Linear(d_model, hq) if cfg.gate == "headwise" else None
        self.k_proj = Linear(d_model, kv_width)
        self.v_proj = Linear(d_model, kv_width)
        self.o_proj = Linear(hq * hd, d_model)
        self.q_norm = RMSNorm(hd, norm_eps) if cfg.qk_norm else nn.Identity()
        self.k_norm = RMSNorm(hd, norm_eps) if cfg.qk_norm else nn.Identity()
        self.temp_w = nn.Parameter(torch.zeros(hq)) if cfg.temperature != "fixed" else None
        self.cap = rope_cap(cfg)
        self.cp_query = None      # (head, after the temperature?) when the Copy-Paste pointer shares one of this layer's heads (models/cp_head.py)
        self._q_plain = None
        if cfg.normalizer not in ("softmax", "asentmax"):
            raise ValueError(f"attention.normalizer {cfg.normalizer!r}: 'softmax' or 'asentmax'")
        self.entmax = cfg.normalizer == "asentmax"
        if self.entmax:
            # alpha = 1.5 entmax with a learned scale on q: c = 1 + softplus(x w_b + b_b) ln(pos + 2)^(2 tanh(x w_g + b_g)), x the
            # layer's normed input. The two heads are built without touching the global generator and started by the model
            # from a generator of their own, so every other tensor starts as in the softmax model
            # (reference: ced/model/attention.py:32-43, 693-709).
            if cfg.asentmax_chunk < 0:
                raise ValueError(f"attention.asentmax_chunk {cfg.asentmax_chunk}: query rows per chunk, 0 for auto")
            if cfg.temperature != "fixed" or self.cap is not None or self.grid is not None:
                raise ValueError("attention.normalizer 'asentmax' has its own scale on q: temperature 'fixed', no rotary distance "
                                 "cap and kv_sharing 'gqa'")
            with torch.random.fork_rng(devices=[]):
                self.beta_proj = nn.Linear(d_model, hq, bias=True)
                self.gamma_proj = nn.Linear(d_model, hq, bias=True)
            for lin in (self.beta_proj, self.gamma_proj):
                lin.own_init = True
            self.reset_asentmax_parameters()

    @torch.no_grad()
    def reset_asentmax_parameters(self, generator: torch.Generator | None = None) -> None:
        for lin in (self.beta_proj, self.gamma_proj):
            if generator is None or lin.weight.is_meta:
                with torch.random.fork_rng(devices=[]):
                    nn.init.normal_(lin.weight, mean=0.0, std=0.02)
            else:
                lin.weight.copy_(torch.empty(lin.weight.shape, dtype=torch.float32).normal_(0.0, 0.02, generator=generator))
            lin.bias.zero_()

    def asentmax_scale(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """c (B, L, Hq) in >= float32."""
        dt = torch.promote_types(x.dtype, torch.float32)
        F = torch.nn.functional
        with torch.autocast(x.device.type, enabled=False):
            xf = x.to(dt)
            beta = F.softplus(F.linear(xf, self.beta_proj.weight.to(dt), self.beta_proj.bias.to(dt)))
            gamma = 2.0 * torch.tanh(F.linear(xf, self.gamma_proj.weight.to(dt), self.gamma_proj.bias.to(dt)))
            return 1.0 + beta * torch.pow(torch.log((pos + 2).to(dt))[:, :, None], gamma)

    # ------------------------------------------------------------------ pieces

    def query_factor(self, pos: torch.Tensor, dtype: torch.dtype):
        cfg = self.cfg
        if cfg.temperature == "fixed":
            return None
        f = (1.0 + self.temp_w.to(dtype))[:, None]
        if cfg.temperature == "ssmax":
            n = (pos + 1).to(dtype)
            f = f * (1.0 + torch.log(n / cfg.temperature_ref_len) / math.log(cfg.temperature_ref_len))[:, :, None, None]
        return f

    def _rot(self, x, pos):
        return apply_rope(x, pos, self.cfg.rope_fraction, self.cfg.rope_theta)

    def queries(self, x: torch.Tensor, rot_pos: torch.Tensor, pos: torch.Tensor):
        """(q, q_far or None, gate): normed query rotated at its position, and under the cap also by the cap itself;
        the temperature multiplies both."""
        B, L = pos.shape           # the input may be a token shard (tensor parallel); projections return all tokens
        hq, hd = self.cfg.n_q_heads, self.cfg.head_dim
        gate = None
        if self.cfg.gate == "elementwise":
            q, gate = self.q_proj(x).view(B, L, hq, 2 * hd).chunk(2, dim=-1)
        else:
            q = self.q_proj(x).view(B, L, hq, hd)
            if self.g_proj is not None:
                gate = self.g_proj(x).view(B, L, hq, 1)
        qn = self.q_norm(q)
        q = self._rot(qn, rot_pos)
        self._q_plain = q if self.cp_query is not None else None        # the shared head's query before the temperature
        q_far = self._rot(qn, rot_pos.new_full((1, 1), self.cap)) if self.cap is not None else None
        f = self.query_factor(pos, torch.promote_types(q.dtype, torch.float32))
        if self.entmax:
            f = self.asentmax_scale(x, pos)[..., None]
        if f is not None:
            q = (q.to(f.dtype) * f).to(q.dtype)
            if q_far is not None:
                q_far = (q_far.to(f.dtype) * f).to(q_far.dtype)
        return q, q_far, gate

    def keys(self, k_raw: torch.Tensor, rot_pos: torch.Tensor):
        """(k, k_far or None) from projected keys (B, S, Hkv, hd) (grid: raw components (B, S, 1, width))."""
        if self.grid is not None:
            k_raw = assemble_grid(k_raw, self.grid)
        kn = self.k_norm(k_raw)
        return self._rot(kn, rot_pos), (kn if self.cap is not None else None)

    def output(self, o: torch.Tensor, gate: torch.Tensor | None) -> torch.Tensor:
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return self.o_proj(o.flatten(2))

    def fused_prep_ok(self, x: torch.Tensor) -> bool:
        """One kernel does QK-norm, both rotations and the far copies when the layer has the common shape: head
        dimension 64, QK-norm on, fixed temperature, grouped (not grid) keys, 0 or a power of two (<= 32) rotary pairs."""
        cfg = self.cfg
        r2 = rotary_dims(cfg.head_dim, cfg.rope_fraction) // 2
        return (ops.use_native(x) and not self.entmax and self.cp_query is None and x.dtype == torch.bfloat16 and self.grid is None and cfg.qk_norm and cfg.temperature == "fixed"
                and cfg.head_dim == 64 and cfg.gate in ("elementwise", "none") and r2 in (0, 2, 4, 8, 16, 32))

    def _forward_fused(self, x, ctx, cache, rot_pos, cap):
        from ..ops import attention_native as an
        B, L = ctx.doc.shape
        cfg = self.cfg
        hq, hkv, hd = cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim
        r = rotary_dims(hd, cfg.rope_fraction)
        key = ("attn_rot", r, cfg.rope_theta, cap, ctx.rope_scale if self.cap is not None else 1)
        tables = ctx.memo.get(key) if hasattr(ctx, "memo") else None
        if tables is None:
            if r:
                tables = an.rotary_tables(rot_pos, r, cfg.rope_theta, cap)
            else:
                z = torch.zeros(1, dtype=torch.float32, device=x.device)
                tables = (z, z, None, None)
            if hasattr(ctx, "memo"):
                ctx.memo[key] = tables
        interleaved = cfg.gate == "elementwise"
        slot = an.GradSlot() if interleaved and torch.is_grad_enabled() else None
        qg = self.q_proj(x)
        q, q_far, k_new, kf_new = an._AttnPrep.apply(qg, self.k_proj(x), self.q_norm.weight, self.k_norm.weight, *tables,
                                                     self.q_norm.eps, hq, hkv, interleaved, slot)
        if cap is None:
            q_far = kf_new = None
        ok = torch.ones_like(ctx.doc, dtype=torch.bool)
        new = KeySet(k=k_new, v=self.v_proj(x).view(B, L, hkv, hd), idx=ctx.idx, doc=ctx.doc, ok=ok, k_far=kf_new)
        keys = KeySet.cat(cache, new)
        o = ops.attention(q, keys.k, keys.v, ctx.idx, ctx.doc, keys.idx, keys.doc, None if cache is None else keys.ok,
                          q_far=q_far, k_far=keys.k_far, cap=cap, self_aligned=cache is None, q_pos=ctx.pos,
                          single_doc=ctx.single_doc)
        if interleaved:
            o = an._GateOut.apply(o, qg, slot)
        return self.o_proj(o.flatten(2)), keys

    # ------------------------------------------------------------------ forward

    def forward(self, x: torch.Tensor, ctx: SeqContext, cache: KeySet | None = None):
        """Causal self-attention over this chunk plus the cached entries. Returns (y, KeySet incl. this chunk)."""
        B, L = ctx.doc.shape
        cfg = self.cfg
        hkv, hd = cfg.n_kv_heads, cfg.head_dim
        scaled = ctx.rope_scale != 1 and self.cap is not None   # token-scale rotary acts on the capped layers only
        rot_pos = ctx.pos * ctx.rope_scale if scaled else ctx.pos
        cap = self.cap
        if cap is not None and scaled:
            cap = cap // ctx.rope_scale
            if cap < 1:
                raise ValueError("rope_max_distance under token-scale rotary leaves no near key")
        if self.fused_prep_ok(x):
            return self._forward_fused(x, ctx, cache, rot_pos, cap)
        q, q_far, gate = self.queries(x, rot_pos, ctx.pos)
        ok = torch.ones_like(ctx.doc, dtype=torch.bool)
        if self.grid is not None:
            kw = self.grid.width
            new = KeySet(k=self.k_proj(x).view(B, L, 1, kw), v=self.v_proj(x).view(B, L, 1, kw), idx=ctx.idx,
                         doc=ctx.doc, ok=ok, pos=rot_pos)
            keys = KeySet.cat(cache, new)
            k, k_far = self.keys(keys.k, keys.pos)
            v = assemble_grid(keys.v, self.grid)
        else:
            k_new, kf_new = self.keys(self.k_proj(x).view(B, L, hkv, hd), rot_pos)
            new = KeySet(k=k_new, v=self.v_proj(x).view(B, L, hkv, hd), idx=ctx.idx, doc=ctx.doc, ok=ok, k_far=kf_new)
            keys = KeySet.cat(cache, new)
            k, k_far, v = keys.k, keys.k_far, keys.v
            if self.cp_query is not None:      # this chunk's query of the shared head and the key of the key head that serves it
                import dataclasses

                head, after_temperature = self.cp_query
                keys = dataclasses.replace(keys, cp_q=(q if after_temperature else self._q_plain)[:, :, head], cp_k=k_new[:, :, head // (cfg.n_q_heads // hkv)])
                self._q_plain = None
        if self.entmax:      # the exact tensor-op statement on every path
            o = ops.ref.entmax_attention(q, k, v, ctx.idx, ctx.doc, keys.idx, keys.doc, None if cache is None else keys.ok,
                                         chunk=self.cfg.asentmax_chunk)
            return self.output(o, gate), keys
        o = ops.attention(q, k, v, ctx.idx, ctx.doc, keys.idx, keys.doc, None if cache is None else keys.ok,
                          q_far=q_far, k_far=k_far, cap=cap, self_aligned=cache is None, q_pos=ctx.pos,
                          single_doc=ctx.single_doc)
        return self.output(o, gate), keys
