"""Gated DeltaProduct with the second step on a subset of the tokens (`gdn.dprod.stride` s, `summary`, `conv: false`,
`first_beta`; n_h 2).

    S_t = R(k2, v2, beta2) R(k1_t, v1_t, beta1_t) (a_t S_{t-1})    for the carrying tokens: row index p with p mod s = s - 1
    S_t =                  R(k1_t, v1_t, beta1_t) (a_t S_{t-1})    otherwise;     o_t = S_t^T q_t

with R(k, v, beta) S = (I - beta k k^T) S + beta k v^T, the decay once before step 1 and the read after the token's last
update. The second step of a carrying token comes from

    summary none     the token's own x:  k2 = unit(SiLU(W_k x)), v2 = SiLU(W_v x), beta2 = M sigmoid(w_b x), with
                     `dprod.in_proj_kv` / `dprod.in_proj_b` run on the carrying rows only and no short conv
    summary xmean    the same matrices on the mean of x over the tokens of the group of s that are in the carrying (last)
                     token's document
    summary kvmean   no matrix: k2 = unit(mean of k1), v2 = mean of v1 over the same tokens, beta2 = M sigmoid(c),
                     c = `dprod.beta_const` (H_v,) zeros

M = `dprod.beta_max`. Step 1's beta is M sigmoid(b) on a carrying token and sigmoid(b) elsewhere (`first_beta: carry`, so a
token that does not carry is the plain layer's token) or M sigmoid(b) everywhere (`first_beta: all`). An update never
crosses a document boundary, and a group summarises only its last token's document.

How it runs here. The loop (`sparse_recurrence`) is the rule as written. The chunked form runs the ordinary chunked delta
rule on a ROW layout: one row per token plus one row after each carrying token, (k1, v1, beta1, g, q = 0) then
(k2, v2, beta2, g = 0, q); the layout is one concatenation [tokens ; extra rows] followed by one gather through an index
that depends on (L, s, phase) only and is built on the host, and the outputs come back through the inverse gather. A cached
forward needs the phase (the absolute index of the call's first token, one host read) and, with a summary, the running
sums of the group still open (`GDNState.acc`, `GDNState.cnt`). `dprod.sparse_path` names copy strategies of the same
function in the reference; every value runs this one layout. Tensor ops on every device
(reference: ced/model/gdn_dprod_sparse.py:1-701, ced/model/gdn_dprod_sparse_fast.py:39).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .linear import Linear

SUMMARIES = ("none", "xmean", "kvmean")
FIRST_BETAS = ("carry", "all")
PATHS = (None, "plain", "fast", "rows")


@dataclass(frozen=True)
class SparseKeys:
    stride: int
    summary: str
    conv: bool
    first_beta: str

    def moved(self) -> list:
        """The names of the keys that are off their defaults."""
        plain = dict(stride=1, summary="none", conv=True, first_beta="carry")
        return [n for n, v in plain.items() if getattr(self, n) != v]


def keys_of(cfg) -> SparseKeys:
    d = cfg.dprod
    if type(d.stride) is not int or d.stride < 1:
        raise ValueError(f"gdn.dprod.stride {d.stride!r}: an integer >= 1 (1: the second step on every token)")
    for name, allowed in (("summary", SUMMARIES), ("first_beta", FIRST_BETAS), ("sparse_path", PATHS)):
        if getattr(d, name) not in allowed:
            raise ValueError(f"gdn.dprod.{name} {getattr(d, name)!r}: one of {tuple(a for a in allowed if a is not None)}" + (" (or not set)" if None in allowed else ""))
    if type(d.conv) is not bool:
        raise ValueError(f"gdn.dprod.conv {d.conv!r}: true or false")
    return SparseKeys(d.stride, d.summary, d.conv, d.first_beta)


def is_sparse(cfg) -> bool:
    """The layer runs this module: key proj with a stride other than 1, a summary, or conv false."""
    k = keys_of(cfg)
    return cfg.dprod.key == "proj" and (k.stride > 1 or k.summary != "none" or not k.conv)


def check_keys(cfg) -> None:
    k, d = keys_of(cfg), cfg.dprod
    path_moved = d.sparse_path not in (None, "plain")
    used = k.moved() + (["sparse_path"] if path_moved else [])
    what = f"stride {k.stride} / summary {k.summary!r} / conv {k.conv}"
    if d.n_h == 1:
        second_untouched = (d.key, d.value, d.beta, d.rank, d.perm) == ("proj", "proj", "proj", 16, "roll")
        if used and second_untouched:
            raise ValueError(f"gdn.dprod.{', '.join(used)} set with dprod.n_h 1: these keys place the second step and are read only with n_h 2")
        return
    if d.key != "proj":
        clash = [n for n in used if n != "conv"]
        if clash:
            raise ValueError(f"gdn.dprod.{', '.join(clash)} with dprod.key {d.key!r}: the strided and summarised second step is not built together "
                             "with a second step derived from the first")
        return
    if not is_sparse(cfg):
        if path_moved:
            raise ValueError(f"gdn.dprod.sparse_path {d.sparse_path!r} with the stride, summary and conv at their defaults: the key would change nothing")
        return
    if d.n_h != 2:
        raise ValueError(f"gdn.dprod.n_h {d.n_h} with {what}: the second step on a subset of the tokens is n_h 2 only")
    if k.conv:
        raise ValueError(f"gdn.dprod.conv true with {what}: the strided and summarised second step has no short conv (set dprod.conv=false)")
    fixed = dict(value="proj", beta="proj", rank=16, perm="roll", route="interleave", beta_init=None)
    stray = [n for n, v in fixed.items() if getattr(d, n) != v]
    if stray:
        raise ValueError(f"gdn.dprod.{', '.join(stray)} with {what}: not built together")


def params_per_layer(d_model: int, cfg) -> int:
    if cfg.dprod.summary == "kvmean":
        return cfg.n_v_heads
    return d_model * (cfg.n_k_heads * cfg.k_head_dim + cfg.n_v_heads * cfg.v_head_dim + cfg.n_v_heads)


# ------------------------------------------------------------------------------------------------ the layout (host integers)

def first_carry(pos0: int, s: int) -> int:
    """The call index of the first carrying token when the call starts at absolute index pos0."""
    return (-(pos0 + 1)) % s


def carry_flags(L: int, s: int, pos0: int = 0) -> list:
    first = first_carry(pos0, s)
    return [i >= first and (i - first) % s == 0 for i in range(L)]


def row_maps(L: int, s: int, off: int):
    """For a call of L tokens whose first carrying token is at index `off`: (rows, last) as Python lists. rows[r] is where
    row r of the layout comes from in [tokens ; extra rows] (token i at i, the j-th extra row at L + j); last[i] is the row
    token i's output is read on (its extra row when it carries)."""
    rows, last, extra = [], [], 0
    for i in range(L):
        rows.append(i)
        if i >= off and (i - off) % s == 0:
            rows.append(L + extra)
            extra += 1
        last.append(len(rows) - 1)
    return rows, last, extra


def _windows(L: int, s: int, off: int, device):
    """(ends (n_c,), win (n_c, s)): each carrying token's call index and the call indices of its group (negative: before the call)."""
    ends = torch.arange(off, L, s, device=device)
    return ends, ends[:, None] - (s - 1) + torch.arange(s, device=device)[None, :]


def group_sums(u, doc, s: int, off: int, carry_in=None):
    """The sums of the features u (B, L, F) and the token counts over each group closed in the call, restricted to the
    tokens in the document of the group's last token: (sums (B, n_c, F), counts (B, n_c)). One gather of every group's
    window and one masked sum. carry_in (acc, cnt, ok): the sums of the head group's tokens seen in earlier calls, added
    where ok (the carried tokens are in the closing token's document)."""
    ends, win = _windows(u.shape[1], s, off, u.device)
    inside = win >= 0
    at = win.clamp(min=0)
    member = (inside[None] & (doc[:, at] == doc[:, ends][..., None])).to(u.dtype)            # (B, n_c, s)
    sums = (u[:, at] * member[..., None]).sum(2)
    counts = member.sum(2)
    if carry_in is not None and ends.numel() and int(ends[0]) < s - 1:                      # the head group began before the call
        acc, cnt, ok = carry_in
        head_sum = sums[:, 0] + ok[:, None] * acc
        head_cnt = counts[:, 0] + ok * cnt
        sums = torch.cat([head_sum[:, None], sums[:, 1:]], dim=1)
        counts = torch.cat([head_cnt[:, None], counts[:, 1:]], dim=1)
    return sums, counts


def tail_sums(u, doc, s: int, off: int, carry_in=None):
    """The sums over the group still open when the call ends (zeros on a group boundary), restarted at a document start."""
    B, L = u.shape[:2]
    closed = len(range(off, L, s))
    open_from = off + (closed - 1) * s + 1 if closed else 0
    if open_from >= L:
        return u.new_zeros(B, u.shape[-1]), u.new_zeros(B)
    member = (doc[:, open_from:] == doc[:, -1:]).to(u.dtype)
    acc, cnt = torch.einsum("bl,blf->bf", member, u[:, open_from:]), member.sum(1)
    if carry_in is not None and closed == 0:                 # the open group continues one that began earlier
        acc, cnt = acc + carry_in[2][:, None] * carry_in[0], cnt + carry_in[2] * carry_in[1]
    return acc, cnt


def _write(S, key, value, strength):
    """One delta-rule write S <- S + k (x) strength (v - S^T k)."""
    return S + torch.einsum("bhk,bhv->bhkv", key, strength.unsqueeze(-1) * (value - torch.einsum("bhkv,bhk->bhv", S, key)))


def sparse_recurrence(q, k1, v1, g, beta1, is_doc_start, S, carry, k2, v2, beta2):
    """The rule one token at a time. q, k1 (B, L, H, dk) at the value heads; carry: L bools; k2 / v2 / beta2 (B, n_c, ...)."""
    reads, used = [], 0
    for t, carries in enumerate(carry):
        keep = is_doc_start[:, t].logical_not().to(S.dtype)[:, None, None, None]
        S = _write(S * keep * g[:, t].exp()[:, :, None, None], k1[:, t], v1[:, t], beta1[:, t])
        if carries:
            S = _write(S, k2[:, used], v2[:, used], beta2[:, used])
            used += 1
        reads.append(torch.einsum("bhkv,bhk->bhv", S, q[:, t]))
    return torch.stack(reads, dim=1), S


# ------------------------------------------------------------------------------------------------ tensors and forward

class SparseSteps(nn.Module):
    n_extra = 1

    def __init__(self, d_model: int, cfg):
        super().__init__()
        check_keys(cfg)
        k = keys_of(cfg)
        self.stride, self.summary, self.conv, self.first_beta = k.stride, k.summary, k.conv, k.first_beta
        self.channels = cfg.n_k_heads * cfg.k_head_dim + cfg.n_v_heads * cfg.v_head_dim
        self.in_proj_kv = self.in_proj_b = None
        if self.summary == "kvmean":
            self.beta_const = nn.Parameter(torch.zeros(cfg.n_v_heads))
        else:
            with torch.random.fork_rng(devices=[]):
                self.in_proj_kv, self.in_proj_b = Linear(d_model, self.channels), Linear(d_model, cfg.n_v_heads)
            self.in_proj_kv.own_init = self.in_proj_b.own_init = True
        self._maps: dict = {}
        self.reset_own(torch.Generator().manual_seed(0xD9_0D), 0.02)

    @torch.no_grad()
    def reset_own(self, g: torch.Generator, std: float) -> None:
        """in_proj_kv then in_proj_b ~ N(0, std); the constant of kvmean is zeros and draws nothing."""
        if self.in_proj_kv is None:
            self.beta_const.zero_()
            return
        for lin in (self.in_proj_kv, self.in_proj_b):
            w = lin.weight
            if not w.is_meta:
                w.copy_(torch.randn(w.shape, generator=g, dtype=torch.float32).mul(std).to(w))

    def maps(self, L: int, off: int, device):
        key = (L, off, str(device))
        if key not in self._maps:
            rows, last, _ = row_maps(L, self.stride, off)
            self._maps[key] = (torch.tensor(rows, dtype=torch.long, device=device), torch.tensor(last, dtype=torch.long, device=device))
        return self._maps[key]

    def second_step(self, layer, x, k1, v1, ctx, off: int, n_c: int, bmax, carry_in):
        """(k2, v2, beta2) of the carrying tokens, (B, n_c, ...), and the features the summary pools (None without one)."""
        cfg = layer.cfg
        B, L = ctx.doc.shape
        n_k, n_v, d_k, d_v = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim
        feats = None
        if self.summary == "xmean":
            feats = x
        elif self.summary == "kvmean":
            feats = torch.cat([k1.flatten(2), v1.flatten(2)], dim=-1)
        if feats is not None:
            feats = feats.to(torch.promote_types(feats.dtype, torch.float32))
        if n_c == 0:
            return None, None, None, feats
        pooled = None
        if feats is not None:
            total, count = group_sums(feats, ctx.doc, self.stride, off, carry_in)
            pooled = total / count.unsqueeze(-1)
        if self.summary == "kvmean":
            key_mean, value_mean = pooled.split([n_k * d_k, n_v * d_v], dim=-1)
            strength = (bmax * self.beta_const.sigmoid()).expand(B, n_c, n_v)
            return _unit(key_mean.unflatten(-1, (n_k, d_k)).to(k1.dtype)), value_mean.unflatten(-1, (n_v, d_v)).to(v1.dtype), strength, feats
        source = x[:, off::self.stride] if pooled is None else pooled.to(x.dtype)
        key_part, value_part = F.silu(self.in_proj_kv(source)).split([n_k * d_k, n_v * d_v], dim=-1)
        return _unit(key_part.unflatten(-1, (n_k, d_k))), value_part.unflatten(-1, (n_v, d_v)), bmax * self.in_proj_b(source).sigmoid(), feats


def _unit(x):
    return ops.ref.l2_normalize(x.to(torch.promote_types(x.dtype, torch.float32))).to(x.dtype)


def forward(layer, x, ctx, state):
    """(o, conv history, its document ids, S, acc, cnt)."""
    cfg, steps = layer.cfg, layer.dprod
    B, L = ctx.doc.shape
    n_k, n_v, d_k, d_v = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim
    stride, bmax = steps.stride, cfg.dprod.beta_max
    u = layer.in_proj_qkv(x)
    if state is not None and state.conv_input.shape[-1] != u.shape[-1]:
        raise ValueError(f"this GDN cache holds {state.conv_input.shape[-1]} conv channels; a layer with the strided second step carries {u.shape[-1]}")
    past = (None, None) if state is None else (state.conv_input, state.conv_doc)
    q, k1, v1, conv_input, conv_doc = ops.ref.gdn_prep(u, ctx.doc, layer.conv_weight, n_k, n_v, d_k, d_v, *past)
    phase = int(ctx.idx[0, 0]) if state is not None else 0          # the absolute index of the call's first token (one host read with a cache)
    off = first_carry(phase, stride)
    carries = carry_flags(L, stride, phase)
    n_c = sum(carries)
    g, beta1 = ops.ref.gdn_gates(layer.in_proj_a(x), layer.in_proj_b(x), layer.A_log, layer.dt_bias)
    if bmax != 1:                                                   # step 1: M sigmoid(b) on a carrying token, and elsewhere too under first_beta "all"
        everywhere = steps.first_beta == "all" or stride == 1
        lift = torch.tensor([bmax if (c or everywhere) else 1 for c in carries], dtype=beta1.dtype, device=x.device)
        beta1 = beta1 * lift[None, :, None]
    carry_in = None
    if steps.summary != "none" and state is not None and phase % stride:        # the call's first group began in an earlier call
        if state.acc is None:
            raise ValueError("this GDN cache has no running sums: it was not written by a layer with a summarised second step")
        unbroken = ctx.is_doc_start[:, :min(off + 1, L)].any(dim=1).logical_not()
        carry_in = tuple(t.to(torch.promote_types(x.dtype, torch.float32)) for t in (state.acc, state.cnt, unbroken))
    k2, v2, beta2, feats = steps.second_step(layer, x, k1, v1, ctx, off, n_c, bmax, carry_in)
    acc = cnt = None
    if feats is not None:
        acc, cnt = tail_sums(feats, ctx.doc, stride, off, carry_in)
    work = ops.ref.work_dtype(q)
    group = n_v // n_k
    query, key1 = q.repeat_interleave(group, dim=2).to(work), k1.repeat_interleave(group, dim=2).to(work)
    value1, decay, strength1 = v1.to(work), g.to(work), beta1.to(work)
    if n_c:
        key2, value2, strength2 = k2.repeat_interleave(group, dim=2).to(work), v2.to(work), beta2.to(work)
    else:
        key2, value2, strength2 = key1[:, :0], value1[:, :0], strength1[:, :0]
    S0 = state.S.to(work) if state is not None else x.new_zeros(B, n_v, d_k, d_v, dtype=work)
    if cfg.kernel == "recurrence" or L == 1:
        o, S = sparse_recurrence(query, key1, value1, decay, strength1, ctx.is_doc_start, S0, carries, key2, value2, strength2)
        return o, conv_input, conv_doc, S, acc, cnt
    rows, last = steps.maps(L, off, x.device)
    layout = lambda tokens, extra: torch.cat([tokens, extra], dim=1).index_select(1, rows)      # noqa: E731
    not_carrying = torch.tensor([not c for c in carries], device=x.device).to(work)
    q_rows = layout(query * not_carrying[None, :, None, None], query[:, off::stride])           # q is read on a token's last row only
    starts = layout(ctx.is_doc_start, ctx.is_doc_start.new_zeros(B, n_c))
    o_rows, S = ops.ref.chunked_delta_rule(q_rows, layout(key1, key2), layout(value1, value2), layout(decay, torch.zeros_like(strength2)),
                                           layout(strength1, strength2), starts, S0, cfg.chunk_size)
    return o_rows.index_select(1, last), conv_input, conv_doc, S, acc, cnt
