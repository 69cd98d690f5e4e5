"""GDN state diagnostics by position: does the recurrent state of the Gated DeltaNet layers drift at lengths the model
never trained at?

Two views of one row (one document from position 0).

`encoder_gdn_diag` reads the row in blocks through the cache and measures every GDN layer's state S (B, Hv, dk, dv) after
each block: Frobenius norm, largest singular value, stable rank and the relative change since the last block. Cheap, on
the model's own kernels.

`GDNDiagHooks` + `GDNStats` walk the recurrence again from each layer's own input

    S_t = alpha_t S_{t-1} + k_t (x) beta_t (v_t - (alpha_t S_{t-1})^T k_t),   alpha_t = exp(g_t),   o_t = S_t^T q_t

in float32 (the layer's projections, conv and gates through the reference statements; read-only), and at sample
positions p of every position bucket take, per value head, from the state after p and after p - 1:

    norm       ||S_p||_F                                erank   exp(H(sigma / sum sigma)), the effective rank of S_p
    srank      ||S_p||_F^2 / sigma_max^2                sigma_max
    delta      ||S_p - S_{p-1}||_F                      rel_delta = delta / ||S_{p-1}||_F
    decay      (1 - alpha_p) ||S_{p-1}||_F              the part of the change that is forgetting
    write      ||beta_p (v_p - (alpha_p S_{p-1})^T k_p)||   the part that is the new write (||k|| = 1)
    read       ||o_p|| = ||S_p^T q_p||                  what the layer reads out (before its output norm and gate)

and over EVERY position of a bucket the gate statistics per head: mean log decay g, mean decay alpha, mean write gate
beta and the half-life ln 2 / mean(-g) in tokens (a head whose half-life exceeds the training row still holds, beyond
it, state written further back than any row it trained on). Buckets default to 0 / 2k / 8k / 16k / ... / 256k; the
reference bucket is the last one inside the training length, and `GDNStats.result` gives every statistic per layer and
bucket with its ratio to the reference bucket (the drift) and the layers whose ratio leaves [1 / threshold, threshold].
The hooks are forward pre-hooks on every GatedDeltaNet of an eager model: any forward of the model over one row adds
that row's statistics, also a forward in blocks through the cache (the walk carries its own state between blocks).
Layers with a per-channel decay, an erase direction or several sub-steps per token are not walked (their rule is not
the one above). Reference: ced/eval/gdn_diag.py:64-486.
"""

from __future__ import annotations

import math

import torch

from ..models.gdn import GatedDeltaNet
from ..ops import reference as ref

STATS = ("norm", "erank", "srank", "sigma_max", "delta", "rel_delta", "decay", "write", "read")
DRIFT_STATS = ("norm", "erank", "rel_delta", "read", "write")
GATES = ("g", "alpha", "beta")
BASE_LEN = 8192


def default_edges(base: int = BASE_LEN) -> tuple[int, ...]:
    return (0, base // 4, base, 2 * base, 4 * base, 8 * base, 16 * base, 32 * base)


def bucket_names(edges) -> list[str]:
    short = lambda n: f"{n // 1024}k" if n >= 1024 and n % 1024 == 0 else str(n)
    return [f"{short(a)}-{short(b)}" for a, b in zip(edges[:-1], edges[1:])] + [f"{short(edges[-1])}+"]


def bucket_index(positions: torch.Tensor, edges) -> torch.Tensor:
    return torch.bucketize(positions, torch.tensor(list(edges[1:]), device=positions.device), right=True)


def sample_positions(n_valid: int, edges, per_bucket: int = 16) -> torch.Tensor:
    """At most `per_bucket` evenly spaced positions p >= 1 inside each bucket's part of [0, n_valid), increasing."""
    out = []
    bounds = list(edges) + [max(n_valid, edges[-1])]
    for a, b in zip(bounds[:-1], bounds[1:]):
        a, b = max(a, 1), min(b, n_valid)
        if b <= a:
            continue
        k = min(per_bucket, b - a)
        out += sorted({a + (i * (b - a)) // k + (b - a) // (2 * k) for i in range(k)})
    return torch.tensor(sorted(set(p for p in out if p < n_valid)), dtype=torch.long)


def state_measures(S: torch.Tensor) -> dict[str, torch.Tensor]:
    """Per head of S (..., dk, dv): norm, sigma_max, srank, erank (and the older names fro / stable_rank)."""
    Sf = S.float()
    sv = torch.linalg.svdvals(Sf)
    fro = sv.pow(2).sum(-1).sqrt()
    top = sv[..., 0]
    p = sv / sv.sum(-1, keepdim=True).clamp_min(1e-30)
    ent = -(p * torch.log(p.clamp_min(1e-30))).sum(-1)
    srank = (fro / top.clamp_min(1e-30)) ** 2
    return {"norm": fro, "sigma_max": top, "srank": srank, "erank": torch.exp(ent), "fro": fro, "stable_rank": srank}


@torch.no_grad()
def encoder_gdn_diag(model, tokens: torch.Tensor, doc_ids: torch.Tensor, block: int = 2048, autocast_dtype=None) -> list[dict]:
    """One record per block: position reached and, per GDN layer, the head-averaged measures of the cached state."""
    dev = next(model.parameters()).device
    tokens, doc_ids = tokens.to(dev), doc_ids.to(dev)
    cache, prev, out = None, {}, []
    for s in range(0, tokens.shape[1], block):
        with torch.autocast(dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
            res = model.forward(tokens[:, s:s + block], doc_ids[:, s:s + block], cache=cache, return_cache=True, return_hidden=True)
        cache = res.cache
        rec = {"position": min(s + block, tokens.shape[1]), "layers": {}}
        for i, (layer, c) in enumerate(zip(model.encoder.layers, cache.encoder)):
            if layer.kind != "gdn" or c is None or c.S is None:
                continue
            m = {k: float(v.mean()) for k, v in state_measures(c.S).items()}
            if i in prev:
                m["rel_change"] = float((c.S.float() - prev[i]).norm() / prev[i].norm().clamp_min(1e-30))
            prev[i] = c.S.float().clone()
            rec["layers"][i] = m
        out.append(rec)
    return out


# ------------------------------------------------------------------------------------------------------------ the state walk

def layer_inputs(mixer: GatedDeltaNet, x, ctx, state, arms, x_write, x_read):
    """(q, k, v, g, beta) of one call of a GDN layer at the value heads, float32, through the reference statements."""
    cfg = mixer.cfg
    hk, hv, dk, dv = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim
    u_pre, a_lin, b_lin = mixer.project(x, arms, x_write, x_read)
    hist, hist_doc = (None, None) if state is None else (state.conv_input, state.conv_doc)
    q, k, v, _, _ = ref.gdn_prep(u_pre.float(), ctx.doc, mixer.conv_weight.float(), hk, hv, dk, dv,
                                 None if hist is None else hist.float(), hist_doc)
    g, beta = ref.gdn_gates(a_lin.float(), b_lin.float(), mixer.A_log.float(), mixer.dt_bias.float(), ctx.gdn_scale, ctx.gdn_beta_power)
    beta = beta * mixer.beta_max
    rep = hv // hk
    if rep > 1:
        q, k = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
    return q, k, v, g, beta


def walk(q, k, v, g, beta, is_doc_start, S, positions: list[int], chunk: int = 64):
    """The recurrence over one call's L positions from state S; at every local position p of `positions` (increasing) the
    per-head statistics of STATS as a dict of (Hv,) tensors. Returns ({p: stats}, final state)."""
    out, at = {}, 0
    L = q.shape[1]
    seg = lambda a, b: tuple(t[:, a:b] for t in (q, k, v, g, beta, is_doc_start))
    for p in positions:
        if p > at:                                     # up to and including p - 1
            _, S = ref.chunked_delta_rule(*seg(at, p), S, chunk)
        prev = S
        o, S = ref.delta_rule_recurrence(*seg(p, p + 1), S)
        alpha = torch.exp(g[0, p])
        kept = prev[0] * (0.0 if bool(is_doc_start[0, p]) else 1.0)
        pred = torch.einsum("hkv,hk->hv", kept * alpha[:, None, None], k[0, p])
        m = state_measures(S[0])
        prev_norm = kept.flatten(-2).norm(dim=-1)
        delta = (S[0] - kept).flatten(-2).norm(dim=-1)
        out[p] = {"norm": m["norm"], "erank": m["erank"], "srank": m["srank"], "sigma_max": m["sigma_max"], "delta": delta,
                  "rel_delta": delta / prev_norm.clamp_min(1e-30), "decay": (1 - alpha) * prev_norm,
                  "write": (beta[0, p][:, None] * (v[0, p] - pred)).norm(dim=-1), "read": o[0, 0].norm(dim=-1)}
        at = p + 1
    if at < L:
        _, S = ref.chunked_delta_rule(*seg(at, L), S, chunk)
    return out, S


class GDNStats:
    """Accumulates, per GDN layer and position bucket, the sampled state statistics and the all-position gate statistics of
    the rows it is given; `result` averages them and relates every bucket to the reference bucket."""

    def __init__(self, edges=None, per_bucket: int = 16, train_len: int = BASE_LEN):
        self.edges = tuple(edges) if edges is not None else default_edges(train_len)
        self.per_bucket, self.train_len = per_bucket, train_len
        self.names = bucket_names(self.edges)
        self.sums: dict = {}           # layer -> bucket -> stat -> [sum over samples (Hv,), count]
        self.gates: dict = {}          # layer -> bucket -> gate -> [sum over positions (Hv,), count]
        self.rows = 0

    def add_samples(self, layer: int, position: int, stats: dict) -> None:
        b = int(bucket_index(torch.tensor([position]), self.edges))
        cell = self.sums.setdefault(layer, {}).setdefault(b, {})
        for name, value in stats.items():
            acc = cell.setdefault(name, [torch.zeros_like(value, dtype=torch.float64), 0])
            acc[0] += value.double()
            acc[1] += 1

    def add_gates(self, layer: int, first_position: int, g: torch.Tensor, beta: torch.Tensor) -> None:
        """g, beta (L, Hv) of consecutive positions starting at first_position."""
        pos = torch.arange(first_position, first_position + g.shape[0])
        which = bucket_index(pos, self.edges)
        for b in which.unique().tolist():
            sel = which == b
            cell = self.gates.setdefault(layer, {}).setdefault(int(b), {})
            for name, value in (("g", g[sel]), ("alpha", torch.exp(g[sel])), ("beta", beta[sel])):
                acc = cell.setdefault(name, [torch.zeros(value.shape[1], dtype=torch.float64), 0])
                acc[0] += value.double().sum(0)
                acc[1] += int(sel.sum())

    def reference_bucket(self) -> int:
        """The last bucket that lies inside the training length."""
        inside = [i for i, (a, b) in enumerate(zip(self.edges[:-1], self.edges[1:])) if b <= self.train_len]
        return inside[-1] if inside else 0

    def result(self, threshold: float = 2.0) -> dict:
        ref_b = self.reference_bucket()
        layers, flagged = {}, []
        for layer in sorted(self.sums):
            table = {}
            for b in sorted(self.sums[layer]):
                row = {name: (acc[0] / max(acc[1], 1)) for name, acc in self.sums[layer][b].items()}
                rec = {name: float(v.mean()) for name, v in row.items()}
                rec["per_head"] = {name: [round(float(x), 6) for x in v] for name, v in row.items() if name in DRIFT_STATS}
                rec["samples"] = next(iter(self.sums[layer][b].values()))[1]
                gates = self.gates.get(layer, {}).get(b, {})
                for name in GATES:
                    if name in gates:
                        rec[name] = float((gates[name][0] / max(gates[name][1], 1)).mean())
                if "g" in gates:
                    mean_g = gates["g"][0] / max(gates["g"][1], 1)
                    rec["half_life"] = [float(math.log(2.0) / max(-float(x), 1e-12)) for x in mean_g]
                    rec["heads_beyond_training"] = int(sum(h > self.train_len for h in rec["half_life"]))
                table[self.names[b]] = rec
            base = table.get(self.names[ref_b])
            if base is not None:
                for name, rec in table.items():
                    rec["drift"] = {s: (rec[s] / base[s] if base[s] else float("nan")) for s in DRIFT_STATS}
                    out_of_band = [s for s, r in rec["drift"].items() if r == r and not (1.0 / threshold <= r <= threshold)]
                    if out_of_band and name != self.names[ref_b]:
                        flagged.append({"layer": layer, "bucket": name, "stats": out_of_band})
            layers[layer] = table
        return {"edges": list(self.edges), "buckets": self.names, "reference_bucket": self.names[ref_b], "threshold": threshold, "rows": self.rows,
                "layers": layers, "flagged": flagged}


class GDNDiagHooks:
    """Forward pre-hooks on every plain GatedDeltaNet of `model` (eager): each forward over ONE row adds its statistics to
    `stats`. A row may be fed in blocks through the cache; call `new_row()` before each new row."""

    def __init__(self, model, stats: GDNStats, n_valid: int | None = None, chunk: int = 64):
        self.model, self.stats, self.n_valid, self.chunk = model, stats, n_valid, chunk
        self.handles, self.state, self.offset, self.skipped = [], {}, {}, []

    def new_row(self, n_valid: int | None = None) -> None:
        self.state.clear()
        self.offset.clear()
        self.n_valid = n_valid
        self.stats.rows += 1

    def __enter__(self):
        index = 0
        for i, layer in enumerate(self.model.encoder.layers):
            mixer = getattr(layer, "mixer", None)
            if not isinstance(mixer, GatedDeltaNet):
                continue
            if mixer.kda is not None or mixer.erase is not None or mixer.dprod is not None:
                self.skipped.append(i)
                continue
            self.handles.append(mixer.register_forward_pre_hook(self._hook(i, mixer), with_kwargs=True))
            index += 1
        self.stats.rows += 1
        return self

    def __exit__(self, *exc):
        for h in self.handles:
            h.remove()
        self.handles = []

    def _hook(self, layer: int, mixer: GatedDeltaNet):
        def hook(module, args, kwargs):
            names = ("x", "ctx", "state", "arms", "x_write", "x_read")
            call = dict(zip(names, args))
            call.update({k: v for k, v in kwargs.items() if k in names})
            x, ctx = call["x"], call["ctx"]
            if x.shape[0] != 1:
                raise ValueError("the GDN diagnostics walk one row at a time")
            with torch.no_grad():
                q, k, v, g, beta = layer_inputs(mixer, x, ctx, call.get("state"), call.get("arms"), call.get("x_write"), call.get("x_read"))
                first = self.offset.get(layer, 0)
                L = q.shape[1]
                total = first + L if self.n_valid is None else self.n_valid
                wanted = sample_positions(max(total, first + L), self.stats.edges, self.stats.per_bucket).tolist()
                local = [p - first for p in wanted if first <= p < min(first + L, total)]
                S = self.state.get(layer)
                if S is None:
                    S = torch.zeros(1, q.shape[2], q.shape[3], v.shape[3], dtype=torch.float32, device=q.device)
                found, S = walk(q, k, v, g, beta, ctx.is_doc_start, S, local, self.chunk)
                for p, st in found.items():
                    self.stats.add_samples(layer, first + p, {n: t.cpu() for n, t in st.items()})
                keep = max(0, min(L, total - first))
                self.stats.add_gates(layer, first, g[0, :keep].cpu(), beta[0, :keep].cpu())
                self.state[layer], self.offset[layer] = S, first + L
            return None
        return hook


@torch.no_grad()
def gdn_position_diag(model, tokens: torch.Tensor, doc_ids: torch.Tensor, edges=None, per_bucket: int = 16, train_len: int = BASE_LEN,
                      block: int | None = None, autocast_dtype=None, threshold: float = 2.0) -> dict:
    """The bucketed statistics of one row (1, L): the model is run once (in blocks of `block` through the cache when given)
    under the hooks. Returns `GDNStats.result`."""
    dev = next(model.parameters()).device
    tokens, doc_ids = tokens.to(dev), doc_ids.to(dev)
    stats = GDNStats(edges, per_bucket, train_len)
    was_training = model.training
    model.eval()
    try:
        with GDNDiagHooks(model, stats, n_valid=tokens.shape[1]):
            step = block or tokens.shape[1]
            cache = None
            for s in range(0, tokens.shape[1], step):
                with torch.autocast(dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
                    res = model.forward(tokens[:, s:s + step], doc_ids[:, s:s + step], cache=cache, return_cache=True, return_hidden=True)
                cache = res.cache
    finally:
        model.train(was_training)
    return stats.result(threshold)
