"""Optimizer construction: parameter groups by name, flat parameter / gradient / moment buffers, AdamW over them.

Group rules (reference: ced/train/optim.py:198-470): no weight decay for the token embedding (= the tied head),
`A_log`, `dt_bias`; with `optim.zero_gate_decay: none` also the zero-initialised mix lambdas; with
`optim.mix_query_decay` the named depth-mix pseudo-queries. Under `optim.name: muon` 2-D hidden matrices go to Muon
and everything else (embeddings, norm gains, conv, gates, in_proj_a/b, depth readers) to AdamW.

Layout: every parameter is a view into ONE flat float32 master buffer (64-element aligned), its gradient a view into
one flat float32 gradient buffer, and — on CUDA — its bfloat16 compute copy a view into one flat bfloat16 buffer that
the update kernel refreshes in the same pass that applies AdamW. Flat buffers are what the data-parallel collectives
and the fused reduce-scatter + update kernels operate on; their element ranges are the ZeRO shards.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

NO_DECAY_SUFFIXES = ("embed.weight", ".A_log", ".dt_bias", ".temp_w", ".skip_gain", ".x0_gain", ".beta_proj.weight", ".beta_proj.bias",
                     ".gamma_proj.weight", ".gamma_proj.bias",
                     # a looped middle's injection (models/recur.py): B starts at the identity and w near 1, decay would pull both
                     # away from their starts; A_log / dt_bias are covered by the GDN suffixes above
                     "injection.B", ".recur_mix",
                     # the lanes of the looped encoder-decoder (models/looped_decoder.py) start as the plain loop: no pull toward 0
                     "hyper_connections.read_weights", "hyper_connections.mix_weights", "hyper_connections.write_weights",
                     # the Copy-Paste head's <copy> row (the LM head's rule) and its QK-norm gain (the pointer's temperature)
                     "cp_head.w_copy", "cp_head.qk_gain")
ZERO_GATE_SUFFIXES = (".gdn_arms.ccr_gate", ".gdn_arms.write_lambda", ".gdn_arms.qmix_lambda", ".erase.scale", ".dprod.beta_const")
# The cross-read's query translators (models/ccr.py): D = M - I, (H_k, d_k, d_k) a reader, never a Muon matrix (3-D). One
# AdamW group of their own, the last, at the depth readers' learning rate; optim.ccr_translator_decay "none": no decay,
# "identity": the run's weight decay, which on D pulls M toward the identity (reference: ced/train/optim.py:283-312).
CCR_TRANSLATOR_SUFFIX = ".gdn_arms.ccr_translator_delta"
RECUR_B, RECUR_B_MODES = "encoder.recur_injection.B", ("adamw", "muon", "muon_no_decay")     # reference: ced/train/optim.py:427-441, 956-971
SKIP_GAIN = "encoder.skip_gain"
CCR_TRANSLATOR_DECAY_MODES = ("none", "identity")
MIX_QUERY_DECAY = {"decay": (), "none_qmix": (".gdn_arms.qmix_query.query",),
                   "none_write_qmix": (".gdn_arms.write_query.query", ".gdn_arms.qmix_query.query")}
ADAMW_MATRIX_SUFFIXES = ("in_proj_a.weight", "in_proj_b.weight", "beta_proj.weight", "gamma_proj.weight", ".kda.f_down.weight",
                         ".kda.f_up.weight", ".erase.e_down.weight", ".erase.e_up.weight", ".erase.in_proj_gamma.weight",
                         ".dprod.k_down.weight", ".dprod.k_up.weight")      # the derived second key's low-rank address pair
ALIGN = 64


def no_decay_suffixes(o) -> tuple:
    if o.zero_gate_decay not in ("decay", "none"):
        raise ValueError(f"optim.zero_gate_decay {o.zero_gate_decay!r}: 'decay' or 'none'")
    if o.mix_query_decay not in MIX_QUERY_DECAY:
        raise ValueError(f"optim.mix_query_decay {o.mix_query_decay!r}: one of {list(MIX_QUERY_DECAY)}")
    extra = ZERO_GATE_SUFFIXES if o.zero_gate_decay == "none" else ()
    return NO_DECAY_SUFFIXES + extra + MIX_QUERY_DECAY[o.mix_query_decay]


def is_muon_param(name: str, p: torch.Tensor) -> bool:
    if p.ndim != 2 or name.endswith(("embed.weight", "conv_weight") + ADAMW_MATRIX_SUFFIXES):
        return False
    # loop-boundary tensors (injection, lanes, loop embedding), routers, depth mixers and the copy head stay on AdamW
    return not any(part in name for part in (".attn_res.", "injection", "hyper_connections", "router", "loop_embedding")) and not name.startswith("cp_head.")


GDN_MUP_BASE_WIDTH = 512


def gdn_mup_names(model) -> tuple[list[str], list[str]]:
    """(gate projection weights, gate scalars) of every GatedDeltaNet, by parameter name, in the model's order."""
    from ..models.gdn import GatedDeltaNet

    gates, scalars = set(), set()
    for prefix, m in model.named_modules():
        if isinstance(m, GatedDeltaNet):
            if m.kda is not None or m.erase is not None or m.dprod is not None:
                raise ValueError("optim.gdn_mup scales in_proj_a / in_proj_b and the per-head gate scalars: not built with "
                                 "gdn.kda.decay 'channel' or gdn.erase.mode 'eda'")
            gates.update(f"{prefix}.{n}.weight" for n in ("in_proj_a", "in_proj_b"))
            scalars.update(f"{prefix}.{n}" for n in ("A_log", "dt_bias"))
    names = [n for n, _ in model.named_parameters()]
    return [n for n in names if n in gates], [n for n in names if n in scalars]


def _gdn_mup_spec(spec, model, o, base_scale: float):
    """muP grouping of the GDN gates under AdamW: the gate projections leave their groups for one group per fan-in with
    the learning rate scaled by base_width / fan_in (and the run's weight decay); A_log and dt_bias for one group at the
    plain scale without decay. Every other tensor keeps its group and place (reference: ced/train/optim.py:654-712)."""
    if type(o.gdn_mup_base_width) is not int or o.gdn_mup_base_width < 1:
        raise ValueError(f"optim.gdn_mup_base_width {o.gdn_mup_base_width!r}: a positive integer")
    gates, scalars = gdn_mup_names(model)
    if not gates:
        raise ValueError("optim.gdn_mup groups a model's GDN gates and scalars: this model has no GatedDeltaNet layer")
    moved = set(gates) | set(scalars)
    named = dict(model.named_parameters())
    out = [(k, [(n, p) for n, p in items if n not in moved], wd, s) for k, items, wd, s in spec]
    for fan_in in sorted({named[n].shape[1] for n in gates}):
        out.append(("adamw", [(n, named[n]) for n in gates if named[n].shape[1] == fan_in], o.weight_decay,
                    base_scale * o.gdn_mup_base_width / fan_in))
    out.append(("adamw", [(n, named[n]) for n in scalars], 0.0, base_scale))
    return out


@torch.no_grad()
def gdn_mup_init_(model, base_width: int = GDN_MUP_BASE_WIDTH) -> None:
    """The gate projections as drawn times sqrt(base_width / fan_in): variance proportional to 1 / fan_in, today's at the
    base width. No random number is drawn (reference: ced/train/optim.py:715-727)."""
    named = dict(model.named_parameters())
    for n in gdn_mup_names(model)[0]:
        named[n].mul_((base_width / named[n].shape[1]) ** 0.5)


def param_groups(model, o, trainable=None) -> list[dict]:
    """Groups as dicts {"names", "params", "weight_decay", "lr_scale", "kind"}; kind "adamw" or "muon". trainable: an
    optional predicate over parameter names (a frozen trunk): the tensors it rejects keep their place in the flat buffers
    in AdamW groups of learning-rate scale 0 and no decay, so an update leaves their bytes as they are."""
    suffixes = no_decay_suffixes(o)
    named = list(model.named_parameters())
    if o.name == "adamw":
        decay = [(n, p) for n, p in named if not n.endswith(suffixes)]
        plain = [(n, p) for n, p in named if n.endswith(suffixes)]
        spec = [("adamw", decay, o.weight_decay, 1.0), ("adamw", plain, 0.0, 1.0)]
    elif o.name == "muon":
        b_muon = o.recur_b == "muon"            # the looped middle's dense injection matrix as one more Muon tensor (optim.recur_b)
        mats = [(n, p) for n, p in named if is_muon_param(n, p) or (b_muon and n == RECUR_B)]
        rest = [(n, p) for n, p in named if not is_muon_param(n, p) and not (o.recur_b != "adamw" and n == RECUR_B)]
        decay = [(n, p) for n, p in rest if not n.endswith(suffixes)]
        plain = [(n, p) for n, p in rest if n.endswith(suffixes)]
        spec = [("muon", mats, o.weight_decay, 1.0), ("adamw", decay, o.weight_decay, o.adamw_lr_scale),
                ("adamw", plain, 0.0, o.adamw_lr_scale)]
    else:
        raise ValueError(f"optim.name {o.name!r}: 'adamw' or 'muon'")
    if o.recur_b not in RECUR_B_MODES:
        raise ValueError(f"optim.recur_b {o.recur_b!r}: one of {RECUR_B_MODES}")
    if o.recur_b != "adamw":
        if o.name != "muon":
            raise ValueError(f"optim.recur_b {o.recur_b!r} is read under optim.name 'muon', not {o.name!r} (there every tensor is on AdamW)")
        own = [(n, p) for n, p in named if n == RECUR_B and p.ndim == 2]
        if not own:
            raise ValueError(f"optim.recur_b {o.recur_b!r} is for the dense matrix {RECUR_B} of a looped middle's injection (model.loop.recur_layers "
                             "with injection 'parcae' and recur_inject_b 'dense'); this model has none")
        if o.recur_b == "muon_no_decay":        # the Muon update in a group of its own without weight decay, after the groups above
            spec.append(("muon", own, 0.0, 1.0))
    a_scale = o.layer_scalar_a_lr_scale
    if isinstance(a_scale, bool) or not isinstance(a_scale, (int, float)) or not a_scale > 0 or a_scale != a_scale or a_scale == float("inf"):
        raise ValueError(f"optim.layer_scalar_a_lr_scale {a_scale!r}: a finite number above 0")
    if a_scale != 1.0:      # the residual scalars' a alone at its own learning rate: a group of its own, the last of these, without decay
        gain = [(n, p) for n, p in named if n == SKIP_GAIN]
        if not gain:
            raise ValueError(f"optim.layer_scalar_a_lr_scale {a_scale!r} scales the LR of {SKIP_GAIN} (model.encoder.layer_scalars with a stored a); this model has none: leave it 1.0")
        spec = [(k, [(n, p) for n, p in items if n != SKIP_GAIN], wd, sc) for k, items, wd, sc in spec]
        spec.append(("adamw", gain, 0.0, (1.0 if o.name == "adamw" else o.adamw_lr_scale) * a_scale))
    if o.gdn_mup_base_width != GDN_MUP_BASE_WIDTH and not o.gdn_mup:
        raise ValueError(f"optim.gdn_mup_base_width {o.gdn_mup_base_width!r} is read with optim.gdn_mup true: leave it {GDN_MUP_BASE_WIDTH}")
    if o.gdn_mup:
        spec = _gdn_mup_spec(spec, model, o, 1.0 if o.name == "adamw" else o.adamw_lr_scale)
    # A gated second pass's own tensors (models/second_pass.py): AdamW groups of their own at optim.pass2_lr_scale x the LR of
    # the other AdamW tensors; the pass-2 embedding with the run's weight decay, the gate without (reference: ced/train/optim.py:388-398).
    from ..models.second_pass import PASS2_PARAMETERS

    later = [(n, p) for n, p in named if n in PASS2_PARAMETERS]
    if not (isinstance(o.pass2_lr_scale, (int, float)) and o.pass2_lr_scale > 0):
        raise ValueError(f"optim.pass2_lr_scale {o.pass2_lr_scale!r}: a positive multiplier")
    if later:
        taken = {n for n, _ in later}
        base = (1.0 if o.name == "adamw" else o.adamw_lr_scale) * o.pass2_lr_scale
        spec = [(k, [(n, p) for n, p in items if n not in taken], wd, sc) for k, items, wd, sc in spec]
        spec.append(("adamw", [(n, p) for n, p in later if not n.endswith("_gate")], o.weight_decay, base))
        spec.append(("adamw", [(n, p) for n, p in later if n.endswith("_gate")], 0.0, base))
    elif o.pass2_lr_scale != 1.0:
        raise ValueError(f"optim.pass2_lr_scale {o.pass2_lr_scale!r} scales the LR of a gated second pass's tensors (model.loop.pass2_gate); this model has none: leave it 1.0")
    if o.ccr_translator_decay not in CCR_TRANSLATOR_DECAY_MODES:
        raise ValueError(f"optim.ccr_translator_decay {o.ccr_translator_decay!r}: one of {CCR_TRANSLATOR_DECAY_MODES}")
    mats = [(n, p) for n, p in named if n.endswith(CCR_TRANSLATOR_SUFFIX)]
    if not mats and o.ccr_translator_decay != "none":
        raise ValueError(f"optim.ccr_translator_decay {o.ccr_translator_decay!r} is read for the cross-read's query translators "
                         "(model.encoder.gdn_ccr_translator 'key_head'); this model has none: leave it 'none'")
    if mats:
        taken = {n for n, _ in mats}
        spec = [(k, [(n, p) for n, p in items if n not in taken], wd, sc) for k, items, wd, sc in spec]
        spec.append(("adamw", mats, 0.0 if o.ccr_translator_decay == "none" else o.weight_decay, 1.0 if o.name == "adamw" else o.adamw_lr_scale))
    if trainable is not None:
        frozen = [(n, p) for _, items, _, _ in spec for n, p in items if not trainable(n)]
        spec = [(k, [(n, p) for n, p in items if trainable(n)], wd, sc) for k, items, wd, sc in spec] + [("adamw", frozen, 0.0, 0.0)]
    return [{"kind": k, "names": [n for n, _ in items], "params": [p for _, p in items], "weight_decay": wd, "lr_scale": s}
            for k, items, wd, s in spec if items]


@dataclass
class Segment:
    name: str
    offset: int
    numel: int
    shape: tuple
    group: int


class FlatBuffers:
    """The model's parameters re-homed into flat buffers, group by group (each group one contiguous range)."""

    def __init__(self, model, groups: list[dict], device, lp_dtype=None, order=None):
        """order: optional key function over parameter names; a group's tensors are laid out sorted by it (stable), so
        tensors whose gradients finish together can be made neighbours (bucketed gradient reduction)."""
        self.segments: list[Segment] = []
        self.group_ranges: list[tuple[int, int]] = []
        at = 0
        for gi, g in enumerate(groups):
            lo = at
            members = list(zip(g["names"], g["params"]))
            if order is not None:
                members.sort(key=lambda np_: order(np_[0]))
            for n, p in members:
                self.segments.append(Segment(n, at, p.numel(), tuple(p.shape), gi))
                at += -(-p.numel() // ALIGN) * ALIGN
            self.group_ranges.append((lo, at))
        self.size = -(-at // 1024) * 1024
        self.params = torch.zeros(self.size, dtype=torch.float32, device=device)
        self.grads = torch.zeros(self.size, dtype=torch.float32, device=device)
        self.lp = torch.zeros(self.size, dtype=lp_dtype, device=device) if lp_dtype is not None else None
        by_name = dict(model.named_parameters())
        self.by_name = {}
        for s in self.segments:
            p = by_name[s.name]
            view = self.params[s.offset:s.offset + s.numel].view(s.shape)
            view.copy_(p.data)
            p.data = view
            p.grad = self.grads[s.offset:s.offset + s.numel].view(s.shape)
            p.main_grad = p.grad        # where weight-gradient GEMMs may accumulate directly (`wgrad_accum: fp32`)
            self.by_name[s.name] = s
        if self.lp is not None:
            self.refresh_lp()
            mods = dict(model.named_modules())
            for s in self.segments:
                owner, _, leaf = s.name.rpartition(".")
                m = mods.get(owner)
                if leaf == "weight" and hasattr(m, "weight_lp"):
                    m.weight_lp = self.lp[s.offset:s.offset + s.numel].view(s.shape)
            head = "embed.weight" if model.out_embed is None else "out_embed.weight"
            s = self.by_name[head]
            model.head_weight_lp = self.lp[s.offset:s.offset + s.numel].view(s.shape)

    def rebind(self, model, params, grads, lp) -> None:
        """Move the model onto other flat buffers of at least this size (symmetric memory, grown ZeRO buffers): the
        contents must already be there; parameters, gradients and bf16 copies become views of the new buffers."""
        self.params, self.grads, self.lp = params, grads, lp
        self.size = params.numel()
        named = dict(model.named_parameters())
        mods = dict(model.named_modules())
        for s in self.segments:
            p = named[s.name]
            p.data = params[s.offset:s.offset + s.numel].view(s.shape)
            p.grad = grads[s.offset:s.offset + s.numel].view(s.shape)
            p.main_grad = p.grad
            owner, _, leaf = s.name.rpartition(".")
            if lp is not None and leaf == "weight" and hasattr(mods.get(owner), "weight_lp"):
                mods[owner].weight_lp = lp[s.offset:s.offset + s.numel].view(s.shape)
        if lp is not None:
            head = "embed.weight" if model.out_embed is None else "out_embed.weight"
            model.head_weight_lp = self.view(lp, head)

    def refresh_lp(self) -> None:
        if self.lp is not None:
            if self.params.is_cuda:
                from ..ops import native

                native.cast_bf16_(self.params, self.lp)
            else:
                self.lp.copy_(self.params)

    def view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        s = self.by_name[name]
        return flat[s.offset:s.offset + s.numel].view(s.shape)

    def rebind_grads(self, model) -> None:
        """Point every parameter's .grad at its flat view again (after something set it to None)."""
        for n, p in model.named_parameters():
            p.grad = self.view(self.grads, n)
            p.main_grad = p.grad


class FlatAdamW:
    """AdamW on flat buffers with decoupled weight decay, bias correction as torch.optim.AdamW.

    shard (lo, hi): the element range this rank updates (ZeRO); moments exist for that range only. On CUDA the update
    of a group is one launch of the fused kernel (moments, master weight and bf16 copy in one pass)."""

    def __init__(self, flat: FlatBuffers, groups: list[dict], betas, eps: float, shard=None):
        """shard: None (everything), one (lo, hi) element range, or a list of disjoint ascending ranges (a rank's slices
        of several buckets); the moments are stored range after range."""
        self.flat, self.groups = flat, groups
        self.betas, self.eps = tuple(betas), eps
        ranges = [(0, flat.size)] if shard is None else ([tuple(shard)] if isinstance(shard[0], int) else [tuple(r) for r in shard])
        self.ranges, n = [], 0          # (lo, hi, offset of the range in the moment buffers)
        for lo, hi in ranges:
            self.ranges.append((lo, hi, n))
            n += hi - lo
        self.lo, self.hi = ranges[0][0], ranges[-1][1]
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=flat.params.device)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=flat.params.device)
        self.steps = 0
        self.param_groups = [{"lr": 0.0, "lr_scale": g["lr_scale"], "weight_decay": g["weight_decay"], "kind": g["kind"]}
                             for g in groups]
        # the order torch.optim numbers parameters in: group after group, each in the model's parameter order (the flat
        # layout may order a group's tensors differently; checkpoints are written and read in this order)
        self.torch_order = [[n for n in g["names"]] for g in groups]

    def owned(self, gi: int) -> list[tuple[int, int, int]]:
        """(first element, end, offset in the moment buffers) of every owned piece of group gi."""
        glo, ghi = self.flat.group_ranges[gi]
        return [(max(glo, lo), min(ghi, hi), off + max(glo, lo) - lo) for lo, hi, off in self.ranges if min(ghi, hi) > max(glo, lo)]

    def pieces(self, s: Segment) -> list[tuple[int, int, int]]:
        """(first element, end, offset in the moment buffers) of the owned pieces of one tensor."""
        return [(max(s.offset, lo), min(s.offset + s.numel, hi), off + max(s.offset, lo) - lo) for lo, hi, off in self.ranges
                if min(s.offset + s.numel, hi) > max(s.offset, lo)]

    @torch.no_grad()
    def step(self, lr: float, grad_scale: torch.Tensor | float = 1.0, kinds=("adamw",)) -> None:
        """One update at learning rate lr (times each group's lr_scale). grad_scale multiplies the gradient first
        (the clip coefficient; a 0-dim device tensor avoids a host sync)."""
        self.steps += 1
        b1, b2 = self.betas
        c1, c2 = 1.0 - b1 ** self.steps, 1.0 - b2 ** self.steps
        for gi, g in enumerate(self.param_groups):
            g["lr"] = lr * g["lr_scale"]
            if g["kind"] not in kinds:
                continue
            for a, b, off in self.owned(gi):
                p, gr = self.flat.params[a:b], self.flat.grads[a:b]
                m, v = self.exp_avg[off:off + b - a], self.exp_avg_sq[off:off + b - a]
                lp = None if self.flat.lp is None else self.flat.lp[a:b]
                if p.is_cuda:
                    from ..ops import native

                    native.adamw_(p, gr, m, v, lp, g["lr"], b1, b2, self.eps, g["weight_decay"], c1, c2, grad_scale)
                    continue
                gs = gr * grad_scale
                p.mul_(1.0 - g["lr"] * g["weight_decay"])
                m.lerp_(gs, 1.0 - b1)
                v.mul_(b2).addcmul_(gs, gs, value=1.0 - b2)
                p.addcdiv_(m, (v / c2).sqrt_().add_(self.eps), value=-g["lr"] / c1)
                if lp is not None:
                    lp.copy_(p)

    # ---- torch.optim-shaped state for checkpoints (reference: ced/train/trainer.py:3602-3627 saves optimizer.state_dict())
    # Parameters are numbered as torch.optim.AdamW built over the same groups numbers them, and each group carries
    # torch's own keys, so the file loads into a torch.optim.AdamW (the reference's optimizer) and the other way round.
    TORCH_GROUP_KEYS = {"amsgrad": False, "maximize": False, "foreach": None, "capturable": False, "differentiable": False, "fused": None,
                        "decoupled_weight_decay": True}

    def state_dict(self) -> dict:
        state, index, names = {}, 0, []
        packed_groups = []
        for gi, g in enumerate(self.param_groups):
            ids = []
            for name in self.torch_order[gi]:
                s = self.flat.by_name[name]
                own = self.pieces(s)
                if g["kind"] == "adamw" and self.steps > 0 and len(own) == 1 and own[0][1] - own[0][0] == s.numel:      # wholly this rank's
                    a = own[0][2]
                    state[index] = {"step": torch.tensor(float(self.steps)),
                                    "exp_avg": self.exp_avg[a:a + s.numel].view(s.shape).clone(),
                                    "exp_avg_sq": self.exp_avg_sq[a:a + s.numel].view(s.shape).clone()}
                ids.append(index)
                names.append(name)
                index += 1
            packed_groups.append({**self.TORCH_GROUP_KEYS, **g, "betas": self.betas, "eps": self.eps, "params": ids})
        return {"state": state, "param_groups": packed_groups, "names": names}

    def load_state_dict(self, sd: dict) -> None:
        names = sd.get("names") or [n for group in self.torch_order for n in group]       # a torch.optim file: numbered in torch's order
        self.reset_moments()
        for index, name in enumerate(names):
            st = sd["state"].get(index)
            s = self.flat.by_name.get(name)
            if st is None or s is None:
                continue
            for a, b, off in self.pieces(s):      # by name, so a state written at another world size or layout loads
                self.exp_avg[off:off + b - a].copy_(st["exp_avg"].reshape(-1)[a - s.offset:b - s.offset])
                self.exp_avg_sq[off:off + b - a].copy_(st["exp_avg_sq"].reshape(-1)[a - s.offset:b - s.offset])
            self.steps = int(st["step"])

    def reset_moments(self) -> None:
        self.exp_avg.zero_()
        self.exp_avg_sq.zero_()
        self.steps = 0


def grad_norm(flat: FlatBuffers, lo: int = 0, hi: int | None = None) -> torch.Tensor:
    g = flat.grads[lo:hi if hi is not None else flat.size]
    if g.is_cuda:
        from ..ops import native

        return native.sumsq(g).sqrt()
    return g.double().pow(2).sum().sqrt().float()


def build_optimizer(model, cfg_optim, device, lp_dtype=None, shard=None, trainable=None):
    """(flat buffers, optimizer) for `optim.name` 'adamw' or 'muon' (reference: ced/train/optim.py:927-979)."""
    groups = param_groups(model, cfg_optim, trainable)
    flat = FlatBuffers(model, groups, device, lp_dtype)
    if cfg_optim.name == "muon":
        from .muon import MuonWithAdamW

        return flat, MuonWithAdamW(flat, groups, cfg_optim, shard)
    return flat, FlatAdamW(flat, groups, cfg_optim.betas, cfg_optim.eps, shard)
