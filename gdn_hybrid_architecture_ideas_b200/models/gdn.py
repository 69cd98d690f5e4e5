"""Gated DeltaNet mixer.

in_proj_qkv -> causal document-masked conv (K taps) -> SiLU -> split q,k,v -> L2-normalise q,k (q scaled dk^-0.5);
beta = sigmoid(in_proj_b x); g = -exp(A_log) softplus(in_proj_a x + dt_bias); gated delta rule; out_proj of the gated
RMSNorm of the readout with z = in_proj_z x. Value head j reads key head j // (Hv/Hk)
(reference: ced/model/gdn.py:261-375, 599-849).

The write/query depth mixes ("arms", reference: ced/model/gdn_arms.py:809-928) change which input each row range of
the projections reads: with x_w = x + lambda (m' - x) and x_q = x + lambda_q (m'_q - x), variant "qmix" projects the
q rows from x_q and the k, v, decay and beta rows from x_w. `project` below holds that routing for every variant.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import ops
from ..config import GDNConfig
from . import gdn_dprod, gdn_dprod_derived, gdn_dprod_sparse, gdn_erase, gdn_kda
from .linear import Linear
from .norms import GatedRMSNorm
from .sequence import SeqContext

READ_MIX_VARIANTS = ("qmix", "kqmix")


@dataclass
class GDNState:
    conv_input: torch.Tensor   # (B, K-1, C) last pre-conv inputs
    conv_doc: torch.Tensor     # (B, K-1) their document ids (-1: none)
    S: torch.Tensor | None     # (B, Hv, dk, dv)
    ckpt: torch.Tensor | None = None    # a cross-read writer only: the checkpoint the next token reads (B, Hv, dk, dv)
    ccr: object | None = None           # the record a writer's call hands its readers; taken out by the stack, never cached
    k_prev: torch.Tensor | None = None  # gdn.dprod.key 'prev' only: the unit key of the last token processed (B, Hk, dk)
    pass1: object | None = None         # the record a read-only second pass reads (models/second_pass.py); taken out by the model, never cached
    acc: torch.Tensor | None = None     # gdn.dprod.summary only: the sums (B, F) and the count (B,) of the group of tokens still open
    cnt: torch.Tensor | None = None


class GDNArms(nn.Module):
    """What one GDN layer holds of the write / query mixes and of the checkpoint cross-read: the write mix's lambda and,
    from the second block on, its depth query over the finished blocks; for qmix / kqmix the same for the query mix; for
    a cross-read reader its gate (H_v,) and, with a translator, D = M - I (H_k, d_k, d_k). Lambdas, queries and D are zeros
    at the start and the gates start at `gate_init` (0 unless asked), so the layer starts as the plain layer.

    ccr: None, or a dict(read, write, spacing, layer, source, target, translator, gate_init, gate_floor, hk, hv, dk) of
    plain attributes (models/ccr.py); write_mix "none": a layer that only takes part in the cross-read."""

    def __init__(self, d: int, eps: float, has_query: bool, variant: str, write_mix: str = "layer", ccr: dict | None = None):
        super().__init__()
        from .depth_mix import DepthQuery

        self.write_mix = write_mix
        self.variant = variant if write_mix != "none" else "none"
        self.write_query = DepthQuery(d, eps) if has_query and write_mix != "none" else None
        if write_mix != "none":       # "layer": one scalar; "head": one a key head, then one a value head
            self.write_lambda = nn.Parameter(torch.zeros(1 if write_mix == "layer" else (ccr or {}).get("heads", 1)))
        if self.variant in READ_MIX_VARIANTS:
            self.qmix_lambda = nn.Parameter(torch.zeros(1))
            self.qmix_query = DepthQuery(d, eps) if has_query else None
        c = ccr or {}
        self.ccr_read, self.ccr_write, self.spacing = bool(c.get("read")), bool(c.get("write")), int(c.get("spacing", 0))
        self.layer, self.ccr_source, self.ccr_target = c.get("layer"), c.get("source"), c.get("target", "previous")
        self.translator = c.get("translator", "none") if self.ccr_read else "none"
        self.gate_floor = float(c.get("gate_floor", 0.0)) if self.ccr_read else 0.0
        if self.ccr_read:
            init = float(c.get("gate_init", 0.0))
            self.ccr_gate = nn.Parameter(torch.zeros(c["hv"]) if init == 0 else torch.full((c["hv"],), init))
            if self.translator == "key_head":
                self.ccr_translator_delta = nn.Parameter(torch.zeros(c["hk"], c["dk"], c["dk"]))
        self.qmix_static = False        # True once qmix_keep holds a choice (models/qmix_select.py)
        self.n_sources = 0

    def register_qmix_keep(self, n_sources: int) -> None:
        """Under model.encoder.gdn_qmix_select_step, for a layer whose query mix reads more than two sources: the persistent
        buffer qmix_keep ((2,) int64, -1 = not chosen) and a post-load hook that sets `qmix_static` from it, so every loader
        of a state dict reads the form the weights were trained in (reference: ced/model/gdn_arms.py:616-641)."""
        from .qmix_select import KEEP

        self.n_sources = n_sources
        if n_sources <= KEEP or getattr(self, "qmix_query", None) is None:
            return
        self.register_buffer("qmix_keep", torch.full((KEEP,), -1, dtype=torch.long))
        self.register_load_state_dict_post_hook(_sync_qmix_static)

    def chosen_sources(self) -> list | None:
        """The chosen pair (ascending) or None before the choice; one host read."""
        keep = getattr(self, "qmix_keep", None)
        if keep is None or int(keep[0]) < 0:
            return None
        return [int(i) for i in keep.detach().cpu().tolist()]

    def read_mix(self, sources: list) -> torch.Tensor:
        """The query mix over `sources`: the softmax over all of them, or over the chosen pair once there is one."""
        if self.qmix_static:
            from .qmix_select import depth_mix_pair

            return depth_mix_pair(sources, self.qmix_query, self.qmix_keep)
        return self.qmix_query(sources)


def _sync_qmix_static(module: "GDNArms", incompatible_keys) -> None:
    chosen = module.chosen_sources()
    if chosen is not None and not 0 <= chosen[0] < chosen[1] < module.n_sources:
        raise ValueError(f"qmix_keep {chosen} is not 2 ascending sources of the layer's {module.n_sources}")
    module.qmix_static = chosen is not None


class GatedDeltaNet(nn.Module):
    def __init__(self, d_model: int, cfg: GDNConfig, norm_eps: float, norm_gain: str = "channel", dprod_carry: tuple | None = None):
        super().__init__()
        if cfg.n_v_heads % cfg.n_k_heads:
            raise ValueError("gdn.n_v_heads must be a multiple of gdn.n_k_heads")
        # Write strength range: beta = beta_max * sigmoid(b). With 2 the transition's eigenvalue along k spans
        # (-alpha, alpha) (negative eigenvalues; reference: ced/model/gdn_negeig.py:37-61). The kernels use beta as a
        # multiplier only, so nothing else changes.
        m = cfg.negeig.beta_max
        if isinstance(m, bool) or m not in (1, 2):
            raise ValueError(f"gdn.negeig.beta_max {m!r}: 1 (beta = sigmoid(b)) or 2 (beta = 2 sigmoid(b))")
        self.beta_max = m
        self.cfg = cfg
        hk, hv, dk, dv = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim
        self.conv_channels = 2 * hk * dk + hv * dv
        self.in_proj_qkv = Linear(d_model, self.conv_channels)
        self.in_proj_z = Linear(d_model, hv * dv)
        self.in_proj_b = Linear(d_model, hv)
        # Per-channel decay (gdn.kda.decay 'channel'): the gate's tensors stand where in_proj_a and the per-head dt_bias
        # were; None for the scalar decay, and then nothing is built and no random number drawn.
        gdn_kda.check_config(cfg)
        self.kda = gdn_kda.KDAGate(d_model, cfg) if gdn_kda.is_on(cfg) else None
        if self.kda is None:
            self.in_proj_a = Linear(d_model, hv)
        self.conv_weight = nn.Parameter(torch.empty(self.conv_channels, cfg.conv_kernel))
        self.A_log = nn.Parameter(torch.empty(hv))
        if self.kda is None:
            self.dt_bias = nn.Parameter(torch.empty(hv))
        self.norm = GatedRMSNorm(dv, norm_eps, gate=cfg.output_gate, gain=norm_gain)
        self.out_proj = Linear(hv * dv, d_model)
        self.reset_gate_parameters(cfg.init)
        bound = 1.0 / math.sqrt(cfg.conv_kernel)
        nn.init.uniform_(self.conv_weight, -bound, bound)
        self.write_mix = "none"
        self.keep_record = False        # set for one forward by a model with a second pass: the layer also leaves what that pass reads
        self.arms_attached = False      # set by the encoder on a layer that holds GDNArms (a write mix, a cross-read, or both)
        # The erase direction (gdn.erase.mode 'eda'): its tensors come last and draw nothing from the global stream.
        gdn_erase.check_config(cfg)
        self.erase = gdn_erase.EraseGate(d_model, cfg) if gdn_erase.is_on(cfg) else None
        # Gated DeltaProduct (gdn.dprod.n_h >= 2): the extra steps' tensors, from a stream of their own as well.
        gdn_dprod.check_config(cfg)
        self.dprod = gdn_dprod.build_steps(d_model, cfg, dprod_carry)

    @torch.no_grad()
    def reset_gate_parameters(self, scheme: str) -> None:
        """"fla": A ~ U(0,16), dt ~ logU(1e-3, 1e-1) clamped at 1e-4, dt_bias = softplus^-1(dt);
        "hf": A ~ U(0.01, 16), dt_bias = 1 (reference: ced/model/gdn.py:375-399)."""
        hv = self.cfg.n_v_heads
        if scheme == "fla":
            A = torch.empty(hv).uniform_(0, 16)
            dt = torch.exp(torch.rand(hv) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3)).clamp(min=1e-4)
            bias = dt + torch.log(-torch.expm1(-dt))
        elif scheme == "hf":
            A = torch.empty(hv).uniform_(0.01, 16)
            bias = torch.ones(hv)
        else:
            raise ValueError(f"unknown GDN init scheme {scheme!r}")
        self.A_log.copy_(torch.log(A))
        if self.kda is None:
            self.dt_bias.copy_(bias)
        else:
            self.kda.reset_dt_bias(scheme)

    # ------------------------------------------------------------------ projections

    def project(self, x, arms: GDNArms | None, x_write, x_read):
        """(u_pre, a_lin, b_lin): the pre-conv in-projection and the decay / beta pre-activations, each row range
        reading the input its variant assigns."""
        hk, dk = self.cfg.n_k_heads, self.cfg.k_head_dim
        nq, C = hk * dk, self.conv_channels
        if arms is None or arms.write_mix == "none":
            return self.in_proj_qkv(x), self.in_proj_a(x), self.in_proj_b(x)
        if arms.write_mix == "head":
            # One lambda per head: entry i < H_k the k channels of key head i, entry H_k + j the v channels, the write strength
            # and the decay of value head j. By linearity P(x_w^h) = P(x) + lambda_h P(m' - x): one more projection of the k, v,
            # a and b rows on the difference (reference: ced/model/gdn_arms.py:919-928).
            hv, dv = self.cfg.n_v_heads, self.cfg.v_head_dim
            lam = arms.write_lambda
            d = (x_write - x).to(x.dtype)
            u = self.in_proj_qkv(x)
            lam_kv = torch.cat([lam[:hk].repeat_interleave(dk), lam[hk:].repeat_interleave(dv)]).to(u.dtype)
            kv = u[..., nq:] + torch.nn.functional.linear(d, self.in_proj_qkv.weight[nq:].to(d.dtype)) * lam_kv
            lam_v = lam[hk:]
            a0, b0 = self.in_proj_a(x), self.in_proj_b(x)
            a = a0 + self.in_proj_a(d) * lam_v.to(a0.dtype)
            b = b0 + self.in_proj_b(d) * lam_v.to(b0.dtype)
            return torch.cat([u[..., :nq], kv.to(u.dtype)], dim=-1), a.to(a0.dtype), b.to(b0.dtype)
        v = arms.variant
        W = self.in_proj_qkv
        reads = v in READ_MIX_VARIANTS
        xw, xr = ops.input_mixes(x, x_write, arms.write_lambda, x_read if reads else None, arms.qmix_lambda if reads else None)
        # (rows [0, split) read `first`, rows [split, C) read `second`)
        if v == "none":
            u = ops.split_linear(x, xw, W, nq)
        elif v == "qmix":
            u = ops.split_linear(xr, xw, W, nq)
        elif v == "kqmix":
            u = ops.split_linear(xr, xw, W, 2 * nq)
        elif v == "korig":
            u = ops.split_linear(x, xw, W, 2 * nq)
        elif v == "vonly":
            return ops.split_linear(x, xw, W, 2 * nq), self.in_proj_a(x), self.in_proj_b(x)
        elif v == "qshare":
            u = W(xw)
        elif v == "qshare_kv":
            return W(xw), self.in_proj_a(x), self.in_proj_b(x)
        elif v == "qshare_bd":
            u = ops.split_linear(xw, x, W, nq)
        else:
            raise ValueError(f"gdn_write_variant {v!r}")
        return u, self.in_proj_a(xw), self.in_proj_b(xw)

    # ------------------------------------------------------------------ forward

    def forward(self, x: torch.Tensor, ctx: SeqContext, state: GDNState | None = None, arms: GDNArms | None = None,
                x_write: torch.Tensor | None = None, x_read: torch.Tensor | None = None, need_state: bool = True, ccr=None):
        """x (B, L, d) normed layer input. Returns (y, GDNState). state: the cache of earlier chunks (None: the row
        starts here). need_state False (training) lets the kernel skip the final state. ccr: the record of the layer
        this one cross-reads (models/ccr.py), for a reader only."""
        if (arms is None) == self.arms_attached:
            raise ValueError("a GDN layer with write/query mixes or the cross-read is called with its arms (through its encoder layer)")
        if self.kda is not None or self.erase is not None or self.dprod is not None:
            return self.forward_kda(x, ctx, state, arms)
        if arms is not None and (arms.ccr_read or arms.ccr_write):
            return self.forward_ccr(x, ctx, state, arms, x_write, x_read, ccr)
        if self.keep_record:
            from .second_pass import gdn_forward_keep

            y, new_state, new_state.pass1 = gdn_forward_keep(self, x, ctx, state)
            return y, new_state
        B, L = ctx.doc.shape       # the input may be a token shard (tensor parallel); projections return all tokens
        cfg = self.cfg
        hk, hv, dk, dv = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim
        u_pre, a_lin, b_lin = self.project(x, arms, x_write, x_read)
        hist, hist_doc = (None, None) if state is None else (state.conv_input, state.conv_doc)
        qkv, conv_input, conv_doc = ops.gdn_prep(u_pre, ctx.doc, self.conv_weight, hk, hv, dk, dv, hist, hist_doc,
                                                 single_doc=ctx.single_doc, packed=True)
        g, beta = ops.gdn_gates(a_lin, b_lin, self.A_log, self.dt_bias, ctx.gdn_scale, ctx.gdn_beta_power)
        if self.beta_max != 1:
            if ctx.gdn_scale != 1 and ctx.gdn_beta_power:
                raise ValueError("gdn.negeig.beta_max 2 with the bag write-strength power (tst.gdn_resolution_gates 'decay_beta'): "
                                 "1 - (1 - beta)^s is written for beta in (0, 1)")
            beta = beta * self.beta_max
        S0 = None if state is None else state.S
        kernel = "recurrence" if cfg.kernel == "recurrence" else "chunked"
        o, S = ops.delta_rule_packed(qkv, hk, hv, dk, dv, g, beta, ctx.is_doc_start, S0, kernel=kernel,
                                     chunk_size=cfg.chunk_size, need_state=need_state, inplace_state=bool(ctx.memo.get("inplace_state")))
        z = self.in_proj_z(x).view(B, L, hv, dv)
        y = self.out_proj(self.norm(o, z).flatten(2))
        return y, GDNState(conv_input=conv_input, conv_doc=conv_doc, S=S)

    def forward_ccr(self, x, ctx: SeqContext, state: GDNState | None, arms, x_write, x_read, rec):
        """The layer under the checkpoint cross-read (models/ccr.py): the scalar layer's input preparation, gates and
        output norm; a writer's delta rule also takes the states its readers' checkpoints name, a reader adds
        gate (*) ckpt^T q to the rule's output before the gated norm (reference: ced/model/gdn.py:715-823)."""
        from . import ccr as ccr_mod

        if (rec is not None) != arms.ccr_read:
            raise ValueError("a cross-read reader takes its source's record, and only a reader does")
        if ctx.gdn_scale != 1:
            raise ValueError("model.encoder.gdn_ccr_spacing is not built with TST's resolution-explicit gates (a bag phase)")
        cfg = self.cfg
        B, L = ctx.doc.shape
        hk, hv, dk, dv = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim
        u_pre, a_lin, b_lin = self.project(x, arms, x_write, x_read)
        hist, hist_doc = (None, None) if state is None else (state.conv_input, state.conv_doc)
        q, k, v, conv_input, conv_doc = ops.gdn_prep(u_pre, ctx.doc, self.conv_weight, hk, hv, dk, dv, hist, hist_doc, single_doc=ctx.single_doc)
        g, beta = ops.gdn_gates(a_lin, b_lin, self.A_log, self.dt_bias)
        if self.beta_max != 1:
            beta = beta * self.beta_max
        cross = ccr_mod.read(arms, rec, q, hv) if rec is not None else None
        kernel = "recurrence" if cfg.kernel == "recurrence" else "chunked"
        ckpt = out = None
        if arms.ccr_write:
            if state is not None and state.ckpt is None:
                raise ValueError("this cache was written without the cross-read's checkpoints")
            rep = hv // hk
            S0 = x.new_zeros(B, hv, dk, dv, dtype=g.dtype) if state is None else state.S
            o, S, out, ckpt = ccr_mod.write(q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2), v, g, beta, ctx, S0,
                                            None if state is None else state.ckpt, arms.spacing, kernel, cfg.chunk_size, arms.layer)
        else:
            o, S = ops.delta_rule(q, k, v, g, beta, ctx.is_doc_start, None if state is None else state.S, kernel=kernel, chunk_size=cfg.chunk_size)
        if cross is not None:
            o = (o + arms.ccr_gate[:, None] * cross).to(o.dtype)
        z = self.in_proj_z(x).view(B, L, hv, dv)
        y = self.out_proj(self.norm(o.to(x.dtype), z).flatten(2))
        return y, GDNState(conv_input=conv_input, conv_doc=conv_doc, S=S, ckpt=ckpt, ccr=out)

    def forward_kda(self, x, ctx: SeqContext, state: GDNState | None, arms):
        """The layer with one decay per key channel and / or the erase direction: the scalar layer's input preparation
        and output norm around the tensor-op rules (reference: ced/model/gdn_kda.py:481-549,
        ced/model/gdn_erase.py:428-506)."""
        if arms is not None or ctx.gdn_scale != 1:
            raise ValueError("gdn.kda.decay 'channel' / gdn.erase.mode 'eda' / gdn.dprod.n_h >= 2 are not built with the GDN write / query mixes "
                             "(model.encoder.gdn_write_mix) nor with TST's resolution-explicit gates (a bag phase)")
        cfg = self.cfg
        B, L = ctx.doc.shape
        hk, hv, dk, dv = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim
        if isinstance(self.dprod, gdn_dprod_sparse.SparseSteps):
            o, conv_input, conv_doc, S, acc, cnt = gdn_dprod_sparse.forward(self, x, ctx, state)
            z = self.in_proj_z(x).view(B, L, hv, dv)
            y = self.out_proj(self.norm(o.to(x.dtype), z).flatten(2))
            return y, GDNState(conv_input=conv_input, conv_doc=conv_doc, S=S, acc=acc, cnt=cnt)
        if isinstance(self.dprod, gdn_dprod_derived.DerivedSteps):
            o, conv_input, conv_doc, S, k_prev = gdn_dprod_derived.forward(self, x, ctx, state)
            z = self.in_proj_z(x).view(B, L, hv, dv)
            y = self.out_proj(self.norm(o.to(x.dtype), z).flatten(2))
            return y, GDNState(conv_input=conv_input, conv_doc=conv_doc, S=S, k_prev=k_prev)
        if self.dprod is not None:
            o, conv_input, conv_doc, S = gdn_dprod.forward(self, x, ctx, state)
            z = self.in_proj_z(x).view(B, L, hv, dv)
            y = self.out_proj(self.norm(o.to(x.dtype), z).flatten(2))
            return y, GDNState(conv_input=conv_input, conv_doc=conv_doc, S=S)
        hist, hist_doc = (None, None) if state is None else (state.conv_input, state.conv_doc)
        q, k, v, conv_input, conv_doc = ops.gdn_prep(self.in_proj_qkv(x), ctx.doc, self.conv_weight, hk, hv, dk, dv, hist, hist_doc,
                                                     single_doc=ctx.single_doc)
        if self.kda is not None:
            g, beta = gdn_kda.gates(self, x)
        else:
            g, beta = ops.ref.gdn_gates(self.in_proj_a(x), self.in_proj_b(x), self.A_log, self.dt_bias)
        rep = hv // hk
        q, k = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
        S0 = x.new_zeros(B, hv, dk, dv, dtype=g.dtype) if state is None else state.S
        if self.erase is not None:
            e = self.erase.direction(x).repeat_interleave(rep, dim=2)
            o, S = gdn_erase.rule(q, k, v, g, beta, e, self.erase.strength(x), ctx.is_doc_start, S0, cfg.kernel, cfg.chunk_size)
        elif cfg.kernel != "recurrence" and L > 1:
            o, S = ops.ref.kda_chunked(q, k, v, g, beta, ctx.is_doc_start, S0, cfg.chunk_size)
        else:
            o, S = ops.ref.kda_recurrence(q, k, v, g, beta, ctx.is_doc_start, S0)
        z = self.in_proj_z(x).view(B, L, hv, dv)
        y = self.out_proj(self.norm(o.to(x.dtype), z).flatten(2))
        return y, GDNState(conv_input=conv_input, conv_doc=conv_doc, S=S)
