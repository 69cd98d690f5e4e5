"""Encoder layer (Peri-LN) and the layer stack with block-entry depth mixing and the GDN write/query mixes.

Layer: y = x + s * out_norm(mixer(in_norm(x))); y = y + s * mlp_out_norm(mlp(mlp_in_norm(y))), s a fixed float from
the config (reference: ced/model/encoder.py:193-318). Layer i is attention iff (i + 1) % full_attn_interval == 0.

Block walk ("block_entry"): sources = [b_0 = embedding output]; block n starts from start_n = mix(sources) (block 1
from b_0 itself), runs its layers, and appends b_n = x_end - start_n; the stack returns mix(sources) with the last
layer's `out` reader. A GDN layer with arms additionally forms m' = in_norm(mix_w(sources)) and (qmix) m'_q over the
same sources (reference: ced/model/attn_res.py:700-797, ced/model/gdn_arms.py:766-777).
"""

from __future__ import annotations

import hashlib
import math

import torch
import torch.nn as nn

from .. import ops
from ..config import ModelConfig
from . import act_checkpoint
from . import ccr as ccr_mod
from .attention import GatedAttention
from .depth_mix import DepthQuery, EntryLayer, LayerQueries, reader_factory
from .gdn import READ_MIX_VARIANTS, GatedDeltaNet, GDNArms
from .mlp import dense_ffn
from .norms import RMSNorm, round_stream
from .qmix_select import check_config as check_qmix_select, record_query_weights
from .sequence import SeqContext


def residual_scale(cfg: ModelConfig) -> float:
    """Fixed residual-branch multiplier of the encoder (reference: ced/model/scaling.py:16-45)."""
    rs = cfg.residual_scale
    if rs.mode in ("none", "inverse_loops"):
        return 1.0
    if rs.mode in ("completep_effective_depth", "loop_factored"):
        return rs.lam * rs.depth_base / cfg.encoder.n_layers
    raise ValueError(f"unknown residual scale mode {rs.mode!r}")


LAYER_SCALARS = ("none", "skip_x0", "skip_x0_span", "x0", "skip")
SPAN_CLAMP = 3.0


def layer_scalar_parameters(mode: str) -> tuple[str, ...]:
    """Names of the (n_layers,) tensors a residual-scalar form stores on the encoder, in state-dict order."""
    if mode not in LAYER_SCALARS:
        raise ValueError(f"model.encoder.layer_scalars {mode!r}: one of {LAYER_SCALARS}")
    return {"none": (), "x0": ("x0_gain",), "skip": ("skip_gain",)}.get(mode, ("skip_gain", "x0_gain"))


def layer_scalar_terms(mode: str, skip_gain, x0_gain, span: float = 4.0):
    """(a - 1, b) of every layer, each (n_layers,) or None, for x <- a x + b x0 + f(x).

    "skip_x0": the stored tensors. "skip": a - 1 stored, b = 0 (None). "x0": a = 1 (None), b stored with b_0 = 0.
    "skip_x0_span": the stored u gives S_k = (ln(span) / 2) tanh(clamp(u_k, +-3)) (gradient passed straight through the
    clamp), a_i = exp(S_{i+1} - S_i) with S_0 = 0, so every product of consecutive a stays inside (1 / span, span);
    b as in "x0" (reference: ced/model/encoder.py:60-100)."""
    if mode == "skip_x0":
        return skip_gain, x0_gain
    if mode == "skip":
        return skip_gain, None
    b = torch.cat([x0_gain.new_zeros(1), x0_gain[1:]])
    if mode == "x0":
        return None, b
    u = skip_gain.detach().clamp(-SPAN_CLAMP, SPAN_CLAMP) + (skip_gain - skip_gain.detach())
    cum = (0.5 * math.log(span)) * torch.tanh(u)
    return torch.expm1(cum - torch.cat([cum.new_zeros(1), cum[:-1]])), b


def apply_layer_scalars(out, x, x0, a_minus_1, b):
    """out + (a - 1) x + b x0 in at least float32, returned in out's dtype (reference: ced/model/encoder.py:103-140)."""
    dtype = torch.promote_types(out.dtype, torch.float32)
    extra = None
    if a_minus_1 is not None:
        extra = x.to(dtype) * a_minus_1.to(dtype)
    if b is not None:
        inj = x0.to(dtype) * b.to(dtype)
        extra = inj if extra is None else extra + inj
    return out if extra is None else (out.to(dtype) + extra).to(out.dtype)


class CanonLayer(nn.Module):
    """h' = h + causal depthwise convolution (kernel K) of h inside each document, on the normed input of a global
    attention layer; taps zeros as built, so the layer starts as the identity. conv_weight (d, K), [:, K-1] on the current
    input, the layout of the GDN short convolution (reference: ced/model/canon.py:118-152)."""

    def __init__(self, d_model: int, kernel: int):
        super().__init__()
        self.kernel = kernel
        self.conv_weight = nn.Parameter(torch.zeros(d_model, kernel))

    @torch.no_grad()
    def init_uniform(self, generator: torch.Generator) -> None:
        bound = 1.0 / math.sqrt(self.kernel)
        drawn = torch.empty(tuple(self.conv_weight.shape), dtype=torch.float32).uniform_(-bound, bound, generator=generator)
        if not self.conv_weight.is_meta:
            self.conv_weight.copy_(drawn)

    def forward(self, h, doc, hist=None, hist_doc=None):
        out, hist, hist_doc = ops.ref.causal_doc_conv(h, doc, self.conv_weight, hist, hist_doc)
        return (h + out).to(h.dtype), hist, hist_doc


def canon_generator(seed: int, layer: int) -> torch.Generator:
    """CPU generator of one Canon layer's uniform start, a function of (run seed, layer index) only
    (reference: ced/model/canon.py:92-98)."""
    digest = hashlib.blake2b(f"canon-taps:{seed}:{layer}".encode(), digest_size=8).digest()
    return torch.Generator(device="cpu").manual_seed(int.from_bytes(digest, "little") & (2 ** 63 - 1))


class EncoderLayer(nn.Module):
    def __init__(self, kind: str, cfg: ModelConfig, scale: float, attention=None, gdn=None):
        super().__init__()
        d, eps, gain = cfg.d_model, cfg.norm_eps, cfg.encoder.block_norm_gain
        self.kind = kind
        self.residual_scale = scale
        self.stream_bf16 = cfg.encoder.residual_dtype == "bf16"
        self.mixer_in_norm = RMSNorm(d, eps, gain=gain)
        self.mixer_out_norm = RMSNorm(d, eps, gain=gain)
        self.mlp_in_norm = RMSNorm(d, eps, gain=gain)
        self.mlp_out_norm = RMSNorm(d, eps, gain=gain)
        if kind == "gdn":
            gdn_cfg, carry = gdn if isinstance(gdn, tuple) else (gdn or cfg.encoder.gdn, None)
            self.mixer = GatedDeltaNet(d, gdn_cfg, eps, norm_gain=gain, dprod_carry=carry)
        elif kind == "attention":
            self.mixer = GatedAttention(d, attention or cfg.encoder.attention, eps)
        else:
            raise ValueError(kind)
        self.mlp = dense_ffn(d, cfg.ffn_hidden, cfg.ffn_activation)
        self.canon = CanonLayer(d, cfg.encoder.canon_kernel) if kind == "attention" and cfg.encoder.canon_kernel else None

    def forward(self, x: torch.Tensor, ctx: SeqContext, cache=None, sources: list | None = None, need_state: bool = True,
                scalars: tuple | None = None, premixed: tuple | None = None, ccr=None):
        """scalars: (x0, a - 1, b) of this layer's residual scalars, applied as the last term of the layer's own sum.
        premixed: (write mix, query mix) of this layer over `sources`, already formed by the stack (one kernel for all the
        readers of a block); an entry that is None is formed here. ccr: the record of the GDN layer this one
        cross-reads (models/ccr.py); a writer leaves its own in the new cache entry's `ccr`."""
        x_in = x
        h, x = ops.prenorm(x, self.mixer_in_norm.weight, self.mixer_in_norm.eps)      # x: the stream, now read by the residual add only
        if self.canon is not None:
            if cache is not None and cache.canon_input is None:
                raise ValueError("this cache was written without a Canon layer: it cannot be continued with one")
            h, canon_input, canon_doc = self.canon(h, ctx.doc, None if cache is None else cache.canon_input,
                                                   None if cache is None else cache.canon_doc)
        arms: GDNArms | None = getattr(self, "gdn_arms", None)
        if arms is not None and arms.write_mix == "none":       # the cross-read alone
            mixed, new_cache = self.mixer(h, ctx, cache, arms=arms, need_state=need_state, ccr=ccr)
        elif arms is not None:
            if sources is None:
                raise ValueError("a GDN layer with write/query mixes is called with the finished blocks (sources)")
            pre_w, pre_q = premixed if premixed is not None else (None, None)
            if pre_w is None:
                pre_w = arms.write_query(sources) if arms.write_query is not None else sources[0]
            x_write = self.mixer_in_norm(pre_w)
            x_read = None
            if arms.variant in READ_MIX_VARIANTS:
                x_read = x_write if arms.qmix_query is None else self.mixer_in_norm(pre_q if pre_q is not None else arms.read_mix(sources))
            mixed, new_cache = self.mixer(h, ctx, cache, arms=arms, x_write=x_write, x_read=x_read, need_state=need_state, ccr=ccr)
        elif self.kind == "gdn":
            mixed, new_cache = self.mixer(h, ctx, cache, need_state=need_state)
        else:
            mixed, new_cache = self.mixer(h, ctx, cache)
        y = ops.norm_add(x, mixed, self.mixer_out_norm.weight, self.mixer_out_norm.eps, self.residual_scale)
        if self.stream_bf16:
            y = round_stream(y)
        h2, y = ops.prenorm(y, self.mlp_in_norm.weight, self.mlp_in_norm.eps)
        y = ops.norm_add(y, self.mlp(h2), self.mlp_out_norm.weight, self.mlp_out_norm.eps, self.residual_scale)
        if self.stream_bf16:
            y = round_stream(y)
        if scalars is not None:
            y = apply_layer_scalars(y, x_in, *scalars)
        if self.canon is not None:
            new_cache.canon_input, new_cache.canon_doc = canon_input, canon_doc
        return y, new_cache


class Encoder(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        enc = cfg.encoder
        self.cfg = cfg
        scale = residual_scale(cfg)
        if enc.gdn_shape_by_layer and enc.gdn_write_mix != "none":
            raise ValueError("model.encoder.gdn_shape_by_layer is not built with model.encoder.gdn_write_mix "
                             "(reference: ced/model/gdn_dprod_place.py:185-203)")
        per_global, per_gdn = iter(enc.global_attention()), iter(enc.gdn_layer_configs())
        self.layers = nn.ModuleList(
            EncoderLayer(kind, cfg, scale, attention=next(per_global) if kind == "attention" else None,
                         gdn=next(per_gdn) if kind == "gdn" else None)
            for kind in enc.layer_kinds())
        self.block = enc.full_attn_interval
        self.block_entry = enc.attn_res == "block_entry"
        check_qmix_select(cfg)
        self.qmix_record: dict | None = None      # set for one forward by the trainer: every query mix's weight sums (models/qmix_select.py)
        self.block_every = enc.attn_res == "block"        # every sublayer reads the blocks
        self.ldm = enc.attn_res == "ldm"                  # linear depth memory: a per-position memory beside the stream
        self.activation_checkpoint = "none"
        self.host_pool = None
        # bucketed data parallelism (parallel/zero.py): an object with forward_enter(block) / backward_done(block), told when
        # the forward is about to read a block's matrices and when the gradient of a block's input is complete
        self.stage_hooks = None
        d, eps, S, n = cfg.d_model, cfg.norm_eps, self.block, enc.n_layers
        H = enc.attn_res_heads
        if type(H) is not int or H < 1 or d % H:
            raise ValueError(f"model.encoder.attn_res_heads {H!r}: a whole number of heads that divides d_model {d}")
        if enc.attn_res_query not in ("static", "token"):
            raise ValueError(f"model.encoder.attn_res_query {enc.attn_res_query!r}: 'static' or 'token'")
        self.token_query = enc.attn_res_query == "token"
        if self.token_query and (not self.block_entry or enc.gdn_write_mix != "none"):
            raise ValueError("model.encoder.attn_res_query 'token' is built for model.encoder.attn_res 'block_entry' (its readers) "
                             "without the GDN write / query mixes")
        if enc.attn_res_query_hidden and not self.token_query:
            raise ValueError("model.encoder.attn_res_query_hidden is read with model.encoder.attn_res_query 'token' only: leave it 0")
        query_hidden = (enc.attn_res_query_hidden or max(1, d // 32)) if self.token_query else 0
        if H != 1 and (not self.block_entry or enc.gdn_write_mix != "none"):
            raise ValueError(f"model.encoder.attn_res_heads {H} is built for model.encoder.attn_res 'block_entry' (its readers) "
                             "without the GDN write / query mixes")
        if self.block_every:
            if S <= 0 or n % S:
                raise ValueError("model.encoder.attn_res 'block' needs n_layers to be a multiple of full_attn_interval")
            if enc.gdn_write_mix != "none":
                raise ValueError("model.encoder.gdn_write_mix reads the finished blocks of attn_res 'block_entry', not 'block'")
            for i, layer in enumerate(self.layers):
                layer.attn_res = LayerQueries(d, eps, first=i % S == 0, has_mixer_query=i > 0, last=i == n - 1)
        if self.ldm:
            from . import ldm

            if enc.gdn_write_mix != "none" or self.token_query or H != 1 or enc.canon_kernel:
                raise ValueError("model.encoder.attn_res 'ldm' is built on the plain stack: no GDN write / query mixes, token queries, "
                                 "reader heads or Canon layers")
            ldm.build(cfg, self.layers)
        if self.block_entry:
            if S <= 0 or n % S:
                raise ValueError("model.encoder.attn_res 'block_entry' needs n_layers to be a multiple of full_attn_interval")
            for i, layer in enumerate(self.layers):
                opens, closes = i > 0 and i % S == 0, i % S == S - 1
                if opens or closes:
                    layer.attn_res = EntryLayer(reader_factory(d, eps, enc.attn_res_heads, query_hidden), bool(query_hidden), opens, closes, i == n - 1)
        if enc.gdn_write_mix not in ("none", "layer", "head"):
            raise ValueError(f"model.encoder.gdn_write_mix {enc.gdn_write_mix!r}: 'none', 'layer' or 'head'")
        if enc.gdn_write_mix == "head" and (enc.gdn_write_variant != "none" or cfg.fp8.mode != "none" or cfg.nvfp4.mode != "none"):
            raise ValueError("model.encoder.gdn_write_mix 'head' (one lambda a head) is built without a write variant and without model.fp8 / model.nvfp4")
        if enc.gdn_write_mix != "none" and not self.block_entry:
            raise ValueError("model.encoder.gdn_write_mix reads the finished blocks of attn_res 'block_entry'")
        ccr_mod.check_config(cfg)
        reads, writes = ccr_mod.sources(cfg), set(ccr_mod.writers(cfg))
        self.ccr = bool(reads)
        for i, layer in enumerate(self.layers):
            if layer.kind != "gdn":
                continue
            write = enc.gdn_write_mix if enc.gdn_write_mix != "none" and i > 0 else "none"
            if write == "none" and i not in reads and i not in writes:
                continue
            g = enc.gdn
            heads = {"heads": g.n_k_heads + g.n_v_heads}
            cross = heads if not self.ccr else dict(heads=heads["heads"], 
                read=i in reads, write=i in writes, spacing=enc.gdn_ccr_spacing, layer=i, source=reads.get(i), target=enc.gdn_ccr_target,
                translator=enc.gdn_ccr_translator, gate_init=enc.gdn_ccr_gate_init, gate_floor=enc.gdn_ccr_gate_floor,
                hk=g.n_k_heads, hv=g.n_v_heads, dk=g.k_head_dim)
            layer.gdn_arms = GDNArms(d, eps, has_query=i // S >= 1 if S > 0 else False, variant=enc.gdn_write_variant, write_mix=write, ccr=cross)
            layer.mixer.write_mix, layer.mixer.arms_attached = write, True
            if enc.gdn_qmix_select_step:
                layer.gdn_arms.register_qmix_keep(i // S + 1)
        # Canon layers: zeros as built; "uniform" draws each layer's taps from its own seeded CPU generator, so no other
        # parameter's start changes (reference: ced/model/canon.py:101-115, ced/model/control.py:1195-1243).
        K = enc.canon_kernel
        if isinstance(K, bool) or not isinstance(K, int) or K < 0 or K == 1:
            raise ValueError(f"model.encoder.canon_kernel {K!r}: 0 (no Canon layer) or an integer >= 2")
        if enc.canon_init not in ("zeros", "uniform") or (not K and enc.canon_init != "zeros"):
            raise ValueError(f"model.encoder.canon_init {enc.canon_init!r} with canon_kernel {K}: 'zeros' or (with a kernel) 'uniform'")
        if K and (self.block <= 0 or enc.layer_scalars != "none" or cfg.nvfp4.mode != "none"):
            raise ValueError("model.encoder.canon_kernel needs a global attention layer and is not built together with "
                             "layer_scalars or nvfp4")
        if K and enc.canon_init == "uniform":
            seed = torch.initial_seed()
            for i, layer in enumerate(self.layers):
                if layer.canon is not None:
                    layer.canon.init_uniform(canon_generator(seed, i))
        # Per-layer residual scalars x <- a x + b x0 + f(x): (n_layers,) zeros after the layers' own tensors.
        self.scalar_form = enc.layer_scalars
        self.scalar_span = float(enc.layer_scalars_span)
        names = layer_scalar_parameters(self.scalar_form)
        if not (math.isfinite(self.scalar_span) and self.scalar_span > 1.0):
            raise ValueError(f"model.encoder.layer_scalars_span {enc.layer_scalars_span!r}: a finite width above 1")
        if names and cfg.nvfp4.mode != "none":
            raise ValueError("model.encoder.layer_scalars is not built together with model.nvfp4")
        if names and (self.block_entry or self.block_every):
            raise ValueError("model.encoder.layer_scalars is not built together with model.encoder.attn_res: both replace "
                             "the layers' residual add (reference: ced/model/attn_res.py:166-168)")
        for name in names:
            setattr(self, name, nn.Parameter(torch.zeros(n)))
        # A looped middle (models/recur.py): the layers first .. end - 1 run T times; what a pass reads is the injection's.
        from . import recur as recur_mod

        recur_mod.check_config(cfg)
        self.recur = tuple(cfg.loop.recur_layers) or None
        self.recur_norm = self.recur_injection = self.recur_mix = self.recur_depth = None
        if self.recur is not None:
            lc = cfg.loop
            self.recur_state_init = lc.recur_state_init
            if lc.injection == "parcae":
                if lc.recur_prelude_norm:
                    self.recur_norm = RMSNorm(d, eps)
                self.recur_injection = recur_mod.RecurInjection(d, lc.parcae_init_decay, lc.recur_inject_b)
            elif lc.injection == "mix":
                self.recur_mix = nn.Parameter(torch.tensor(float(lc.recur_mix_init)))
            elif lc.injection == "depth_mix":
                self.recur_depth = DepthQuery(d, eps)

    def layer_scalar_args(self, x0):
        """Per layer (x0, a - 1, b) as 0-dim tensors, or None without the scalars."""
        if self.scalar_form == "none":
            return None
        a, b = layer_scalar_terms(self.scalar_form, getattr(self, "skip_gain", None), getattr(self, "x0_gain", None), self.scalar_span)
        return [(x0 if b is not None else None, None if a is None else a[i], None if b is None else b[i]) for i in range(len(self.layers))]

    @torch.no_grad()
    def project_layer_scalars(self) -> None:
        """After an optimizer step: the span form's stored u back into [-3, 3] (reference: ced/train/trainer.py:3135)."""
        if self.scalar_form == "skip_x0_span":
            self.skip_gain.clamp_(-SPAN_CLAMP, SPAN_CLAMP)

    def _stage(self, b: int, x: torch.Tensor) -> None:
        """Block b starts at stream x: tell the data-parallel plan (if one listens) now, and again when x's gradient is
        complete — by then every backward node of the block's layers has run, so their matrices' gradients are final."""
        h = self.stage_hooks
        if h is None:
            return
        h.forward_enter(b)
        if torch.is_grad_enabled() and x.requires_grad:
            x.register_hook(lambda g, b=b: h.backward_done(b))

    def _run_walk(self, walk, layer, x, ctx, cache, sources, need_state, scalars=None, premixed=None):
        """`_run` for a stack with the checkpoint cross-read: a layer that takes part is called with the record it reads
        and its own record is taken out of its new cache entry for the layers after it (models/ccr.py `Walk`). Under
        activation_checkpoint "layer" the record is an input and an output of the layer's checkpointed call."""
        arms = getattr(layer, "gdn_arms", None)
        if walk is None or arms is None or not (arms.ccr_read or arms.ccr_write):
            return self._run(layer, x, ctx, cache, sources, need_state, scalars, premixed)
        rec = walk.record_in(arms)
        mode = self.activation_checkpoint
        if mode != "none" and cache is None and torch.is_grad_enabled() and x.requires_grad:
            if mode not in ccr_mod.CHECKPOINT_MODES:
                raise ValueError(f"model.encoder.gdn_ccr_spacing runs with activation_checkpoint {ccr_mod.CHECKPOINT_MODES}, not {mode!r}")

            def call(x_, states, slot, *src):
                r = None if states is None else ccr_mod.Record(states, slot, rec.source)
                y_, c_ = layer(x_, ctx, None, list(src) if src else None, False, None, None, r)
                return y_ if c_.ccr is None else (y_, c_.ccr.states, c_.ccr.slot)
            out = act_checkpoint.run_checkpointed(call, x, None if rec is None else rec.states, None if rec is None else rec.slot, *(sources or ()))
            y, own = (out, None) if isinstance(out, torch.Tensor) else (out[0], ccr_mod.Record(out[1], out[2], arms.layer))
            walk.hand_record(arms, own)
            return y, None
        y, new_cache = layer(x, ctx, cache, sources, need_state, None, premixed, rec)
        return y, walk.hand(arms, new_cache)

    def _run(self, layer, x, ctx, cache, sources, need_state, scalars=None, premixed=None):
        """One layer call under the stack's activation memory mode (models/act_checkpoint.py)."""
        mode = self.activation_checkpoint
        training = cache is None and torch.is_grad_enabled() and x.requires_grad
        if scalars is not None:
            if mode != "none" and training:
                raise ValueError("model.encoder.layer_scalars runs with activation_checkpoint 'none'")
            return layer(x, ctx, cache, sources, need_state, scalars)
        if premixed is not None:
            if mode in ("host", "host_overlap") and training:
                if self.host_pool is None or self.host_pool.device != x.device:
                    self.host_pool = act_checkpoint.HostPool(x.device, overlap=mode == "host_overlap")
                with self.host_pool.offload():
                    return layer(x, ctx, cache, sources, need_state, None, premixed)
            return layer(x, ctx, cache, sources, need_state, None, premixed)
        if mode == "layer" and training and not getattr(layer, "keep_record", False):     # a layer a second pass reads again keeps its outputs
            def call(x_, *src):
                return layer(x_, ctx, None, list(src) if src else None, False)[0]
            return act_checkpoint.run_checkpointed(call, x, *(sources or ())), None
        if mode in ("host", "host_overlap") and training:
            if self.host_pool is None or self.host_pool.device != x.device:
                self.host_pool = act_checkpoint.HostPool(x.device, overlap=mode == "host_overlap")
            with self.host_pool.offload():
                return layer(x, ctx, cache, sources, need_state)
        return layer(x, ctx, cache, sources, need_state)

    def _run_block(self, b, x, ctx, sources):
        """The layers of block b as one recomputed unit ("block" mode)."""
        S = self.block
        layers = [self.layers[i] for i in range(b * S, (b + 1) * S)]

        def call(x_, *src):
            for layer in layers:
                use = list(src) if getattr(layer, "gdn_arms", None) is not None else None
                x_ = layer(x_, ctx, None, use, False)[0]
            return x_
        return act_checkpoint.run_checkpointed(call, x, *sources)

    def _block_mixes(self, b: int, sources: list) -> dict:
        """Every depth mix block b takes over the finished blocks, formed together: the block's entry ("entry") and each GDN
        layer's write ((i, "w")) and query ((i, "q")) mix. They read the same sources with different pseudo-queries, so on
        CUDA one kernel reads each source once for all of them and one backward kernel writes each source's gradient once
        (ops.depth_mix_multi). Empty when there is nothing to share."""
        if len(sources) < 2 or not ops.use_native(sources[0]) or self.token_query:
            return {}
        S = self.block
        keys, readers = [], []
        if b > 0:
            keys.append("entry")
            readers.append(self.layers[b * S].attn_res.entry)
        for i in range(b * S, (b + 1) * S):
            arms = getattr(self.layers[i], "gdn_arms", None)
            if arms is None:
                continue
            if arms.write_query is not None:
                keys.append((i, "w"))
                readers.append(arms.write_query)
            if arms.variant in READ_MIX_VARIANTS and arms.qmix_query is not None and not arms.qmix_static:
                keys.append((i, "q"))
                readers.append(arms.qmix_query)
        if len(readers) < 2 or len(readers) > 8 or any(r.heads > 1 for r in readers):
            return {}
        outs = ops.depth_mix_multi(sources, [(r.query, r.key_norm.weight) for r in readers], readers[0].key_norm.eps)
        return dict(zip(keys, outs))

    def _forward_block_every(self, x, ctx, get, need_state):
        """attn_res "block": each sublayer's input is a depth mix over the finished blocks and the current block's partial
        sum, and a block's sum starts with its first sublayer's output (reference: ced/model/attn_res.py:580-625, 645-660)."""
        if self.activation_checkpoint != "none" and torch.is_grad_enabled() and x.requires_grad:
            raise ValueError("model.encoder.attn_res 'block' runs with activation_checkpoint 'none'")
        done, new_caches = [], []
        for i, layer in enumerate(self.layers):
            res, scale = layer.attn_res, layer.residual_scale
            sources = [*done, x]
            h = x if res.pre_mixer is None else res.pre_mixer(sources)
            if layer.kind == "gdn":
                mixed, c = layer.mixer(layer.mixer_in_norm(h), ctx, get(i), need_state=need_state)
            else:
                mixed, c = layer.mixer(layer.mixer_in_norm(h), ctx, get(i))
            f = scale * layer.mixer_out_norm(mixed, out_dtype=x.dtype)
            if res.first:
                seen, partial = sources, f.to(x.dtype)
            else:
                seen, partial = done, x + f
            h = res.pre_mlp([*seen, partial])
            partial = partial + scale * layer.mlp_out_norm(layer.mlp(layer.mlp_in_norm(h)), out_dtype=x.dtype)
            new_caches.append(c)
            if res.out is not None:
                return res.out([*seen, partial]), new_caches
            if res.first:
                done = done + [x]
            x = partial
        return x, new_caches

    def forward_recur(self, x: torch.Tensor, ctx: SeqContext, caches: list | None, need_state: bool, T: int):
        """The stack with its looped middle at T passes (models/recur.py). `caches` and the returned list hold one entry per
        layer application, in running order."""
        from . import recur as recur_mod

        if type(T) is not int or T < 1:
            raise ValueError(f"T={T!r}: a pass count >= 1")
        if self.activation_checkpoint == "block" and torch.is_grad_enabled() and x.requires_grad:
            raise ValueError("activation_checkpoint 'block' is not built for a looped middle: use 'layer' or 'none'")
        first, end = self.recur
        want = recur_mod.cache_length(self.recur, len(self.layers), T)
        if caches is not None and len(caches) != want:
            raise ValueError(f"this cache holds {len(caches)} layer entries; a forward at T = {T} needs {want} (a cached sequence keeps its T)")
        new_caches: list = []

        def segment(h, layers):
            for layer in layers:
                h, c = self._run(layer, h, ctx, None if caches is None else caches[len(new_caches)], None, need_state)
                new_caches.append(c)
            return h

        layers = list(self.layers)
        x0 = x
        p = segment(x, layers[:first])
        if self.recur_depth is not None:
            sources, z = [x0, p], None
            for _ in range(T):
                z = segment(self.recur_depth(sources), layers[first:end])
                sources = sources + [z]
            return segment(z, layers[end:]), new_caches
        inject, mix = self.recur_injection, self.recur_mix
        if inject is None:
            e, z = (None if mix is None else p), p
        else:
            e = p if self.recur_norm is None else self.recur_norm(p, out_dtype=p.dtype)
            z = e if self.recur_state_init == "prelude" else None
        for k in range(T):
            if inject is not None:
                u = inject(z, e)
            elif mix is not None and k > 0:
                u = recur_mod.input_mix(e, z, mix)
            else:
                u = z
            z = segment(u, layers[first:end])
        return segment(z, layers[end:]), new_caches

    def forward(self, x: torch.Tensor, ctx: SeqContext, caches: list | None = None, need_state: bool = True, T: int | None = None):
        """x: embedding-stage output (B, L, d). Returns (stream entering final_norm, per-layer caches). T: the pass count of a
        looped middle (models/recur.py); ignored by a stack without one."""
        if self.recur is not None:
            return self.forward_recur(x, ctx, caches, need_state, self.cfg.loop.t_eval if T is None else T)
        new_caches = []
        get = (lambda i: None) if caches is None else (lambda i: caches[i])
        walk = ccr_mod.Walk() if self.ccr else None
        if walk is not None and self.activation_checkpoint not in ccr_mod.CHECKPOINT_MODES and caches is None and torch.is_grad_enabled() and x.requires_grad:
            raise ValueError(f"model.encoder.gdn_ccr_spacing runs with activation_checkpoint {ccr_mod.CHECKPOINT_MODES}, not {self.activation_checkpoint!r}")
        sc = self.layer_scalar_args(x)
        scal = (lambda i: None) if sc is None else (lambda i: sc[i])
        if self.block_every:
            return self._forward_block_every(x, ctx, get, need_state)
        if self.ldm:
            from .ldm import layer_forward

            if self.activation_checkpoint != "none" and torch.is_grad_enabled() and x.requires_grad:
                raise ValueError("model.encoder.attn_res 'ldm' runs with activation_checkpoint 'none'")
            M = None
            for i, layer in enumerate(self.layers):
                x, M, c = layer_forward(layer, x, M, ctx, get(i), need_state)
                new_caches.append(c)
            return x, new_caches
        if not self.block_entry:
            for i, layer in enumerate(self.layers):
                if self.block > 0 and i % self.block == 0 and len(self.layers) % self.block == 0:
                    self._stage(i // self.block, x)
                x, c = self._run_walk(walk, layer, x, ctx, get(i), None, need_state, scal(i))
                new_caches.append(c)
            return x, new_caches
        sources = [x]
        S = self.block
        recompute = self.activation_checkpoint in ("layer", "block") and caches is None and torch.is_grad_enabled() and x.requires_grad
        for b in range(len(self.layers) // S):
            first = self.layers[b * S]
            mixes = {} if recompute else self._block_mixes(b, sources)
            if b == 0:
                start = x
            elif "entry" in mixes:
                start = mixes["entry"]
            else:       # a token-dependent query is formed from the stream where the block before ended
                start = first.attn_res.entry(sources, x) if self.token_query else first.attn_res.entry(sources)
            if b > 0 and first.stream_bf16:
                start = round_stream(start)
            x = start
            self._stage(b, x)
            if self.activation_checkpoint == "block" and sc is None and caches is None and torch.is_grad_enabled() and x.requires_grad:
                x = self._run_block(b, x, ctx, sources)
                new_caches.extend([None] * S)
                sources = sources + [x - start]
                continue
            for i in range(b * S, (b + 1) * S):
                layer = self.layers[i]
                src = sources if getattr(layer, "gdn_arms", None) is not None else None
                pre = (mixes.get((i, "w")), mixes.get((i, "q"))) if (src is not None and mixes) else None
                if self.qmix_record is not None:
                    record_query_weights(self.qmix_record, i, layer, src)
                x, c = self._run_walk(walk, layer, x, ctx, get(i), src, need_state, scal(i), pre)
                new_caches.append(c)
            sources = sources + [x - start]
        last = self.layers[-1].attn_res
        if getattr(self, "keep_sources", False):       # the Copy-Paste pointer's readers read the same [b_0 .. b_N] (models/cp_head.py)
            ctx.memo["cp_pointer_sources"] = sources
        return (last.out(sources, x) if self.token_query else last.out(sources)), new_caches
