"""Encoder layer (Peri-LN) and the layer stack with block-entry depth mixing and the GDN write/query mixes.

Layer: y = x + s * out_norm(mixer(in_norm(x))); y = y + s * mlp_out_norm(mlp(mlp_in_norm(y))), s a fixed float from
the config (reference: ced/model/encoder.py:193-318). Layer i is attention iff (i + 1) % full_attn_interval == 0.

Block walk ("block_entry"): sources = [b_0 = embedding output]; block n starts from start_n = mix(sources) (block 1
from b_0 itself), runs its layers, and appends b_n = x_end - start_n; the stack returns mix(sources) with the last
layer's `out` reader. A GDN layer with arms additionally forms m' = in_norm(mix_w(sources)) and (qmix) m'_q over the
same sources (reference: ced/model/attn_res.py:700-797, ced/model/gdn_arms.py:766-777).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..config import ModelConfig
from . import act_checkpoint
from .attention import GatedAttention
from .depth_mix import EntryLayer
from .gdn import READ_MIX_VARIANTS, GatedDeltaNet, GDNArms
from .mlp import dense_ffn
from .norms import RMSNorm, round_stream
from .sequence import SeqContext


def residual_scale(cfg: ModelConfig) -> float:
    """Fixed residual-branch multiplier of the encoder (reference: ced/model/scaling.py:16-45)."""
    rs = cfg.residual_scale
    if rs.mode in ("none", "inverse_loops"):
        return 1.0
    if rs.mode in ("completep_effective_depth", "loop_factored"):
        return rs.lam * rs.depth_base / cfg.encoder.n_layers
    raise ValueError(f"unknown residual scale mode {rs.mode!r}")


class EncoderLayer(nn.Module):
    def __init__(self, kind: str, cfg: ModelConfig, scale: float, attention=None):
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
            self.mixer = GatedDeltaNet(d, cfg.encoder.gdn, eps, norm_gain=gain)
        elif kind == "attention":
            self.mixer = GatedAttention(d, attention or cfg.encoder.attention, eps)
        else:
            raise ValueError(kind)
        self.mlp = dense_ffn(d, cfg.ffn_hidden, cfg.ffn_activation)

    def forward(self, x: torch.Tensor, ctx: SeqContext, cache=None, sources: list | None = None, need_state: bool = True):
        h = self.mixer_in_norm(x)
        arms: GDNArms | None = getattr(self, "gdn_arms", None)
        if arms is not None:
            if sources is None:
                raise ValueError("a GDN layer with write/query mixes is called with the finished blocks (sources)")
            x_write = self.mixer_in_norm(arms.write_query(sources) if arms.write_query is not None else sources[0])
            x_read = None
            if arms.variant in READ_MIX_VARIANTS:
                x_read = x_write if arms.qmix_query is None else self.mixer_in_norm(arms.qmix_query(sources))
            mixed, new_cache = self.mixer(h, ctx, cache, arms=arms, x_write=x_write, x_read=x_read, need_state=need_state)
        elif self.kind == "gdn":
            mixed, new_cache = self.mixer(h, ctx, cache, need_state=need_state)
        else:
            mixed, new_cache = self.mixer(h, ctx, cache)
        y = ops.norm_add(x, mixed, self.mixer_out_norm.weight, self.mixer_out_norm.eps, self.residual_scale)
        if self.stream_bf16:
            y = round_stream(y)
        y = ops.norm_add(y, self.mlp(self.mlp_in_norm(y)), self.mlp_out_norm.weight, self.mlp_out_norm.eps, self.residual_scale)
        if self.stream_bf16:
            y = round_stream(y)
        return y, new_cache


class Encoder(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        enc = cfg.encoder
        self.cfg = cfg
        scale = residual_scale(cfg)
        per_global = iter(enc.global_attention())
        self.layers = nn.ModuleList(
            EncoderLayer(kind, cfg, scale, attention=next(per_global) if kind == "attention" else None)
            for kind in enc.layer_kinds())
        self.block = enc.full_attn_interval
        self.block_entry = enc.attn_res == "block_entry"
        self.activation_checkpoint = "none"
        self.host_pool = None
        d, eps, S, n = cfg.d_model, cfg.norm_eps, self.block, enc.n_layers
        if self.block_entry:
            if S <= 0 or n % S:
                raise ValueError("model.encoder.attn_res 'block_entry' needs n_layers to be a multiple of full_attn_interval")
            for i, layer in enumerate(self.layers):
                opens, closes = i > 0 and i % S == 0, i % S == S - 1
                if opens or closes:
                    layer.attn_res = EntryLayer(d, eps, entry=opens, closes=closes, last=i == n - 1)
        if enc.gdn_write_mix == "layer":
            if not self.block_entry:
                raise ValueError("model.encoder.gdn_write_mix reads the finished blocks of attn_res 'block_entry'")
            for i, layer in enumerate(self.layers):
                if layer.kind == "gdn" and i > 0:
                    layer.gdn_arms = GDNArms(d, eps, has_query=i // S >= 1, variant=enc.gdn_write_variant)
                    layer.mixer.write_mix = "layer"
        elif enc.gdn_write_mix != "none":
            raise ValueError(f"model.encoder.gdn_write_mix {enc.gdn_write_mix!r}: 'none' or 'layer'")

    def _run(self, layer, x, ctx, cache, sources, need_state):
        """One layer call under the stack's activation memory mode (models/act_checkpoint.py)."""
        mode = self.activation_checkpoint
        training = cache is None and torch.is_grad_enabled() and x.requires_grad
        if mode == "layer" and training:
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

    def forward(self, x: torch.Tensor, ctx: SeqContext, caches: list | None = None, need_state: bool = True):
        """x: embedding-stage output (B, L, d). Returns (stream entering final_norm, per-layer caches)."""
        new_caches = []
        get = (lambda i: None) if caches is None else (lambda i: caches[i])
        if not self.block_entry:
            for i, layer in enumerate(self.layers):
                x, c = self._run(layer, x, ctx, get(i), None, need_state)
                new_caches.append(c)
            return x, new_caches
        sources = [x]
        S = self.block
        for b in range(len(self.layers) // S):
            first = self.layers[b * S]
            start = x if b == 0 else first.attn_res.entry(sources)
            if b > 0 and first.stream_bf16:
                start = round_stream(start)
            x = start
            if self.activation_checkpoint == "block" and caches is None and torch.is_grad_enabled() and x.requires_grad:
                x = self._run_block(b, x, ctx, sources)
                new_caches.extend([None] * S)
                sources = sources + [x - start]
                continue
            for i in range(b * S, (b + 1) * S):
                layer = self.layers[i]
                src = sources if getattr(layer, "gdn_arms", None) is not None else None
                x, c = self._run(layer, x, ctx, get(i), src, need_state)
                new_caches.append(c)
            sources = sources + [x - start]
        return self.layers[-1].attn_res.out(sources), new_caches
