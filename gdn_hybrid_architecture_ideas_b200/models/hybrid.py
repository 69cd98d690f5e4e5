"""HybridLM: embedding -> embed_norm -> encoder -> final_norm -> (tied) LM head, with prefill/extend caches.

State-dict names follow the reference's control architecture (ced/model/control.py:342-415): `embed.weight`,
`embed_norm.weight`, `encoder.layers.<i>...`, `final_norm.weight`, `out_embed.weight` when untied. Tokens may be bags
(B, L, s) for token-superposition training: a position is then the mean of s embeddings (control.py:436-455).
"""

from __future__ import annotations

import os

from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import ops
from ..config import ModelConfig, require_supported
from .encoder import Encoder
from .norms import RMSNorm
from .sequence import SeqState, sequence_context


@dataclass
class ControlCache:
    seq: SeqState
    encoder: list
    T: int = 1


@dataclass
class ModelOutput:
    logits: torch.Tensor | None
    hidden_aux: torch.Tensor | None = None
    kept: torch.Tensor | None = None
    n_dropped: torch.Tensor | None = None
    cache: ControlCache | None = None


def lm_head(h: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Logits in at least float32 (reference: ced/model/looped_ced.py:107-117)."""
    dt = torch.promote_types(h.dtype, torch.float32)
    return torch.nn.functional.linear(h.to(dt), weight.to(dt))


class HybridLM(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        if cfg.arch != "control":
            raise ValueError(f"model.arch {cfg.arch!r}: this framework builds arch 'control' (the hybrid stack)")
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.embed_norm = RMSNorm(cfg.d_model, cfg.norm_eps) if cfg.embed_norm else nn.Identity()
        self.encoder = Encoder(cfg)
        self.final_norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.out_embed = None if cfg.tie_embeddings else nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.head_weight_lp: torch.Tensor | None = None  # bf16 shadow of the head matrix (set by the engine)
        self.tp = None      # tensor-parallel context (parallel.tp_model.apply): the stream is then this rank's token shard
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)) and not getattr(m, "own_init", False):
                nn.init.normal_(m.weight, mean=0.0, std=cfg.init_std)
        entmax_layers = [m for m in self.modules() if getattr(m, "entmax", False)]
        if entmax_layers:           # the scale heads: one CPU generator of their own, in model order (reference: ced/model/looped_ced.py:145-155)
            g = torch.Generator().manual_seed((torch.initial_seed() + 0xA5E_2506_16640) % (1 << 63))
            for m in entmax_layers:
                m.reset_asentmax_parameters(g)
        if cfg.encoder.gdn.erase.mode != "none":        # the erase's tensors: a generator of their own as well
            from .gdn_erase import check_model, init_own_parameters as init_erase

            check_model(cfg)
            init_erase(self, cfg.init_std)
        if cfg.encoder.gdn.dprod.n_h != 1:               # Gated DeltaProduct's extra steps: their own generator
            from . import gdn_dprod

            gdn_dprod.check_model(cfg)
            gdn_dprod.init_own_parameters(self, cfg.init_std)
        if cfg.encoder.attn_res_query == "token" or cfg.encoder.attn_res == "ldm":       # address networks: from a generator of their own, after every other tensor
            from .depth_mix import init_own_parameters

            init_own_parameters(self, cfg.init_std)

    def head_weight(self) -> torch.Tensor:
        return self.embed.weight if self.out_embed is None else self.out_embed.weight

    lm_head_weight = head_weight

    def embed_tokens(self, tokens: torch.Tensor) -> torch.Tensor:
        e = ops.embedding(tokens, self.embed.weight)
        return self.embed_norm(e, out_dtype=e.dtype) if self.cfg.embed_norm else e   # the residual stream keeps the table's dtype

    def forward(self, tokens: torch.Tensor, doc_ids: torch.Tensor, dec_mask=None, T=None, capacity=None,
                cache: ControlCache | None = None, return_cache: bool = False, return_hidden: bool = False,
                varlen: dict | None = None, rope_scale: int = 1, gdn_scale: int = 1, gdn_beta_power: bool = False,
                single_doc: bool = False) -> ModelOutput:
        """tokens (B, L) or bags (B, L, s); doc_ids (B, L). return_hidden: give the head input instead of logits
        (the fused loss consumes it). single_doc: the caller guarantees every row is one document (kernels skip
        the document masks). T: the pass count of a looped middle (models/recur.py; default loop.t_eval, or the cache's own T;
        ignored by every other model). dec_mask and capacity are accepted for call compatibility and ignored
        (reference: ced/model/control.py:716-872)."""
        if self.encoder.recur is not None:
            if cache is not None:
                if T is not None and T != cache.T:
                    raise ValueError(f"this cache was prefilled at T = {cache.T}; a cached sequence keeps its pass count (got T = {T})")
                T = cache.T
            elif T is None:
                T = int(os.environ.get("GHB_LOOP_T", self.cfg.loop.t_eval))
        else:
            T = None
        ctx, seq_state = sequence_context(doc_ids, cache.seq if cache else None)
        ctx.single_doc = bool(single_doc) and cache is None
        if varlen is not None:
            ctx.cu_seqlens, ctx.cu_seqlens_cpu = varlen.get("enc"), varlen.get("enc_cpu")
        if tokens.dim() == 3 or rope_scale != 1 or gdn_scale != 1:
            if cache is not None or return_cache:
                raise ValueError("bags of tokens, rope_scale and gdn_scale run without a cache")
            ctx.rope_scale, ctx.gdn_scale, ctx.gdn_beta_power = int(rope_scale), int(gdn_scale), bool(gdn_beta_power)
        B, L = tokens.shape[:2]
        need_state = return_cache or cache is not None
        if self.tp is not None:
            if need_state:
                raise ValueError("tensor parallel runs training forwards only (no cache)")
            tp = self.tp
            tp.batch_shape = (B, L)
            per = B * L // tp.world
            tokens = tokens.reshape(B * L, *tokens.shape[2:])[tp.rank * per:(tp.rank + 1) * per][None]     # this rank's token shard
        h, caches = self.encoder(self.embed_tokens(tokens), ctx, cache.encoder if cache else None, need_state=need_state, T=T)
        hidden = self.final_norm(h)
        logits = None if return_hidden else lm_head(hidden, self.head_weight())
        return ModelOutput(
            logits=logits, hidden_aux=hidden if return_hidden else None,
            kept=torch.zeros(B, L, dtype=torch.bool, device=tokens.device),
            n_dropped=torch.zeros(B, dtype=torch.long, device=tokens.device),
            cache=ControlCache(seq=seq_state, encoder=caches, T=T or 1) if return_cache else None)

    @torch.no_grad()
    def prefill(self, tokens, doc_ids, dec_mask=None, T=None) -> ModelOutput:
        return self.forward(tokens, doc_ids, return_cache=True, T=T)

    @torch.no_grad()
    def extend(self, tokens, doc_ids, dec_mask, cache: ControlCache, T=None) -> ModelOutput:
        return self.forward(tokens, doc_ids, cache=cache, return_cache=True, T=T)


def build_model(cfg: ModelConfig) -> HybridLM:
    """Validated model with initial weights: every Linear/Embedding N(0, init_std); norm gains, depth queries and mix
    lambdas zero; GDN gates by `gdn.init`; low-precision recipes applied last (reference: ced/model/control.py:1246-1346)."""
    require_supported(cfg)
    from .mtp import attach_mtp, check_mtp

    check_mtp(cfg)
    model = HybridLM(cfg)
    if cfg.mtp.enabled:
        attach_mtp(model)       # drawn after every trunk tensor: the trunk starts as the model without the key
    from .lowp import apply_low_precision

    apply_low_precision(model, cfg)
    return model
