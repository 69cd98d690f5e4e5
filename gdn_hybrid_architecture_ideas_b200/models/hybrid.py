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
    copy: object | None = None      # the Copy-Paste head's keys of every position so far (models/cp_head.py CopyCache)


@dataclass
class ModelOutput:
    logits: torch.Tensor | None
    hidden_aux: torch.Tensor | None = None
    kept: torch.Tensor | None = None
    n_dropped: torch.Tensor | None = None
    cache: ControlCache | None = None
    cp_pointer: object | None = None      # the Copy-Paste pointer's own inputs (models/cp_head.py `PointerInputs`; pointer_input 'mix')


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
        from . import second_pass

        second_pass.check_config(cfg)
        self.gated = second_pass.is_on(cfg)                      # a read-only second pass through the top `pass2_layers` layers
        self.pass2_from = cfg.encoder.n_layers - (cfg.loop.pass2_layers if self.gated else 0)
        from . import pass_counts

        self.schedule = pass_counts.schedule_of(cfg.loop) if self.gated else None      # pass counts by segment (models/pass_counts.py)
        self.n_passes = pass_counts.built_passes(cfg.loop) if self.gated else 1
        self.pass_scheduler = None           # per-position counts from the tokens when a caller gives none; built at first use from loop.segment_tokenizer
        if self.gated and cfg.loop.loop_embedding:
            self.loop_embedding_pass2 = nn.Parameter(torch.zeros(cfg.d_model))
            if self.n_passes > 2:
                self.loop_embedding_pass3 = nn.Parameter(torch.zeros(cfg.d_model))
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.embed_norm = RMSNorm(cfg.d_model, cfg.norm_eps) if cfg.embed_norm else nn.Identity()
        self.encoder = Encoder(cfg)
        self.final_norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.out_embed = None if cfg.tie_embeddings else nn.Embedding(cfg.vocab_size, cfg.d_model)
        if self.gated:
            self.hyper_connections = second_pass.SecondPassGate(self.n_passes)
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
        from . import cp_head as cp_mod

        cp_mod.check_config(cfg)
        if cfg.cp_head.enabled:          # the Copy-Paste head: after every other tensor, from a generator of its own
            cp_mod.attach(self)

    def lm_head_weight(self) -> torch.Tensor:
        """The (V, d) LM head matrix: the input embedding when tied. With a Copy-Paste head this is p_LM's head."""
        return self.embed.weight if self.out_embed is None else self.out_embed.weight

    def head_weight(self) -> torch.Tensor:
        """`lm_head_weight`, refused in eval mode for a model whose next-token distribution is the Copy-Paste mixture: a
        scoring path that applies the bare head to hidden states would score p_LM by mistake (models/cp_head.py
        `head_token_ce` scores the mixture)."""
        if not self.training and getattr(self, "cp_head", None) is not None and self.cp_head.gated:
            from .cp_head import score_mode

            if score_mode(self) == "mixture" and not self.cfg.cp_head.force_lambda_zero:
                raise ValueError("this model has a Copy-Paste head: its next-token distribution is the mixture, not softmax(h W^T). Score it with "
                                 "models.cp_head.head_token_ce or the forward's logits (log p); lm_head_weight() is p_LM's head")
        return self.lm_head_weight()

    def embed_tokens(self, tokens: torch.Tensor) -> torch.Tensor:
        e = ops.embedding(tokens, self.embed.weight)
        return self.embed_norm(e, out_dtype=e.dtype) if self.cfg.embed_norm else e   # the residual stream keeps the table's dtype

    def pass2_parameter_names(self) -> list[str]:
        from .second_pass import PASS2_PARAMETERS

        return [n for n, _ in self.named_parameters() if n in PASS2_PARAMETERS] if self.gated else []

    def alpha(self):
        """The second pass's gate (0-dim, detached) or None."""
        return self.hyper_connections.pass2_gate.detach() if self.gated else None

    def forward(self, tokens: torch.Tensor, doc_ids: torch.Tensor, dec_mask=None, T=None, capacity=None,
                cache: ControlCache | None = None, return_cache: bool = False, return_hidden: bool = False,
                varlen: dict | None = None, rope_scale: int = 1, gdn_scale: int = 1, gdn_beta_power: bool = False,
                single_doc: bool = False, pass2_mask: torch.Tensor | None = None, pass2_capacity: int | None = None,
                pass_counts: torch.Tensor | None = None, scored: torch.Tensor | None = None) -> ModelOutput:
        """tokens (B, L) or bags (B, L, s); doc_ids (B, L). return_hidden: give the head input instead of logits
        (the fused loss consumes it). single_doc: the caller guarantees every row is one document (kernels skip
        the document masks). T: the pass count of a looped middle (models/recur.py; default loop.t_eval, or the cache's own T)
        or of a stack with a gated second pass (models/second_pass.py: 1 or 2, default loop.t_eval; at T = 2 pass 2 runs at
        every position, or is kept at the first pass2_capacity positions of each row that pass2_mask marks, and `kept` /
        `n_dropped` say where); ignored by every other model. With a pass schedule (loop.segment_passes / unscored_passes) a
        forward at T = 2 runs, at each position, the passes of pass_counts ((B, L) integers 1 .. 3) or, when none are given,
        of the model's own scheduler over the tokens (whole rows, no cache; `scored` (B, L) for the unscored rule);
        pass2_mask then marks the positions whose logits are read, every other one runs pass 1 only. dec_mask and capacity
        are accepted for call compatibility and ignored (reference: ced/model/control.py:716-872)."""
        two = False
        if self.gated:
            T = self.cfg.loop.t_eval if T is None else T
            if T not in (1, 2):
                raise ValueError(f"T={T!r}: a stack with a second pass runs T = 1 or T = 2")
            two = T == 2 and not (pass2_mask is not None and pass2_capacity == 0)
            if pass_counts is not None and self.schedule is None:
                raise ValueError("pass_counts are for a model with a pass schedule (model.loop.segment_passes / unscored_passes)")
        elif pass2_mask is not None or pass2_capacity is not None or pass_counts is not None:
            raise ValueError("pass2_mask / pass2_capacity belong to a model with a gated second pass (model.loop.pass2_gate)")
        if self.encoder.recur is not None:
            if cache is not None:
                if T is not None and T != cache.T:
                    raise ValueError(f"this cache was prefilled at T = {cache.T}; a cached sequence keeps its pass count (got T = {T})")
                T = cache.T
            elif T is None:
                T = int(os.environ.get("GHB_LOOP_T", self.cfg.loop.t_eval))
        elif not self.gated:
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
        kept = n_dropped = None
        if two:
            from . import second_pass

            if tokens.dim() == 3 or rope_scale != 1 or gdn_scale != 1 or self.tp is not None:
                raise ValueError("bags of tokens, rope_scale, gdn_scale and tensor parallel run on the one-pass stack")
            block = list(self.encoder.layers)[self.pass2_from:]
            for layer in block:
                layer.keep_record = layer.mixer.keep_record = True
            try:
                z1, caches = self.encoder(self.embed_tokens(tokens), ctx, cache.encoder if cache else None, need_state=need_state)
            finally:
                for layer in block:
                    layer.keep_record = layer.mixer.keep_record = False
            records = []
            for layer, c in zip(block, caches[self.pass2_from:]):
                if layer.kind == "gdn":
                    records.append(c.pass1)
                    c.pass1 = None                                   # the cache is pass 1's: the record does not travel with it
                else:
                    records.append(c)
            checkpoint = cache is None and self.encoder.activation_checkpoint == "layer" and torch.is_grad_enabled() and z1.requires_grad
            if self.schedule is not None:
                if pass2_capacity is not None:
                    raise ValueError("pass2_capacity is the dense second pass's slot count; under a pass schedule the counts say where a pass runs")
                counts = self._pass_counts(tokens, doc_ids, pass_counts, scored, cache)
                if pass2_mask is not None:
                    counts = torch.where(pass2_mask.bool().to(counts.device), counts, torch.ones_like(counts))
                top = int(counts.max())                               # counts come from the host: no device wait
                h, kept = second_pass.scheduled_passes(self, z1, ctx, records, counts.to(z1.device), top, checkpoint)
                n_dropped = torch.zeros(B, dtype=torch.long, device=z1.device)
                self.last_counts = counts
            else:
                h, kept, n_dropped = second_pass.second_pass(self, z1, ctx, records, pass2_mask, pass2_capacity, checkpoint)
            self.last_loop_usage = second_pass.loop_usage(z1.detach(), h.detach(), kept)
        else:
            h, caches = self.encoder(self.embed_tokens(tokens), ctx, cache.encoder if cache else None, need_state=need_state,
                                     T=None if self.gated else T)
        hidden = self.final_norm(h)
        copy_cache = pointer = None
        if getattr(self, "cp_head", None) is not None and self.cfg.cp_head.pointer_input == "shared":
            import dataclasses

            from .cp_head import PointerInputs

            entry = caches[self.cp_head.shared_layer]
            if entry is None or entry.cp_q is None:
                raise ValueError("model.cp_head.pointer_input 'shared': the shared layer handed over no query and key (activation checkpointing drops a layer's key set)")
            pointer = PointerInputs(entry.cp_q, entry.cp_k)
            caches = list(caches)
            caches[self.cp_head.shared_layer] = dataclasses.replace(entry, cp_q=None, cp_k=None)       # a cache keeps keys only
        if getattr(self, "cp_head", None) is not None and self.cfg.cp_head.pointer_input == "mix":
            from .cp_head import SOURCES_KEY

            sources = ctx.memo.pop(SOURCES_KEY)
            if self.training and self.cfg.cp_head.train_mode == "addon":      # the add-on head's readers send no gradient into the stack
                sources = [b.detach() for b in sources]
            if self.cp_head.gated or self.training:       # a pointer trained on its auxiliary loss is dropped at evaluation
                pointer = self.cp_head.mix(sources)
        if return_hidden:
            logits = None
        elif getattr(self, "cp_head", None) is not None and self.cp_head.gated:
            from .cp_head import forward_logits

            if tokens.dim() != 2 or self.tp is not None:
                raise ValueError("the Copy-Paste head's output is for token rows on one device, not bags or a token shard")
            logits, copy_cache = forward_logits(self, hidden, tokens, doc_ids, ctx.idx, cache.copy if cache else None, pointer)
        else:
            logits = lm_head(hidden, self.lm_head_weight())
        if return_cache and copy_cache is None and getattr(self, "cp_head", None) is not None and self.cp_head.gated:
            raise ValueError("a cache of a Copy-Paste model is built by a forward that returns logits (prefill / extend)")
        return ModelOutput(
            logits=logits, hidden_aux=hidden if return_hidden else None, cp_pointer=pointer,
            kept=torch.zeros(B, L, dtype=torch.bool, device=tokens.device) if kept is None else kept,
            n_dropped=torch.zeros(B, dtype=torch.long, device=tokens.device) if n_dropped is None else n_dropped,
            cache=ControlCache(seq=seq_state, encoder=caches, T=T or 1, copy=copy_cache) if return_cache else None)

    def _pass_counts(self, tokens, doc_ids, given, scored, cache) -> torch.Tensor:
        """The (B, L) pass counts of a scheduled forward, on the host: the caller's, or the model's own scheduler's over whole rows."""
        if given is not None:
            counts = given.detach().to("cpu", torch.long)
            if counts.shape != tokens.shape[:2] or int(counts.min()) < 1 or int(counts.max()) > self.n_passes:
                raise ValueError(f"pass_counts {tuple(counts.shape)}: (B, L) integers from 1 to {self.n_passes}")
            return counts
        if cache is not None:
            raise ValueError("a cached forward of a model with a pass schedule takes its pass_counts from the caller (the segment of a position "
                             "depends on the tokens before the chunk)")
        if self.pass_scheduler is None:
            from .pass_counts import PassScheduler

            self.pass_scheduler = PassScheduler.from_tokenizer(self.schedule, self.cfg.loop.segment_tokenizer)
        return self.pass_scheduler.counts(tokens, doc_ids, scored=scored)

    def _pass2_at(self, dec_mask, T) -> dict:
        """prefill / extend: a decoder mask marks the positions whose logits are read, so pass 2 is kept there alone, with as
        many slots as the fullest row has marked positions (one host read of the mask: inference only)."""
        if dec_mask is None or not self.gated or (self.cfg.loop.t_eval if T is None else T) == 1:
            return {}
        if self.schedule is not None:            # the counts say where a pass runs; the mask whose logits are read
            return {"pass2_mask": dec_mask.bool()}
        return {"pass2_mask": dec_mask.bool(), "pass2_capacity": int(dec_mask.bool().sum(1).max())}

    @torch.no_grad()
    def prefill(self, tokens, doc_ids, dec_mask=None, T=None, pass_counts=None) -> ModelOutput:
        return self.forward(tokens, doc_ids, return_cache=True, T=T, pass_counts=pass_counts, **self._pass2_at(dec_mask, T))

    @torch.no_grad()
    def extend(self, tokens, doc_ids, dec_mask, cache: ControlCache, T=None, pass_counts=None) -> ModelOutput:
        return self.forward(tokens, doc_ids, cache=cache, return_cache=True, T=T, pass_counts=pass_counts, **self._pass2_at(dec_mask, T))


def build_model(cfg: ModelConfig):
    """Validated model with initial weights: every Linear/Embedding N(0, init_std); norm gains, depth queries and mix
    lambdas zero; GDN gates by `gdn.init`; low-precision recipes applied last (reference: ced/model/control.py:1246-1346).
    arch 'looped_ced' builds the looped encoder-decoder (models/looped_decoder.py)."""
    require_supported(cfg)
    if cfg.arch == "looped_ced":
        from .looped_decoder import LoopedCED

        return LoopedCED(cfg)
    from .mtp import attach_mtp, check_mtp

    check_mtp(cfg)
    model = HybridLM(cfg)
    if cfg.mtp.enabled:
        attach_mtp(model)       # drawn after every trunk tensor: the trunk starts as the model without the key
    from .lowp import apply_low_precision

    apply_low_precision(model, cfg)
    return model
