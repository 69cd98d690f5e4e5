"""The looped encoder-decoder (`model.arch: looped_ced`): a causal encoder over every position and a shared decoder block
that runs T times at the decoder positions only (the positions whose next token the model generates).

    h      = Encoder(embed(x))                                   every position
    aux    = head(RMSNorm_aux(h))                                every position (its loss counts at the context positions)
    memory = (k, v) of RMSNorm(h) through `memory_kv`            offered by the context positions
    e      = RMSNorm_inj(h at the slots);  Y = lanes(e)          the decoder slots
    pass k = 0 .. T - 1:   z = read_k(Y);  u = inject(z, e) + loop_embedding[k];  s = layers(u);  Y = write_k(Y, z, s)
    dec    = head(RMSNorm_dec(collapse(Y)))                      at the slots, put back at their positions

Slots. A row of L positions reserves C = min(L, round_up(ceil(p L), m)) decoder slots (p = `decoder.capacity_fraction`,
m = `decoder.capacity_multiple`); the first C decoder positions of the row take them in order, which is prefix-stable
(whether position t is kept depends on dec_mask[: t + 1] alone), later ones are dropped and count as context. An empty
slot has index L, document -1 and position 0. Every shape is fixed by (B, L, C): the slots' positions come from one
cumulative sum and one sorted search, reads and writes are gathers through the map and its inverse (`Slots`), and no
boolean indexing runs.

A decoder layer (Peri-LN: u += eps Norm(mixer(Norm(u))); u += eps Norm(FFN(Norm(u)))) is a memory-attention layer
(`decoder.memory_attn_interval`-th layers) or a Gated DeltaNet over the row's slot sequence with a state of its own per
pass. A memory-attention query at position t, pass k, layer l reads in ONE softmax the memory of the context positions
s <= t of its document and the pass-k layer-l keys of the decoder positions s <= t of its document, itself included;
every position offers exactly one kind of key, so teacher forcing (a pass over all slots at once) and cached decoding
(each position through all passes before the next) are the same function. An empty slot reads the empty slots of its
row alone (document -1), which keeps its softmax finite; nothing reads its result.

Loop boundary: the diagonal Parcae injection (`loop.injection: parcae`; `none` passes z through), a loop-index embedding
(zeros), static hyper-connections over K lanes (`loop.hyper_connections: static`: per pass a read vector, a lane mixing
matrix and write weights, started so that the lanes reproduce the plain loop), depth attention (`loop.depth_attention:
layer`: one head over the position's own stack of layer applications, output projection zeros), mixers untied per pass
(`decoder.untie_mixers`), a routed FFN (`decoder.ffn_experts`), intermediate readouts through norms of their own (the
drafts). The fixed residual multipliers follow `model.residual_scale` at the reference loop count.

Tensor ops on the encoder's kernels (the encoder is the hybrid stack's). Reference: ced/model/looped_ced.py:158-379,
ced/model/decoder.py:34-241, ced/model/loop.py:26-190, ced/model/capacity.py:26-70, ced/model/scaling.py:16-45.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config import ModelConfig
from .attention import GatedAttention, KeySet, rope_cap
from .encoder import Encoder
from .gdn import GatedDeltaNet, GDNState
from .mlp import RoutedSwiGLU, dense_ffn
from .norms import RMSNorm
from .recur import RecurInjection
from .rope import apply_rope
from .sequence import SeqContext, SeqState, sequence_context

UNTIE = ("none", "attention", "all")
HYPER = ("none", "static")
INJECTIONS = ("none", "parcae")


# ------------------------------------------------------------------------------------------------------------- slots

def decoder_capacity(length: int, fraction: float, multiple: int) -> int:
    wanted = math.ceil(fraction * length)
    return min(length, -(-wanted // multiple) * multiple)


@dataclass
class Slots:
    index: torch.Tensor        # (B, C) the position in each slot, L for an empty slot
    valid: torch.Tensor        # (B, C) bool
    kept: torch.Tensor         # (B, L) bool: the positions that run the decoder
    inverse: torch.Tensor      # (B, L) the slot of each kept position, C elsewhere
    n_dropped: torch.Tensor    # (B,) decoder positions beyond the capacity

    def take(self, x: torch.Tensor, fill=0) -> torch.Tensor:
        """x (B, L, ...) -> (B, C, ...); an empty slot reads `fill`."""
        return _rows(x, self.index, fill)

    def put(self, base: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
        """base (B, L, ...) with values (B, C, ...) at the slots' positions; a gather through the inverse map."""
        spread = _rows(values, self.inverse, 0)
        return torch.where(self.kept.view(*self.kept.shape, *([1] * (base.dim() - 2))), spread.to(base.dtype), base)


def _rows(x: torch.Tensor, index: torch.Tensor, fill) -> torch.Tensor:
    """out[b, j] = x[b, index[b, j]], the row one past the end reading `fill`."""
    padded = torch.cat([x, torch.full_like(x[:, :1], fill)], dim=1)
    return torch.gather(padded, 1, index.view(*index.shape, *([1] * (x.dim() - 2))).expand(*index.shape, *x.shape[2:]))


def select_slots(dec_mask: torch.Tensor, capacity: int) -> Slots:
    """The first `capacity` decoder positions of each row, in order. The count of decoder positions up to t is
    nondecreasing in t, so slot c holds the first position where it reaches c + 1: one sorted search."""
    B, L = dec_mask.shape
    count = dec_mask.long().cumsum(1)
    wanted = torch.arange(1, capacity + 1, device=dec_mask.device).expand(B, capacity)
    index = torch.searchsorted(count, wanted.contiguous())                  # L where the row has fewer
    kept = dec_mask & (count <= capacity)
    inverse = torch.where(kept, count - 1, torch.full_like(count, capacity))
    return Slots(index, index < L, kept, inverse, count[:, -1] - kept.long().sum(1))


@dataclass
class SlotContext:
    """The gathered slots of a chunk: absolute index (-1 empty), document (-1 empty), position in the document, valid."""

    idx: torch.Tensor
    doc: torch.Tensor
    pos: torch.Tensor
    valid: torch.Tensor
    memo: dict = field(default_factory=dict)

    def as_sequence(self, past: GDNState | None) -> SeqContext:
        """The slots as a sequence for a GDN layer over decoder positions: a document starts at a valid slot whose
        document differs from the slot before it (across chunks: the last entry of the conv history)."""
        before = self.doc.new_full((self.doc.shape[0], 1), -1) if past is None else past.conv_doc[:, -1:]
        prev = torch.cat([before, self.doc[:, :-1]], dim=1)
        return SeqContext(idx=self.idx, doc=self.doc, pos=self.pos, is_doc_start=self.valid & (self.doc != prev))


# ----------------------------------------------------------------------------------------------------- loop boundary

class NoInjection(nn.Module):
    def forward(self, z, e):
        return z


class _Injection(RecurInjection):
    """decay z + dt (B e) with the dense B (the stack's looped middle uses the same tensors)."""

    def forward(self, z, e):
        return super().forward(z, e)


class SingleState(nn.Module):
    """No lanes: the state is the block's output."""

    def start(self, e):
        return e

    def read(self, Y, k):
        return Y

    def write(self, Y, z, s, k):
        return s

    def finish(self, Y):
        return Y


class StaticLanes(nn.Module):
    """K lanes that start as copies of e. Pass k reads r = sum_j a_k[j] Y_j and writes Y_i <- sum_j M_k[i, j] Y_j + b_k[i] w
    with w = s - r (`hc_write: delta`) or s (`full`); a_k = one_hot(k mod K), M_k = I, b_k = 1 at the start, which is the
    plain loop. The lanes' mean is the result."""

    def __init__(self, loop):
        super().__init__()
        K, T = loop.hc_streams, loop.t_max
        if loop.hc_write not in ("delta", "full"):
            raise ValueError(f"model.loop.hc_write {loop.hc_write!r}: 'delta' or 'full'")
        self.lanes, self.full = K, loop.hc_write == "full"
        self.read_weights = nn.Parameter(F.one_hot(torch.arange(T) % K, K).float())
        self.mix_weights = nn.Parameter(torch.eye(K).expand(T, K, K).clone())
        self.write_weights = nn.Parameter(torch.ones(T, K))

    def start(self, e):
        return e.unsqueeze(-2).repeat_interleave(self.lanes, dim=-2)

    def read(self, Y, k):
        return (self.read_weights[k].to(Y.dtype).unsqueeze(-1) * Y).sum(-2)

    def write(self, Y, z, s, k):
        moved = s if self.full else s - z
        return self.mix_weights[k].to(Y.dtype) @ Y + self.write_weights[k].to(Y.dtype).unsqueeze(-1) * moved.unsqueeze(-2)

    def finish(self, Y):
        return Y.mean(-2)


class DepthAttention(nn.Module):
    """One head, per position, over the position's own stack of layer applications (entry j = pass k, layer l:
    j = k n_layers + l), rotary over the depth index; a residual branch beside the mixer whose output projection starts at
    zero. The stack lives for the position's step only."""

    def __init__(self, d_model: int, head_dim: int, theta: float, eps: float):
        super().__init__()
        self.head_dim, self.theta = head_dim, theta
        self.qkv = nn.Linear(d_model, 3 * head_dim, bias=False)
        self.q_norm, self.k_norm = RMSNorm(head_dim, eps), RMSNorm(head_dim, eps)
        self.out = nn.Linear(head_dim, d_model, bias=False)

    def forward(self, h, depth: int, stack: list):
        q, k, v = self.qkv(h).split(self.head_dim, dim=-1)
        at = torch.full(h.shape[:2], depth, dtype=torch.long, device=h.device)
        turn = lambda t, norm: apply_rope(norm(t).unsqueeze(2), at, 1.0, self.theta).squeeze(2)      # noqa: E731
        q = turn(q, self.q_norm)
        stack.append((turn(k, self.k_norm), v))
        wide = torch.promote_types(q.dtype, torch.float32)
        keys, values = (torch.stack([entry[i] for entry in stack], dim=2).to(wide) for i in (0, 1))       # (B, C, depth + 1, hd)
        share = ((keys @ q.to(wide).unsqueeze(-1)).squeeze(-1) * self.head_dim ** -0.5).softmax(-1)
        return self.out((share.unsqueeze(-2) @ values).squeeze(-2).to(h.dtype))


# ------------------------------------------------------------------------------------------------------------ layers

class MemoryKV(nn.Module):
    """The keys and values the context positions offer the decoder: one projection of RMSNorm(h), a key norm of its own and
    the decoder's rotary embedding, formed once and read by every pass (and, unless `memory_kv_per_layer`, every layer)."""

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.attn = cfg.decoder.attention
        self.in_norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.proj = nn.Linear(cfg.d_model, 2 * self.attn.n_kv_heads * self.attn.head_dim, bias=False)
        self.k_norm = RMSNorm(self.attn.head_dim, cfg.norm_eps) if self.attn.qk_norm else nn.Identity()

    def forward(self, h, ctx: SeqContext, ok) -> KeySet:
        a = self.attn
        k, v = self.proj(self.in_norm(h)).unflatten(-1, (2, a.n_kv_heads, a.head_dim)).unbind(2)
        plain = self.k_norm(k)
        return KeySet(k=apply_rope(plain, ctx.pos, a.rope_fraction, a.rope_theta), v=v, idx=ctx.idx, doc=ctx.doc, ok=ok,
                      k_far=plain if rope_cap(a) is not None else None)


def gdn_over_slots(mixer: GatedDeltaNet, h, slots: SlotContext, past: GDNState | None):
    """A Gated DeltaNet layer over the slot sequence, the empty slots (a suffix) neither decaying nor writing the state;
    the conv history kept is that of the last real slots."""
    cfg = mixer.cfg
    B, C = slots.doc.shape
    seq = slots.as_sequence(past)
    hist, hist_doc = (None, None) if past is None else (past.conv_input, past.conv_doc)
    pre = mixer.in_proj_qkv(h)
    K = mixer.conv_weight.shape[1]
    first = (pre.new_zeros(B, K - 1, pre.shape[-1]), slots.doc.new_full((B, K - 1), -1)) if hist is None else (hist.to(pre.dtype), hist_doc)
    q, k, v, _, _ = ops.ref.gdn_prep(pre, slots.doc, mixer.conv_weight, cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim, *first)
    real = slots.valid.long().sum(1, keepdim=True) + torch.arange(K - 1, device=h.device)               # the K - 1 inputs before the first empty slot
    conv_input = torch.gather(torch.cat([first[0], pre], dim=1), 1, real.unsqueeze(-1).expand(B, K - 1, pre.shape[-1]))
    conv_doc = torch.gather(torch.cat([first[1], slots.doc], dim=1), 1, real)
    g, beta = ops.ref.gdn_gates(mixer.in_proj_a(h), mixer.in_proj_b(h), mixer.A_log, mixer.dt_bias)
    live = slots.valid.unsqueeze(-1)
    g, beta = g * live.to(g.dtype), beta * live.to(beta.dtype) * mixer.beta_max
    group = cfg.n_v_heads // cfg.n_k_heads
    S0 = h.new_zeros(B, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim, dtype=ops.ref.work_dtype(q)) if past is None else past.S
    rule = ops.ref.delta_rule_recurrence if cfg.kernel == "recurrence" or C == 1 else (lambda *a: ops.ref.chunked_delta_rule(*a, cfg.chunk_size))
    work = S0.dtype
    o, S = rule(q.repeat_interleave(group, dim=2).to(work), k.repeat_interleave(group, dim=2).to(work), v.to(work), g.to(work), beta.to(work),
                seq.is_doc_start, S0)
    z = mixer.in_proj_z(h).unflatten(-1, (cfg.n_v_heads, cfg.v_head_dim))
    return mixer.out_proj(mixer.norm(o.to(h.dtype), z).flatten(2)), GDNState(conv_input=conv_input, conv_doc=conv_doc, S=S)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, kind: str, scale: float):
        super().__init__()
        d, eps, dec = cfg.d_model, cfg.norm_eps, cfg.decoder
        self.kind, self.residual_scale = kind, scale
        for name in ("attn_in_norm", "attn_out_norm", "mlp_in_norm", "mlp_out_norm"):
            setattr(self, name, RMSNorm(d, eps))
        if dec.untie_mixers not in UNTIE:
            raise ValueError(f"model.decoder.untie_mixers {dec.untie_mixers!r}: one of {UNTIE}")
        own_per_pass = dec.untie_mixers == "all" or (dec.untie_mixers == "attention" and kind == "memory_attention")
        copies = cfg.loop.t_max if own_per_pass else 1
        if kind == "memory_attention":
            if dec.attention.normalizer != "softmax" or dec.attention.kv_sharing != "gqa":
                raise ValueError("model.decoder.attention: the looped decoder's memory attention is softmax over GQA keys")
            self.mixers = nn.ModuleList(GatedAttention(d, dec.attention, eps) for _ in range(copies))
        else:
            self.mixers = nn.ModuleList(GatedDeltaNet(d, dec.gdn, eps) for _ in range(copies))
        lp = cfg.loop
        self.depth_attention = DepthAttention(d, lp.depth_attention_head_dim, lp.depth_attention_rope_theta, eps) if lp.depth_attention == "layer" else None
        if dec.ffn_experts > 0:
            if cfg.ffn_activation != "swiglu":
                raise ValueError("model.decoder.ffn_experts: the routed decoder FFN is SwiGLU (model.ffn_activation 'swiglu')")
            self.mlp = RoutedSwiGLU(d, dec.ffn_experts, dec.ffn_top_k, dec.ffn_expert_hidden or cfg.ffn_hidden // dec.ffn_top_k)
        else:
            self.mlp = dense_ffn(d, cfg.ffn_hidden, cfg.ffn_activation)

    def attend(self, mixer: GatedAttention, h, slots: SlotContext, memory: KeySet, own_past: KeySet | None):
        B, C = slots.doc.shape
        a = mixer.cfg
        q, q_far, gate = mixer.queries(h, slots.pos, slots.pos)
        k, k_far = mixer.keys(mixer.k_proj(h).view(B, C, a.n_kv_heads, a.head_dim), slots.pos)
        # an empty slot (document -1, index -1) is offered too: only the empty slots of its row can read it
        own_now = KeySet(k=k, v=mixer.v_proj(h).view(B, C, a.n_kv_heads, a.head_dim), idx=slots.idx, doc=slots.doc,
                         ok=torch.ones_like(slots.valid), k_far=k_far)
        keys = KeySet.cat(memory, own_past, own_now)
        o = ops.ref.attention(q, keys.k, keys.v, slots.idx, slots.doc, keys.idx, keys.doc, keys.ok, q_far=q_far, k_far=keys.k_far, cap=mixer.cap)
        return mixer.output(o, gate), KeySet.cat(own_past, own_now)

    def forward(self, u, slots: SlotContext, memory: KeySet | None, own_past, k: int, depth: int = 0, stack: list | None = None):
        """u (B, C, d) at pass k; own_past: this (pass, layer)'s cache entry of earlier chunks. Returns (u, the entry)."""
        mixer = self.mixers[k if len(self.mixers) > 1 else 0]
        h = self.attn_in_norm(u)
        if self.kind == "memory_attention":
            mixed, entry = self.attend(mixer, h, slots, memory, own_past)
        else:
            mixed, entry = gdn_over_slots(mixer, h, slots, own_past)
        u = u + self.residual_scale * self.attn_out_norm(mixed)
        if self.depth_attention is not None:
            u = u + self.residual_scale * self.depth_attention(h, depth, stack)
        x = self.mlp_in_norm(u)
        out = self.mlp(x, valid=slots.valid) if isinstance(self.mlp, RoutedSwiGLU) else self.mlp(x)
        return u + self.residual_scale * self.mlp_out_norm(out), entry


# ------------------------------------------------------------------------------------------------------------- model

def residual_scales(cfg: ModelConfig) -> tuple[float, float]:
    """(encoder, decoder) multipliers of the residual branches, from the config alone (never the sampled T)."""
    rs, n_enc, n_dec = cfg.residual_scale, cfg.encoder.n_layers, cfg.decoder.n_layers
    t_ref = rs.t_ref if rs.t_ref is not None else max(cfg.loop.t_choices)
    if rs.mode == "none":
        return 1.0, 1.0
    if rs.mode == "completep_effective_depth":
        both = rs.lam * rs.depth_base / (n_enc + t_ref * n_dec)
        return both, both
    if rs.mode == "loop_factored":
        return rs.lam * rs.depth_base / n_enc, rs.lam / (t_ref * math.sqrt(n_dec / rs.l_ref))
    if rs.mode == "inverse_loops":
        return 1.0, rs.lam / t_ref
    raise ValueError(f"unknown residual scale mode {rs.mode!r}")


@dataclass
class LoopedCache:
    """seq: index / document bookkeeping; encoder: one entry per encoder layer; memory: per memory projection, the
    memory of all past positions (decoder positions have ok False); own[k][l]: pass k, decoder layer l over the past
    decoder slots (a KeySet or a GDNState); T: the pass count the cache was built at."""

    seq: SeqState
    encoder: list
    memory: list
    own: list
    T: int


@dataclass
class Chunk:
    """What the passes need of a chunk: the bookkeeping and caches after its encoder, the memory of all positions so far,
    the aux head's input, the slots and the injected input e (B, C, d)."""

    seq_state: SeqState
    encoder: list
    memory: list
    aux_hidden: torch.Tensor
    slots: Slots
    at: SlotContext
    e: torch.Tensor

    @property
    def seq(self):
        return self.seq_state


@dataclass
class LoopedOutput:
    logits: torch.Tensor | None          # (B, L, V): the decoder head at the kept positions, the aux head elsewhere
    kept: torch.Tensor
    n_dropped: torch.Tensor
    cache: LoopedCache | None = None
    draft_logits: list | None = None     # [k - 1]: the readout after pass k < T, at the slots
    slot_index: torch.Tensor | None = None
    slot_valid: torch.Tensor | None = None
    aux_loss: torch.Tensor | None = None
    hidden_aux: torch.Tensor | None = None       # return_hidden: head inputs instead of logits
    hidden_dec: torch.Tensor | None = None
    hidden_drafts: list | None = None
    slots: Slots | None = None


def check_config(cfg: ModelConfig) -> None:
    lp, dec = cfg.loop, cfg.decoder
    if lp.injection not in INJECTIONS:
        raise ValueError(f"model.loop.injection {lp.injection!r} on arch 'looped_ced': one of {INJECTIONS}")
    if lp.hyper_connections not in HYPER:
        raise ValueError(f"model.loop.hyper_connections {lp.hyper_connections!r}: one of {HYPER}")
    if lp.depth_attention not in ("none", "layer"):
        raise ValueError(f"model.loop.depth_attention {lp.depth_attention!r}: 'none' or 'layer'")
    if "memory_attention" not in dec.layer_kinds():
        raise ValueError("model.decoder: the decoder needs at least one memory-attention layer to read the context (memory_attn_interval <= n_layers)")
    off = {"model.loop.recur_layers": bool(lp.recur_layers), "model.loop.pass2_gate": lp.pass2_gate != "none", "model.cp_head.enabled": bool(cfg.cp_head.enabled),
           "model.mtp.enabled": bool(cfg.mtp.enabled), "model.fp8.mode": cfg.fp8.mode != "none", "model.nvfp4.mode": cfg.nvfp4.mode != "none",
           "model.encoder.attn_res": cfg.encoder.attn_res != "none", "model.decoder.self_kv": bool(dec.self_kv),
           "attention.rope_max_distance (encoder or decoder)": cfg.encoder.attention.rope_max_distance is not None or dec.attention.rope_max_distance is not None,
           "model.decoder.gdn (kda / erase / dprod / negeig)": (dec.gdn.kda.decay, dec.gdn.erase.mode, dec.gdn.dprod.n_h) != ("scalar", "none", 1)}
    hit = [k for k, v in off.items() if v]
    if hit:
        raise ValueError(f"model.arch 'looped_ced' is not built together with: {', '.join(hit)}")
    if not 1 <= lp.t_eval <= lp.t_max or any(not 1 <= t <= lp.t_max for t in lp.t_choices):
        raise ValueError(f"model.loop.t_eval {lp.t_eval} / t_choices {list(lp.t_choices)!r}: pass counts in 1 .. t_max ({lp.t_max})")


class LoopedCED(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        if cfg.arch != "looped_ced":
            raise ValueError(f"model.arch {cfg.arch!r}: LoopedCED builds arch 'looped_ced'")
        check_config(cfg)
        self.cfg = cfg
        d, eps, lp = cfg.d_model, cfg.norm_eps, cfg.loop
        _, dec_scale = residual_scales(cfg)
        self.embed = nn.Embedding(cfg.vocab_size, d)
        self.embed_norm = RMSNorm(d, eps) if cfg.embed_norm else nn.Identity()
        self.encoder = Encoder(cfg)
        self.aux_norm = RMSNorm(d, eps)
        kinds = cfg.decoder.layer_kinds()
        readers = [l for l, kind in enumerate(kinds) if kind == "memory_attention"]
        self.memory_of = {l: (i if cfg.decoder.memory_kv_per_layer else 0) for i, l in enumerate(readers)}
        self.memory_kv = nn.ModuleList(MemoryKV(cfg) for _ in range(len(readers) if cfg.decoder.memory_kv_per_layer else 1))
        self.inject_norm = RMSNorm(d, eps)
        self.injection = _Injection(d, lp.parcae_init_decay) if lp.injection == "parcae" else NoInjection()
        self.loop_embedding = nn.Parameter(torch.zeros(lp.t_max, d)) if lp.loop_embedding else None
        self.hyper_connections = StaticLanes(lp) if lp.hyper_connections == "static" else SingleState()
        self.decoder_layers = nn.ModuleList(DecoderLayer(cfg, kind, dec_scale) for kind in kinds)
        self.decoder_norm = RMSNorm(d, eps)
        self.readout_norms = nn.ModuleList(RMSNorm(d, eps) for _ in range(lp.t_max - 1))
        self.out_embed = None if cfg.tie_embeddings else nn.Embedding(cfg.vocab_size, d)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)) and not getattr(m, "own_init", False):
                nn.init.normal_(m.weight, mean=0.0, std=cfg.init_std)
        for layer in self.decoder_layers:
            if layer.depth_attention is not None:
                nn.init.zeros_(layer.depth_attention.out.weight)

    def head_weight(self) -> torch.Tensor:
        return self.embed.weight if self.out_embed is None else self.out_embed.weight

    lm_head_weight = head_weight

    def capacity(self, length: int) -> int:
        return decoder_capacity(length, self.cfg.decoder.capacity_fraction, self.cfg.decoder.capacity_multiple)

    def _head(self, hidden):
        wide = torch.promote_types(hidden.dtype, torch.float32)
        return F.linear(hidden.to(wide), self.head_weight().to(wide))

    def encode(self, tokens, doc_ids, dec_mask, capacity: int, cache) -> "Chunk":
        """The encoder over a chunk's positions, the aux head's input, the slots, the memory and the injected input. cache:
        anything with `seq`, `encoder` and `memory` of the earlier chunks (or None)."""
        ctx, seq_state = sequence_context(doc_ids, cache.seq if cache else None)
        h, enc_caches = self.encoder(self.embed_norm(self.embed(tokens)), ctx, cache.encoder if cache else None)
        slots = select_slots(dec_mask, capacity)
        memory = [KeySet.cat(cache.memory[i] if cache else None, mem(h, ctx, ~slots.kept)) for i, mem in enumerate(self.memory_kv)]
        at = SlotContext(idx=slots.take(ctx.idx, -1), doc=slots.take(ctx.doc, -1), pos=slots.take(ctx.pos, 0), valid=slots.valid)
        return Chunk(seq_state, enc_caches, memory, self.aux_norm(h), slots, at, self.inject_norm(slots.take(h)))

    def run_pass(self, k: int, chunk: "Chunk", Y, own_past: list | None, stacks: list | None = None):
        """Pass k of the shared block over the chunk's slots: (the lanes after it, this pass's cache entries by layer)."""
        lanes = self.hyper_connections
        z = lanes.read(Y, k)
        u = self.injection(z, chunk.e)
        if self.loop_embedding is not None:
            u = u + self.loop_embedding[k]
        entries = []
        for l, layer in enumerate(self.decoder_layers):
            mem = chunk.memory[self.memory_of[l]] if layer.kind == "memory_attention" else None
            u, entry = layer(u, chunk.at, mem, own_past[l] if own_past else None, k, depth=k * len(self.decoder_layers) + l,
                             stack=None if stacks is None else stacks[l])
            entries.append(entry)
        return lanes.write(Y, z, u, k), entries

    def slot_logits(self, Y, passes_done: int, T: int):
        """(B, C, V) from the lanes after `passes_done` passes: the decoder head's when all T ran, else that draft's."""
        norm = self.decoder_norm if passes_done == T else self.readout_norms[passes_done - 1]
        return self._head(norm(self.hyper_connections.finish(Y)))

    def forward(self, tokens, doc_ids, dec_mask, T: int | None = None, capacity: int | None = None, cache: LoopedCache | None = None,
                return_cache: bool = False, return_drafts: bool = False, return_hidden: bool = False) -> LoopedOutput:
        """tokens, doc_ids (B, L); dec_mask (B, L) bool, True where the position's next token is generated. capacity: the
        slots a row reserves (default the training capacity of L; prefill and cached steps pass L so nothing is dropped)."""
        cfg = self.cfg
        B, L = tokens.shape
        T = cfg.loop.t_eval if T is None else T
        if not 1 <= T <= cfg.loop.t_max:
            raise ValueError(f"T={T} outside 1 .. t_max = {cfg.loop.t_max}")
        if cache is not None and cache.T != T:
            raise ValueError(f"this cache was built at T = {cache.T}; a cached sequence keeps its pass count")
        capacity = self.capacity(L) if capacity is None else capacity
        routed = [layer.mlp for layer in self.decoder_layers if isinstance(layer.mlp, RoutedSwiGLU)]
        for mlp in routed:
            mlp.reset_stats()
        chunk = self.encode(tokens, doc_ids, dec_mask, capacity, cache)
        slots, aux_hidden, lanes = chunk.slots, chunk.aux_hidden, self.hyper_connections
        Y = lanes.start(chunk.e)
        stacks = [[] for _ in self.decoder_layers] if cfg.loop.depth_attention == "layer" else None
        own, drafts = [], []
        for k in range(T):
            Y, entries = self.run_pass(k, chunk, Y, cache.own[k] if cache else None, stacks)
            own.append(entries)
            if return_drafts and k < T - 1:
                drafts.append(self.readout_norms[k](lanes.finish(Y)))
        final = self.decoder_norm(lanes.finish(Y))
        seq_state, enc_caches, memory = chunk.seq_state, chunk.encoder, chunk.memory
        logits = None if return_hidden else slots.put(self._head(aux_hidden), self._head(final))
        aux_loss = None
        if routed:
            dec = cfg.decoder
            aux_loss = dec.moe_balance_weight * torch.stack([m.balance_loss() for m in routed]).mean()
            if dec.router_z_weight > 0:
                aux_loss = aux_loss + dec.router_z_weight * torch.stack([m.z_loss() for m in routed]).mean()
        new_cache = LoopedCache(seq_state, enc_caches, memory, own, T) if return_cache else None
        return LoopedOutput(logits=logits, kept=slots.kept, n_dropped=slots.n_dropped, cache=new_cache,
                            draft_logits=[self._head(x) for x in drafts] if return_drafts and not return_hidden else None,
                            slot_index=slots.index, slot_valid=slots.valid, aux_loss=aux_loss, hidden_aux=aux_hidden if return_hidden else None,
                            hidden_dec=final if return_hidden else None, hidden_drafts=drafts if return_drafts and return_hidden else None, slots=slots)

    @torch.no_grad()
    def prefill(self, tokens, doc_ids, dec_mask, T=None) -> LoopedOutput:
        return self.forward(tokens, doc_ids, dec_mask, T=T, capacity=tokens.shape[1], return_cache=True)

    @torch.no_grad()
    def extend(self, tokens, doc_ids, dec_mask, cache: LoopedCache) -> LoopedOutput:
        return self.forward(tokens, doc_ids, dec_mask, T=cache.T, capacity=tokens.shape[1], cache=cache, return_cache=True)

    @torch.no_grad()
    def generate(self, prompt, prompt_doc_ids, prompt_dec_mask, max_new_tokens: int, T=None, greedy: bool = True, generator=None):
        """(tokens (B, N), logits (B, N, V)): every generated token is fed back as a decoder position. The prompt ends at a
        decoder position (the assistant header)."""
        if not bool(prompt_dec_mask[:, -1].all()):
            raise ValueError("the prompt must end at a decoder position")
        out = self.prefill(prompt, prompt_doc_ids, prompt_dec_mask, T=T)
        doc, picked, seen = prompt_doc_ids[:, -1:], [], []
        for _ in range(max_new_tokens):
            step = out.logits[:, -1]
            tok = step.argmax(-1, keepdim=True) if greedy else torch.multinomial(step.softmax(-1), 1, generator=generator)
            picked.append(tok)
            seen.append(step)
            out = self.extend(tok, doc, torch.ones_like(tok, dtype=torch.bool), out.cache)
        if not picked:
            return prompt.new_empty(prompt.shape[0], 0), out.logits.new_empty(prompt.shape[0], 0, out.logits.shape[-1])
        return torch.cat(picked, dim=1), torch.stack(seen, dim=1)


def two_head_loss(model: LoopedCED, out: LoopedOutput, targets, valid, n_valid: float, n_dec: float, n_aux: float, z_loss: float = 0.0,
                  aux_weight: float = 1.0, normalization: str = "global_token_mean", draft_weight: float = 0.0, micro_share: float = 1.0):
    """(loss, sums) of a forward with return_hidden: the decoder head at the kept slots whose target counts, the aux head at
    the other positions whose target counts, each CE + z LSE^2; `global_token_mean` divides both by the batch's valid
    targets, `per_head_mean` each by its own count; the drafts add draft_weight x their CE over the decoder count; a routed
    FFN adds its balance term at the micro-batch's share."""
    from .cp_head import token_lse_zy

    W = model.head_weight()
    slots = out.slots
    lse_a, zy_a = token_lse_zy(out.hidden_aux, W, targets)
    t_slots = slots.take(targets, 0)
    on_dec = slots.take(valid, False) & slots.valid
    on_aux = valid & ~slots.kept
    lse_d, zy_d = token_lse_zy(out.hidden_dec, W, t_slots)
    term = lambda lse, zy, on: ((lse - zy + z_loss * lse * lse) * on.to(lse.dtype)).sum()       # noqa: E731
    sum_dec, sum_aux = term(lse_d, zy_d, on_dec), term(lse_a, zy_a, on_aux)
    if normalization == "global_token_mean":
        loss = (sum_dec + aux_weight * sum_aux) / n_valid
    elif normalization == "per_head_mean":
        loss = sum_dec / n_dec + aux_weight * sum_aux / n_aux
    else:
        raise ValueError(f"loss.normalization {normalization!r}: 'global_token_mean' or 'per_head_mean'")
    sums = {"ce_dec": ((lse_d - zy_d) * on_dec.to(lse_d.dtype)).sum().detach(), "ce_aux": ((lse_a - zy_a) * on_aux.to(lse_a.dtype)).sum().detach()}
    for i, hidden in enumerate(out.hidden_drafts or []):
        lse_k, zy_k = token_lse_zy(hidden, W, t_slots)
        d_sum = ((lse_k - zy_k) * on_dec.to(lse_k.dtype)).sum()
        loss = loss + draft_weight * d_sum / n_dec
        sums[f"ce_draft_loop{i + 1}"] = d_sum.detach()
    if out.aux_loss is not None:
        loss = loss + out.aux_loss * micro_share
        sums["moe_balance"] = out.aux_loss.detach() * micro_share
    return loss, sums
