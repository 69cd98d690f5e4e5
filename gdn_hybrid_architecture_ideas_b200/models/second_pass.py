"""The gated second pass of the plain hybrid stack (`model.loop.pass2_gate: scalar`, `pass2_layers` n, T = 2).

    z_1 = Stack(embed(x))                      pass 1: the single-pass model at every position
    s_2 = Block(z_1 + e_2)                     pass 2: the top n layers again, WRITING NOTHING
    z_2 = z_1 + alpha (s_2 - z_1)              alpha one trained scalar, e_2 a (d,) embedding; both start at 0
    logits = Head(RMSNorm_final(z_2))

In pass 2 a layer is the same layer (weights, norms, residual scale) in read-only mode:
  * a global-attention layer puts pass 2's own query at t (rotary at t's document position, the temperature's key count
    pos_t + 1) over THAT layer's pass-1 keys and values at s <= t of t's document. No key or value is projected.
  * a GDN layer reads the state pass 1 left after t (t's own write included) with pass 2's query, whose short convolution
    reads pass 1's inputs at t-K+1 .. t-1 and pass 2's at t. That read is one more call of the delta rule over pass 1's
    k, v, g, beta with q = q_2, so on a GPU it is the layer's own kernel. No key, value, gate or state is formed.
Nothing of pass 2 enters the cache: the cache of a chunk is pass 1's whatever T, and read tokens need one pass. The
output at t depends on pass-1 quantities at s <= t and on z_1(t) alone, never on which other positions run pass 2. So
where a mask names the positions whose next token is generated (`pass2_mask`, with `pass2_capacity` slots a row), pass 2
is computed at every position of the chunk and kept at the first `capacity` marked ones (the same values as a gather
into slots, with fixed shapes); `kept` / `n_dropped` say where it ran and how many marked positions had no slot. Pass 1's
records are not detached: pass 2's loss trains pass 1's keys, values and states.

New tensors: `hyper_connections.pass2_gate` (alpha, 0-dim) and, with `loop.loop_embedding`, `loop_embedding_pass2` (d);
a T = 1 checkpoint of the same stack loads into the rest. Reference: ced/model/control.py:19-54 (definition), :201-242
(refusals), :511-560 (the pass), ced/model/encoder.py:349-400 (read-only layers), ced/model/gdn.py:851-975 (the GDN read),
ced/model/loop.py:312-352 (the gate). Pass counts by segment (`loop.segment_passes` / `unscored_passes`, a third pass):
models/pass_counts.py gives the counts, `scheduled_passes` here runs them.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from . import act_checkpoint

PASS2_PARAMETERS = ("loop_embedding_pass2", "hyper_connections.pass2_gate", "loop_embedding_pass3", "hyper_connections.pass3_gate")


def is_on(cfg) -> bool:
    return cfg.loop.pass2_gate != "none"


def check_config(cfg) -> None:
    lc, e = cfg.loop, cfg.encoder
    from .pass_counts import schedule_of

    if schedule_of(lc) is not None and not is_on(cfg):
        raise ValueError("model.loop.segment_passes / unscored_passes set the passes of a gated second pass (model.loop.pass2_gate 'scalar'): this model has none")
    if not is_on(cfg):
        if lc.pass2_layers:
            raise ValueError(f"model.loop.pass2_layers {lc.pass2_layers!r} without loop.pass2_gate 'scalar': set both, or leave pass2_layers 0")
        return
    if lc.pass2_gate != "scalar":
        raise ValueError(f"model.loop.pass2_gate {lc.pass2_gate!r}: 'none' or 'scalar' (this stack has no hyper-connection lanes, so the 'hc' form does not exist for it)")
    n = e.n_layers
    if type(lc.pass2_layers) is not int or not 1 <= lc.pass2_layers <= n:
        raise ValueError(f"model.loop.pass2_layers {lc.pass2_layers!r}: the number of top layers the second pass runs through, 1 .. {n}")
    if lc.t_max != 2:
        raise ValueError(f"model.loop.pass2_gate is built for T = 2 (loop.t_max = 2), not t_max = {lc.t_max}")
    if lc.t_eval not in (1, 2):
        raise ValueError(f"model.loop.t_eval {lc.t_eval!r}: 1 or 2 for a stack with a second pass")
    refused = [(bool(lc.recur_layers), "loop.recur_layers (the looped middle is the other loop: set one)"),
               (e.attn_res != "none", f"encoder.attn_res {e.attn_res!r} (a read-only layer call would add to a block's sum)"),
               (e.gdn_write_mix != "none" or bool(e.gdn_ccr_spacing), "encoder.gdn_write_mix / gdn_ccr_spacing"),
               (e.layer_scalars != "none", "encoder.layer_scalars"), (bool(e.canon_kernel), "encoder.canon_kernel"),
               (bool(e.nope_global_layers), "encoder.nope_global_layers"), (bool(e.gdn_shape_by_layer), "encoder.gdn_shape_by_layer"),
               (e.attention.normalizer != "softmax", f"attention.normalizer {e.attention.normalizer!r}"),
               (e.attention.kv_sharing != "gqa", f"attention.kv_sharing {e.attention.kv_sharing!r}"),
               (e.gdn.kda.decay != "scalar" or e.gdn.erase.mode != "none" or e.gdn.dprod.n_h != 1, "gdn.kda.decay 'channel' / gdn.erase.mode 'eda' / gdn.dprod.n_h >= 2"),
               (cfg.nvfp4.mode != "none" or cfg.fp8.mode != "none", "model.nvfp4 / model.fp8 (pass 2 applies the q rows of a GDN in-projection directly)"),
               (bool(cfg.mtp.enabled), "model.mtp")]
    bad = [why for cond, why in refused if cond]
    if bad:
        raise ValueError(f"model.loop.pass2_gate 'scalar' is not built with: {'; '.join(bad)}")


class SecondPassGate(nn.Module):
    """z_2 = z_1 + alpha (s_2 - z_1): a multiply and two sums in the stream's dtype, so alpha = 0 gives z_1 exactly; alpha gets a
    gradient at once, the block's pass-2 path exactly zero until alpha moves."""

    def __init__(self, n_passes: int = 2):
        super().__init__()
        self.n_passes = n_passes
        self.pass2_gate = nn.Parameter(torch.zeros(()))
        if n_passes == 3:          # only through a 3 in model.loop.segment_passes
            self.pass3_gate = nn.Parameter(torch.zeros(()))

    def forward(self, z: torch.Tensor, s: torch.Tensor, k: int = 1) -> torch.Tensor:
        """The state after the pass with 0-based index k from the state before it (z) and the block's output (s)."""
        gate = self.pass2_gate if k == 1 else self.pass3_gate
        return z + gate.to(z.dtype) * (s - z)

    @torch.no_grad()
    def is_identity(self) -> bool:
        return bool(self.pass2_gate == 0) and (self.n_passes < 3 or bool(self.pass3_gate == 0))


@dataclass
class GDNPass1:
    """What a GDN layer's pass 1 leaves for a read-only second pass. q_inputs (B, K-1+L, H_k d_k): the q channels before
    the convolution over [history ; chunk]; q_docs (B, K-1+L) their documents; the rest: the delta rule's inputs."""

    q_inputs: torch.Tensor
    q_docs: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    g: torch.Tensor
    beta: torch.Tensor
    is_doc_start: torch.Tensor
    S0: torch.Tensor | None


def gdn_forward_keep(mixer, x, ctx, state):
    """The GDN layer's forward (the plain scalar-decay layer) that also returns its record: (y, GDNState, GDNPass1)."""
    from .gdn import GDNState

    cfg = mixer.cfg
    B, L = ctx.doc.shape
    hk, hv, dk, dv, K = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim, cfg.conv_kernel
    u_pre = mixer.in_proj_qkv(x)
    hist, hist_doc = (None, None) if state is None else (state.conv_input, state.conv_doc)
    q, k, v, conv_input, conv_doc = ops.gdn_prep(u_pre, ctx.doc, mixer.conv_weight, hk, hv, dk, dv, hist, hist_doc, single_doc=ctx.single_doc)
    g, beta = ops.gdn_gates(mixer.in_proj_a(x), mixer.in_proj_b(x), mixer.A_log, mixer.dt_bias)
    if mixer.beta_max != 1:
        beta = beta * mixer.beta_max
    S0 = None if state is None else state.S
    kernel = "recurrence" if cfg.kernel == "recurrence" else "chunked"
    o, S = ops.delta_rule(q, k, v, g, beta, ctx.is_doc_start, S0, kernel=kernel, chunk_size=cfg.chunk_size)
    z = mixer.in_proj_z(x).view(B, L, hv, dv)
    y = mixer.out_proj(mixer.norm(o, z).flatten(2))
    nq = hk * dk
    past = u_pre.new_zeros(B, K - 1, nq) if hist is None else hist[..., :nq].to(u_pre.dtype)
    past_doc = torch.full((B, K - 1), -1, dtype=ctx.doc.dtype, device=ctx.doc.device) if hist_doc is None else hist_doc
    rec = GDNPass1(q_inputs=torch.cat([past, u_pre[..., :nq]], dim=1), q_docs=torch.cat([past_doc, ctx.doc], dim=1), k=k, v=v, g=g, beta=beta,
                   is_doc_start=ctx.is_doc_start, S0=S0)
    return y, GDNState(conv_input=conv_input, conv_doc=conv_doc, S=S), rec


def gdn_read_all(mixer, x, doc, rec: GDNPass1) -> torch.Tensor:
    """The read-only GDN layer at every position: o2_t = S1_t^T q2_t through one more delta-rule call with q = q2."""
    cfg = mixer.cfg
    B, L, _ = x.shape
    hk, hv, dk, dv, K = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim, cfg.conv_kernel
    nq = hk * dk
    w = mixer.conv_weight[:nq].to(x.dtype)
    out = F.linear(x, mixer.in_proj_qkv.weight[:nq].to(x.dtype)) * w[:, K - 1]      # tap 0: pass 2's own input
    for j in range(1, K):                                                            # tap j looks j steps back, into pass 1's inputs
        s = K - 1 - j
        same = (rec.q_docs[:, s:s + L] == doc).to(x.dtype)
        out = out + rec.q_inputs[:, s:s + L].to(x.dtype) * same[..., None] * w[:, K - 1 - j]
    q2 = (ops.ref.l2_normalize(F.silu(out).view(B, L, hk, dk)) * dk ** -0.5).to(rec.k.dtype)
    kernel = "recurrence" if cfg.kernel == "recurrence" else "chunked"
    o2, _ = ops.delta_rule(q2, rec.k, rec.v, rec.g, rec.beta, rec.is_doc_start, rec.S0, kernel=kernel, chunk_size=cfg.chunk_size, need_state=False)
    z2 = mixer.in_proj_z(x).view(B, L, hv, dv)
    return mixer.out_proj(mixer.norm(o2, z2).flatten(2))


def attention_read(mixer, x, ctx, keys) -> torch.Tensor:
    """Pass 2's queries over the layer's pass-1 key set (this chunk's and the cache's): the causal and document mask, the rotary
    positions and the temperature's key counts are pass 1's."""
    rot_pos = ctx.pos
    q, q_far, gate = mixer.queries(x, rot_pos, ctx.pos)
    aligned = keys.k.shape[1] == x.shape[1]          # no cache: queries and keys are the same positions, the training kernel's case
    o = ops.attention(q, keys.k, keys.v, ctx.idx, ctx.doc, keys.idx, keys.doc, None if aligned else keys.ok, q_far=q_far, k_far=keys.k_far,
                      cap=mixer.cap, self_aligned=aligned, q_pos=ctx.pos, single_doc=ctx.single_doc and aligned)
    return mixer.output(o, gate)


def layer_read_all(layer, x, ctx, record) -> torch.Tensor:
    """One layer in read-only mode at every position of the chunk."""
    h = layer.mixer_in_norm(x)
    mixed = gdn_read_all(layer.mixer, h, ctx.doc, record) if layer.kind == "gdn" else attention_read(layer.mixer, h, ctx, record)
    x = x + layer.residual_scale * layer.mixer_out_norm(mixed, out_dtype=x.dtype)
    return x + layer.residual_scale * layer.mlp_out_norm(layer.mlp(layer.mlp_in_norm(x)), out_dtype=x.dtype)


def select_kept(mask: torch.Tensor, capacity: int | None):
    """(kept (B, L): the first `capacity` marked positions of each row, n_dropped (B,): the marked positions without a slot)."""
    if capacity is None:
        return mask, torch.zeros(mask.shape[0], dtype=torch.long, device=mask.device)
    rank = mask.long().cumsum(1)
    kept = mask & (rank <= capacity)
    return kept, (mask.long().sum(1) - kept.long().sum(1))


def loop_usage(z1, z, kept) -> torch.Tensor:
    """The mean over the positions where pass 2 ran of ||z_2 - z_1|| / ||z_2|| (0 when it ran nowhere)."""
    num = torch.linalg.vector_norm((z - z1).float(), dim=-1)
    den = torch.linalg.vector_norm(z.float(), dim=-1).clamp_min(1e-20)
    k = kept.to(num.dtype)
    return ((num / den) * k).sum() / k.sum().clamp_min(1.0)


def block_read_all(model, u, ctx, records: list, checkpoint: bool):
    """The top block's layers in read-only mode at every position, from the stream u."""
    block = list(model.encoder.layers)[model.pass2_from:]
    for layer, record in zip(block, records):
        if checkpoint:
            flat, rebuild = _flatten(record)
            u = act_checkpoint.run_checkpointed(lambda u_, *t, layer=layer, rebuild=rebuild: layer_read_all(layer, u_, ctx, rebuild(t)), u, *flat)
        else:
            u = layer_read_all(layer, u, ctx, record)
    return u


def scheduled_passes(model, z1, ctx, records: list, counts: torch.Tensor, max_count: int, checkpoint: bool):
    """(z, kept): every position's state after the LAST pass its count asks for (models/pass_counts.py). counts (B, L) integer
    on z1's device; max_count: its largest value, known on the host (a pass no position runs is not computed)."""
    z = z1
    for k in range(1, min(max_count, model.hyper_connections.n_passes)):
        e = getattr(model, f"loop_embedding_pass{k + 1}", None)
        s = block_read_all(model, z if e is None else z + e.to(z.dtype), ctx, records, checkpoint)
        z = torch.where((counts > k)[..., None], model.hyper_connections(z, s, k), z)
    return z, counts >= 2


def second_pass(model, z1, ctx, records: list, pass2_mask, capacity, checkpoint: bool):
    """(z, kept, n_dropped): z_2 where pass 2 is kept and z_1 elsewhere."""
    B, L, _ = z1.shape
    e2 = getattr(model, "loop_embedding_pass2", None)
    u = block_read_all(model, z1 if e2 is None else z1 + e2.to(z1.dtype), ctx, records, checkpoint)
    z2 = model.hyper_connections(z1, u)
    if pass2_mask is None:
        return z2, torch.ones(B, L, dtype=torch.bool, device=z1.device), torch.zeros(B, dtype=torch.long, device=z1.device)
    kept, n_dropped = select_kept(pass2_mask.bool(), capacity)
    return torch.where(kept[..., None], z2, z1), kept, n_dropped


def _flatten(record):
    """A record as a tuple of tensors (a checkpointed call's inputs) and the function that puts it back together."""
    import dataclasses

    names = [f.name for f in dataclasses.fields(record)]
    values = [getattr(record, n) for n in names]
    return tuple(values), (lambda t, cls=type(record), names=names: cls(**dict(zip(names, t))))
