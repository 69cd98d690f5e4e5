"""Multi-token-prediction drafter of depth 1 on a frozen trunk (`model.mtp.enabled`).

    h'_i = M [ RMSNorm_h(h_i) ; RMSNorm_e(Emb(t_{i+1})) ]        M: (d, 2d), no bias ("eh_proj")
    y_i  = Block(h'_1 .. h'_i)                                    one causal gated-attention encoder layer
    p_i  = softmax(head(RMSNorm_o(y_i)))                          the distribution of t_{i+2}

h_i is the trunk's head input (after its final norm), Emb the trunk's own input embedding (its raw rows) and `head` the
trunk's own output matrix: both shared and frozen. The head's tensors live under `mtp.` in the state dict and are drawn
after every trunk tensor, so the trunk starts as the model without the key. `HybridLM.forward` never calls the head
(reference: ced/model/mtp.py:1-230; its trainer refuses the key and trains the head with the trunk frozen, which is
what `train_step` below does; a depth-k draft applies the head again on its own output).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ..config import ModelConfig
from .encoder import EncoderLayer, residual_scale
from .hybrid import lm_head
from .linear import Linear
from .norms import RMSNorm
from .sequence import SeqContext, sequence_context

PREFIX = "mtp."
MTP_TRUNKS = ("none", "block_entry")


def check_mtp(cfg: ModelConfig) -> None:
    """Refuse the drafter where it is not built (reference: ced/model/mtp.py:70-116)."""
    m, e = cfg.mtp, cfg.encoder
    if type(m.enabled) is not bool:
        raise ValueError(f"model.mtp.enabled {m.enabled!r}: true or false")
    if m.block != "attention":
        raise ValueError(f"model.mtp.block {m.block!r}: 'attention'")
    if not m.enabled:
        return
    if e.canon_kernel:
        raise ValueError("model.mtp is not built together with model.encoder.canon_kernel")
    if e.attn_res not in MTP_TRUNKS:
        raise ValueError(f"model.mtp is built on model.encoder.attn_res in {MTP_TRUNKS}")
    if e.attn_res == "block_entry" and e.gdn_write_mix != "none":
        raise ValueError("model.mtp on a depth-mixing trunk is built for its own form only: model.encoder.gdn_write_mix 'none'")
    if e.layer_scalars != "none":
        raise ValueError("model.mtp is not built together with model.encoder.layer_scalars")
    if cfg.nvfp4.mode != "none" or cfg.fp8.mode != "none":
        raise ValueError("model.mtp is not built together with model.nvfp4 / model.fp8 (the head trains on a frozen bf16 trunk)")


class MTPHead(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        d, eps = cfg.d_model, cfg.norm_eps
        self.hnorm = RMSNorm(d, eps)
        self.enorm = RMSNorm(d, eps)
        self.eh_proj = Linear(2 * d, d)
        self.block = EncoderLayer("attention", cfg, residual_scale(cfg), cfg.encoder.attention)
        self.out_norm = RMSNorm(d, eps)

    def forward(self, hidden: torch.Tensor, next_tokens: torch.Tensor, embed: nn.Embedding, ctx: SeqContext, cache=None):
        """hidden (B, L, d): the trunk's head input at positions i (or the head's own output of the position before, at a
        deeper draft); next_tokens (B, L): t_{i+1}. Returns (y (B, L, d), the block's key set including these positions)."""
        e = embed(next_tokens)
        u = self.eh_proj(torch.cat([self.hnorm(hidden), self.enorm(e)], dim=-1).to(hidden.dtype)).to(hidden.dtype)
        return self.block(u, ctx, cache)


def attach_mtp(model: nn.Module) -> nn.Module:
    """model.mtp = a new head, N(0, init_std) on its linear weights, drawn after every trunk tensor."""
    head = MTPHead(model.cfg)
    for m in head.modules():
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, mean=0.0, std=model.cfg.init_std)
    model.mtp = head
    return model


def freeze_trunk(model: nn.Module) -> list[nn.Parameter]:
    """requires_grad False on every trunk tensor, True on the head's; returns the head's parameters."""
    if getattr(model, "mtp", None) is None:
        raise ValueError("the model has no MTP head (model.mtp.enabled)")
    head = []
    for name, p in model.named_parameters():
        own = name.startswith(PREFIX)
        p.requires_grad_(own)
        if own:
            head.append(p)
    return head


def assert_trunk_frozen(model: nn.Module) -> None:
    for name, p in model.named_parameters():
        if not name.startswith(PREFIX):
            assert not p.requires_grad and p.grad is None, f"trunk tensor {name} requires or holds a gradient"


def mtp_targets(targets: torch.Tensor, target_valid: torch.Tensor):
    """(B, L) data targets t_{i+1} and validity -> the head's targets t_{i+2} and validity (t_{i+1} and t_{i+2} both
    continue position i's document; the row's last position has none)."""
    t2 = torch.cat([targets[:, 1:], torch.zeros_like(targets[:, :1])], dim=1)
    v2 = torch.cat([target_valid[:, :-1] & target_valid[:, 1:], torch.zeros_like(target_valid[:, :1])], dim=1)
    return t2, v2


@torch.no_grad()
def trunk_hidden(model: nn.Module, tokens: torch.Tensor, doc_ids: torch.Tensor, cache=None, return_cache: bool = False):
    out = model(tokens, doc_ids, cache=cache, return_cache=return_cache, return_hidden=True)
    return (out.hidden_aux, out.cache) if return_cache else out.hidden_aux


def mtp_loss(model: nn.Module, tokens: torch.Tensor, doc_ids: torch.Tensor, targets: torch.Tensor, target_valid: torch.Tensor):
    """(mean CE of t_{i+2} over valid positions, top-1 accuracy of the draft, number of valid positions). The trunk runs
    without a gradient; the head reads (h_i, t_{i+1}) with t_{i+1} = targets."""
    hidden = trunk_hidden(model, tokens, doc_ids)
    ctx, _ = sequence_context(doc_ids)
    t2, v2 = mtp_targets(targets, target_valid)
    y, _ = model.mtp(hidden.detach(), targets.clamp_min(0), model.embed, ctx)
    logits = lm_head(model.mtp.out_norm(y), model.head_weight().detach())
    ce = torch.nn.functional.cross_entropy(logits.flatten(0, 1), t2.flatten(), reduction="none")
    w = v2.flatten().to(ce.dtype)
    n = w.sum().clamp_min(1.0)
    acc = ((logits.argmax(-1) == t2) & v2).sum() / n
    return (ce * w).sum() / n, acc, int(v2.sum())


def train_step(model: nn.Module, optimizer: torch.optim.Optimizer, tokens, doc_ids, targets, target_valid) -> dict:
    """One optimizer step of the head on a frozen trunk."""
    assert_trunk_frozen(model)
    optimizer.zero_grad(set_to_none=True)
    loss, acc, n = mtp_loss(model, tokens, doc_ids, targets, target_valid)
    loss.backward()
    optimizer.step()
    return {"loss": float(loss.detach()), "draft_accuracy": float(acc), "positions": n}


@torch.no_grad()
def draft(model: nn.Module, hidden_last: torch.Tensor, next_token: torch.Tensor, ctx: SeqContext, depth: int = 1, cache=None):
    """Greedy drafts of t_{i+2} .. t_{i+1+depth} from the trunk's last head input (B, 1, d) and the verified t_{i+1}
    (B, 1): the head is applied again on its own output for depth > 1. Returns (drafted tokens (B, depth), key set)."""
    out, h, t = [], hidden_last, next_token
    for k in range(depth):
        step_ctx = ctx if k == 0 else SeqContext(idx=ctx.idx + k, doc=ctx.doc, pos=ctx.pos + k, is_doc_start=torch.zeros_like(ctx.is_doc_start))
        y, cache = model.mtp(h, t, model.embed, step_ctx, cache)
        t = lm_head(model.mtp.out_norm(y), model.head_weight()).argmax(-1)
        out.append(t)
        h = y
    return torch.cat(out, dim=1), cache
