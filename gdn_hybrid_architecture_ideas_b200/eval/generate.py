"""Greedy generation on the model's caches.

`generate_greedy`: one prompt at a time (chunked prefill, then one token per step). `generate_greedy_batched`:
prompts of different lengths in one batch, left-padded; the padding is a document of its own, so document isolation
keeps it out of every read; prefill runs in chunks; the head runs on the last position only; stop conditions are
checked on the host every `check_every` steps (reference: ced/eval/recall_ruler_gen.py:43-216).
"""

from __future__ import annotations

from typing import Callable

import torch

from ..models.hybrid import lm_head


def _last_logits(model, hidden_last: torch.Tensor) -> torch.Tensor:
    return lm_head(hidden_last, model.head_weight())


def _step(model, tokens, docs, cache, ac):
    """One cached forward: (cache, what the next token is read from at the last position). A model with a Copy-Paste head builds
    its cache in a forward that returns logits (log p of the mixture, over the copy cache); every other model hands the last
    hidden state to the head."""
    copy = getattr(model, "cp_head", None) is not None and model.cp_head.gated
    with torch.autocast(**ac):
        out = model.forward(tokens, docs, cache=cache, return_cache=True, return_hidden=not copy)
    return out.cache, (out.logits[:, -1:] if copy else out.hidden_aux[:, -1:]), copy


@torch.no_grad()
def generate_greedy(model, prompt: list[int], max_new: int, is_done: Callable[[int, list[int]], bool] | None = None,
                    eos_id: int | None = None, prefill_chunk: int = 1024, autocast_dtype=None) -> list[int]:
    return generate_greedy_batched(model, [prompt], max_new, is_done=is_done, eos_id=eos_id, prefill_chunk=prefill_chunk,
                                   autocast_dtype=autocast_dtype)[0]


@torch.no_grad()
def generate_greedy_batched(model, prompts: list[list[int]], max_new: int, is_done: Callable[[int, list[int]], bool] | None = None,
                            eos_id: int | None = None, pad_id: int = 0, prefill_chunk: int = 1024, check_every: int = 8,
                            autocast_dtype=None) -> list[list[int]]:
    dev = next(model.parameters()).device
    was_training = model.training
    model.eval()
    B, width = len(prompts), max(len(p) for p in prompts)
    tokens = torch.full((B, width), pad_id, dtype=torch.long)
    docs = torch.ones(B, width, dtype=torch.long)
    for b, p in enumerate(prompts):
        tokens[b, width - len(p):] = torch.tensor(p, dtype=torch.long)
        docs[b, :width - len(p)] = 0                       # the left padding is document 0, the prompt document 1
    tokens, docs = tokens.to(dev), docs.to(dev)
    cache, hidden = None, None
    ac = dict(device_type=dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None)
    copy = False
    for s in range(0, width, prefill_chunk):
        cache, hidden, copy = _step(model, tokens[:, s:s + prefill_chunk], docs[:, s:s + prefill_chunk], cache, ac)
    one = torch.ones(B, 1, dtype=torch.long, device=dev)
    generated = torch.zeros(B, max_new, dtype=torch.long, device=dev)
    done = [False] * B
    lengths = [max_new] * B
    for step in range(max_new):
        nxt = (hidden if copy else _last_logits(model, hidden)).argmax(-1)       # (B, 1)
        generated[:, step] = nxt[:, 0]
        if (step + 1) % check_every == 0 or step == max_new - 1:
            host = generated[:, :step + 1].cpu()
            for b in range(B):
                if done[b]:
                    continue
                seq = host[b].tolist()
                for n in range(max(0, step + 1 - check_every), step + 1):
                    if (eos_id is not None and seq[n] == eos_id) or (is_done is not None and is_done(b, seq[:n + 1])):
                        done[b], lengths[b] = True, n + 1
                        break
            if all(done):
                break
        if step + 1 < max_new:
            cache, hidden, copy = _step(model, nxt, one, cache, ac)
    model.train(was_training)
    host = generated.cpu()
    return [host[b, :lengths[b]].tolist() for b in range(B)]


@torch.no_grad()
def full_forward_argmax(model, ids: list[int], positions: list[int], autocast_dtype=None) -> list[int]:
    """Argmax of an uncached forward at the given positions (cross-check of cached generation)."""
    dev = next(model.parameters()).device
    tok = torch.tensor([ids], dtype=torch.long, device=dev)
    with torch.autocast(dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
        logits = model(tok, torch.zeros_like(tok)).logits
    return [int(logits[0, p].argmax()) for p in positions]
