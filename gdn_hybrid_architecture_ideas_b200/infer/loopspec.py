"""LoopSpec: greedy speculative decoding of the looped encoder-decoder at T = 2 from its own first pass.

The readout after pass 1 at position p (the model's draft head) proposes the token at p + 1 before pass 2 has run. One
pipeline step then does, for the committed position p and the proposed p + 1,

    pass 2 at p          -> the target's greedy token at p + 1                      (needs nothing of p + 1)
    encoder + pass 1 at p + 1 with the proposed token -> the next proposal

and compares: equal, the proposal is committed and the work at p + 1 stands; different, the work at p + 1 is dropped, the
target's token is committed and its encoder + pass 1 run again (a bubble). Every committed token is the target's greedy
token, so the output is exactly `LoopedCED.generate(..., T=2, greedy=True)`; what changes is that the two halves of a step
are independent and can run side by side (two rows of one decoder pass on a GPU). The caches here are the model's
functional ones (a chunk's entries are concatenated into new tensors), so dropping the work at p + 1 is keeping the old
references: nothing is copied or restored. One row at a time.
Reference: ced/infer/engine.py:677-741 (there on the engine's static buffers, with a snapshot and restore).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..models.looped_decoder import Chunk, LoopedCED


@dataclass
class SpecStats:
    steps: int = 0
    accepted: int = 0
    flags: list = field(default_factory=list)

    @property
    def acceptance(self) -> float:
        return self.accepted / max(self.steps, 1)


@dataclass
class _Front:
    """The encoder-side caches up to and including a position, pass 1's own entries up to it, the position's chunk, its lanes
    after pass 1 and the token its draft head proposes next."""

    base: Chunk
    own_first: list
    lanes: torch.Tensor
    proposal: int


class LoopSpec:
    def __init__(self, model: LoopedCED):
        if model.cfg.arch != "looped_ced" or model.cfg.loop.t_max < 2:
            raise ValueError("LoopSpec drafts from the first pass of a looped encoder-decoder with t_max >= 2")
        if model.cfg.loop.depth_attention != "none":
            raise ValueError("LoopSpec is not built with model.loop.depth_attention (a position's depth stack spans both passes)")
        self.model, self.T, self.stats = model, 2, SpecStats()

    def _advance(self, token: int, doc: torch.Tensor, behind, own_first: list) -> _Front:
        """Encoder and pass 1 for one committed or proposed token after the caches `behind`."""
        m = self.model
        tok = torch.tensor([[token]], device=doc.device)
        chunk = m.encode(tok, doc, torch.ones_like(tok, dtype=torch.bool), 1, behind)
        lanes, entries = m.run_pass(0, chunk, m.hyper_connections.start(chunk.e), own_first)
        return _Front(chunk, entries, lanes, int(m.slot_logits(lanes, 1, self.T)[0, -1].argmax()))

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, doc_ids: torch.Tensor, dec_mask: torch.Tensor, max_new_tokens: int) -> tuple[list, SpecStats]:
        """prompt, doc_ids, dec_mask (1, P), the last position a decoder position. Returns (tokens, statistics)."""
        m = self.model
        if prompt.shape[0] != 1 or not bool(dec_mask[0, -1]):
            raise ValueError("LoopSpec decodes one row whose prompt ends at a decoder position")
        self.stats = SpecStats()
        if max_new_tokens < 1:
            return [], self.stats
        start = m.prefill(prompt, doc_ids, dec_mask, T=self.T)
        out = [int(start.logits[0, -1].argmax())]               # the first token comes straight from the target
        doc = doc_ids[:, -1:]
        own_second = start.cache.own[1]
        front = self._advance(out[0], doc, start.cache, start.cache.own[0])
        while len(out) < max_new_tokens:
            ahead = self._advance(front.proposal, doc, front.base, front.own_first)                  # encoder + pass 1 at the next position
            lanes, own_second = m.run_pass(1, front.base, front.lanes, own_second)                    # pass 2 at this one
            target = int(m.slot_logits(lanes, 2, self.T)[0, -1].argmax())
            hit = target == front.proposal
            self.stats.steps += 1
            self.stats.accepted += int(hit)
            self.stats.flags.append(hit)
            out.append(target)
            front = ahead if hit else self._advance(target, doc, front.base, front.own_first)        # a miss: the work ahead is dropped
        return out, self.stats
