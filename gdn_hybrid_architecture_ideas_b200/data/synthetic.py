"""Deterministic synthetic batches: every batch is a pure function of (seed, step, row), so a resume needs only the
step counter and a data-parallel rank's rows are the single process's rows of the same index
(reference: ced/train/data.py:21-72, 147-202).

Two generators: `SyntheticPackedData` packs short documents drawn from a fixed first-order Markov chain (something a
small model can learn), `UniformTokens` draws token ids uniformly (one document per row), which is the shape the
throughput benchmarks name. Both build rows with vectorised tensor ops so data never bounds a step.
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass

import torch

from ..config import DataConfig


@dataclass
class Batch:
    tokens: torch.Tensor          # (B, L) inputs, or (B, L, s) bags
    targets: torch.Tensor         # (B, L) next tokens
    target_valid: torch.Tensor    # (B, L) bool; False where the target belongs to the next document
    doc_ids: torch.Tensor         # (B, L) increasing along the row
    dec_mask: torch.Tensor | None = None
    multi_targets: torch.Tensor | None = None   # (B, L, s) bag targets (token-superposition training)
    multi_valid: torch.Tensor | None = None
    loss_mask: torch.Tensor | None = None
    single_doc: bool = False      # host-known: every row is one document

    def pin(self) -> "Batch":
        for name in ("tokens", "targets", "target_valid", "doc_ids", "dec_mask", "multi_targets", "multi_valid", "loss_mask"):
            t = getattr(self, name)
            if isinstance(t, torch.Tensor) and not t.is_pinned() and torch.cuda.is_available():
                setattr(self, name, t.pin_memory())
        return self

    def to(self, device, non_blocking: bool = True) -> "Batch":
        moved = {}
        for name in ("tokens", "targets", "target_valid", "doc_ids", "dec_mask", "multi_targets", "multi_valid", "loss_mask"):
            t = getattr(self, name)
            moved[name] = t.to(device, non_blocking=non_blocking) if isinstance(t, torch.Tensor) else t
        return Batch(single_doc=self.single_doc, **moved)

    _TENSORS = ("tokens", "targets", "target_valid", "doc_ids", "dec_mask", "multi_targets", "multi_valid", "loss_mask")

    def clone_static(self) -> "Batch":
        """A copy on fixed buffers (CUDA-graph replay reads its inputs from them)."""
        got = {n: (getattr(self, n).clone() if isinstance(getattr(self, n), torch.Tensor) else getattr(self, n)) for n in self._TENSORS}
        return Batch(single_doc=self.single_doc, **got)

    def copy_from(self, other: "Batch") -> None:
        for n in self._TENSORS:
            mine, theirs = getattr(self, n), getattr(other, n)
            if isinstance(mine, torch.Tensor):
                mine.copy_(theirs, non_blocking=True)

    def h2d_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.tokens, self.targets, self.target_valid, self.doc_ids, self.loss_mask)
                   if isinstance(t, torch.Tensor))


def short_rows(data, first: int, count: int, length: int, full_length: int) -> Batch:
    """Rows first .. first + count - 1 of the run's rows cut to `length` tokens (batch-shape schedules): base row g of
    full_length tokens is cut into full_length / length consecutive pieces, piece j holding its tokens [j length, j length +
    length] (inputs and the last one's target), so short row i is piece i % n of base row i // n. A piece that starts
    inside a document keeps the document (its ids are re-based to start at 0 for the row)."""
    if length == full_length:
        return data.rows(first, count)
    n = full_length // length
    g0, g1 = first // n, (first + count - 1) // n
    base = data.rows(g0, g1 - g0 + 1)
    seq = torch.cat([base.tokens, base.targets[:, -1:]], dim=1)
    last_doc = torch.where(base.target_valid[:, -1], base.doc_ids[:, -1], base.doc_ids[:, -1] + 1)
    docs = torch.cat([base.doc_ids, last_doc[:, None]], dim=1)
    toks, dcs = [], []
    for i in range(first, first + count):
        r, j = i // n - g0, i % n
        toks.append(seq[r, j * length: j * length + length + 1])
        d = docs[r, j * length: j * length + length + 1]
        dcs.append(d - d[0])
    t, d = torch.stack(toks), torch.stack(dcs)
    return Batch(tokens=t[:, :-1].contiguous(), targets=t[:, 1:].contiguous(), target_valid=(d[:, 1:] == d[:, :-1]).contiguous(),
                 doc_ids=d[:, :-1].contiguous(), single_doc=base.single_doc)


def counter_generator(seed: int, step: int, stream: int) -> torch.Generator:
    """Generator seeded from blake2b("seed:step:stream"): counter-based randomness, distinct triples never alias."""
    digest = hashlib.blake2b(f"{seed}:{step}:{stream}".encode(), digest_size=8).digest()
    g = torch.Generator()
    g.manual_seed(int.from_bytes(digest, "little") & (2 ** 63 - 1))
    return g


class SyntheticPackedData:
    """Rows of seq_len + 1 tokens packed with documents of doc_len_min .. doc_len_max tokens; inside a document a
    token follows its predecessor through one of 4 fixed successors with probability 0.8, else is uniform."""

    def __init__(self, cfg: DataConfig, vocab_size: int, capacity: int | None = None):
        """capacity: decoder positions a row marks in spans (the looped encoder-decoder; data/spans.py), None for no mask."""
        self.cfg = cfg
        self.vocab_size = vocab_size
        self.capacity = capacity
        g = counter_generator(cfg.seed, -1, 0)
        self.successors = torch.randint(0, vocab_size, (vocab_size, 4), generator=g)

    def _spans(self, g: torch.Generator) -> torch.Tensor:
        from .spans import sample_spans

        c = self.cfg
        return sample_spans(c.seq_len, self.capacity, g, distribution=c.span_distribution, median=c.span_median, sigma=c.span_sigma,
                            span_min=c.span_min, span_max=c.span_max)

    def _row(self, g: torch.Generator):
        c, n = self.cfg, self.cfg.seq_len + 1
        lengths = torch.randint(c.doc_len_min, c.doc_len_max + 1, (n,), generator=g)
        ends = lengths.cumsum(0)
        docs = torch.searchsorted(ends, torch.arange(n), right=True)
        starts = torch.ones(n, dtype=torch.bool)
        starts[1:] = docs[1:] != docs[:-1]
        follow = (torch.rand(n, generator=g) < 0.8) & ~starts
        which = torch.randint(0, 4, (n,), generator=g)
        uniform = torch.randint(0, self.vocab_size, (n,), generator=g)
        tokens = uniform.clone()
        # A run of "follow" positions is a chain from the last non-follow token: resolve by doubling is not possible
        # for a table lookup, so walk the (few) maximal runs with a vectorised step per offset inside runs.
        run_id = (~follow).cumsum(0)
        offset = torch.arange(n) - torch.zeros(n, dtype=torch.long).scatter_reduce(
            0, run_id, torch.arange(n), reduce="amin", include_self=False)[run_id]
        for k in range(1, int(offset.max()) + 1):
            at = (offset == k).nonzero(as_tuple=True)[0]
            tokens[at] = self.successors[tokens[at - 1], which[at]]
        return tokens, docs

    def batch(self, step: int, first: int = 0, count: int | None = None) -> Batch:
        B = self.cfg.batch_size
        return self.rows(step * B + first, B - first if count is None else count)

    def rows(self, first: int, count: int) -> Batch:
        """Base rows first .. first + count - 1 of the run's row sequence (row g is row g % B of step g // B)."""
        B = self.cfg.batch_size
        rows = [self._row(counter_generator(self.cfg.seed, g // B, 1000 + g % B)) for g in range(first, first + count)]
        seq = torch.stack([r[0] for r in rows])
        docs = torch.stack([r[1] for r in rows])
        dec = None
        if self.capacity is not None:        # a generator of the row's own, apart from its tokens'
            dec = torch.stack([self._spans(counter_generator(self.cfg.seed, g // B, 2000 + g % B)) for g in range(first, first + count)])
        return Batch(tokens=seq[:, :-1].contiguous(), targets=seq[:, 1:].contiguous(),
                     target_valid=(docs[:, 1:] == docs[:, :-1]).contiguous(), doc_ids=docs[:, :-1].contiguous(), dec_mask=dec,
                     single_doc=self.cfg.doc_len_min > self.cfg.seq_len)


class UniformTokens:
    """Token ids uniform on [0, vocab), one document per row (data.kind "uniform"): the synthetic shape of the
    throughput benchmarks."""

    def __init__(self, cfg: DataConfig, vocab_size: int):
        self.cfg, self.vocab_size = cfg, vocab_size

    def batch(self, step: int, first: int = 0, count: int | None = None) -> Batch:
        B = self.cfg.batch_size
        return self.rows(step * B + first, B - first if count is None else count)

    def rows(self, first: int, count: int) -> Batch:
        """Base rows first .. first + count - 1 of the run's row sequence (row g is row g % B of step g // B)."""
        B, L = self.cfg.batch_size, self.cfg.seq_len
        seq = torch.stack([torch.randint(0, self.vocab_size, (L + 1,), generator=counter_generator(self.cfg.seed, g // B, 1000 + g % B))
                           for g in range(first, first + count)])
        B = seq.shape[0]
        return Batch(tokens=seq[:, :-1].contiguous(), targets=seq[:, 1:].contiguous(),
                     target_valid=torch.ones(B, L, dtype=torch.bool), doc_ids=torch.zeros(B, L, dtype=torch.long),
                     single_doc=True)


def make_data(cfg: DataConfig, vocab_size: int, capacity: int | None = None):
    if cfg.kind == "synthetic":
        return SyntheticPackedData(cfg, vocab_size, capacity)
    if capacity is not None:
        raise ValueError(f"data.kind {cfg.kind!r}: the looped encoder-decoder's decoder positions are placed on data.kind 'synthetic'")
    if cfg.kind == "uniform":
        return UniformTokens(cfg, vocab_size)
    if cfg.kind == "shards":
        from .shards import ShardPacker
        from .shard_format import open_shards

        dirs = [cfg.shard_dir, *cfg.extra_shard_dirs]
        return ShardPacker(open_shards(dirs, order=cfg.union_order), cfg)
    raise ValueError(f"data.kind {cfg.kind!r}: 'synthetic', 'uniform' or 'shards'")
