"""CUDA-graph replay of the training micro-batch (forward, fused head + loss, backward).

After `warmup` eager micro-batches the runner captures one micro-batch on static input buffers (tokens, targets,
document ids, valid mask, position-in-document, the 1 / n_targets scalar) and replays it for every later micro-batch
of the same shape: one graph launch in place of a few thousand kernel launches and the Python between them. The
gradients accumulate into the flat gradient buffer, which is static memory, so the optimizer (and the data-parallel
step) run outside the graph exactly as in eager mode. Capture needs fixed shapes and no host decision inside the
step, so it is refused (by name) with token superposition, shape schedules, tensor parallelism and activation
checkpointing modes that park tensors on the host (reference: ced/train/cuda_graphs.py:179-999, GraphRunner :414).
"""

from __future__ import annotations

import torch


def refusals(cfg, trainer) -> list[str]:
    bad = []
    if trainer.device.type != "cuda":
        bad.append("cuda_graphs needs a CUDA device")
    if cfg.tst.schedule:
        bad.append("cuda_graphs with tst.schedule (the bag size changes the step's shapes)")
    if cfg.shape_schedule:
        bad.append("cuda_graphs with shape_schedule")
    if cfg.tensor_parallel > 1:
        bad.append("cuda_graphs with tensor_parallel (the fused collectives carry per-call sequence numbers from the host)")
    if cfg.activation_checkpoint in ("host", "host_overlap"):
        bad.append("cuda_graphs with activation_checkpoint host modes (host copies are ordered by host events)")
    if any(getattr(m, "precision", "bf16") != "bf16" for m in trainer.model.modules()):
        bad.append("cuda_graphs with low-precision recipes (their non-finite flags are read on the host)")
    return bad


class GraphRunner:
    def __init__(self, trainer, warmup: int = 3):
        bad = refusals(trainer.cfg, trainer)
        if bad:
            raise ValueError("cuda_graphs refused: " + "; ".join(bad))
        self.trainer, self.warmup = trainer, warmup
        self.seen = 0
        self.graph = None
        self.static = None
        self.inv_n = torch.zeros((), dtype=torch.float32, device=trainer.device)
        self.out = None
        self.shape = None

    def _fill(self, mb, n_global: int):
        if self.static is None:
            self.static = mb.clone_static()
            self.shape = tuple(mb.tokens.shape)
        else:
            if tuple(mb.tokens.shape) != self.shape or mb.single_doc != self.static.single_doc:
                raise ValueError(f"cuda_graphs: micro-batch shape changed from {self.shape} to {tuple(mb.tokens.shape)}")
            self.static.copy_from(mb)
        self.inv_n.fill_(1.0 / max(n_global, 1))

    def micro(self, mb, n_global: int):
        """Runs one micro-batch (eagerly during warm-up, then by graph replay). Returns (loss, ce_sum) device tensors;
        gradients are accumulated into the flat gradient buffer either way."""
        t = self.trainer
        self._fill(mb, n_global)
        if self.graph is None and self.seen >= self.warmup:
            torch.cuda.synchronize(t.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                loss, ce = t._micro_loss(self.static, self.inv_n)
                loss.backward()
                self.out = torch.stack([loss.detach().float(), ce.float()])
            self.graph = graph
            # the capture pass itself ran no kernel: replay it for this micro-batch
        self.seen += 1
        if self.graph is not None:
            self.graph.replay()
            return self.out[0].clone(), self.out[1].clone()
        loss, ce = t._micro_loss(self.static, self.inv_n)
        loss.backward()
        return loss.detach().float(), ce.float()
