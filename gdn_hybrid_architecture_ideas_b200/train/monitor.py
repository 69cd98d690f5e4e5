"""Run observability beside metrics.jsonl: a best-effort Weights & Biases logger, gradient norms per parameter family,
the depth-mix readers' state, the residual stream's RMS per layer, and named NVTX ranges around the step's phases.

Everything here is read-only with respect to training: a monitor never changes a gradient, a weight or the RNG, and a
logger that fails warns once and is dropped (reference: ced/train/trainer.py:4231-4260, 4717-4725 for W&B;
:3020-3070 for the family gradient norms; ced/model/attn_res.py:1390-1409 for the reader summary;
ced/model/encoder.py:1169 for the stream RMS).
"""

from __future__ import annotations

import contextlib

import torch

FAMILIES = (("embed", ("embed.", "out_embed.")), ("gdn", (".mixer.in_proj_", ".mixer.out_proj", ".mixer.conv_weight", ".mixer.A_log", ".mixer.dt_bias")),
            ("attention", (".mixer.q_proj", ".mixer.k_proj", ".mixer.v_proj", ".mixer.o_proj", ".mixer.g_proj")), ("mlp", (".mlp.",)),
            ("depth_mix", (".attn_res.", ".gdn_arms.")), ("norm", ("_norm.weight", "final_norm.")))


def family_of(name: str) -> str:
    for family, marks in FAMILIES:
        if any(m in name or name.startswith(m) for m in marks):
            return family
    return "other"


class WandbLogger:
    """W&B as an optional sink: `mode` "disabled" builds nothing; otherwise the package is imported and a run opened, and any
    failure (package absent, no network, a dead run) prints one line and turns the sink off. Training never waits on it."""

    def __init__(self, wcfg, run_id: str | None, config: dict, log=print, directory=None):
        self.run, self.run_id, self._log = None, run_id, log
        if wcfg.mode == "disabled":
            return
        try:
            import wandb

            self.run_id = run_id or wandb.util.generate_id()
            self.run = wandb.init(project=wcfg.project, entity=wcfg.entity, name=wcfg.run_name, id=self.run_id, resume="allow", mode=wcfg.mode,
                                  config=config, dir=None if directory is None else str(directory))
        except Exception as e:  # noqa: BLE001 - a logger must never stop a run
            log(f"W&B unavailable ({type(e).__name__}: {e}); continuing with metrics.jsonl only")
            self.run = None

    def call(self, method: str, *args, **kwargs) -> None:
        if self.run is None:
            return
        try:
            getattr(self.run, method)(*args, **kwargs)
        except Exception as e:  # noqa: BLE001
            self._log(f"W&B {method} failed ({type(e).__name__}: {e}); continuing without W&B")
            self.run = None

    def log(self, metrics: dict, step: int) -> None:
        self.call("log", {k: v for k, v in metrics.items() if isinstance(v, (int, float))}, step=step)

    def finish(self) -> None:
        self.call("finish")
        self.run = None


@torch.no_grad()
def family_grad_norms(flat) -> torch.Tensor:
    """Gradient norm per parameter family, before clipping, as ONE device tensor in FAMILIES order (+ "other"): the host
    reads it with the step's other numbers, so the monitor adds no synchronisation of its own."""
    names = [f for f, _ in FAMILIES] + ["other"]
    sums = {n: [] for n in names}
    for s in flat.segments:
        sums[family_of(s.name)].append(flat.grads[s.offset:s.offset + s.numel].float().pow(2).sum())
    zero = torch.zeros((), device=flat.grads.device)
    return torch.stack([torch.stack(v).sum().sqrt() if v else zero for v in (sums[n] for n in names)])


def family_names() -> list[str]:
    return [f for f, _ in FAMILIES] + ["other"]


@torch.no_grad()
def depth_reader_summary(model) -> dict:
    """Every depth-mix reader's pseudo-query norm (how far it has moved from the uniform mix it starts as) and its key gain's
    largest deviation from 1, by module name. Two host reads in all."""
    from ..models.depth_mix import DepthQuery

    items = [(n, m) for n, m in model.named_modules() if isinstance(m, DepthQuery)]
    if not items:
        return {}
    norms = torch.stack([torch.linalg.vector_norm(m.query.double()) for _, m in items]).cpu().tolist()
    gains = torch.stack([m.key_norm.weight.double().abs().max() for _, m in items]).cpu().tolist()
    return {"readers": [n for n, _ in items], "query_norm": norms, "key_gain_dev": gains}


@torch.no_grad()
def ccr_summary(model) -> dict:
    """The checkpoint cross-read's tensors as they are now: per reader layer its gate's values and, with a translator,
    ||M - I||_F per key head (0 at the start). One host read each (reference: ced/model/gdn_arms.py:1262-1314)."""
    rows = [(i, a) for i, a in ((i, getattr(layer, "gdn_arms", None)) for i, layer in enumerate(model.encoder.layers))
            if a is not None and a.ccr_read]
    if not rows:
        return {}
    out = {"layers": [i for i, _ in rows], "ccr_gate": torch.stack([a.ccr_gate.double() for _, a in rows]).cpu().tolist()}
    if any(a.translator != "none" for _, a in rows):
        out["ccr_translator_dev"] = torch.stack([torch.linalg.matrix_norm(a.ccr_translator_delta.double()) for _, a in rows]).cpu().tolist()
    return out


class StreamRMS:
    """Root-mean-square of the residual stream leaving each layer, collected by forward hooks during ONE forward
    (`with StreamRMS(model) as rms: ...; rms.values()`): the growth of the stream along the depth."""

    def __init__(self, model):
        self.model, self._handles, self._rms = model, [], []

    def __enter__(self):
        for layer in self.model.encoder.layers:
            self._handles.append(layer.register_forward_hook(self._hook))
        return self

    def _hook(self, module, args, out):
        x = out[0] if isinstance(out, tuple) else out
        if isinstance(x, torch.Tensor):
            self._rms.append(x.detach().float().pow(2).mean().sqrt())

    def __exit__(self, *exc):
        for h in self._handles:
            h.remove()
        self._handles = []

    def values(self) -> list[float]:
        return torch.stack(self._rms).cpu().tolist() if self._rms else []


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool = True):
    """A named range on the profiler timeline (forward+backward of a micro-batch, gradient synchronisation, optimizer)."""
    on = enabled and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()
